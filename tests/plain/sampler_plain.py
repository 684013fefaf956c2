"""Plain host sampler: the oracle of the device sampler, one row at a time in numpy.

The pipeline is the reference's (vllm-oxide, crates/vllm-oxide/src/sampler.rs:207-261): greedy
short-circuit for temperature 0 or top_k 1 (:228-230), logits * (1/T) (:235-238), top-k with ties
at the threshold kept (:349-364), top-p over the survivors (:373-408), Gumbel-max (:265-287),
argmax ties to the lowest index (:293-305).  Two rules are the engine's own and restated here:
uniforms come from a counter-based generator keyed per row, and top-p keeps every token whose
logit is >= the boundary token's (probability mass summed as 40-bit fixed point).
"""
import numpy as np

_GOLD = np.uint64(0x9E3779B97F4A7C15)
_M1 = np.uint64(0xBF58476D1CE4E5B9)
_M2 = np.uint64(0x94D049BB133111EB)


def counter_uniform(key: int, n: int) -> np.ndarray:
    with np.errstate(over="ignore"):
        idx = np.arange(1, n + 1, dtype=np.uint64)
        z = np.uint64(key) + idx * _GOLD
        z = (z ^ (z >> np.uint64(30))) * _M1
        z = (z ^ (z >> np.uint64(27))) * _M2
        z = z ^ (z >> np.uint64(31))
    return ((z >> np.uint64(40)).astype(np.float32) + np.float32(0.5)) * np.float32(1.0 / 16777216.0)


def apply_penalties(logits, history, presence, frequency, repetition):
    """sampler.rs:320-345: once per distinct token: /= repetition (if != 0), -= presence, -= frequency*count."""
    out = logits.astype(np.float32).copy()
    toks, counts = np.unique(np.asarray(history, dtype=np.int64), return_counts=True)
    for t, c in zip(toks, counts):
        if 0 <= t < len(out):
            if repetition != 0.0:
                out[t] = out[t] / np.float32(repetition)
            out[t] -= np.float32(presence)
            if frequency != 0.0:
                out[t] -= np.float32(frequency) * np.float32(c)
    return out


def surviving_mask(logits, temperature, top_k, top_p):
    """Which tokens can still be sampled after temperature, top-k and top-p."""
    V = len(logits)
    x = logits.astype(np.float32) * (np.float32(1.0) / np.float32(temperature))
    keep = np.ones(V, dtype=bool)
    if top_k and 1 <= top_k < V:
        thr = np.sort(x)[::-1][top_k - 1]
        keep &= x >= thr
    if top_p is not None and 0.0 < top_p < 1.0:
        mx = x[keep].max()
        mass = (np.exp((x - mx).astype(np.float32)).astype(np.float32) * np.float32(1099511627776.0)).astype(np.uint64)
        mass[~keep] = 0
        order = np.argsort(-x, kind="stable")
        order = order[keep[order]]
        cum = np.cumsum(mass[order], dtype=np.uint64)
        target = max(1, int(float(np.float32(top_p)) * float(int(cum[-1]))))
        boundary = int(np.searchsorted(cum, np.uint64(target), side="left"))
        keep &= x >= x[order[boundary]]
    return x, keep


def sample_row(logits, temperature, top_k, top_p, key):
    logits = np.asarray(logits, dtype=np.float32)
    if temperature <= 0.0 or top_k == 1:
        return int(np.argmax(logits))
    x, keep = surviving_mask(logits, temperature, top_k, top_p)
    u = counter_uniform(key, len(logits))
    g = -np.log(-np.log(u, dtype=np.float32), dtype=np.float32)
    score = np.where(keep, x + g, -np.inf).astype(np.float32)
    return int(np.argmax(score))
