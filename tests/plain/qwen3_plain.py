"""Plain, slow Qwen3 (dense) forward pass: whole sequences, no cache, one function per part.

This file is the oracle the engine is compared with.  It shares no code with the
package: it reads config.json and model.safetensors with its own few lines, and every
function restates one formula of the reference project (vllm-oxide, paths relative to
its root; `SRC/` = `crates/vllm-oxide/src/`).

It rests on the formulas only: the reference's model code is a Rust crate on candle that
cannot be compiled here (no Rust toolchain) and refuses to run attention without CUDA
(SRC/models/qwen3.rs:214-217), so no output of the reference's own code stands behind
these functions.  The closed-form vectors of the reference's unit tests are restated in
tests/test_plain.py.

`dt` is the model dtype.  With torch.bfloat16 every tensor is rounded where the reference
rounds it (after each matrix product, after the norm's division, after the rotation ...);
with torch.float32 or torch.float64 nothing is rounded below that type.
"""
import json
import math
import struct

import torch

_ST_DTYPES = {"F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16,
              "F64": torch.float64, "I32": torch.int32, "I64": torch.int64}


def read_folder(path):
    """config.json as a dict and model.safetensors as {name: tensor}.

    safetensors layout: 8-byte little-endian header length, JSON header
    {name: {dtype, shape, data_offsets}}, raw little-endian data.
    """
    with open(f"{path}/config.json") as f:
        cfg = json.load(f)
    with open(f"{path}/model.safetensors", "rb") as f:
        blob = f.read()
    (n,) = struct.unpack("<Q", blob[:8])
    header = json.loads(blob[8:8 + n])
    weights = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        a, b = meta["data_offsets"]
        t = torch.frombuffer(bytearray(blob[8 + n + a:8 + n + b]), dtype=_ST_DTYPES[meta["dtype"]])
        weights[name] = t.reshape(meta["shape"]).clone()
    return cfg, weights


def sizes(cfg):
    """The numbers of SRC/models/qwen3.rs:26-58 (head_dim falls back to hidden/heads, :48-51)."""
    hd = cfg.get("head_dim") or cfg["hidden_size"] // cfg["num_attention_heads"]
    return dict(H=cfg["hidden_size"], L=cfg["num_hidden_layers"], nh=cfg["num_attention_heads"],
                kvh=cfg["num_key_value_heads"], hd=hd, I=cfg["intermediate_size"],
                V=cfg["vocab_size"], eps=cfg["rms_norm_eps"],
                theta=cfg.get("rope_theta", 1_000_000.0),
                max_pos=cfg["max_position_embeddings"],
                tied=bool(cfg.get("tie_word_embeddings", False)))


def layer_window(cfg, layer):
    """Window of a layer, or None for all keys.

    The reference reads none of `use_sliding_window`, `sliding_window`,
    `max_window_layers` (SRC/models/qwen3.rs:26-44); the rule here is the architecture's
    own: with `use_sliding_window`, layers from `max_window_layers` on see the last
    `sliding_window` keys (the query's own position included).
    """
    if cfg.get("use_sliding_window") and cfg.get("sliding_window"):
        if layer >= cfg.get("max_window_layers", 0):
            return int(cfg["sliding_window"])
    return None


def _internal(dt):
    # SRC/layers/rmsnorm.rs:52-56: half types compute in f32, others stay as they are.
    return torch.float32 if dt in (torch.bfloat16, torch.float16) else dt


def embedding(table, token_ids, dt):
    """h0[t] = E[id[t]]  (SRC/models/qwen3.rs:296)."""
    return table.to(dt)[token_ids.long()]


def linear(x, w, dt, bias=None):
    """x @ W^T (+ b), W stored [out, in]  (SRC/layers/linear.rs:84-90).

    The product accumulates above `dt` and is rounded to `dt` once.
    """
    it = _internal(dt)
    y = x.to(it) @ w.to(dt).to(it).t()
    y = y.to(dt)
    if bias is not None:
        y = y + bias.to(dt)
    return y


def add_rms_norm(x, residual, weight, eps, dt):
    """(y, residual') of SRC/layers/rmsnorm.rs:51-81.

    s = x + residual in the internal type; residual' = s rounded to dt; y is computed from
    the unrounded s: (s / sqrt(mean(s^2) + eps)) rounded to dt, then times w in dt.
    With residual None no add happens and residual' = x (:65-69).
    """
    it = _internal(dt)
    if residual is None:
        s = x.to(it)
        new_res = x
    else:
        s = x.to(it) + residual.to(it)
        new_res = s.to(dt)
    var = (s * s).sum(-1, keepdim=True) / s.shape[-1]
    normed = s / torch.sqrt(var + eps)
    return normed.to(dt) * weight.to(dt), new_res


def split_qkv(qkv, nh, kvh, hd):
    """q, k, v as [T, heads, hd] from the merged product (SRC/models/qwen3.rs:161-170)."""
    T = qkv.shape[0]
    q = qkv[:, :nh * hd].reshape(T, nh, hd)
    k = qkv[:, nh * hd:(nh + kvh) * hd].reshape(T, kvh, hd)
    v = qkv[:, (nh + kvh) * hd:(nh + 2 * kvh) * hd].reshape(T, kvh, hd)
    return q, k, v


def head_rms_norm(x, weight, eps, dt):
    """q_norm / k_norm: RMSNorm over head_dim per head, no residual
    (SRC/models/qwen3.rs:171-178 with SRC/layers/rmsnorm.rs:51-81)."""
    return add_rms_norm(x, None, weight, eps, dt)[0]


def rope_table(hd, max_pos, theta):
    """[max_pos, hd] = cos || sin, all in f32 (SRC/layers/rope.rs:50-88).

    inv_freq[i] = 1 / theta^(2i/hd) with f32 pow; angle = f32(p) * inv_freq.
    """
    half = hd // 2
    i = torch.arange(half, dtype=torch.float32)
    inv_freq = 1.0 / torch.pow(torch.tensor(theta, dtype=torch.float32), (2 * i) / hd)
    t = torch.arange(max_pos, dtype=torch.float32)
    freqs = t[:, None] * inv_freq[None, :]
    return torch.cat([freqs.cos(), freqs.sin()], dim=-1)


def apply_rope(x, positions, table, dt):
    """Rotate-half over the whole head (SRC/layers/rope.rs:129-159).

    y = [x1*c - x2*s || x2*c + x1*s], computed above dt, rounded to dt.
    """
    it = torch.float64 if dt == torch.float64 else torch.float32
    hd = x.shape[-1]
    cs = table[positions.long()].to(it)
    c, s = cs[:, None, :hd // 2], cs[:, None, hd // 2:]
    xf = x.to(it)
    x1, x2 = xf[..., :hd // 2], xf[..., hd // 2:]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1).to(dt)


def attention(q, k, v, positions, window, dt):
    """Causal grouped-query attention of one whole sequence.

    Query head h reads kv head h // (nh/kvh); scale 1/sqrt(hd) (SRC/models/qwen3.rs:204);
    key j is seen by query i iff pos_j <= pos_i (SRC/attention/flash_attn.rs:26-36), and
    with a window iff also pos_i - pos_j < window.  Scores, softmax and the weighted sum
    are computed above dt; the result is rounded to dt.
    """
    it = _internal(dt)
    T, nh, hd = q.shape
    kvh = k.shape[1]
    g = nh // kvh
    scale = 1.0 / math.sqrt(hd)
    out = torch.empty(T, nh, hd, dtype=it, device=q.device)
    pi, pj = positions[:, None].long(), positions[None, :].long()
    allowed = pj <= pi
    if window is not None:
        allowed &= (pi - pj) < window
    for h in range(nh):
        s = (q[:, h].to(it) @ k[:, h // g].to(it).t()) * scale
        s = s.masked_fill(~allowed, float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[:, h] = p @ v[:, h // g].to(it)
    return out.to(dt).reshape(T, nh * hd)


def swiglu(x, w_gate, w_up, w_down, dt):
    """down( silu(gate(x)) * up(x) )  (SRC/models/qwen3.rs:82-86, SRC/layers/activation.rs:17-21).

    silu(z) = z / (1 + e^-z) evaluated above dt and rounded, then the product in dt.
    """
    it = _internal(dt)
    g = linear(x, w_gate, dt)
    u = linear(x, w_up, dt)
    gi = g.to(it)
    silu = (gi / (1.0 + torch.exp(-gi))).to(dt)
    return linear(silu * u, w_down, dt)


def lm_head(h, cfg, weights, dt):
    """logits = h @ Wlm^T in dt then f32 (SRC/models/qwen3.rs:322-331,384-386; SRC/engine/mod.rs:148)."""
    w = weights["model.embed_tokens.weight"] if sizes(cfg)["tied"] else weights["lm_head.weight"]
    return linear(h, w, dt).to(torch.float64 if dt == torch.float64 else torch.float32)


def decoder_layer(cfg, weights, i, hidden, residual, positions, table, dt, trace=None):
    """One layer in the reference's order (SRC/models/qwen3.rs:247-258): add+norm, attention,
    add+norm, feed-forward; returns (mlp output, residual)."""
    z = sizes(cfg)
    p = f"model.layers.{i}."
    normed, residual = add_rms_norm(hidden, residual, weights[p + "input_layernorm.weight"], z["eps"], dt)
    has_bias = bool(cfg.get("attention_bias", False))
    bias = (lambda n: weights[p + f"self_attn.{n}_proj.bias"]) if has_bias else (lambda n: None)
    q = linear(normed, weights[p + "self_attn.q_proj.weight"], dt, bias("q"))
    k = linear(normed, weights[p + "self_attn.k_proj.weight"], dt, bias("k"))
    v = linear(normed, weights[p + "self_attn.v_proj.weight"], dt, bias("v"))
    q, k, v = split_qkv(torch.cat([q, k, v], dim=-1), z["nh"], z["kvh"], z["hd"])
    q = head_rms_norm(q, weights[p + "self_attn.q_norm.weight"], z["eps"], dt)
    k = head_rms_norm(k, weights[p + "self_attn.k_norm.weight"], z["eps"], dt)
    q = apply_rope(q, positions, table, dt)
    k = apply_rope(k, positions, table, dt)
    a = attention(q, k, v, positions, layer_window(cfg, i), dt)
    a = linear(a, weights[p + "self_attn.o_proj.weight"], dt)
    normed, residual = add_rms_norm(a, residual, weights[p + "post_attention_layernorm.weight"], z["eps"], dt)
    m = swiglu(normed, weights[p + "mlp.gate_proj.weight"], weights[p + "mlp.up_proj.weight"],
               weights[p + "mlp.down_proj.weight"], dt)
    if trace is not None:
        trace.append(dict(q=q, k=k, v=v, attn=a, mlp=m, residual=residual))
    return m, residual


def forward_logits(cfg, weights, token_ids, dt=torch.float32, trace=None):
    """Logits [T, V] at every position of one whole sequence (SRC/models/qwen3.rs:295-304,384-386).

    Everything happens where the weights lie (the tests at the layer sizes of large checkpoints hand in
    weights on the GPU, so that a float64 run takes seconds); the table of angles is made on the CPU
    either way, so that its values do not depend on the device."""
    z = sizes(cfg)
    dev = weights["model.embed_tokens.weight"].device
    ids = torch.as_tensor(token_ids, dtype=torch.int64).to(dev)
    positions = torch.arange(len(ids)).to(dev)
    table = rope_table(z["hd"], z["max_pos"], z["theta"]).to(dev)
    hidden = embedding(weights["model.embed_tokens.weight"], ids, dt)
    residual = None
    for i in range(z["L"]):
        hidden, residual = decoder_layer(cfg, weights, i, hidden, residual, positions, table, dt, trace)
    hf, _ = add_rms_norm(hidden, residual, weights["model.norm.weight"], z["eps"], dt)
    return lm_head(hf, cfg, weights, dt)


def greedy_generate(cfg, weights, prompt, n_new, dt=torch.float32):
    """n_new tokens by argmax, lowest index on ties (SRC/sampler.rs:293-305), recomputing the
    whole sequence each time."""
    ids = list(prompt)
    out = []
    for _ in range(n_new):
        logits = forward_logits(cfg, weights, ids, dt)[-1]
        tok = int(torch.argmax(logits))  # torch returns the first maximum
        out.append(tok)
        ids.append(tok)
    return out
