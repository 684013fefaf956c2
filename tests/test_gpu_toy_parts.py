"""Generality of the parts: a toy architecture, defined HERE, is registered, built and stepped
without a change to the framework's files.

The toy model has a mixer with state of its own (a decaying sum per request, kept in the cache
manager's state slots, no pages), names one attention layer twice in its order (each run with a
cache plane of its own), and lets a last attention layer read the keys and values that the first
run wrote.  It is compared, whole and in portions and mixed with another request, with a plain
implementation written below from the plain parts.
"""
import math
from dataclasses import dataclass

import numpy as np
import pytest
import torch

from plain import qwen3_plain as P

pytestmark = pytest.mark.gpu

H, NH, KVH, HD, I, V, EPS, THETA, MAXPOS, DECAY = 48, 3, 1, 16, 72, 97, 1e-5, 1000.0, 256, 0.75


def register_toy():
    from vllm_oxide_b200.models import ExecStep, ModelPlan, register_architecture
    from vllm_oxide_b200.parts import Mixer, PartSpec, StateSpec, register_part
    from vllm_oxide_b200.weights import TensorSpec

    class DecayMixer(Mixer):
        """y_t = (s_t) W^T with s_t = decay * s_{t-1} + x_t, s kept per request in a state slot."""

        def __init__(self, hidden_size, decay, prefix, **_):
            self.H, self.decay, self.prefix = hidden_size, decay, prefix

        def tensor_specs(self):
            return [TensorSpec(self.prefix + "mix.weight", (self.H, self.H), "matrix", self.H)]

        def load(self, tensors):
            self.w = tensors[self.prefix + "mix.weight"]

        def state_spec(self):
            return StateSpec((self.H,), torch.float32)

        def forward(self, x, ctx, cache, state, write_cache=True):
            assert cache is None and state is not None
            cu = ctx.host_view("cu_q")
            slots = ctx.host_view("state_slots")
            out = torch.empty_like(x)
            for r in range(ctx.num_requests):
                s = state[int(slots[r])].clone()
                for t in range(int(cu[r]), int(cu[r + 1])):
                    s = self.decay * s + x[t].float()
                    out[t] = (s @ self.w.float().t()).to(x.dtype)
                state[int(slots[r])] = s
            return out

    register_part("mixer", "toy_decay", DecayMixer)

    @dataclass
    class ToyConfig:
        raw: dict

        @classmethod
        def from_dict(cls, d):
            return cls(d)

    def norm(name):
        return PartSpec("rmsnorm", dict(size=H, eps=EPS, weight_name=name))

    def toy_plan(cfg):
        def attn_layer(i):
            p = f"toy.layers.{i}."
            return PartSpec("pre_norm", dict(
                mixer=PartSpec("attention", dict(hidden_size=H, num_heads=NH, num_kv_heads=KVH, head_dim=HD, eps=EPS,
                                                 qkv_bias=False, qk_norm=True, window=None, position="rope",
                                                 prefix=p + "self_attn.")),
                feed_forward=PartSpec("swiglu", dict(hidden_size=H, intermediate_size=I, prefix=p + "mlp.")),
                input_norm=norm(p + "input_layernorm.weight"), post_mixer_norm=norm(p + "post_attention_layernorm.weight")))
        decay_layer = PartSpec("pre_norm", dict(
            mixer=PartSpec("toy_decay", dict(hidden_size=H, decay=DECAY, prefix="toy.layers.1.")),
            feed_forward=PartSpec("swiglu", dict(hidden_size=H, intermediate_size=I, prefix="toy.layers.1.mlp.")),
            input_norm=norm("toy.layers.1.input_layernorm.weight"),
            post_mixer_norm=norm("toy.layers.1.post_attention_layernorm.weight")))
        return ModelPlan(
            architecture="ToyDecayForCausalLM", hidden_size=H, vocab_size=V, max_position=MAXPOS,
            embedding_name="toy.embed.weight", lm_head_name=None, final_norm=norm("toy.norm.weight"),
            positions={"rope": PartSpec("rope", dict(head_dim=HD, max_position=MAXPOS, theta=THETA))},
            layers=[attn_layer(0), decay_layer, attn_layer(2)],
            # layer 0 runs twice (planes 0 and 2); layer 2 reads what the first run of layer 0 wrote
            order=[ExecStep(0, 0), ExecStep(1, 1), ExecStep(0, 2), ExecStep(2, 0, write_cache=False)])

    register_architecture("ToyDecayForCausalLM", ToyConfig.from_dict, toy_plan)


def plain_toy(weights, tokens, dt):
    """The toy model, whole sequence, from the plain parts."""
    ids = torch.as_tensor(tokens)
    pos = torch.arange(len(tokens))
    table = P.rope_table(HD, MAXPOS, THETA)
    hidden, residual = P.embedding(weights["toy.embed.weight"], ids, dt), None
    kept = {}

    def attn_block(i, hidden, residual, write_to=None, read_from=None):
        p = f"toy.layers.{i}."
        normed, residual = P.add_rms_norm(hidden, residual, weights[p + "input_layernorm.weight"], EPS, dt)
        q = P.linear(normed, weights[p + "self_attn.q_proj.weight"], dt)
        k = P.linear(normed, weights[p + "self_attn.k_proj.weight"], dt)
        v = P.linear(normed, weights[p + "self_attn.v_proj.weight"], dt)
        q, k, v = P.split_qkv(torch.cat([q, k, v], -1), NH, KVH, HD)
        q = P.apply_rope(P.head_rms_norm(q, weights[p + "self_attn.q_norm.weight"], EPS, dt), pos, table, dt)
        k = P.apply_rope(P.head_rms_norm(k, weights[p + "self_attn.k_norm.weight"], EPS, dt), pos, table, dt)
        if write_to is not None:
            kept[write_to] = (k, v)
        if read_from is not None:
            k, v = kept[read_from]
        a = P.linear(P.attention(q, k, v, pos, None, dt), weights[p + "self_attn.o_proj.weight"], dt)
        normed, residual = P.add_rms_norm(a, residual, weights[p + "post_attention_layernorm.weight"], EPS, dt)
        return P.swiglu(normed, weights[p + "mlp.gate_proj.weight"], weights[p + "mlp.up_proj.weight"],
                        weights[p + "mlp.down_proj.weight"], dt), residual

    hidden, residual = attn_block(0, hidden, residual, write_to=0)
    normed, residual = P.add_rms_norm(hidden, residual, weights["toy.layers.1.input_layernorm.weight"], EPS, dt)
    s = torch.zeros(H, dtype=torch.float32 if dt != torch.float64 else dt)
    mixed = torch.empty_like(normed)
    for t in range(len(tokens)):
        s = DECAY * s + normed[t].to(s.dtype)
        mixed[t] = (s @ weights["toy.layers.1.mix.weight"].to(dt).to(s.dtype).t()).to(dt)
    normed, residual = P.add_rms_norm(mixed, residual, weights["toy.layers.1.post_attention_layernorm.weight"], EPS, dt)
    hidden = P.swiglu(normed, weights["toy.layers.1.mlp.gate_proj.weight"], weights["toy.layers.1.mlp.up_proj.weight"],
                      weights["toy.layers.1.mlp.down_proj.weight"], dt)
    hidden, residual = attn_block(0, hidden, residual, write_to=2)
    hidden, residual = attn_block(2, hidden, residual, read_from=0)
    hf, _ = P.add_rms_norm(hidden, residual, weights["toy.norm.weight"], EPS, dt)
    return P.linear(hf, weights["toy.embed.weight"], dt).double().numpy()


@pytest.fixture(scope="module")
def toy_folder(tmp_path_factory):
    register_toy()
    from vllm_oxide_b200.engine.loading import write_random_model_folder
    folder = str(tmp_path_factory.mktemp("toy"))
    write_random_model_folder(folder, dict(architectures=["ToyDecayForCausalLM"]), 11, "fan_in", torch.float32)
    return folder


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_architecture_steps_like_its_plain_form(toy_folder, dtype):
    from vllm_oxide_b200.engine.trace import TraceRunner
    _, weights = P.read_folder(toy_folder)
    g = torch.Generator().manual_seed(4)
    a = torch.randint(0, V, (75,), generator=g).tolist()
    b = torch.randint(0, V, (40,), generator=g).tolist()
    dt = torch.float64 if dtype == "float32" else torch.bfloat16
    want_a, want_b = plain_toy(weights, a, dt), plain_toy(weights, b, dt)

    def close(got, want, what):
        scale = np.abs(want).max()
        worst = np.abs(np.asarray(got, np.float64) - want).max() / scale
        assert worst < (2e-5 if dtype == "float32" else 0.04), f"{what}: {worst:.3e}"

    r = TraceRunner(toy_folder, dtype, 128, 16)
    assert len(r.cache.planes) == 3 and r.cache.planes[1] is None and r.cache.states[1].shape[1:] == (H,)
    assert r.cache.states[0] is None and len(r.cache.groups) == 1 and r.cache.groups[0].planes == [0, 2]
    close(r.step([dict(id="a", tokens=a, want=list(range(75)))], ["a"]), want_a, "whole")
    # in portions, mixed with a second request whose state lives in another slot; b reuses a's slot later
    r = TraceRunner(toy_folder, dtype, 128, 16)
    got_a, got_b = [], []
    got_a.append(r.step([dict(id="a", tokens=a[:30], want=list(range(30)))], []))
    out = r.step([dict(id="a", tokens=a[30:33], want=[0, 1, 2]), dict(id="b", tokens=b[:17], want=list(range(17)))], [])
    got_a.append(out[:3]); got_b.append(out[3:])
    for t in range(33, 75):
        out = r.step([dict(id="a", tokens=[a[t]], want=[0])] + ([dict(id="b", tokens=[b[t - 16]], want=[0])] if t - 16 < 40 else []),
                     ["a"] if t == 74 else [])
        got_a.append(out[:1])
        if out.shape[0] > 1:
            got_b.append(out[1:])
    close(np.concatenate(got_a), want_a, "portions a")
    close(np.concatenate(got_b), want_b[:len(np.concatenate(got_b))], "portions b")
    # a new request takes the slot that a gave back: its state must start from zero
    c = r.step([dict(id="c", tokens=b, want=list(range(40)))], ["c"])
    close(c, want_b, "state slot used again")


E, RI, RL = 3, 40, 2          # experts, their width, layers of the routed toy


def toy_angles():
    """[max_pos, hd] = cos || sin of angles that grow linearly with the pair index (not a power law)."""
    i = torch.arange(HD // 2, dtype=torch.float32)
    t = torch.arange(MAXPOS, dtype=torch.float32)
    ang = t[:, None] * (0.02 * (i + 1.0))[None, :]
    return torch.cat([ang.cos(), ang.sin()], dim=-1)


def register_routed_toy():
    from vllm_oxide_b200.models import ExecStep, ModelPlan, register_architecture
    from vllm_oxide_b200.parts import FeedForward, PartSpec, PositionEncoding, register_part
    from vllm_oxide_b200.weights import TensorSpec

    class LinearAngles(PositionEncoding):
        """Another table for the attention part's rotation: the interface is `rotation_rule()`."""

        def __init__(self, device=None, **_):
            self.cos_sin = toy_angles().contiguous().to(device)

        def rotation_rule(self):
            from vllm_oxide_b200.parts import RotationRule
            return RotationRule(self.cos_sin, HD, False)

    class Top1Experts(FeedForward):
        """Each token goes to the expert with the largest router logit (float, ties to the lowest index):
        y = down_e(relu(up_e(x)))."""

        def __init__(self, hidden_size, width, experts, prefix, **_):
            self.H, self.W, self.E, self.prefix = hidden_size, width, experts, prefix

        def tensor_specs(self):
            p = self.prefix
            specs = [TensorSpec(p + "router.weight", (self.E, self.H), "norm")]          # kept in float
            for e in range(self.E):
                specs += [TensorSpec(f"{p}experts.{e}.up.weight", (self.W, self.H), "matrix", self.H),
                          TensorSpec(f"{p}experts.{e}.down.weight", (self.H, self.W), "matrix", self.W)]
            return specs

        def load(self, tensors):
            p = self.prefix
            self.router = tensors[p + "router.weight"]
            self.up = [tensors[f"{p}experts.{e}.up.weight"] for e in range(self.E)]
            self.down = [tensors[f"{p}experts.{e}.down.weight"] for e in range(self.E)]

        def forward(self, x, ctx):
            logits = x.float() @ self.router.float().t()
            choice = logits.argmax(dim=-1)
            out = torch.zeros_like(x)
            for e in range(self.E):
                rows = (choice == e).nonzero().flatten()
                if rows.numel():
                    h = torch.relu((x[rows].float() @ self.up[e].float().t()).to(x.dtype))
                    out[rows] = (h.float() @ self.down[e].float().t()).to(x.dtype)
            return out

    register_part("position", "toy_linear_angles", LinearAngles)
    register_part("feed_forward", "toy_top1", Top1Experts)

    @dataclass
    class RoutedConfig:
        raw: dict

        @classmethod
        def from_dict(cls, d):
            return cls(d)

    def norm(name):
        return PartSpec("rmsnorm", dict(size=H, eps=EPS, weight_name=name))

    def plan(cfg):
        def layer(i):
            p = f"routed.layers.{i}."
            return PartSpec("pre_norm", dict(
                mixer=PartSpec("attention", dict(hidden_size=H, num_heads=NH, num_kv_heads=KVH, head_dim=HD, eps=EPS,
                                                 qkv_bias=False, qk_norm=False, window=None, position="angles",
                                                 prefix=p + "self_attn.")),
                feed_forward=PartSpec("toy_top1", dict(hidden_size=H, width=RI, experts=E, prefix=p + "moe.")),
                input_norm=norm(p + "input_layernorm.weight"), post_mixer_norm=norm(p + "post_attention_layernorm.weight")))
        return ModelPlan(
            architecture="ToyRoutedForCausalLM", hidden_size=H, vocab_size=V, max_position=MAXPOS,
            embedding_name="routed.embed.weight", lm_head_name=None, final_norm=norm("routed.norm.weight"),
            positions={"angles": PartSpec("toy_linear_angles", {})},
            layers=[layer(i) for i in range(RL)], order=[ExecStep(i, i) for i in range(RL)])

    register_architecture("ToyRoutedForCausalLM", RoutedConfig.from_dict, plan)


def plain_routed(weights, tokens, dt):
    """The routed toy, whole sequence, from the plain parts; returns the logits and each layer's expert choices."""
    ids = torch.as_tensor(tokens)
    pos = torch.arange(len(tokens))
    table = toy_angles()
    it = torch.float64 if dt == torch.float64 else torch.float32
    hidden, residual = P.embedding(weights["routed.embed.weight"], ids, dt), None
    choices, margins = [], []
    for i in range(RL):
        p = f"routed.layers.{i}."
        normed, residual = P.add_rms_norm(hidden, residual, weights[p + "input_layernorm.weight"], EPS, dt)
        q = P.linear(normed, weights[p + "self_attn.q_proj.weight"], dt)
        k = P.linear(normed, weights[p + "self_attn.k_proj.weight"], dt)
        v = P.linear(normed, weights[p + "self_attn.v_proj.weight"], dt)
        q, k, v = P.split_qkv(torch.cat([q, k, v], -1), NH, KVH, HD)
        q, k = P.apply_rope(q, pos, table, dt), P.apply_rope(k, pos, table, dt)
        a = P.linear(P.attention(q, k, v, pos, None, dt), weights[p + "self_attn.o_proj.weight"], dt)
        normed, residual = P.add_rms_norm(a, residual, weights[p + "post_attention_layernorm.weight"], EPS, dt)
        logits = normed.to(it) @ weights[p + "moe.router.weight"].to(it).t()
        top = logits.topk(2, dim=-1).values
        margins.append((top[:, 0] - top[:, 1]).double())
        choice = logits.argmax(dim=-1)
        choices.append(choice)
        hidden = torch.zeros_like(normed)
        for e in range(E):
            rows = (choice == e).nonzero().flatten()
            if rows.numel():
                h = torch.relu(P.linear(normed[rows], weights[f"{p}moe.experts.{e}.up.weight"], dt))
                hidden[rows] = P.linear(h, weights[f"{p}moe.experts.{e}.down.weight"], dt)
    hf, _ = P.add_rms_norm(hidden, residual, weights["routed.norm.weight"], EPS, dt)
    return P.linear(hf, weights["routed.embed.weight"], dt).double().numpy(), choices, torch.stack(margins).min(dim=0).values


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_routed_feed_forward_and_another_position_encoding(tmp_path, dtype):
    register_routed_toy()
    from vllm_oxide_b200.engine.loading import write_random_model_folder
    from vllm_oxide_b200.engine.trace import TraceRunner
    folder = str(tmp_path / "routed")
    write_random_model_folder(folder, dict(architectures=["ToyRoutedForCausalLM"]), 23, "fan_in", torch.float32)
    _, weights = P.read_folder(folder)
    g = torch.Generator().manual_seed(9)
    a = torch.randint(0, V, (60,), generator=g).tolist()
    dt = torch.float64 if dtype == "float32" else torch.bfloat16
    want, choices, margin = plain_routed(weights, a, dt)
    assert all(len(set(c.tolist())) == E for c in choices), "every expert must be used, or routing is not tested"
    # a token whose two best router logits nearly tie may be routed otherwise after rounding: it is left out
    sure = (margin > (1e-4 if dtype == "float32" else 0.05)).numpy()
    assert sure.sum() > 40

    def close(got, what):
        scale = np.abs(want).max()
        worst = np.abs(np.asarray(got, np.float64) - want)[sure].max() / scale
        assert worst < (2e-5 if dtype == "float32" else 0.04), f"{what}: {worst:.3e}"

    r = TraceRunner(folder, dtype, 128, 16)
    close(r.step([dict(id="a", tokens=a, want=list(range(60)))], ["a"]), "whole")
    r = TraceRunner(folder, dtype, 128, 16)
    got = [r.step([dict(id="a", tokens=a[:37], want=list(range(37)))], [])]
    got.append(r.step([dict(id="a", tokens=a[37:39], want=[0, 1])], []))
    for t in range(39, 60):
        got.append(r.step([dict(id="a", tokens=[a[t]], want=[0])], []))
    close(np.concatenate(got), "portions and single tokens")


def test_unknown_parts_and_bad_orders_are_refused():
    register_toy()
    from vllm_oxide_b200.models import ExecStep, ModelPlan
    from vllm_oxide_b200.parts import PartSpec, build_part, known_parts
    assert "toy_decay" in known_parts("mixer") and "attention" in known_parts("mixer")
    with pytest.raises(KeyError, match="no mixer part of kind 'nope'"):
        build_part("mixer", PartSpec("nope"))
    plan = ModelPlan("x", 8, 8, 8, "e", None, PartSpec("rmsnorm"), {}, [PartSpec("pre_norm")],
                     [ExecStep(0, 0, write_cache=False)])
    with pytest.raises(ValueError, match="before any run has written"):
        plan.validate()
    plan.order = [ExecStep(0, 0), ExecStep(0, 0)]
    with pytest.raises(ValueError, match="written by two runs"):
        plan.validate()


# ---------------------------------------------------------------------------------------------------------------------
# Another position rule for the STOCK attention part: the first half of every head rotated in neighbouring pairs in one
# layer, no rotation at all in the next.  Only a plan is defined here; parts and kernels are the framework's.
ROT = HD // 2


def register_partial_rotary_toy():
    from vllm_oxide_b200.models import ExecStep, ModelPlan, register_architecture
    from vllm_oxide_b200.parts import PartSpec

    @dataclass
    class ToyConfig:
        raw: dict

        @classmethod
        def from_dict(cls, d):
            return cls(d)

    def norm(name):
        return PartSpec("rmsnorm", dict(size=H, eps=EPS, weight_name=name))

    def plan(cfg):
        def layer(i, position):
            p = f"toy.layers.{i}."
            return PartSpec("pre_norm", dict(
                mixer=PartSpec("attention", dict(hidden_size=H, num_heads=NH, num_kv_heads=KVH, head_dim=HD, eps=EPS,
                                                 qkv_bias=False, qk_norm=True, window=None, position=position,
                                                 prefix=p + "self_attn.")),
                feed_forward=PartSpec("swiglu", dict(hidden_size=H, intermediate_size=I, prefix=p + "mlp.")),
                input_norm=norm(p + "input_layernorm.weight"), post_mixer_norm=norm(p + "post_attention_layernorm.weight")))
        return ModelPlan(
            architecture="ToyPartialRotaryForCausalLM", hidden_size=H, vocab_size=V, max_position=MAXPOS,
            embedding_name="toy.embed.weight", lm_head_name=None, final_norm=norm("toy.norm.weight"),
            positions={"front_pairs": PartSpec("rope", dict(head_dim=HD, max_position=MAXPOS, theta=THETA, rotary_dim=ROT,
                                                            interleaved=True))},
            layers=[layer(0, "front_pairs"), layer(1, None)],
            order=[ExecStep(0, 0), ExecStep(1, 1)])

    register_architecture("ToyPartialRotaryForCausalLM", ToyConfig.from_dict, plan)


def plain_partial_rotary(weights, tokens, dt):
    """The same model from the plain parts; the rotation is restated here: elements 2i and 2i + 1 (i < ROT / 2) of a head
    turn by angle i of the position, the rest of the head passes through."""
    ids = torch.as_tensor(tokens)
    pos = torch.arange(len(tokens))
    table = P.rope_table(ROT, MAXPOS, THETA)           # [max_pos, ROT]: cos of ROT/2 angles, then sin

    def rotate_front_pairs(x):
        it = torch.float64 if dt == torch.float64 else torch.float32
        cs = table[pos].to(it)
        c, s = cs[:, None, :ROT // 2], cs[:, None, ROT // 2:]
        xf = x.to(it)
        x1, x2 = xf[..., 0:ROT:2], xf[..., 1:ROT:2]
        y = torch.stack([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1).flatten(-2)
        return torch.cat([y, xf[..., ROT:]], dim=-1).to(dt)

    hidden, residual = P.embedding(weights["toy.embed.weight"], ids, dt), None
    for i, rotate in ((0, rotate_front_pairs), (1, lambda x: x)):
        p = f"toy.layers.{i}."
        normed, residual = P.add_rms_norm(hidden, residual, weights[p + "input_layernorm.weight"], EPS, dt)
        q = P.linear(normed, weights[p + "self_attn.q_proj.weight"], dt)
        k = P.linear(normed, weights[p + "self_attn.k_proj.weight"], dt)
        v = P.linear(normed, weights[p + "self_attn.v_proj.weight"], dt)
        q, k, v = P.split_qkv(torch.cat([q, k, v], -1), NH, KVH, HD)
        q = rotate(P.head_rms_norm(q, weights[p + "self_attn.q_norm.weight"], EPS, dt))
        k = rotate(P.head_rms_norm(k, weights[p + "self_attn.k_norm.weight"], EPS, dt))
        a = P.linear(P.attention(q, k, v, pos, None, dt), weights[p + "self_attn.o_proj.weight"], dt)
        normed, residual = P.add_rms_norm(a, residual, weights[p + "post_attention_layernorm.weight"], EPS, dt)
        hidden = P.swiglu(normed, weights[p + "mlp.gate_proj.weight"], weights[p + "mlp.up_proj.weight"],
                          weights[p + "mlp.down_proj.weight"], dt)
    hf, _ = P.add_rms_norm(hidden, residual, weights["toy.norm.weight"], EPS, dt)
    return P.linear(hf, weights["toy.embed.weight"], dt).double().numpy()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_another_position_rule_needs_only_a_plan(tmp_path, dtype):
    """Partial rotation in neighbouring pairs in one layer and no rotation in the other, with the stock attention part
    and its kernels: whole, and decoded token by token after a portion, against the plain form above."""
    from vllm_oxide_b200.engine.loading import write_random_model_folder
    from vllm_oxide_b200.engine.trace import TraceRunner
    register_partial_rotary_toy()
    folder = str(tmp_path / "partial")
    write_random_model_folder(folder, dict(architectures=["ToyPartialRotaryForCausalLM"]), 21, "fan_in", torch.float32)
    _, weights = P.read_folder(folder)
    g = torch.Generator().manual_seed(6)
    toks = torch.randint(0, V, (70,), generator=g).tolist()
    dt = torch.float64 if dtype == "float32" else torch.bfloat16
    want = plain_partial_rotary(weights, toks, dt)
    scale = np.abs(want).max()
    bound = 2e-5 if dtype == "float32" else 0.04
    r = TraceRunner(folder, dtype, 80, 16)
    whole = r.step([dict(id="w", tokens=toks, want=list(range(70)))], ["w"])
    assert np.abs(whole.astype(np.float64) - want).max() / scale < bound
    rows = [r.step([dict(id="d", tokens=toks[:37], want=list(range(37)))], [])]
    rows += [r.step([dict(id="d", tokens=[t], want=[0])], []) for t in toks[37:]]
    assert np.abs(np.concatenate(rows).astype(np.float64) - want).max() / scale < bound
    # and the rule matters: the stock rule on the same weights gives other logits
    assert np.abs(want - plain_toy_stock_rule(weights, toks, dt)).max() / scale > 3 * bound


def plain_toy_stock_rule(weights, tokens, dt):
    """The two layers with the reference's rule (the whole head in halves, both layers), to show that the test above
    would see a rule that was not applied."""
    ids = torch.as_tensor(tokens)
    pos = torch.arange(len(tokens))
    table = P.rope_table(HD, MAXPOS, THETA)
    hidden, residual = P.embedding(weights["toy.embed.weight"], ids, dt), None
    for i in (0, 1):
        p = f"toy.layers.{i}."
        normed, residual = P.add_rms_norm(hidden, residual, weights[p + "input_layernorm.weight"], EPS, dt)
        q = P.linear(normed, weights[p + "self_attn.q_proj.weight"], dt)
        k = P.linear(normed, weights[p + "self_attn.k_proj.weight"], dt)
        v = P.linear(normed, weights[p + "self_attn.v_proj.weight"], dt)
        q, k, v = P.split_qkv(torch.cat([q, k, v], -1), NH, KVH, HD)
        q = P.apply_rope(P.head_rms_norm(q, weights[p + "self_attn.q_norm.weight"], EPS, dt), pos, table, dt)
        k = P.apply_rope(P.head_rms_norm(k, weights[p + "self_attn.k_norm.weight"], EPS, dt), pos, table, dt)
        a = P.linear(P.attention(q, k, v, pos, None, dt), weights[p + "self_attn.o_proj.weight"], dt)
        normed, residual = P.add_rms_norm(a, residual, weights[p + "post_attention_layernorm.weight"], EPS, dt)
        hidden = P.swiglu(normed, weights[p + "mlp.gate_proj.weight"], weights[p + "mlp.up_proj.weight"],
                          weights[p + "mlp.down_proj.weight"], dt)
    hf, _ = P.add_rms_norm(hidden, residual, weights["toy.norm.weight"], EPS, dt)
    return P.linear(hf, weights["toy.embed.weight"], dt).double().numpy()


# ---------------------------------------------------------------------------------------------------------------------
# A mixer that keeps ONE tensor a token in pages (a latent), in pages of its own size and in float32, beside a stock
# attention layer that keeps keys and values in the engine's pages: two cache groups, two block tables per request.
LW, LATENT_PAGE = 24, 8


def register_latent_toy():
    from vllm_oxide_b200.models import ExecStep, ModelPlan, register_architecture
    from vllm_oxide_b200.parts import CacheSpec, Mixer, PartSpec, register_part
    from vllm_oxide_b200.weights import TensorSpec

    class LatentMeanMixer(Mixer):
        """c_t = x_t Wc^T is written to the pages (one float32 tensor of LW elements a token); y_t = mean(c_0..c_t) Wo^T
        is computed from the pages through the block table, so it sees earlier portions and nothing of other requests."""

        def __init__(self, hidden_size, latent, prefix, **_):
            self.H, self.L, self.prefix = hidden_size, latent, prefix

        def tensor_specs(self):
            return [TensorSpec(self.prefix + "compress.weight", (self.L, self.H), "matrix", self.H),
                    TensorSpec(self.prefix + "expand.weight", (self.H, self.L), "matrix", self.L)]

        def load(self, tensors):
            self.wc, self.wo = tensors[self.prefix + "compress.weight"], tensors[self.prefix + "expand.weight"]

        def cache_spec(self):
            return CacheSpec(kv_heads=1, head_dim=self.L, tensors=1, block_size=LATENT_PAGE, dtype=torch.float32)

        def forward(self, x, ctx, cache, state, write_cache=True):
            assert cache.v is None and cache.k.dtype == torch.float32 and cache.block_size == LATENT_PAGE
            T = ctx.num_tokens
            c = x[:T].float() @ self.wc.float().t()
            flat = cache.k.view(-1, self.L)                                  # [pages * page size, L]: one row a slot
            flat[ctx.slot_mapping[cache.group][:T].long()] = c
            cu, lens = ctx.host_view("cu_q"), ctx.host_view("context_lens")
            out = torch.zeros_like(x)
            for r in range(ctx.num_requests):
                n, end = int(cu[r + 1] - cu[r]), int(lens[r])
                pages = ctx.block_tables[cache.group][r, :(end + LATENT_PAGE - 1) // LATENT_PAGE].long()
                seen = cache.k[pages].reshape(-1, self.L)[:end]              # the latents of positions 0 .. end-1
                means = seen.cumsum(0)[end - n:] / torch.arange(end - n + 1, end + 1, device=x.device)[:, None]
                out[int(cu[r]):int(cu[r + 1])] = (means @ self.wo.float().t()).to(x.dtype)
            return out

    register_part("mixer", "toy_latent_mean", LatentMeanMixer)

    @dataclass
    class ToyConfig:
        raw: dict

        @classmethod
        def from_dict(cls, d):
            return cls(d)

    def norm(name):
        return PartSpec("rmsnorm", dict(size=H, eps=EPS, weight_name=name))

    def plan(cfg):
        def layer(i, mixer):
            p = f"toy.layers.{i}."
            return PartSpec("pre_norm", dict(
                mixer=mixer(p), feed_forward=PartSpec("swiglu", dict(hidden_size=H, intermediate_size=I, prefix=p + "mlp.")),
                input_norm=norm(p + "input_layernorm.weight"), post_mixer_norm=norm(p + "post_attention_layernorm.weight")))
        attention = lambda p: PartSpec("attention", dict(hidden_size=H, num_heads=NH, num_kv_heads=KVH, head_dim=HD, eps=EPS,
                                                        qkv_bias=False, qk_norm=True, window=None, position="rope",
                                                        prefix=p + "self_attn."))
        latent = lambda p: PartSpec("toy_latent_mean", dict(hidden_size=H, latent=LW, prefix=p + "latent."))
        return ModelPlan(
            architecture="ToyLatentForCausalLM", hidden_size=H, vocab_size=V, max_position=MAXPOS,
            embedding_name="toy.embed.weight", lm_head_name=None, final_norm=norm("toy.norm.weight"),
            positions={"rope": PartSpec("rope", dict(head_dim=HD, max_position=MAXPOS, theta=THETA))},
            layers=[layer(0, attention), layer(1, latent)], order=[ExecStep(0, 0), ExecStep(1, 1)])

    register_architecture("ToyLatentForCausalLM", ToyConfig.from_dict, plan)


def plain_latent_toy(weights, tokens, dt):
    ids = torch.as_tensor(tokens)
    pos = torch.arange(len(tokens))
    table = P.rope_table(HD, MAXPOS, THETA)
    hidden, residual = P.embedding(weights["toy.embed.weight"], ids, dt), None
    p = "toy.layers.0."
    normed, residual = P.add_rms_norm(hidden, residual, weights[p + "input_layernorm.weight"], EPS, dt)
    q = P.linear(normed, weights[p + "self_attn.q_proj.weight"], dt)
    k = P.linear(normed, weights[p + "self_attn.k_proj.weight"], dt)
    v = P.linear(normed, weights[p + "self_attn.v_proj.weight"], dt)
    q, k, v = P.split_qkv(torch.cat([q, k, v], -1), NH, KVH, HD)
    q = P.apply_rope(P.head_rms_norm(q, weights[p + "self_attn.q_norm.weight"], EPS, dt), pos, table, dt)
    k = P.apply_rope(P.head_rms_norm(k, weights[p + "self_attn.k_norm.weight"], EPS, dt), pos, table, dt)
    a = P.linear(P.attention(q, k, v, pos, None, dt), weights[p + "self_attn.o_proj.weight"], dt)
    normed, residual = P.add_rms_norm(a, residual, weights[p + "post_attention_layernorm.weight"], EPS, dt)
    hidden = P.swiglu(normed, weights[p + "mlp.gate_proj.weight"], weights[p + "mlp.up_proj.weight"],
                      weights[p + "mlp.down_proj.weight"], dt)
    p = "toy.layers.1."
    normed, residual = P.add_rms_norm(hidden, residual, weights[p + "input_layernorm.weight"], EPS, dt)
    it = torch.float64 if dt == torch.float64 else torch.float32
    c = normed.to(it) @ weights[p + "latent.compress.weight"].to(dt).to(it).t()
    means = c.cumsum(0) / torch.arange(1, len(tokens) + 1)[:, None]
    mixed = (means @ weights[p + "latent.expand.weight"].to(dt).to(it).t()).to(dt)
    normed, residual = P.add_rms_norm(mixed, residual, weights[p + "post_attention_layernorm.weight"], EPS, dt)
    hidden = P.swiglu(normed, weights[p + "mlp.gate_proj.weight"], weights[p + "mlp.up_proj.weight"],
                      weights[p + "mlp.down_proj.weight"], dt)
    hf, _ = P.add_rms_norm(hidden, residual, weights["toy.norm.weight"], EPS, dt)
    return P.linear(hf, weights["toy.embed.weight"], dt).double().numpy()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_mixer_with_one_tensor_a_token_in_pages_of_its_own_size(tmp_path, dtype):
    """The cache allocates what each plane's spec states: keys and values in the engine's pages for the attention layer,
    ONE float32 tensor a token in pages of 8 for the toy mixer; each group has its own pool and block tables, pages of
    both are given back and used again, and the logits are the plain form's, whole and cut and mixed."""
    from vllm_oxide_b200.engine.loading import write_random_model_folder
    from vllm_oxide_b200.engine.trace import TraceRunner
    register_latent_toy()
    folder = str(tmp_path / "latent")
    write_random_model_folder(folder, dict(architectures=["ToyLatentForCausalLM"]), 31, "fan_in", torch.float32)
    _, weights = P.read_folder(folder)
    g = torch.Generator().manual_seed(8)
    reqs = {name: torch.randint(0, V, (n,), generator=g).tolist() for name, n in (("a", 61), ("b", 30), ("c", 45))}
    dt = torch.float64 if dtype == "float32" else torch.bfloat16
    want = {name: plain_latent_toy(weights, toks, dt) for name, toks in reqs.items()}

    def close(got, w, what):
        worst = np.abs(np.asarray(got, np.float64) - w).max() / np.abs(w).max()
        assert worst < (2e-5 if dtype == "float32" else 0.04), f"{what}: {worst:.3e}"

    r = TraceRunner(folder, dtype, 96, 16)                       # 6 pages of 16, and 12 pages of 8 for the latents
    kv, latent = r.cache.planes
    assert len(r.cache.groups) == 2 and {(g.block_size, g.num_blocks) for g in r.cache.groups} == {(16, 6), (8, 12)}
    assert latent.v is None and latent.data.shape == (1, 12, 1, 8, LW) and latent.data.dtype == torch.float32
    assert kv.v is not None and kv.data.shape == (2, 6, KVH, 16, HD) and kv.group != latent.group
    assert not r.manager.prefix_caching
    close(r.step([dict(id="a", tokens=reqs["a"], want=list(range(61)))], ["a"]), want["a"], "whole")
    # a in portions beside b; then c on the pages both gave back
    got = {name: [] for name in reqs}
    out = r.step([dict(id="a", tokens=reqs["a"][:19], want=list(range(19)))], [])
    got["a"].append(out)
    out = r.step([dict(id="a", tokens=reqs["a"][19:21], want=[0, 1]), dict(id="b", tokens=reqs["b"][:9], want=list(range(9)))], [])
    got["a"].append(out[:2]); got["b"].append(out[2:])
    for t in range(21, 61):
        entries = [dict(id="a", tokens=[reqs["a"][t]], want=[0])]
        if t - 12 < 30:
            entries.append(dict(id="b", tokens=[reqs["b"][t - 12]], want=[0]))
        out = r.step(entries, [e["id"] for e in entries if (e["id"] == "a" and t == 60) or (e["id"] == "b" and t - 12 == 29)])
        got["a"].append(out[:1])
        if len(entries) > 1:
            got["b"].append(out[1:])
        assert r.manager.check_invariants() == ""
    got["c"].append(r.step([dict(id="c", tokens=reqs["c"][:40], want=list(range(40)))], []))
    got["c"].append(r.step([dict(id="c", tokens=reqs["c"][40:], want=list(range(5)))], ["c"]))
    for name in reqs:
        close(np.concatenate(got[name]), want[name], f"cut and mixed {name}")
    assert r.manager.num_free_blocks(0) + r.manager.num_free_blocks(1) == 18


# ---------------------------------------------------------------------------------------------------------------------
# What a plan may say beyond its layers: a scale on the embedded tokens, a soft cap on the logits, and a position part
# that adds learned absolute positions to the embedding (its table is a tensor of the checkpoint) while the attention
# layers rotate nothing.
EMB_SCALE, SOFTCAP = math.sqrt(H), 7.5


def register_absolute_toy():
    from vllm_oxide_b200.models import ExecStep, ModelPlan, register_architecture
    from vllm_oxide_b200.parts import PartSpec, PositionEncoding, register_part
    from vllm_oxide_b200.weights import TensorSpec

    class LearnedPositions(PositionEncoding):
        """hidden[t] += table[position[t]]: one row of a learned table per token, added right after the embedding."""
        graph_safe = True       # the same operations whatever the batch holds (rows beyond the batch get row 0)

        def __init__(self, size, max_position, name, **_):
            self.size, self.max_position, self.name = size, max_position, name

        def tensor_specs(self):
            return [TensorSpec(self.name, (self.max_position, self.size), "embedding")]

        def load(self, tensors):
            self.table = tensors[self.name]

        def embed(self, hidden, ctx):
            pos = ctx.positions[:hidden.shape[0]].clamp(0, self.max_position - 1).long()
            hidden += self.table[pos]

    register_part("position", "toy_learned", LearnedPositions)

    @dataclass
    class ToyConfig:
        raw: dict

        @classmethod
        def from_dict(cls, d):
            return cls(d)

    def norm(name):
        return PartSpec("rmsnorm", dict(size=H, eps=EPS, weight_name=name))

    def plan(cfg):
        def layer(i):
            p = f"toy.layers.{i}."
            return PartSpec("pre_norm", dict(
                mixer=PartSpec("attention", dict(hidden_size=H, num_heads=NH, num_kv_heads=KVH, head_dim=HD, eps=EPS,
                                                 qkv_bias=False, qk_norm=True, window=None, position=None,
                                                 prefix=p + "self_attn.")),
                feed_forward=PartSpec("swiglu", dict(hidden_size=H, intermediate_size=I, prefix=p + "mlp.")),
                input_norm=norm(p + "input_layernorm.weight"), post_mixer_norm=norm(p + "post_attention_layernorm.weight")))
        return ModelPlan(
            architecture="ToyAbsoluteForCausalLM", hidden_size=H, vocab_size=V, max_position=MAXPOS,
            embedding_name="toy.embed.weight", lm_head_name=None, final_norm=norm("toy.norm.weight"),
            positions={"learned": PartSpec("toy_learned", dict(size=H, max_position=MAXPOS, name="toy.positions.weight"))},
            layers=[layer(0), layer(1)], order=[ExecStep(0, 0), ExecStep(1, 1)],
            embedding_scale=EMB_SCALE, logit_softcap=SOFTCAP)

    register_architecture("ToyAbsoluteForCausalLM", ToyConfig.from_dict, plan)


def plain_absolute_toy(weights, tokens, dt):
    ids = torch.as_tensor(tokens)
    pos = torch.arange(len(tokens))
    it = torch.float64 if dt == torch.float64 else torch.float32
    emb = (P.embedding(weights["toy.embed.weight"], ids, dt).to(it) * EMB_SCALE).to(dt)
    hidden = (emb.to(it) + weights["toy.positions.weight"].to(dt)[pos].to(it)).to(dt)
    residual = None
    for i in (0, 1):
        p = f"toy.layers.{i}."
        normed, residual = P.add_rms_norm(hidden, residual, weights[p + "input_layernorm.weight"], EPS, dt)
        q = P.linear(normed, weights[p + "self_attn.q_proj.weight"], dt)
        k = P.linear(normed, weights[p + "self_attn.k_proj.weight"], dt)
        v = P.linear(normed, weights[p + "self_attn.v_proj.weight"], dt)
        q, k, v = P.split_qkv(torch.cat([q, k, v], -1), NH, KVH, HD)
        q = P.head_rms_norm(q, weights[p + "self_attn.q_norm.weight"], EPS, dt)
        k = P.head_rms_norm(k, weights[p + "self_attn.k_norm.weight"], EPS, dt)
        a = P.linear(P.attention(q, k, v, pos, None, dt), weights[p + "self_attn.o_proj.weight"], dt)
        normed, residual = P.add_rms_norm(a, residual, weights[p + "post_attention_layernorm.weight"], EPS, dt)
        hidden = P.swiglu(normed, weights[p + "mlp.gate_proj.weight"], weights[p + "mlp.up_proj.weight"],
                          weights[p + "mlp.down_proj.weight"], dt)
    hf, _ = P.add_rms_norm(hidden, residual, weights["toy.norm.weight"], EPS, dt)
    logits = P.linear(hf, weights["toy.embed.weight"], dt).double()
    return (SOFTCAP * torch.tanh(logits / SOFTCAP)).numpy()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_plan_with_an_embedding_scale_a_soft_cap_and_learned_positions(tmp_path, dtype):
    """Nothing of the model walk is edited for it: the plan carries the two constants, the position part brings its
    table with the checkpoint and adds it after the embedding.  Whole, and decoded token by token (from CUDA graphs)."""
    from vllm_oxide_b200.engine.loading import write_random_model_folder
    from vllm_oxide_b200.engine.trace import TraceRunner
    register_absolute_toy()
    folder = str(tmp_path / "absolute")
    write_random_model_folder(folder, dict(architectures=["ToyAbsoluteForCausalLM"]), 41, "fan_in", torch.float32)
    _, weights = P.read_folder(folder)
    assert weights["toy.positions.weight"].shape == (MAXPOS, H)
    g = torch.Generator().manual_seed(10)
    toks = torch.randint(0, V, (60,), generator=g).tolist()
    dt = torch.float64 if dtype == "float32" else torch.bfloat16
    want = plain_absolute_toy(weights, toks, dt)
    assert np.abs(want).max() < SOFTCAP and np.abs(want).max() > 0.8 * SOFTCAP        # the cap is at work
    bound = 2e-5 if dtype == "float32" else 0.04
    r = TraceRunner(folder, dtype, 64, 16)
    whole = r.step([dict(id="w", tokens=toks, want=list(range(60)))], ["w"])
    assert np.abs(whole.astype(np.float64) - want).max() / SOFTCAP < bound
    rows = [r.step([dict(id="d", tokens=toks[:21], want=list(range(21)))], [])]
    rows += [r.step([dict(id="d", tokens=[t], want=[0])], ["d"] if n == 59 else []) for n, t in enumerate(toks) if n >= 21]
    assert np.abs(np.concatenate(rows).astype(np.float64) - want).max() / SOFTCAP < bound
    assert r.core.graph_replays > 0
    # the positions matter: the same tokens at other positions give other logits
    shifted = r.step([dict(id="s", tokens=toks[5:25], want=list(range(20)))], ["s"])
    assert np.abs(shifted.astype(np.float64) - want[5:25]).max() / SOFTCAP > 3 * bound
