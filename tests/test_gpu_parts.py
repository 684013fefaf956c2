"""Each part alone, built from a PartSpec with sizes that are not the engine's, against the plain part."""
import math

import pytest
import torch

from helpers import make_context
from plain import qwen3_plain as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype):
    return dict(rtol=1e-4, atol=1e-4) if dtype == torch.float32 else dict(rtol=3e-2, atol=3e-2)


def manager_with(requests, bs=16, pages=32, windows=(0,)):
    from vllm_oxide_b200 import host
    m = host.KvCacheManager([host.GroupSpec(bs, pages, w) for w in windows], 8, False)
    for rid, n in requests:
        m.add_request(rid)
        assert m.ensure(rid, 0, n)
    return m


@pytest.mark.parametrize("dtype", DTYPES)
def test_rmsnorm_part(dtype):
    from vllm_oxide_b200.parts import PartSpec, build_part
    norm = build_part("norm", PartSpec("rmsnorm", dict(size=88, eps=2e-5, weight_name="n.weight")))
    assert [(s.name, s.shape, s.role) for s in norm.tensor_specs()] == [("n.weight", (88,), "norm")]
    w = (1 + 0.1 * torch.randn(88)).to(dtype).float()
    norm.load({"n.weight": w.to(DEV)})
    ctx = make_context(manager_with([(0, 6)]), [(0, 0, range(6), [5])], dtype)
    x, res = torch.randn(6, 88).to(dtype), torch.randn(6, 88).to(dtype)
    y, r = norm.forward(x.to(DEV), None, ctx)
    wy, wr = P.add_rms_norm(x, None, w.to(dtype), 2e-5, dtype)
    assert torch.allclose(y.cpu().float(), wy.float(), **tol(dtype)) and torch.equal(r.cpu(), x)
    y2, r2 = norm.forward(x.to(DEV), res.to(DEV).clone(), ctx)
    wy, wr = P.add_rms_norm(x, res, w.to(dtype), 2e-5, dtype)
    assert torch.allclose(y2.cpu().float(), wy.float(), **tol(dtype)) and torch.allclose(r2.cpu().float(), wr.float(), atol=1e-6)


def test_rope_part_table_is_the_plain_table():
    from vllm_oxide_b200.parts import PartSpec, build_part
    for hd, n, theta in [(16, 64, 1e4), (48, 300, 5e5), (128, 4096, 1e6)]:
        rope = build_part("position", PartSpec("rope", dict(head_dim=hd, max_position=n, theta=theta)), device=DEV)
        assert torch.equal(rope.cos_sin.cpu(), P.rope_table(hd, n, theta))
    with pytest.raises(ValueError, match="even"):
        build_part("position", PartSpec("rope", dict(head_dim=15, max_position=8, theta=1e4)), device=DEV)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window,bias", [(None, False), (9, False), (None, True)])
def test_attention_part(dtype, window, bias):
    """The mixer alone: two requests, one whole and one continuing from a cached portion."""
    from vllm_oxide_b200.parts import CachePlane, PartSpec, build_part
    Hd, nh, kvh, hd, eps = 40, 6, 3, 16, 1e-5
    rope = build_part("position", PartSpec("rope", dict(head_dim=hd, max_position=128, theta=777.0)), device=DEV)
    att = build_part("mixer", PartSpec("attention", dict(hidden_size=Hd, num_heads=nh, num_kv_heads=kvh, head_dim=hd, eps=eps,
                                                           qkv_bias=bias, qk_norm=not bias, window=window, position="r",
                                                           prefix="x.")),
                     positions={"r": rope}, dtype=dtype, device=DEV)
    g = torch.Generator().manual_seed(3)
    tensors = {}
    for s in att.tensor_specs():
        t = torch.randn(s.shape, generator=g)
        t = (1 + 0.1 * t) if s.role == "norm" else t / math.sqrt(s.shape[-1]) if s.role == "matrix" else 0.1 * t
        tensors[s.name] = t.to(dtype).float() if s.role == "norm" else t.to(dtype)
    att.load({k: v.to(DEV) for k, v in tensors.items()})
    assert att.cache_spec().window == (window or 0) and att.cache_spec().kv_heads == kvh
    m = manager_with([(0, 21), (1, 50)], windows=(window or 0,))
    plane = CachePlane(torch.zeros(32, kvh, 16, hd, dtype=dtype, device=DEV), torch.zeros(32, kvh, 16, hd, dtype=dtype, device=DEV), 0, 16)
    xa, xb = torch.randn(21, Hd, generator=g).to(dtype), torch.randn(50, Hd, generator=g).to(dtype)

    def plain(x):
        n = x.shape[0]
        b = (lambda k: tensors[f"x.{k}_proj.bias"]) if bias else (lambda k: None)
        q = P.linear(x, tensors["x.q_proj.weight"], dtype, b("q"))
        k = P.linear(x, tensors["x.k_proj.weight"], dtype, b("k"))
        v = P.linear(x, tensors["x.v_proj.weight"], dtype, b("v"))
        q, k, v = P.split_qkv(torch.cat([q, k, v], -1), nh, kvh, hd)
        if not bias:
            q = P.head_rms_norm(q, tensors["x.q_norm.weight"].to(dtype), eps, dtype)
            k = P.head_rms_norm(k, tensors["x.k_norm.weight"].to(dtype), eps, dtype)
        table = P.rope_table(hd, 128, 777.0)
        pos = torch.arange(n)
        q, k = P.apply_rope(q, pos, table, dtype), P.apply_rope(k, pos, table, dtype)
        return P.linear(P.attention(q, k, v, pos, window, dtype), tensors["x.o_proj.weight"], dtype)

    # step 1: request 1's first 30 tokens; step 2: request 0 whole beside the rest of request 1
    ctx = make_context(m, [(1, 0, range(30), [])], dtype)
    out1 = att.forward(xb[:30].to(DEV), ctx, plane, None).cpu()
    ctx = make_context(m, [(0, 0, range(21), []), (1, 30, range(20), [])], dtype)
    out2 = att.forward(torch.cat([xa, xb[30:]]).to(DEV), ctx, plane, None).cpu()
    assert ctx.err.item() == 0
    wa, wb = plain(xa), plain(xb)
    assert torch.allclose(out2[:21].float(), wa.float(), **tol(dtype))
    assert torch.allclose(torch.cat([out1, out2[21:]]).float(), wb.float(), **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
def test_swiglu_part(dtype):
    from vllm_oxide_b200.parts import PartSpec, build_part
    ffn = build_part("feed_forward", PartSpec("swiglu", dict(hidden_size=24, intermediate_size=50, prefix="f.")))
    g = torch.Generator().manual_seed(0)
    t = {s.name: (torch.randn(s.shape, generator=g) / math.sqrt(s.shape[-1])).to(dtype) for s in ffn.tensor_specs()}
    ffn.load({k: v.to(DEV) for k, v in t.items()})
    x = torch.randn(11, 24, generator=g).to(dtype)
    ctx = make_context(manager_with([(0, 11)]), [(0, 0, range(11), [])], dtype)
    got = ffn.forward(x.to(DEV), ctx).cpu()
    want = P.swiglu(x, t["f.gate_proj.weight"], t["f.up_proj.weight"], t["f.down_proj.weight"], dtype)
    assert torch.allclose(got.float(), want.float(), **tol(dtype))


def test_a_model_may_mix_parts_layer_by_layer():
    """Window in some layers and not in others gives two cache groups, each with pages of its own."""
    from conftest import TINY
    from vllm_oxide_b200.cache import PagedCache
    from vllm_oxide_b200.models import CausalLM, resolve
    _, plan = resolve(TINY["C"]["config"])
    model = CausalLM(plan, torch.float32, DEV)
    specs = model.cache_specs()
    assert [s.window for s in specs] == [0, 0, 24, 24]
    cache = PagedCache(specs, model.state_specs(), torch.float32, DEV, 16, 10, 4)
    assert [(g.window, g.planes) for g in cache.groups] == [(0, [0, 1]), (24, [2, 3])]
    assert cache.manager.num_groups == 2 and cache.planes[2].group == 1 and cache.planes[0].k.shape == (10, 3, 16, 48)
