"""Each CUDA kernel alone against its plain reference, at sizes other than the engine's."""
import math

import numpy as np
import pytest
import torch

from plain import qwen3_plain as P
from plain import sampler_plain as S

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype):
    return dict(rtol=1e-5, atol=1e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)


def err_word():
    return torch.zeros(1, dtype=torch.int32, device=DEV)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H", [72, 1000])
def test_embedding(dtype, H):
    from vllm_oxide_b200 import kernels
    V = 301
    table = torch.randn(V, H, device=DEV).to(dtype)
    ids = torch.tensor([0, 300, 5, 5, 17], dtype=torch.int32, device=DEV)
    out = torch.empty(5, H, dtype=dtype, device=DEV)
    err = err_word()
    kernels.embedding(table, ids, out, 5, err)
    assert torch.equal(out, P.embedding(table.cpu(), ids.cpu(), dtype).to(DEV)) and err.item() == 0
    bad = torch.tensor([3, 301], dtype=torch.int32, device=DEV)
    kernels.embedding(table, bad, out, 2, err)
    assert err.item() == 1 and torch.equal(out[0], table[3]) and out[1].abs().max() == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H", [100, 4104, 13000])
def test_add_rmsnorm(dtype, H):
    from vllm_oxide_b200 import kernels
    T, eps = 7, 3e-6
    x = torch.randn(T, H, device=DEV).to(dtype)
    res = (3 * torch.randn(T, H, device=DEV)).to(dtype)
    w = (1 + 0.1 * torch.randn(H, device=DEV)).float()
    wq = w.to(dtype)   # the plain formula multiplies in the model dtype; use a weight that is exact in it
    y = torch.empty_like(x)
    r = res.clone()
    err = err_word()
    kernels.add_rmsnorm(x, r, wq.float(), y, eps, True, err)
    ry, rr = P.add_rms_norm(x.cpu(), res.cpu(), wq.cpu(), eps, dtype)
    assert torch.allclose(y.cpu().float(), ry.float(), **tol(dtype))
    assert torch.equal(r.cpu(), rr) if dtype == torch.bfloat16 else torch.allclose(r.cpu(), rr, atol=1e-6)
    # without a residual: residual' = x
    r2 = torch.zeros_like(x)
    kernels.add_rmsnorm(x, r2, wq.float(), y, eps, False, err)
    ry, _ = P.add_rms_norm(x.cpu(), None, wq.cpu(), eps, dtype)
    assert torch.allclose(y.cpu().float(), ry.float(), **tol(dtype)) and torch.equal(r2, x)
    # wanted rows only, residual untouched; the same row gives the same bits as in the full call
    rows = torch.tensor([5, 0, 5], dtype=torch.int32, device=DEV)
    r3 = res.clone()
    yr = torch.empty(3, H, dtype=dtype, device=DEV)
    kernels.add_rmsnorm(x, r3, wq.float(), yr, eps, True, err, rows=rows, n_out=3)
    full = torch.empty_like(x)
    kernels.add_rmsnorm(x, res.clone(), wq.float(), full, eps, True, err)
    assert torch.equal(yr, full[rows.long()]) and torch.equal(r3, res) and err.item() == 0


@pytest.mark.parametrize("dtype", DTYPES)
def test_silu_mul(dtype):
    from vllm_oxide_b200 import kernels
    T, I = 5, 333
    gu = (4 * torch.randn(T, 2 * I, device=DEV)).to(dtype)
    gu[0, 0], gu[0, 1] = -50.0, 0.0
    out = torch.empty(T, I, dtype=dtype, device=DEV)
    kernels.silu_mul(gu, out, T)
    g, u = gu[:, :I].cpu(), gu[:, I:].cpu()
    it = torch.float32
    ref = ((g.to(it) / (1 + torch.exp(-g.to(it)))).to(dtype) * u)
    assert torch.allclose(out.cpu().float(), ref.float(), **tol(dtype))
    assert out[0, 0].abs() < 1e-6 and out[0, 1] == 0
    if I % 8 == 0 or True:
        I2 = 336
        gu2 = (4 * torch.randn(T, 2 * I2, device=DEV)).to(dtype)
        out2 = torch.empty(T, I2, dtype=dtype, device=DEV)
        kernels.silu_mul(gu2, out2, T, interleaved=True)
        v = gu2.cpu().reshape(T, I2 // 8, 2, 8)
        g2, u2 = v[:, :, 0].reshape(T, I2), v[:, :, 1].reshape(T, I2)
        ref2 = ((g2.float() / (1 + torch.exp(-g2.float()))).to(dtype) * u2)
        assert torch.allclose(out2.cpu().float(), ref2.float(), **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,kvh,hd", [(5, 5, 16), (6, 2, 48), (8, 1, 80), (4, 4, 256)])
@pytest.mark.parametrize("norm,bias", [(True, False), (False, True)])
def test_qk_norm_rope_kv_write(dtype, nh, kvh, hd, norm, bias):
    from vllm_oxide_b200 import kernels
    from vllm_oxide_b200.parts import RotationRule
    T, bs, pages, eps, max_pos, theta = 9, 16, 6, 2e-6, 300, 12345.0
    width = (nh + 2 * kvh) * hd
    qkv = torch.randn(T, width, device=DEV).to(dtype)
    b = (0.1 * torch.randn(width, device=DEV)).to(dtype) if bias else None
    wq = (1 + 0.1 * torch.randn(hd, device=DEV)).to(dtype).float() if norm else None
    wk = (1 + 0.1 * torch.randn(hd, device=DEV)).to(dtype).float() if norm else None
    pos = torch.tensor([0, 1, 2, 299, 150, 7, 64, 65, 31], dtype=torch.int32, device=DEV)
    slots = torch.tensor([5, 95, 17, -1, 40, 41, 0, 63, 64], dtype=torch.int32, device=DEV)
    table = P.rope_table(hd, max_pos, theta)
    kc = torch.full((pages, kvh, bs, hd), 7.0, device=DEV).to(dtype)     # [pages, kv heads, slots of a page, hd]
    vc = torch.full((pages, kvh, bs, hd), 7.0, device=DEV).to(dtype)
    out = qkv.clone()
    err = err_word()
    kernels.qk_norm_rope_kv_write(out, b, pos, slots, wq, wk, RotationRule(table.to(DEV), hd), kc, vc, T, nh, kvh, hd, eps, True, err)
    assert err.item() == 0
    x = qkv.cpu()
    if bias:
        x = x + b.cpu()
    q, k, v = P.split_qkv(x, nh, kvh, hd)
    if norm:
        q = P.head_rms_norm(q, wq.cpu().to(dtype), eps, dtype)
        k = P.head_rms_norm(k, wk.cpu().to(dtype), eps, dtype)
    q = P.apply_rope(q, pos.cpu(), table, dtype)
    k = P.apply_rope(k, pos.cpu(), table, dtype)
    got_q = out[:, :nh * hd].reshape(T, nh, hd).cpu()
    assert torch.allclose(got_q.float(), q.float(), **tol(dtype))
    kflat = kc.permute(0, 2, 1, 3).reshape(pages * bs, kvh, hd).cpu()   # by slot
    vflat = vc.permute(0, 2, 1, 3).reshape(pages * bs, kvh, hd).cpu()
    written = torch.zeros(pages * bs, dtype=torch.bool)
    for t in range(T):
        s = int(slots[t])
        if s < 0:
            continue
        written[s] = True
        assert torch.allclose(kflat[s].float(), k[t].float(), **tol(dtype))
        assert torch.equal(vflat[s], v[t].to(dtype))
    assert (kflat[~written] == 7).all() and (vflat[~written] == 7).all()     # nothing else was touched
    # a reader of another layer's cache writes nothing
    kc2 = torch.zeros_like(kc)
    kernels.qk_norm_rope_kv_write(qkv.clone(), b, pos, slots, wq, wk, RotationRule(table.to(DEV), hd), kc2, kc2, T, nh, kvh, hd, eps, False, err)
    assert kc2.abs().max() == 0
    # positions beyond the table and slots beyond the pool are refused, not read
    badpos = pos.clone(); badpos[0] = 300
    kernels.qk_norm_rope_kv_write(qkv.clone(), b, badpos, slots, wq, wk, RotationRule(table.to(DEV), hd), kc, vc, T, nh, kvh, hd, eps, True, err)
    assert err.item() & 2
    err.zero_()
    badslot = slots.clone(); badslot[1] = pages * bs
    kernels.qk_norm_rope_kv_write(qkv.clone(), b, pos, badslot, wq, wk, RotationRule(table.to(DEV), hd), kc, vc, T, nh, kvh, hd, eps, True, err)
    assert err.item() & 4


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,kvh,hd,T", [(32, 8, 128, 300), (16, 8, 64, 257), (3, 1, 32, 300), (6, 2, 48, 300), (8, 1, 80, 256),
                                         (2, 2, 256, 260), (5, 5, 16, 300), (7, 1, 128, 3), (9, 3, 64, 1), (4, 2, 96, 40),
                                         (2, 1, 512, 5), (3, 3, 144, 270)])
def test_qk_norm_rope_kv_write_many_tokens_and_head_sizes(dtype, nh, kvh, hd, T):
    """The rotation kernel picks its shape by head size and token count (16-byte accesses for head sizes that are a power
    of two, four heads a warp from 256 tokens on): each against the plain formulas, with norm and bias together."""
    from vllm_oxide_b200 import kernels
    from vllm_oxide_b200.parts import RotationRule
    bs, eps, max_pos, theta = 32, 1e-5, 700, 1e6
    pages = -(-T // bs) + 2
    g = torch.Generator().manual_seed(T + hd)
    width = (nh + 2 * kvh) * hd
    qkv = torch.randn(T, width, generator=g).to(dtype).to(DEV)
    b = (0.1 * torch.randn(width, generator=g)).to(dtype).to(DEV)
    wq = (1 + 0.1 * torch.randn(hd, generator=g)).to(dtype).float().to(DEV)
    wk = (1 + 0.1 * torch.randn(hd, generator=g)).to(dtype).float().to(DEV)
    pos = torch.randint(0, max_pos, (T,), generator=g).int().to(DEV)
    slots = torch.randperm(pages * bs, generator=g)[:T].int()
    slots[T // 2] = -1                                              # a token whose key goes nowhere
    slots = slots.to(DEV)
    table = P.rope_table(hd, max_pos, theta)
    kc = torch.full((pages, kvh, bs, hd), 7.0, device=DEV).to(dtype)
    vc = torch.full((pages, kvh, bs, hd), 7.0, device=DEV).to(dtype)
    out = qkv.clone()
    err = err_word()
    kernels.qk_norm_rope_kv_write(out, b, pos, slots, wq, wk, RotationRule(table.to(DEV), hd), kc, vc, T, nh, kvh, hd, eps, True, err)
    assert err.item() == 0
    q, k, v = P.split_qkv(qkv.cpu() + b.cpu(), nh, kvh, hd)
    q = P.apply_rope(P.head_rms_norm(q, wq.cpu().to(dtype), eps, dtype), pos.cpu(), table, dtype)
    k = P.apply_rope(P.head_rms_norm(k, wk.cpu().to(dtype), eps, dtype), pos.cpu(), table, dtype)
    assert torch.allclose(out[:, :nh * hd].reshape(T, nh, hd).cpu().float(), q.float(), **tol(dtype))
    kflat = kc.permute(0, 2, 1, 3).reshape(pages * bs, kvh, hd).cpu()
    vflat = vc.permute(0, 2, 1, 3).reshape(pages * bs, kvh, hd).cpu()
    keep = slots.cpu() >= 0
    idx = slots.cpu()[keep].long()
    assert torch.allclose(kflat[idx].float(), k[keep].float(), **tol(dtype))
    assert torch.equal(vflat[idx], v[keep].to(dtype))
    untouched = torch.ones(pages * bs, dtype=torch.bool)
    untouched[idx] = False
    assert (kflat[untouched] == 7).all() and (vflat[untouched] == 7).all()

def plain_rotation(x, positions, table, rot_dim, interleaved, dt):
    """Rotation of the first rot_dim elements of every head, in halves or in neighbouring pairs, restated in plain torch:
    the halves rule with rot_dim = head size is P.apply_rope (crates/vllm-oxide/src/layers/rope.rs:129-159)."""
    if rot_dim == 0:
        return x
    it = torch.float64 if dt == torch.float64 else torch.float32
    cs = table[positions.long()].to(it)
    half = rot_dim // 2
    c, s = cs[:, None, :half], cs[:, None, half:]
    xf = x.to(it)
    rot, rest = xf[..., :rot_dim], xf[..., rot_dim:]
    if interleaved:
        x1, x2 = rot[..., 0::2], rot[..., 1::2]
        y = torch.stack([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1).flatten(-2)
    else:
        x1, x2 = rot[..., :half], rot[..., half:]
        y = torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1)
    return torch.cat([y, rest], dim=-1).to(dt)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,kvh,hd,rot,interleaved", [(4, 2, 64, 32, False), (4, 2, 64, 64, True), (6, 1, 48, 16, True),
                                                        (3, 3, 80, 0, False), (8, 2, 128, 64, False), (2, 1, 16, 2, True)])
def test_qk_norm_rope_kv_write_other_position_rules(dtype, nh, kvh, hd, rot, interleaved):
    """The position rule is an argument of the kernel: a rotation of only the first elements of a head, neighbouring
    pairs instead of halves, or no rotation at all; norm, bias and the cache write as with the stock rule."""
    from vllm_oxide_b200 import kernels
    from vllm_oxide_b200.parts import RotationRule
    T, bs, eps, max_pos, theta = 37, 16, 1e-5, 200, 5e4
    pages = -(-T // bs) + 1
    g = torch.Generator().manual_seed(hd + rot)
    width = (nh + 2 * kvh) * hd
    qkv = torch.randn(T, width, generator=g).to(dtype).to(DEV)
    b = (0.1 * torch.randn(width, generator=g)).to(dtype).to(DEV)
    wq = (1 + 0.1 * torch.randn(hd, generator=g)).to(dtype).float().to(DEV)
    wk = (1 + 0.1 * torch.randn(hd, generator=g)).to(dtype).float().to(DEV)
    pos = torch.randint(0, max_pos, (T,), generator=g).int().to(DEV)
    slots = torch.randperm(pages * bs, generator=g)[:T].int().to(DEV)
    table = P.rope_table(rot, max_pos, theta) if rot else None
    rule = RotationRule(table.to(DEV) if rot else None, rot, interleaved)
    kc = torch.full((pages, kvh, bs, hd), 7.0, device=DEV).to(dtype)
    vc = torch.full((pages, kvh, bs, hd), 7.0, device=DEV).to(dtype)
    out = qkv.clone()
    err = err_word()
    kernels.qk_norm_rope_kv_write(out, b, pos, slots, wq, wk, rule, kc, vc, T, nh, kvh, hd, eps, True, err)
    assert err.item() == 0
    q, k, v = P.split_qkv(qkv.cpu() + b.cpu(), nh, kvh, hd)
    q = plain_rotation(P.head_rms_norm(q, wq.cpu().to(dtype), eps, dtype), pos.cpu(), table, rot, interleaved, dtype)
    k = plain_rotation(P.head_rms_norm(k, wk.cpu().to(dtype), eps, dtype), pos.cpu(), table, rot, interleaved, dtype)
    assert torch.allclose(out[:, :nh * hd].reshape(T, nh, hd).cpu().float(), q.float(), **tol(dtype))
    kflat = kc.permute(0, 2, 1, 3).reshape(pages * bs, kvh, hd).cpu()
    vflat = vc.permute(0, 2, 1, 3).reshape(pages * bs, kvh, hd).cpu()
    idx = slots.cpu().long()
    assert torch.allclose(kflat[idx].float(), k.float(), **tol(dtype))
    assert torch.equal(vflat[idx], v.to(dtype))


def paged_setup(dtype, kvh, hd, bs, ctx_lens, g):
    """Random keys/values for requests of the given context lengths, scattered over shuffled pages."""
    B = len(ctx_lens)
    pages_per = [(c + bs - 1) // bs for c in ctx_lens]
    num_pages = sum(pages_per) + 3
    perm = torch.randperm(num_pages, generator=g).tolist()
    P_max = max(pages_per)
    bt = torch.full((B, P_max), -1, dtype=torch.int32)
    kc = torch.randn(num_pages, kvh, bs, hd, generator=g).to(dtype)   # unused slots hold noise on purpose
    vc = torch.randn(num_pages, kvh, bs, hd, generator=g).to(dtype)
    ks, vs = [], []
    it = iter(perm)
    for b, c in enumerate(ctx_lens):
        k = torch.randn(c, kvh, hd, generator=g).to(dtype)
        v = torch.randn(c, kvh, hd, generator=g).to(dtype)
        for p in range(pages_per[b]):
            page = next(it)
            bt[b, p] = page
            n = min(bs, c - p * bs)
            kc[page, :, :n] = k[p * bs:p * bs + n].transpose(0, 1)
            vc[page, :, :n] = v[p * bs:p * bs + n].transpose(0, 1)
        ks.append(k); vs.append(v)
    return kc, vc, bt, ks, vs


def run_attention(fn, dtype, nh, kvh, hd, bs, window, q_lens, ctx_lens, seed=0, craft=None):
    """Queries are the last q_len positions of each request. Returns (got, want) [T, nh*hd]."""
    g = torch.Generator().manual_seed(seed)
    kc, vc, bt, ks, vs = paged_setup(dtype, kvh, hd, bs, ctx_lens, g)
    T = sum(q_lens)
    q = torch.randn(T, nh, hd, generator=g).to(dtype)
    token_req = torch.tensor([b for b, n in enumerate(q_lens) for _ in range(n)], dtype=torch.int32)
    positions = torch.tensor([c - n + i for n, c in zip(q_lens, ctx_lens) for i in range(n)], dtype=torch.int32)
    if craft is not None:
        craft(q, ks, vs, kc, vc, bt, positions)
    want = torch.empty(T, nh * hd, dtype=dtype)
    t0 = 0
    for b, (n, c) in enumerate(zip(q_lens, ctx_lens)):
        # plain attention over the whole request, then keep the rows of the queries
        qfull = torch.zeros(c, nh, hd, dtype=dtype)
        qfull[c - n:] = q[t0:t0 + n]
        o = P.attention(qfull, ks[b], vs[b], torch.arange(c), window or None, dtype)
        want[t0:t0 + n] = o[c - n:]
        t0 += n
    out = torch.empty(T, nh * hd, dtype=dtype, device=DEV)
    err = err_word()
    cu_q = torch.tensor([0] + list(np.cumsum(q_lens)), dtype=torch.int32)
    fn(q=q.to(DEV), out=out, kc=kc.to(DEV), vc=vc.to(DEV), bt=bt.to(DEV), token_req=token_req.to(DEV),
       positions=positions.to(DEV), cu_q=cu_q.to(DEV), ctx=torch.tensor(ctx_lens, dtype=torch.int32, device=DEV),
       T=T, nh=nh, kvh=kvh, hd=hd, window=window, err=err)
    assert err.item() == 0
    return out.cpu().float(), want.float()


def generic_attention(q, out, kc, vc, bt, token_req, positions, T, nh, kvh, hd, window, err, **_):
    from vllm_oxide_b200 import kernels
    kernels.paged_attention_generic(q.reshape(T, nh * hd), nh * hd, out, kc, vc, bt, token_req, positions, T, nh, kvh, hd,
                                    window, 1.0 / math.sqrt(hd), err)


ATT_CASES = [  # nh, kvh, hd, block_size, window, q_lens, ctx_lens
    (4, 2, 16, 16, 0, [1, 5, 40], [1, 37, 40]),
    (6, 1, 48, 32, 0, [1, 1, 1], [700, 33, 64]),
    (8, 2, 128, 64, 0, [130, 1], [333, 129]),
    (3, 3, 80, 16, 24, [1, 30, 2], [100, 61, 24]),
    (5, 5, 32, 16, 7, [50], [50]),
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", ATT_CASES)
def test_attention_generic(dtype, case):
    nh, kvh, hd, bs, window, q_lens, ctx_lens = case
    got, want = run_attention(generic_attention, dtype, nh, kvh, hd, bs, window, q_lens, ctx_lens)
    assert torch.allclose(got, want, **(dict(rtol=1e-4, atol=2e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)))


def craft_spike(key_pos):
    """Makes one far key dominate every query's scores: the output must be that key's value."""
    def craft(q, ks, vs, kc, vc, bt, positions):
        hd = q.shape[-1]
        bs = kc.shape[2]
        q[:] = 0
        q[..., 0] = 8.0
        for b in range(len(ks)):
            ks[b][:] = 0.01 * ks[b]
            ks[b][key_pos, :, 0] = 8.0 * math.sqrt(hd)
            vs[b][key_pos] = 5.0
            for p in range((ks[b].shape[0] + bs - 1) // bs):
                n = min(bs, ks[b].shape[0] - p * bs)
                kc[bt[b, p], :, :n] = ks[b][p * bs:p * bs + n].transpose(0, 1)
                vc[bt[b, p], :, :n] = vs[b][p * bs:p * bs + n].transpose(0, 1)
    return craft


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("key_pos,window,expect_hit", [
    (3, 0, True),        # a far key among hundreds
    (15, 0, True), (16, 0, True),            # the last slot of a page, the first slot of the next
    (800 - 64, 64, True), (800 - 65, 64, False),   # the window's edge: just inside, just outside
])
def test_attention_generic_reads_the_right_far_key(dtype, key_pos, window, expect_hit):
    got, want = run_attention(generic_attention, dtype, 2, 1, 32, 16, window, [1], [800], craft=craft_spike(key_pos))
    assert torch.allclose(got, want, atol=3e-2)
    assert (got.mean() > 4.9) == expect_hit


def test_attention_generic_does_not_depend_on_the_batch():
    """The same query gives the same bits alone, beside other requests, and from other pages."""
    a_got, _ = run_attention(generic_attention, torch.float32, 4, 2, 64, 16, 0, [3], [200], seed=5)
    g = torch.Generator().manual_seed(5)
    kc, vc, bt, ks, vs = paged_setup(torch.float32, 2, 64, 16, [200], g)
    q = torch.randn(3, 4, 64, generator=g)
    # the same request, now second in a batch of three and on pages chosen by another permutation
    g2 = torch.Generator().manual_seed(99)
    kc2, vc2, bt2, ks2, vs2 = paged_setup(torch.float32, 2, 64, 16, [50, 200, 9], g2)
    for p in range(13):
        n = min(16, 200 - p * 16)
        kc2[bt2[1, p], :, :n] = ks[0][p * 16:p * 16 + n].transpose(0, 1)
        vc2[bt2[1, p], :, :n] = vs[0][p * 16:p * 16 + n].transpose(0, 1)
    qq = torch.cat([torch.randn(1, 4, 64, generator=g2), q, torch.randn(2, 4, 64, generator=g2)])
    token_req = torch.tensor([0, 1, 1, 1, 2, 2], dtype=torch.int32, device=DEV)
    positions = torch.tensor([49, 197, 198, 199, 7, 8], dtype=torch.int32, device=DEV)
    out = torch.empty(6, 256, device=DEV)
    err = err_word()
    generic_attention(qq.to(DEV), out, kc2.to(DEV), vc2.to(DEV), bt2.to(DEV), token_req, positions, 6, 4, 2, 64, 0, err)
    assert torch.equal(out[1:4].cpu(), a_got)


def decode_attention(num_splits, use_tma=True, persistent=False):
    def fn(q, out, kc, vc, bt, cu_q, ctx, T, nh, kvh, hd, window, err, **_):
        from vllm_oxide_b200 import kernels
        B = ctx.shape[0]
        n = kernels.attention_decode_scratch_floats(hd, B, nh, num_splits)
        scratch = torch.full((max(n, 1),), float("nan"), device=DEV)
        pairs = kernels.decode_pairs_counter(DEV) if persistent else None
        for _ in range(2 if persistent else 1):          # twice over one counter: the kernel leaves it at zero
            kernels.attention_decode(q.reshape(T, nh * hd), nh * hd, out, kc, vc, bt, cu_q, ctx, B, nh, kvh, hd, window,
                                     1.0 / math.sqrt(hd), num_splits, scratch if n else None, err, use_tma=use_tma,
                                     pairs=pairs)
        if persistent:
            assert pairs.tolist() == [0, 0]
    return fn


DECODE_CASES = [  # nh, kvh, hd, block_size, window, ctx_lens, splits
    (32, 8, 128, 256, 0, [2048, 1, 700, 64, 65, 63], 4),
    (16, 8, 128, 16, 0, [300, 129], 1),
    (6, 1, 32, 32, 0, [100, 5, 31, 32, 33], 3),
    (4, 2, 16, 16, 0, [40, 1, 17], 2),
    (3, 3, 48, 16, 24, [100, 24, 25, 3], 2),
    (16, 1, 64, 64, 0, [513, 77], 5),
    (8, 2, 256, 64, 100, [400, 99, 101], 3),
    (5, 5, 80, 48, 0, [200], 7),
    (8, 8, 64, 48, 30, [200, 31, 47, 48, 49], 2),
    (12, 3, 192, 32, 0, [333, 1, 65], 3),
    (32, 8, 128, 256, 0, [701], 8),              # the most splits that merge as a cluster
    (32, 8, 128, 256, 0, [2050, 701, 100], 8),
    (8, 2, 64, 64, 0, [1000, 130], 6),
    (32, 8, 128, 256, 0, [2050], 16),            # more: merged by the second kernel
    (32, 8, 128, 256, 0, [16500], 32),           # one long request: 32 splits of 8 tiles
]


@pytest.mark.parametrize("use_tma", [True, False])
@pytest.mark.parametrize("case", DECODE_CASES)
def test_attention_decode(case, use_tma):
    """Head sizes that are a multiple of 64 have two kernels (TMA and cp.async copies); both are checked."""
    nh, kvh, hd, bs, window, ctx_lens, splits = case
    got, want = run_attention(decode_attention(splits, use_tma), torch.bfloat16, nh, kvh, hd, bs, window,
                              [1] * len(ctx_lens), ctx_lens)
    assert torch.allclose(got, want, rtol=2e-2, atol=2e-2)


MANY_DECODE_CASES = [  # nh, kvh, hd, block_size, window, requests: more (request, kv head) pairs than blocks fit the GPU
    (16, 8, 128, 16, 0, 75),
    (32, 8, 128, 256, 0, 80),
    (8, 8, 64, 48, 30, 90),
    (16, 16, 64, 64, 0, 40),
    (32, 2, 128, 64, 0, 160),      # sixteen heads per kv head: the largest merge buffer, fewer blocks fit
    (12, 4, 192, 32, 100, 100),
]


@pytest.mark.parametrize("case", MANY_DECODE_CASES)
def test_attention_decode_of_many_requests_with_persistent_blocks(case):
    """One split, more pairs than resident blocks and a counter: persistent blocks take several pairs each, of very different
    lengths (one key, a page's edge, hundreds of keys), with requests that are no decoding requests among them.
    The result agrees with the plain formula and, bit for bit, with one block per pair."""
    from vllm_oxide_b200 import kernels
    nh, kvh, hd, bs, window, n = case
    g = torch.Generator().manual_seed(n)
    ctx_lens = [int(x) for x in torch.randint(1, 500, (n,), generator=g)]
    ctx_lens[:6] = [1, bs, bs + 1, 63, 64, 65]
    q_lens = [1] * n
    for i in range(7, n, 9):               # portions of prompts: the decode kernel leaves their rows alone
        q_lens[i] = 2
        ctx_lens[i] = max(ctx_lens[i], 2)
    got, want = run_attention(decode_attention(1, persistent=True), torch.bfloat16, nh, kvh, hd, bs, window, q_lens, ctx_lens)
    starts = np.cumsum([0] + q_lens)
    rows = torch.tensor([int(starts[b]) for b in range(n) if q_lens[b] == 1])
    assert torch.allclose(got[rows], want[rows], rtol=2e-2, atol=2e-2)
    per_pair, _ = run_attention(decode_attention(1), torch.bfloat16, nh, kvh, hd, bs, window, q_lens, ctx_lens)
    assert torch.equal(got[rows], per_pair[rows])


@pytest.mark.parametrize("key_pos,window,expect_hit", [(3, 0, True), (255, 0, True), (256, 0, True), (511, 0, True),
                                                       (800 - 64, 64, True), (800 - 65, 64, False), (799, 0, True)])
def test_attention_decode_reads_the_right_far_key(key_pos, window, expect_hit):
    got, want = run_attention(decode_attention(4), torch.bfloat16, 8, 2, 64, 16, window, [1], [800], craft=craft_spike(key_pos))
    assert torch.allclose(got, want, atol=3e-2)
    assert (got.mean() > 4.9) == expect_hit


# the kernels behind attention_prefill: tcgen05 with one or two query tiles a block (head sizes 64 and 128),
# mma.sync with TMA copies (head sizes that are a multiple of 64), mma.sync with cp.async (every head size)
PREFILL_KERNELS = {"tc5x2": dict(query_tiles=2), "tc5x1": dict(query_tiles=1), "tma": dict(use_tc5=False),
                   "cp.async": dict(use_tc5=False, use_tma=False),
                   # the tcgen05 kernel with its query tiles by cp.async and its output stored row by row, as for a caller
                   # that gives it no tensor maps of q and the output
                   "tc5x2-rows": dict(query_tiles=2, tiles_by_tma=False)}


def prefill_attention(q, out, kc, vc, bt, cu_q, ctx, T, nh, kvh, hd, window, err, kernel="tc5x2", **_):
    from vllm_oxide_b200 import kernels
    B = ctx.shape[0]
    max_q = int((cu_q[1:] - cu_q[:-1]).max())
    kernels.attention_prefill(q.reshape(T, nh * hd), nh * hd, out, kc, vc, bt, cu_q, ctx, B, max_q, nh, kvh, hd, window,
                              1.0 / math.sqrt(hd), err, **PREFILL_KERNELS[kernel])


PREFILL_CASES = [  # nh, kvh, hd, block_size, window, q_lens, ctx_lens
    (32, 8, 128, 256, 0, [300, 2, 64], [300, 2, 700]),
    (16, 8, 128, 16, 0, [17, 130], [80, 130]),
    (6, 1, 32, 32, 0, [5, 31, 32, 33, 100], [5, 31, 40, 33, 228]),
    (4, 2, 16, 16, 0, [40, 2, 17], [40, 19, 17]),
    (3, 3, 48, 16, 24, [30, 2, 70], [61, 24, 170]),
    (16, 1, 64, 64, 0, [65, 3], [513, 77]),
    (8, 2, 256, 64, 100, [150, 20], [400, 99]),
    (5, 5, 80, 48, 7, [50], [50]),
    (8, 8, 64, 48, 30, [200, 31, 2], [200, 31, 48]),
    (12, 3, 192, 32, 0, [133, 65], [333, 65]),
    (16, 4, 128, 128, 70, [300, 129], [700, 129]),
    (6, 2, 128, 64, 0, [700], [700]),            # three heads a group: a tile holds 42 tokens, 126 of its 128 rows
    (10, 2, 128, 64, 0, [300, 26, 51], [300, 90, 51]),   # five (Qwen3-14B's 40 over 8): 25 tokens a tile
    (14, 2, 64, 32, 0, [2, 257, 40], [2, 300, 1000]),
]


@pytest.mark.parametrize("kernel", list(PREFILL_KERNELS))
@pytest.mark.parametrize("case", PREFILL_CASES)
def test_attention_prefill(case, kernel):
    """Every kernel that a head size has is checked (a head size without one falls through to the next)."""
    import functools
    nh, kvh, hd, bs, window, q_lens, ctx_lens = case
    got, want = run_attention(functools.partial(prefill_attention, kernel=kernel), torch.bfloat16, nh, kvh, hd, bs,
                              window, q_lens, ctx_lens)
    assert torch.allclose(got, want, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("case", [c for c in PREFILL_CASES if c[2] in (64, 128)])
def test_attention_prefill_tiles_by_tma_are_the_same_bits(case):
    """How the query tiles come in and how whole output tiles leave (copy engine, or cp.async and row stores) changes no
    arithmetic: the two give the same bits, for whole tiles and for tiles that end inside a request."""
    import functools
    nh, kvh, hd, bs, window, q_lens, ctx_lens = case
    a, _ = run_attention(functools.partial(prefill_attention, kernel="tc5x2"), torch.bfloat16, nh, kvh, hd, bs, window,
                         q_lens, ctx_lens)
    b, _ = run_attention(functools.partial(prefill_attention, kernel="tc5x2-rows"), torch.bfloat16, nh, kvh, hd, bs, window,
                         q_lens, ctx_lens)
    assert torch.equal(a, b)


@pytest.mark.parametrize("key_pos,window,expect_hit", [(3, 0, True), (63, 0, True), (64, 0, True), (791, 0, True),
                                                       (792 - 63, 64, True), (792 - 64, 64, False)])
@pytest.mark.parametrize("kernel", ["tc5x2", "tc5x1", "tma"])
def test_attention_prefill_reads_the_right_far_key(key_pos, window, expect_hit, kernel):
    """Eight queries at positions 792..799: the first one decides whether the key is inside its window."""
    import functools
    got, want = run_attention(functools.partial(prefill_attention, kernel=kernel), torch.bfloat16, 8, 2, 64, 16, window, [8],
                              [800], craft=craft_spike(key_pos))
    assert torch.allclose(got, want, atol=3e-2)
    assert (got[0].mean() > 4.9) == expect_hit


@pytest.mark.parametrize("kernel", ["tc5x2", "tc5x1"])
def test_attention_prefill_tc5_many_launches_end_and_repeat(kernel):
    """Thousands of blocks at the head counts of a large model, launched again and again: no bounded wait runs out (a
    softmax thread that reaches the end late must not miss the last product's signal) and the result repeats bit for bit."""
    from vllm_oxide_b200 import kernels
    nh, kvh, hd, bs = 64, 8, 128, 256
    q_lens, ctx_lens = [1580, 1615], [1580, 4049]
    g = torch.Generator().manual_seed(11)
    pages = [-(-c // bs) for c in ctx_lens]
    kc = torch.randn(sum(pages) + 1, kvh, bs, hd, generator=g).bfloat16().to(DEV)
    vc = torch.randn(sum(pages) + 1, kvh, bs, hd, generator=g).bfloat16().to(DEV)
    bt = torch.full((2, max(pages)), -1, dtype=torch.int32)
    bt[0, :pages[0]] = torch.arange(1, 1 + pages[0])
    bt[1, :pages[1]] = torch.arange(1 + pages[0], 1 + pages[0] + pages[1])
    T = sum(q_lens)
    q = torch.randn(T, nh * hd, generator=g).bfloat16().to(DEV)
    cu_q = torch.tensor([0, q_lens[0], T], dtype=torch.int32, device=DEV)
    ctx = torch.tensor(ctx_lens, dtype=torch.int32, device=DEV)
    err = err_word()
    first = None
    for _ in range(40):
        out = torch.zeros(T, nh * hd, dtype=torch.bfloat16, device=DEV)
        kernels.attention_prefill(q, nh * hd, out, kc, vc, bt.to(DEV), cu_q, ctx, 2, max(q_lens), nh, kvh, hd, 0,
                                  1.0 / math.sqrt(hd), err, **PREFILL_KERNELS[kernel])
        torch.cuda.synchronize()
        assert err.item() == 0
        if first is None:
            first = out
            assert torch.isfinite(out.float()).all() and out.float().abs().max() > 0
        else:
            assert torch.equal(out, first)


def test_attention_kernels_agree_with_the_plain_kernel_on_random_batches():
    """Eighty random batches (head counts, groups up to 16, page sizes, windows, pages scattered over the pool, decoding
    requests beside portions): every tensor-core kernel for portions and the decode kernel at several split counts
    against the plain kernel (which the tests above hold to the plain implementation); each writes its own rows only."""
    import random
    from vllm_oxide_b200 import kernels
    rng = random.Random(4)
    for case in range(80):
        hd, kvh = rng.choice([64, 128]), rng.choice([1, 2, 3, 4, 8])
        nh = kvh * rng.choice([1, 2, 3, 4, 8, 16])
        bs = rng.choice([16, 32, 64, 128, 256])
        window = rng.choice([0, 0, 0, rng.randint(1, 300)])
        B = rng.randint(1, 5)
        ctx_lens = [rng.choice([rng.randint(1, 70), rng.randint(1, 700), rng.randint(1, 3000)]) for _ in range(B)]
        q_lens = [1 if (k := rng.random()) < 0.3 else (c if k < 0.6 else rng.randint(1, c)) for c in ctx_lens]
        g = torch.Generator().manual_seed(case)
        pages = [-(-c // bs) for c in ctx_lens]
        total = sum(pages) + 2
        order = torch.randperm(total - 1, generator=g) + 1
        kc = torch.randn(total, kvh, bs, hd, generator=g).bfloat16().to(DEV)
        vc = torch.randn(total, kvh, bs, hd, generator=g).bfloat16().to(DEV)
        bt = torch.full((B, max(pages)), -1, dtype=torch.int32)
        at = 0
        for b in range(B):
            bt[b, :pages[b]] = order[at:at + pages[b]].int()
            at += pages[b]
        bt = bt.to(DEV)
        T = sum(q_lens)
        q = (torch.randn(T, nh * hd, generator=g) * rng.choice([0.3, 1.0, 3.0])).bfloat16().to(DEV)
        cu = [0] + list(np.cumsum(q_lens))
        token_req = torch.tensor([b for b, n in enumerate(q_lens) for _ in range(n)], dtype=torch.int32, device=DEV)
        positions = torch.tensor([c - n + i for n, c in zip(q_lens, ctx_lens) for i in range(n)], dtype=torch.int32, device=DEV)
        cu_q = torch.tensor(cu, dtype=torch.int32, device=DEV)
        ctx = torch.tensor(ctx_lens, dtype=torch.int32, device=DEV)
        scale = 1.0 / math.sqrt(hd)
        err = err_word()
        want = torch.zeros(T, nh * hd, dtype=torch.bfloat16, device=DEV)
        kernels.paged_attention_generic(q, nh * hd, want, kc, vc, bt, token_req, positions, T, nh, kvh, hd, window, scale, err)
        single = torch.tensor([cu[b] for b in range(B) if q_lens[b] == 1], dtype=torch.long, device=DEV)
        portion = torch.tensor([t for b in range(B) if q_lens[b] > 1 for t in range(cu[b], cu[b + 1])], dtype=torch.long, device=DEV)
        what = f"case {case}: nh={nh} kvh={kvh} hd={hd} page={bs} window={window} q={q_lens} ctx={ctx_lens}"
        runs = []
        if len(portion):
            runs += [(name, portion, single, lambda out, kw=kw: kernels.attention_prefill(
                q, nh * hd, out, kc, vc, bt, cu_q, ctx, B, max(q_lens), nh, kvh, hd, window, scale, err, **kw))
                for name, kw in PREFILL_KERNELS.items()]
        if len(single):
            for splits in sorted({1, 2, rng.randint(3, 8), rng.randint(9, 20)}):
                n = kernels.attention_decode_scratch_floats(hd, B, nh, splits)
                scratch = torch.empty(max(n, 1), device=DEV) if n else None
                runs.append((f"decode with {splits} splits", single, portion, lambda out, s=splits, sc=scratch: kernels.attention_decode(
                    q, nh * hd, out, kc, vc, bt, cu_q, ctx, B, nh, kvh, hd, window, scale, s, sc, err)))
        for name, mine, others, launch in runs:
            out = torch.full((T, nh * hd), 777.0, dtype=torch.bfloat16, device=DEV)
            launch(out)
            assert err.item() == 0, (name, what)
            assert (out[mine].float() - want[mine].float()).abs().max() < 4e-2, (name, what)
            assert len(others) == 0 or (out[others] == 777).all(), (name, what)


def test_attention_decode_and_prefill_share_a_mixed_batch():
    def both(q, out, kc, vc, bt, token_req, positions, cu_q, ctx, T, nh, kvh, hd, window, err, **_):
        out.fill_(777.0)
        decode_attention(2)(q=q, out=out, kc=kc, vc=vc, bt=bt, cu_q=cu_q, ctx=ctx, T=T, nh=nh, kvh=kvh, hd=hd,
                            window=window, err=err)
        assert (out[1:6] == 777).all() and (out[0] != 777).all() and (out[6] != 777).all()
        prefill_attention(q=q, out=out, kc=kc, vc=vc, bt=bt, cu_q=cu_q, ctx=ctx, T=T, nh=nh, kvh=kvh, hd=hd,
                          window=window, err=err)

    got, want = run_attention(both, torch.bfloat16, 12, 4, 64, 16, 0, [1, 5, 1], [90, 40, 130])
    assert torch.allclose(got, want, rtol=2e-2, atol=2e-2)


def test_attention_decode_leaves_portions_to_the_other_kernel():
    """In a mixed batch the decode kernel writes only the rows of one-token requests; the plain kernel,
    told to skip those, writes the rest; together they give the whole batch."""
    from vllm_oxide_b200 import kernels

    def both(q, out, kc, vc, bt, token_req, positions, cu_q, ctx, T, nh, kvh, hd, window, err, **_):
        out.fill_(777.0)
        decode_attention(3)(q=q, out=out, kc=kc, vc=vc, bt=bt, cu_q=cu_q, ctx=ctx, T=T, nh=nh, kvh=kvh, hd=hd,
                            window=window, err=err)
        assert (out[1:6] == 777).all() and (out[0] != 777).all() and (out[6] != 777).all()
        kernels.paged_attention_generic(q.reshape(T, nh * hd), nh * hd, out, kc, vc, bt, token_req, positions, T, nh, kvh,
                                        hd, window, 1.0 / math.sqrt(hd), err, skip_single_cu_q=cu_q)

    got, want = run_attention(both, torch.bfloat16, 8, 4, 64, 16, 0, [1, 5, 1], [90, 40, 130])
    assert torch.allclose(got, want, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("M,N,K", [(1, 7, 5), (3, 331, 80), (65, 130, 200), (200, 64, 4097)])
def test_gemm_f32(M, N, K):
    from vllm_oxide_b200 import kernels
    a = torch.randn(M, K, device=DEV)
    w = torch.randn(N, K, device=DEV)
    out = torch.empty(M, N, device=DEV)
    kernels.gemm_f32(a, w, out)
    ref = (a.double() @ w.double().t())
    assert (out.double() - ref).abs().max() <= 2e-6 * math.sqrt(K) * 16
    # a row alone gives the same bits as the row in the batch
    one = torch.empty(1, N, device=DEV)
    kernels.gemm_f32(a[M // 2:M // 2 + 1].contiguous(), w, one)
    assert torch.equal(one[0], out[M // 2])


def test_gemm_f32_is_not_reduced_precision():
    from vllm_oxide_b200 import kernels
    # 1 + 2^-12 squared needs more than TF32's 10 mantissa bits
    a = torch.full((4, 8), 1 + 2.0 ** -12, device=DEV)
    w = torch.full((4, 8), 1 + 2.0 ** -12, device=DEV)
    out = torch.empty(4, 4, device=DEV)
    kernels.gemm_f32(a, w, out)
    assert abs(out[0, 0].item() - 8 * (1 + 2.0 ** -12) ** 2) < 1e-6


@pytest.mark.parametrize("V", [331, 4099, 151936])
def test_sampler_against_the_plain_sampler(V):
    from vllm_oxide_b200.sampling import Sampler, row_key
    g = torch.Generator().manual_seed(V)
    R = 12
    logits = (3 * torch.randn(R, V, generator=g)).float()
    logits[0, 5] = logits[0, 200] = logits[0].max() + 1          # a tie at the top: lowest index wins
    temperature = [0.0, 0.8, 1.0, 1.0, 1.3, 0.7, 1.0, 1.0, 0.5, 2.0, 1.0, 1.0]
    top_k = [0, 0, 8, 1, 0, 50, 0, 3, 0, 20, V, 0]
    top_p = [1.0, 1.0, 1.0, 1.0, 0.9, 0.5, 0.2, 0.9, 1.0, 0.95, 0.3, 0.0]
    keys = [row_key(7, r, 3 * r) for r in range(R)]
    s = Sampler(DEV, 4)
    got = s.forward(logits.to(DEV), temperature, top_k, top_p, keys).cpu().tolist()
    want = [S.sample_row(logits[r].numpy(), temperature[r], top_k[r] or None, top_p[r] if top_p[r] < 1 else None, keys[r])
            for r in range(R)]
    assert got == want
    assert got[0] == 5 and got[3] == int(torch.argmax(logits[3]))
    for r in range(R):
        if temperature[r] > 0 and top_k[r] != 1:
            _, keep = S.surviving_mask(logits[r].numpy(), temperature[r], top_k[r] or None, top_p[r] if 0 < top_p[r] < 1 else None)
            assert keep[got[r]]


def test_sampler_top_p_on_peaked_and_flat_rows():
    """top-p gathers the tokens that can still matter into shared memory when they are few (a peaked row, as a
    language model gives) and searches the whole row when they are many (a flat row): both against the plain sampler."""
    from vllm_oxide_b200.sampling import Sampler, row_key
    g = torch.Generator().manual_seed(3)
    V = 151936
    rows = []
    for spread, lift, n_lifted in [(2.0, 12.0, 30), (1.0, 9.0, 3000), (3.0, 0.0, 0), (0.5, 6.0, 5000), (2.0, 15.0, 1), (1.5, 8.0, 4090)]:
        x = spread * torch.randn(V, generator=g)
        if n_lifted:
            idx = torch.randperm(V, generator=g)[:n_lifted]
            x[idx] += lift + torch.rand(n_lifted, generator=g)
        rows.append(x)
    logits = torch.stack(rows).float()
    R = logits.shape[0]
    temperature = [1.0, 0.8, 1.0, 1.2, 0.7, 1.0]
    top_k = [0, 0, 0, 2000, 0, 0]
    top_p = [0.9, 0.95, 0.9, 0.8, 0.5, 0.99]
    keys = [row_key(11, r, r) for r in range(R)]
    s = Sampler(DEV, 8)
    for trial in range(3):
        keys = [row_key(11 + trial, r, r) for r in range(R)]
        got = s.forward(logits.to(DEV), temperature, top_k, top_p, keys).cpu().tolist()
        want = [S.sample_row(logits[r].numpy(), temperature[r], top_k[r] or None, top_p[r], keys[r]) for r in range(R)]
        assert got == want


def test_sampler_top_k_with_few_and_with_many_tokens_near_the_kth():
    """top-k gathers the tokens that share the k-th largest's sign and exponent range into shared memory when they are
    few, and searches the whole row when they are many (a row whose values lie within one factor of two; negative
    rows; a row of equal values): with and without top-p, against the plain sampler."""
    from vllm_oxide_b200.sampling import Sampler, row_key
    g = torch.Generator().manual_seed(5)
    V = 151936
    peaked = 2.0 * torch.randn(V, generator=g)
    narrow = 2.0 + 0.9 * torch.rand(V, generator=g)          # all of the row in one exponent: nothing to gather
    negative = -3.0 - 0.5 * torch.rand(V, generator=g)
    equal = torch.full((V,), 1.25)
    equal[77] = 1.5
    ties = peaked.clone()
    ties[torch.randperm(V, generator=g)[:300]] = ties.max() + 1   # 300 equal values at the top, k inside them
    rows = [peaked, narrow, negative, equal, ties, peaked, narrow, ties]
    logits = torch.stack(rows).float()
    R = logits.shape[0]
    temperature = [1.0, 0.01, 1.0, 1.0, 0.9, 1.5, 0.02, 1.0]
    top_k = [50, 50, 7, 20, 100, 4000, 5000, 301]
    top_p = [1.0, 1.0, 0.9, 1.0, 1.0, 0.95, 0.7, 0.5]
    s = Sampler(DEV, 8)
    for trial in range(3):
        keys = [row_key(23 + trial, r, 2 * r) for r in range(R)]
        got = s.forward(logits.to(DEV), temperature, top_k, top_p, keys).cpu().tolist()
        want = [S.sample_row(logits[r].numpy(), temperature[r], top_k[r], top_p[r] if top_p[r] < 1 else None, keys[r])
                for r in range(R)]
        assert got == want


def test_sampler_takes_minus_zero_for_zero():
    """-0.0 and 0.0 are one value: among equal maxima the lowest index wins whatever the signs of the zeros, and top-p
    cuts by value (rows of rounded logits against the plain sampler)."""
    from vllm_oxide_b200.sampling import Sampler, row_key
    s = Sampler(DEV, 4)
    x = torch.full((1, 50), -3.0)
    x[0, 7], x[0, 3] = 0.0, -0.0
    assert s.forward(x.to(DEV), [0.0], [0], [1.0], [row_key(1, 0, 0)]).item() == 3
    g = torch.Generator().manual_seed(131)
    rows = torch.round(2 * torch.randn(6, 4097, generator=g)).float()
    assert (rows == 0).any() and torch.signbit(rows[rows == 0]).any()
    keys = [row_key(5, r, r) for r in range(6)]
    got = s.forward(rows.to(DEV), [1.7] * 6, [0] * 6, [0.5] * 6, keys).cpu().tolist()
    assert got == [S.sample_row(rows[r].numpy(), 1.7, None, 0.5, keys[r]) for r in range(6)]


def test_sampler_rows_do_not_depend_on_the_batch_and_follow_the_distribution():
    from vllm_oxide_b200.sampling import Sampler, row_key
    s = Sampler(DEV, 4)
    probs = torch.tensor([0.6, 0.25, 0.1, 0.05])
    logits = probs.log().repeat(3000, 1).to(DEV)
    keys = [row_key(1, 9, i) for i in range(3000)]
    toks = s.forward(logits, [1.0] * 3000, [0] * 3000, [1.0] * 3000, keys).cpu()
    freq = torch.bincount(toks, minlength=4).float() / 3000
    assert (freq - probs).abs().max() < 0.03
    alone = s.forward(logits[17:18], [1.0], [0], [1.0], keys[17:18]).cpu()
    assert alone[0] == toks[17]


def test_penalties_kernel():
    from vllm_oxide_b200.sampling import Sampler
    s = Sampler(DEV, 4)
    logits = torch.full((2, 6), 4.0, device=DEV)
    s.apply_penalties(logits, [[1, 1, 1, 2], None], [0.5, 0.0], [0.25, 0.0], [2.0, 0.0])
    want = S.apply_penalties(np.full(6, 4.0, np.float32), [1, 1, 1, 2], 0.5, 0.25, 2.0)
    assert np.allclose(logits[0].cpu().numpy(), want) and (logits[1] == 4).all()


def test_copy_pages():
    from vllm_oxide_b200 import kernels
    plane = torch.randn(6, 2, 16, 8, device=DEV)
    before = plane.clone()
    pairs = torch.tensor([[0, 4], [2, 5]], dtype=torch.int32, device=DEV)
    kernels.copy_pages(plane, pairs, 2)
    assert torch.equal(plane[4], before[0]) and torch.equal(plane[5], before[2]) and torch.equal(plane[:4], before[:4])


@pytest.mark.parametrize("M,N,K", [(1, 16, 64), (8, 4096, 4096), (3, 331, 128), (16, 24576 // 8, 512), (9, 100, 320),
                                   (5, 517, 192), (16, 48, 12288), (2, 151936 // 16, 1024), (4, 40, 704), (11, 70, 64)])
def test_gemm_skinny(M, N, K):
    from vllm_oxide_b200 import kernels
    g = torch.Generator().manual_seed(M * 1000 + N)
    x = torch.randn(M, K, generator=g).bfloat16().to(DEV)
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).bfloat16().to(DEV)
    assert kernels.gemm_skinny_supported(x, w)
    err = err_word()
    ref = x.double() @ w.double().t()
    out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    kernels.gemm_skinny(x, w, out, kernels.EPI_BF16, err)
    assert torch.allclose(out.double(), ref, rtol=1e-2, atol=1e-2)
    assert torch.equal(out, ref.float().bfloat16()) or (out.double() - ref).abs().max() < 0.02     # one rounding of a float sum
    outf = torch.full((M, N), float("nan"), dtype=torch.float32, device=DEV)
    kernels.gemm_skinny(x, w, outf, kernels.EPI_F32, err)
    assert torch.equal(outf, out.float())                                  # float logits are the bfloat16 values
    # a strided view (rows of a wider buffer) is taken too
    wide = torch.zeros(M, K + 64, dtype=torch.bfloat16, device=DEV)
    wide[:, :K] = x
    out2 = torch.empty_like(out)
    kernels.gemm_skinny(wide[:, :K], w, out2, kernels.EPI_BF16, err)
    assert torch.equal(out2, out) and err.item() == 0


@pytest.mark.parametrize("M,I,K", [(1, 8, 64), (8, 12288 // 4, 1024), (7, 104, 128), (16, 200, 192), (12, 64, 4096)])
def test_gemm_skinny_swiglu(M, I, K):
    from vllm_oxide_b200 import kernels
    g = torch.Generator().manual_seed(M + I)
    x = torch.randn(M, K, generator=g).bfloat16()
    wg = (2 * torch.randn(I, K, generator=g) / math.sqrt(K)).bfloat16()
    wu = (torch.randn(I, K, generator=g) / math.sqrt(K)).bfloat16()
    one = torch.eye(I).bfloat16()
    want = P.swiglu(x, wg, wu, one, torch.bfloat16)          # down = identity: the activation itself
    out = torch.full((M, I), float("nan"), dtype=torch.bfloat16, device=DEV)
    err = err_word()
    if I % 8:
        return      # the fused activation needs groups of eight outputs
    wgu = torch.stack([wg.reshape(I // 8, 8, K), wu.reshape(I // 8, 8, K)], dim=1).reshape(2 * I, K)
    kernels.gemm_skinny(x.to(DEV), wgu.to(DEV), out, kernels.EPI_SWIGLU, err)
    assert torch.allclose(out.cpu().float(), want.float(), rtol=2e-2, atol=2e-2) and err.item() == 0


@pytest.mark.parametrize("M,N,K", [(1, 96, 64), (8, 6144, 4096), (5, 331, 320), (13, 4096, 1024), (16, 520, 192), (3, 9472, 768),
                                   (12, 6400, 256), (16, 128, 64), (9, 20032, 128)])
def test_gemm_skinny_with_the_norm_in_front_and_the_residual_behind(M, N, K):
    """The residual stream kept inside the products: RMSNorm of the tokens applied on the way (plain: norm, then the
    product of the rounded result), and the product added to its output in place."""
    from vllm_oxide_b200 import kernels
    g = torch.Generator().manual_seed(M * 7 + N)
    eps = 1e-5
    x = (3 * torch.randn(M, K, generator=g)).bfloat16()
    wn = (1 + 0.2 * torch.randn(K, generator=g)).bfloat16()
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).bfloat16()
    normed, _ = P.add_rms_norm(x, None, wn, eps, torch.bfloat16)
    want = P.linear(normed, w, torch.bfloat16)
    err = err_word()
    out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    kernels.gemm_skinny(x.to(DEV), w.to(DEV), out, kernels.EPI_BF16, err, norm_weight=wn.float().to(DEV), eps=eps)
    assert torch.allclose(out.cpu().float(), want.float(), rtol=2e-2, atol=2e-2) and err.item() == 0
    # the same product without the norm, added to what is there
    before = torch.randn(M, N, generator=g).bfloat16()
    acc = before.clone().to(DEV)
    kernels.gemm_skinny(x.to(DEV), w.to(DEV), acc, kernels.EPI_ADD, err)
    plain = (P.linear(x, w, torch.bfloat16).float() + before.float()).bfloat16()
    assert torch.allclose(acc.cpu().float(), plain.float(), rtol=2e-2, atol=2e-2) and err.item() == 0
    # the norm in two halves: the adding product leaves stream * weight and the sums of squares behind, the product
    # after it takes them instead of doing the norm's arithmetic itself; against the norm applied on the way, and plain
    if N % 64 == 0:
        wn2 = (1 + 0.2 * torch.randn(N, generator=g)).bfloat16()
        w2 = (torch.randn(72, N, generator=g) / math.sqrt(N)).bfloat16().to(DEV)
        acc2 = before.clone().to(DEV)
        scaled = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
        parts = torch.full((kernels.gemm_skinny_weight_tiles(N) * 16,), float("nan"), device=DEV)
        kernels.gemm_skinny(x.to(DEV), w.to(DEV), acc2, kernels.EPI_ADD, err, emit=(wn2.float().to(DEV), scaled, parts))
        assert torch.equal(acc2, acc)                                       # the stream itself is what it was
        assert torch.equal(scaled.cpu(), (acc.cpu().float() * wn2.float()).bfloat16())
        box = 8 if M <= 8 else 16
        sums = parts[:kernels.gemm_skinny_weight_tiles(N) * box].view(-1, box).sum(0)[:M].cpu()
        assert torch.allclose(sums, acc.cpu().float().pow(2).sum(-1), rtol=1e-5)
        on_the_way = torch.empty(M, 72, dtype=torch.bfloat16, device=DEV)
        kernels.gemm_skinny(acc, w2, on_the_way, kernels.EPI_BF16, err, norm_weight=wn2.float().to(DEV), eps=eps)
        ahead = torch.empty(M, 72, dtype=torch.bfloat16, device=DEV)
        kernels.gemm_skinny(scaled, w2, ahead, kernels.EPI_BF16, err, eps=eps, prenormed=parts)
        normed2, _ = P.add_rms_norm(acc.cpu(), None, wn2, eps, torch.bfloat16)
        want2 = P.linear(normed2, w2.cpu(), torch.bfloat16)
        assert torch.allclose(ahead.cpu().float(), want2.float(), rtol=2e-2, atol=2e-2) and err.item() == 0
        # the two ways differ only in the order the squares are added: a unit of bfloat16 here and there, no more
        assert (ahead.float() - on_the_way.float()).abs().max() <= 2 ** -7 * on_the_way.float().abs().max()
        assert (ahead != on_the_way).float().mean() < 0.01
    # norm in front of the fused activation
    if N % 16 == 0:
        I = N // 2
        wg, wu = w[:I], w[I:]
        want_act = P.swiglu(normed, wg, wu, torch.eye(I).bfloat16(), torch.bfloat16)
        wgu = torch.stack([wg.reshape(I // 8, 8, K), wu.reshape(I // 8, 8, K)], dim=1).reshape(N, K)
        act = torch.full((M, I), float("nan"), dtype=torch.bfloat16, device=DEV)
        kernels.gemm_skinny(x.to(DEV), wgu.to(DEV), act, kernels.EPI_SWIGLU, err, norm_weight=wn.float().to(DEV), eps=eps)
        assert torch.allclose(act.cpu().float(), want_act.float(), rtol=3e-2, atol=3e-2) and err.item() == 0


def test_gemm_skinny_refuses_what_it_cannot_take():
    from vllm_oxide_b200 import kernels
    x = torch.zeros(17, 64, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(8, 64, dtype=torch.bfloat16, device=DEV)
    assert not kernels.gemm_skinny_supported(x, w)
    assert not kernels.gemm_skinny_supported(x[:4, :48], w[:, :48])        # K is not a multiple of 64
    x2 = torch.zeros(4, 136, dtype=torch.bfloat16, device=DEV)
    assert not kernels.gemm_skinny_supported(x2[:, 4:132], torch.zeros(8, 128, dtype=torch.bfloat16, device=DEV))   # misaligned rows
    assert not kernels.gemm_skinny_supported(x[:4].float(), w.float())
    with pytest.raises(kernels.KernelError, match="not supported"):
        kernels.gemm_skinny(x, w, torch.zeros(17, 8, dtype=torch.bfloat16, device=DEV), kernels.EPI_BF16, err_word())


def test_a_wait_that_runs_out_comes_back_as_an_error_word_and_the_next_launch_is_right():
    """Failure detection without a fault: the producers of the weight-streaming product withhold their copies (a flag
    that only this test sets), so every block waits for data that never comes; with the waits shortened to a few hundred
    tries they run out at once: the kernel returns, the error word says 'a bounded wait ran out' and in which kernel,
    nothing was written, and (limit and copies restored) the next ordinary launch on the same context gives the right
    product.  Nothing spins without a bound, nothing faults, and no copy is in flight when a block leaves."""
    from vllm_oxide_b200 import kernels
    M, N, K = 8, 4096, 4096
    g = torch.Generator().manual_seed(3)
    x = torch.randn(M, K, generator=g).bfloat16().to(DEV)
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).bfloat16().to(DEV)
    ref = x.double() @ w.double().t()
    err = err_word()
    out = torch.full((M, N), 7.0, dtype=torch.bfloat16, device=DEV)
    kernels.gemm_skinny_set_wait_limit(300, withhold_copies=True)
    try:
        kernels.gemm_skinny(x, w, out, kernels.EPI_BF16, err)
        torch.cuda.synchronize()
    finally:
        kernels.gemm_skinny_set_wait_limit(0)
    word = int(err.item())
    assert word == 0x20 | 0x100, hex(word)                       # VOB_ERR_TIMEOUT | VOB_WHERE_GEMM_SKINNY
    assert "a bounded wait inside a kernel ran out" in kernels.describe_error_word(word)
    assert "weight-streaming product" in kernels.describe_error_word(word)
    assert bool((out == 7.0).all())                              # a block that gave up wrote nothing
    err.zero_()
    kernels.gemm_skinny(x, w, out, kernels.EPI_BF16, err)
    assert torch.allclose(out.double(), ref, rtol=1e-2, atol=1e-2) and err.item() == 0


@pytest.mark.parametrize("M,N,K", [(14, 17464, 1536), (16, 17472, 1024), (5, 20000, 1280)])
def test_gemm_skinny_a_fast_refill_does_not_overtake_the_readers(M, N, K):
    """A matrix that stays in L2 and gives blocks two tiles each: the copy engine refills a stage of the ring as soon as
    it is released, and must not overwrite what a warp is still reading (one launch in three was wrong before the
    release was preceded by a proxy fence).  Thirty launches, each against a float64 product."""
    from vllm_oxide_b200 import kernels
    g = torch.Generator().manual_seed(1)
    x = torch.randn(M, K, generator=g).bfloat16().to(DEV)
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).bfloat16().to(DEV)
    ref = x.double() @ w.double().t()
    err = err_word()
    for _ in range(30):
        out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
        kernels.gemm_skinny(x, w, out, kernels.EPI_BF16, err)
        assert torch.allclose(out.double(), ref, rtol=1e-2, atol=2e-2) and err.item() == 0


@pytest.mark.parametrize("M,N,K", [(17, 128, 64), (32, 256, 128), (33, 331, 80), (64, 4096, 4096), (100, 517, 200),
                                   (128, 1000, 1024), (8, 128, 64), (64, 24576 // 8, 512), (48, 130, 12288), (40, 24576, 320),
                                   (128, 8192, 1024), (23, 6144, 4096)])
def test_gemm_tc5(M, N, K):
    """The tcgen05 product (accumulator in tensor memory) against a float64 product."""
    from vllm_oxide_b200 import kernels
    g = torch.Generator().manual_seed(M * 1000 + N)
    x = torch.randn(M, K, generator=g).bfloat16().to(DEV)
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).bfloat16().to(DEV)
    assert kernels.gemm_tc5_supported(x, w)
    err = err_word()
    ref = x.double() @ w.double().t()
    out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    kernels.gemm_tc5(x, w, out, kernels.EPI_BF16, err)
    torch.cuda.synchronize()
    assert err.item() == 0
    assert torch.allclose(out.double(), ref, rtol=1e-2, atol=1e-2)
    outf = torch.full((M, N), float("nan"), dtype=torch.float32, device=DEV)
    kernels.gemm_tc5(x, w, outf, kernels.EPI_F32, err)
    assert torch.equal(outf, out.float()) and err.item() == 0
    # split along K over the blocks of a cluster, twice in a row; the choice of the library is one of them
    assert 1 <= kernels.gemm_tc5_cluster(x, w, kernels.EPI_BF16) <= 8
    for cluster in (1, 2, 3, 4, 5, 8):
        k_iters = -(-K // 64)
        if (cluster - 1) * -(-k_iters // cluster) >= k_iters:
            continue                      # a K range would be empty
        for _ in range(2):
            o2 = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
            kernels.gemm_tc5(x, w, o2, kernels.EPI_BF16, err, cluster=cluster)
            assert torch.allclose(o2.double(), ref, rtol=1e-2, atol=1e-2) and err.item() == 0


@pytest.mark.parametrize("M,I,K", [(17, 8, 64), (64, 12288 // 4, 1024), (40, 104, 128), (128, 200, 192)])
def test_gemm_tc5_swiglu(M, I, K):
    from vllm_oxide_b200 import kernels
    g = torch.Generator().manual_seed(M + I)
    x = torch.randn(M, K, generator=g).bfloat16()
    wg = (2 * torch.randn(I, K, generator=g) / math.sqrt(K)).bfloat16()
    wu = (torch.randn(I, K, generator=g) / math.sqrt(K)).bfloat16()
    want = P.swiglu(x, wg, wu, torch.eye(I).bfloat16(), torch.bfloat16)
    wgu = torch.stack([wg.reshape(I // 8, 8, K), wu.reshape(I // 8, 8, K)], dim=1).reshape(2 * I, K)
    out = torch.full((M, I), float("nan"), dtype=torch.bfloat16, device=DEV)
    err = err_word()
    kernels.gemm_tc5(x.to(DEV), wgu.to(DEV), out, kernels.EPI_SWIGLU, err)
    assert torch.allclose(out.cpu().float(), want.float(), rtol=2e-2, atol=2e-2) and err.item() == 0
    if K >= 128:
        out.fill_(float("nan"))
        kernels.gemm_tc5(x.to(DEV), wgu.to(DEV), out, kernels.EPI_SWIGLU, err, cluster=2)
        assert torch.allclose(out.cpu().float(), want.float(), rtol=2e-2, atol=2e-2) and err.item() == 0
