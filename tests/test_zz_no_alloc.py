"""The decode-attention entry point for callers that cannot allocate device memory.

Some users of the kernel library may not call cudaMalloc where they stand: inside a stream capture,
on a thread that must not take the allocator's locks, or in a process whose device memory belongs to
another allocator.  For them `vob_attention_decode_noalloc` keeps the split-key kernel's partial
results in a fixed array inside the library.  This test calls it through its exported C symbol, twice
in a row on different inputs (the second call finds the first call's leftovers in the array), and
checks each result against the ordinary entry point's; it also checks that a launch too large for
the array is refused.  The file is named so that pytest collects it last.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _inputs(seed, B, nh, kvh, hd, bs, ctx_lens):
    g = torch.Generator().manual_seed(seed)
    pages_per = [(c + bs - 1) // bs for c in ctx_lens]
    num_pages = sum(pages_per) + 2
    perm = torch.randperm(num_pages, generator=g).tolist()
    bt = torch.full((B, max(pages_per)), -1, dtype=torch.int32)
    it = iter(perm)
    for b in range(B):
        for p in range(pages_per[b]):
            bt[b, p] = next(it)
    kc = torch.randn(num_pages, kvh, bs, hd, generator=g).bfloat16()
    vc = torch.randn(num_pages, kvh, bs, hd, generator=g).bfloat16()
    q = torch.randn(B, nh * hd, generator=g).bfloat16()
    cu_q = torch.arange(B + 1, dtype=torch.int32)
    ctx = torch.tensor(ctx_lens, dtype=torch.int32)
    return [t.to(DEV) for t in (q, kc, vc, bt, cu_q, ctx)]


def test_no_alloc_entry_point_matches_the_ordinary_one_twice_in_a_row():
    from vllm_oxide_b200 import kernels
    from vllm_oxide_b200.csrc import build
    hd, nh, kvh, bs, splits = 128, 16, 4, 64, 5
    lib = ctypes.CDLL(build.build_attention(hd))
    lib.vob_attention_decode_noalloc_error.restype = ctypes.c_char_p
    lib.vob_attention_decode_noalloc_max_floats.restype = ctypes.c_long
    assert lib.vob_attention_decode_noalloc_max_floats() == 2 * 1024 * 1024
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    for seed, ctx_lens in [(1, [700, 64, 1, 333]), (2, [90, 1500, 65])]:
        B = len(ctx_lens)
        q, kc, vc, bt, cu_q, ctx = _inputs(seed, B, nh, kvh, hd, bs, ctx_lens)
        want = torch.empty(B, nh * hd, dtype=torch.bfloat16, device=DEV)
        n = kernels.attention_decode_scratch_floats(hd, B, nh, splits)
        kernels.attention_decode(q, nh * hd, want, kc, vc, bt, cu_q, ctx, B, nh, kvh, hd, 0, 1 / math.sqrt(hd), splits,
                                 torch.empty(n, device=DEV), err)
        got = torch.full_like(want, float("nan"))
        allocated = torch.cuda.memory_allocated()
        rc = lib.vob_attention_decode_noalloc(p(q), ctypes.c_long(nh * hd), p(got), p(kc), p(vc), p(bt), bt.shape[1],
                                              p(cu_q), p(ctx), B, nh, kvh, bs, 0, ctypes.c_float(1 / math.sqrt(hd)),
                                              ctypes.c_long(kc.shape[0]), splits, p(err), stream)
        assert rc == 0, lib.vob_attention_decode_noalloc_error(rc).decode()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == allocated
        assert err.item() == 0
        assert torch.allclose(got.float(), want.float(), rtol=2e-2, atol=2e-2)
    # 64 requests x 32 heads x 8 splits x 129 floats do not fit into the array: refused, nothing runs
    rc = lib.vob_attention_decode_noalloc(p(q), ctypes.c_long(nh * hd), p(got), p(kc), p(vc), p(bt), bt.shape[1], p(cu_q),
                                          p(ctx), 64, 32, 8, bs, 0, ctypes.c_float(0.1), ctypes.c_long(kc.shape[0]), 8,
                                          p(err), stream)
    assert rc == 2003 and b"exceed the built-in scratch array" in lib.vob_attention_decode_noalloc_error(rc)
