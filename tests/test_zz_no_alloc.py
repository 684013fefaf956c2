"""The decode-attention entry point for callers that cannot allocate device memory.

Some users of the kernel library may not call cudaMalloc where they stand: inside a stream capture,
on a thread that must not take the allocator's locks, or in a process whose device memory belongs to
another allocator.  For them `vob_attention_decode_noalloc` keeps the split-key kernel's partial
results in a fixed array inside the library.  This test calls it through its exported C symbol, several
times in a row on different inputs (every call after the first finds the previous call's leftovers in
the array), and checks each result against the ordinary entry point's and against the plain attention
of the test suite; the device's free memory must not change around a call, and a launch too large for
the array is refused.  The file is named so that pytest collects it last.
"""
import ctypes
import math

import pytest
import torch

from test_gpu_kernels import decode_attention, run_attention

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
HD = 128


def _library():
    from vllm_oxide_b200.csrc import build
    lib = ctypes.CDLL(build.build_attention(HD))
    lib.vob_attention_decode_noalloc_error.restype = ctypes.c_char_p
    lib.vob_attention_decode_noalloc_max_floats.restype = ctypes.c_long
    return lib


def _no_alloc(lib, splits, free_bytes):
    """The new entry point in the shape `run_attention` calls a kernel in; appends the device's free bytes before and
    after the call to `free_bytes`."""
    def fn(q, out, kc, vc, bt, cu_q, ctx, T, nh, kvh, hd, window, err, **_):
        p = lambda t: ctypes.c_void_p(t.data_ptr())
        stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        q2 = q.reshape(T, nh * hd)
        torch.cuda.synchronize()
        before = torch.cuda.mem_get_info()[0]
        rc = lib.vob_attention_decode_noalloc(p(q2), ctypes.c_long(nh * hd), p(out), p(kc), p(vc), p(bt), bt.shape[1],
                                              p(cu_q), p(ctx), ctx.shape[0], nh, kvh, kc.shape[2], window,
                                              ctypes.c_float(1 / math.sqrt(hd)), ctypes.c_long(kc.shape[0]), splits,
                                              p(err), stream)
        assert rc == 0, lib.vob_attention_decode_noalloc_error(rc).decode()
        torch.cuda.synchronize()
        free_bytes.append((before, torch.cuda.mem_get_info()[0]))
    return fn


# nh, kvh, block size, window, context lengths, splits: several splits (the array is used), one split (it is not), a
# window, and contexts that end exactly on a page's edge
CASES = [(16, 4, 64, 0, [700, 64, 1, 333], 5), (16, 4, 64, 0, [90, 1500, 65], 5), (32, 8, 256, 0, [512, 256, 300], 1),
         (8, 2, 64, 100, [400, 99, 101, 128], 3), (16, 4, 16, 0, [160, 16, 48], 2)]


def test_no_alloc_entry_point_matches_the_ordinary_one_and_the_plain_attention():
    lib = _library()
    assert lib.vob_attention_decode_noalloc_max_floats() == 2 * 1024 * 1024
    free_bytes = []
    for seed, (nh, kvh, bs, window, ctx_lens, splits) in enumerate(CASES):
        args = (torch.bfloat16, nh, kvh, HD, bs, window, [1] * len(ctx_lens), ctx_lens)
        got, want = run_attention(_no_alloc(lib, splits, free_bytes), *args, seed=seed)
        # against the plain attention, within what one bfloat16 rounding of the output allows (outputs are of order one)
        assert (got - want).abs().max() < 1.5e-2, (got - want).abs().max()
        ordinary, _ = run_attention(decode_attention(splits, use_tma=False), *args, seed=seed)
        assert torch.equal(got, ordinary)              # the same kernels: the same bits
        with_tma, _ = run_attention(decode_attention(splits, use_tma=True), *args, seed=seed)
        assert torch.allclose(got, with_tma, rtol=2e-2, atol=2e-2)
    # the first call may map the library's array; no later call changes the device's free memory
    assert all(before == after for before, after in free_bytes[1:]), free_bytes


def test_no_alloc_entry_point_refuses_what_does_not_fit():
    lib = _library()
    z = torch.zeros(64, dtype=torch.int32, device=DEV)
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    # 64 requests x 32 heads x 8 splits x 129 floats do not fit into the array: refused, nothing runs
    rc = lib.vob_attention_decode_noalloc(p(z), ctypes.c_long(32 * HD), p(z), p(z), p(z), p(z), 1, p(z), p(z), 64, 32, 8, 64,
                                          0, ctypes.c_float(0.1), ctypes.c_long(1), 8, p(z), stream)
    assert rc == 2003 and b"exceed the built-in scratch array" in lib.vob_attention_decode_noalloc_error(rc)
    # heads that do not divide into groups are refused before anything is looked up
    rc = lib.vob_attention_decode_noalloc(p(z), ctypes.c_long(32 * HD), p(z), p(z), p(z), p(z), 1, p(z), p(z), 1, 32, 5, 64,
                                          0, ctypes.c_float(0.1), ctypes.c_long(1), 2, p(z), stream)
    assert rc == 2001
    torch.cuda.synchronize()
