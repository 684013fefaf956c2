"""ctypes bindings of libvob_kernels.so: one Python function per C entry point.

The library is built in-tree at first use.  There is no fallback: without a CUDA device,
without nvcc or without the built library every call raises `KernelError`.  Tensors are
passed as raw device pointers; every launch goes to torch's current stream, so launches
made inside `torch.cuda.graph(...)` are captured.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .csrc import build as _build


class KernelError(RuntimeError):
    pass


import os as _os

_lib = None
DTYPE_CODES = {torch.float32: 0, torch.bfloat16: 1}

ERR_BITS = {1: "a token id outside the vocabulary", 2: "a position beyond max_position_embeddings",
            4: "a cache slot outside the pool", 8: "a block-table entry that names no page",
            16: "a wanted row outside the batch", 32: "a bounded wait inside a kernel ran out",
            0x100: "(in the weight-streaming product)", 0x200: "(in the tcgen05 product)", 0x400: "(in decode attention)",
            0x800: "(in the attention for portions, mma.sync)", 0x1000: "(in the attention for portions, tcgen05)"}


def lib():
    global _lib
    if _lib is None:
        try:
            path = _build.build_kernels()
            _lib = ctypes.CDLL(path)
        except (OSError, _build.BuildError) as e:
            raise KernelError(f"the CUDA kernel library of vllm_oxide_b200 is not available: {e}") from e
        _lib.vob_error_string.restype = ctypes.c_char_p
        _lib.vob_error_string.argtypes = [ctypes.c_int]
    return _lib


_attn_libs = {}


def attention_lib(head_dim: int):
    """The tensor-core attention library for one head size, built at first use."""
    if head_dim not in _attn_libs:
        try:
            L = ctypes.CDLL(_build.build_attention(head_dim))
        except (OSError, _build.BuildError) as e:
            raise KernelError(f"the attention kernels for head size {head_dim} are not available: {e}") from e
        L.vob_attention_decode_scratch_floats.restype = ctypes.c_long
        _attn_libs[head_dim] = L
    return _attn_libs[head_dim]


def has_fast_attention(dtype, head_dim: int, group: int) -> bool:
    """Whether the tensor-core attention kernels take this case; the plain kernel takes the rest."""
    return dtype == torch.bfloat16 and head_dim % 16 == 0 and 16 <= head_dim <= 256 and group <= 16


def sm_count() -> int:
    """The number of SMs of the current device (the library asks the device once)."""
    return int(lib().vob_sm_count())


launch_count = 0   # launches of this package's own kernels since import (bench.py reports the difference)

# Per-kernel-class device timers, off unless asked for (VOB_KERNEL_TIMERS=1 or enable_kernel_timers()): every launch
# of this package's kernels is then bracketed by two CUDA events on its stream, and kernel_timer_report() adds them up
# by entry point.  It serialises nothing, but events cannot be recorded into a CUDA graph: time with
# EngineOptions(enforce_eager=True).  The event before a launch is recorded where the launch asks for its stream,
# which every binding does as the last thing before it calls the library.
_timers = None          # None: off; else a list of (entry point, start event, end event)
_timer_start = None


def enable_kernel_timers(on: bool = True) -> None:
    global _timers, _timer_start
    _timers, _timer_start = ([] if on else None), None


def kernel_timer_report(reset: bool = True):
    """{entry point: (launches, milliseconds on the device)} since the timers were enabled or last reset."""
    global _timers
    if _timers is None:
        raise KernelError("the kernel timers are off: enable_kernel_timers() or VOB_KERNEL_TIMERS=1")
    torch.cuda.synchronize()
    out = {}
    for what, e0, e1 in _timers:
        n, ms = out.get(what, (0, 0.0))
        out[what] = (n + 1, ms + e0.elapsed_time(e1))
    if reset:
        _timers = []
    return out


def _check(code: int, what: str) -> None:
    global launch_count, _timer_start
    launch_count += 1
    if _timers is not None and _timer_start is not None:
        end = torch.cuda.Event(enable_timing=True)
        end.record(torch.cuda.current_stream(torch.cuda.current_device()))
        _timers.append((what, _timer_start, end))
        _timer_start = None
    if code != 0:
        raise KernelError(f"{what}: {lib().vob_error_string(code).decode()} (code {code})")


def _p(t: Optional[torch.Tensor]):
    return ctypes.c_void_p(t.data_ptr() if t is not None else 0)


def _stream():
    """The current stream's handle.  torch.cuda.current_stream() without a device spends 15 us looking the device up;
    with the index given it is a plain call."""
    global _timer_start
    stream = torch.cuda.current_stream(torch.cuda.current_device())
    if _timers is not None and not torch.cuda.is_current_stream_capturing():
        _timer_start = torch.cuda.Event(enable_timing=True)
        _timer_start.record(stream)
    return ctypes.c_void_p(stream.cuda_stream)


def _code(dtype: torch.dtype) -> int:
    try:
        return DTYPE_CODES[dtype]
    except KeyError:
        raise KernelError(f"dtype {dtype} is not supported (float32 or bfloat16)") from None


def _cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("vllm_oxide_b200 kernels run on CUDA tensors only; there is no CPU path")


def describe_error_word(word: int) -> str:
    return "; ".join(msg for bit, msg in ERR_BITS.items() if word & bit) or f"unknown error bits {word}"


def embedding(table, ids, out, num_tokens: int, err, scale: float = 1.0) -> None:
    """out[t] = table[ids[t]] * scale."""
    _cuda(table, ids, out)
    V, H = table.shape
    _check(lib().vob_embedding(_p(table), _p(ids), _p(out), num_tokens, H, V, ctypes.c_float(scale), _code(table.dtype),
                               _p(err), _stream()), "embedding")


def softcap(logits, num_rows: int, cap: float) -> None:
    """logits = cap * tanh(logits / cap), in place (float32 rows)."""
    _cuda(logits)
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    _check(lib().vob_softcap(_p(logits), ctypes.c_long(logits.stride(0)), num_rows, logits.shape[1], ctypes.c_float(cap),
                             _stream()), "softcap")


def add_rmsnorm(x, residual, weight, y, eps: float, has_residual: bool, err, rows=None, n_out: Optional[int] = None):
    """y = RMSNorm(x + residual) * weight; residual updated in place (unless `rows` selects source rows)."""
    _cuda(x, residual, weight, y, rows)
    assert weight.dtype == torch.float32
    H = x.shape[-1]
    n_src = x.shape[0]
    n = n_src if n_out is None else n_out
    _check(lib().vob_add_rmsnorm(_p(x), _p(residual), _p(weight), _p(y), _p(rows), n, H, n_src,
                                 ctypes.c_float(eps), int(has_residual), _code(x.dtype), _p(err), _stream()),
           "add_rmsnorm")


def silu_mul(gate_up, out, num_tokens: int, interleaved: bool = False) -> None:
    """out = SiLU(gate) * up; gate_up holds [gate | up] per token, or, interleaved, groups of 8 gate + 8 up columns."""
    _cuda(gate_up, out)
    I = out.shape[-1]
    _check(lib().vob_silu_mul(_p(gate_up), _p(out), num_tokens, I, int(interleaved), _code(out.dtype), _stream()),
           "silu_mul")


def qk_norm_rope_kv_write(qkv, bias, positions, slots, wq, wk, rule, kcache, vcache, num_tokens, nh, kvh, hd,
                          eps, write_kv: bool, err) -> None:
    """Bias, per-head norm, rotation and cache write of a merged q|k|v row.  `rule` is the position encoding's
    `RotationRule` (table [max_pos, rotary_dim] float32, rotary_dim, interleaved); a rule with rotary_dim 0 rotates
    nothing."""
    table = rule.table if rule.rotary_dim > 0 else None
    _cuda(qkv, positions, slots, table, kcache, vcache)
    if table is not None and (table.dtype != torch.float32 or table.shape[1] != rule.rotary_dim or not table.is_contiguous()):
        raise KernelError(f"the table of angles must be contiguous float32 [max_pos, {rule.rotary_dim}]")
    num_slots = kcache.shape[0] * kcache.shape[2] if kcache is not None else 0
    block_size = kcache.shape[2] if kcache is not None else 1
    max_pos = table.shape[0] if table is not None else 0
    _check(lib().vob_qk_norm_rope_kv_write(_p(qkv), _p(bias), _p(positions), _p(slots), _p(wq), _p(wk), _p(table),
                                           _p(kcache), _p(vcache), num_tokens, nh, kvh, hd, rule.rotary_dim,
                                           int(rule.interleaved), ctypes.c_float(eps), max_pos, ctypes.c_long(num_slots),
                                           block_size, int(write_kv), _code(qkv.dtype), _p(err), _stream()),
           "qk_norm_rope_kv_write")


def paged_attention_generic(q, q_stride, out, kcache, vcache, block_tables, token_req, positions, num_tokens, nh, kvh,
                            hd, window: int, scale: float, err, skip_single_cu_q=None) -> None:
    """Every token of the batch; with `skip_single_cu_q` (the batch's cu_q) the tokens of requests that
    bring exactly one token are left to the decode kernel."""
    _cuda(q, out, kcache, vcache, block_tables, token_req, positions)
    _check(lib().vob_paged_attention_generic(_p(q), ctypes.c_long(q_stride), _p(out), _p(kcache), _p(vcache),
                                             _p(block_tables), block_tables.shape[-1], _p(token_req), _p(positions),
                                             _p(skip_single_cu_q), num_tokens, nh, kvh, hd, kcache.shape[2], window,
                                             ctypes.c_float(scale), ctypes.c_long(kcache.shape[0]), _code(q.dtype),
                                             _p(err), _stream()), "paged_attention_generic")


def attention_decode_scratch_floats(head_dim: int, num_requests: int, nh: int, num_splits: int) -> int:
    return int(attention_lib(head_dim).vob_attention_decode_scratch_floats(num_requests, nh, num_splits))


def attention_decode(q, q_stride, out, kcache, vcache, block_tables, cu_q, context_lens, num_requests, nh, kvh, hd,
                     window: int, scale: float, num_splits: int, scratch, err, use_tma: bool = True, pairs=None) -> None:
    """Requests that bring exactly one token; the others are skipped.  `pairs`: two int32 zeros on the device that belong
    to this caller (`decode_pairs_counter`); with it, one split and more (request, kv head) pairs than blocks fit the GPU
    run as persistent blocks that draw their pairs from it (the kernel leaves it at zero), without it as one block per
    pair.  Same bits either way."""
    _cuda(q, out, kcache, vcache, block_tables, cu_q, context_lens, scratch, pairs)
    assert pairs is None or (pairs.dtype == torch.int32 and pairs.numel() >= 2)
    assert q.dtype == torch.bfloat16 and kcache.dtype == torch.bfloat16
    L = attention_lib(hd)
    if use_tma and L.vob_attention_decode_has_tma() and kcache.is_contiguous() and vcache.is_contiguous():
        # head sizes that are a multiple of 64: keys and values come in by TMA (about twice cp.async's rate)
        bs = kcache.shape[2]
        keys, slices = L.vob_attention_decode_box_keys(bs), L.vob_attention_decode_box_slices(bs)
        map_k, map_v = tensor_map(kcache.view(-1, hd), keys, slices), tensor_map(vcache.view(-1, hd), keys, slices)
        _check(L.vob_attention_decode_tma(
            map_k, map_v, _p(q), ctypes.c_long(q_stride), _p(out), _p(kcache), _p(vcache), _p(block_tables),
            block_tables.shape[-1], _p(cu_q), _p(context_lens), num_requests, nh, kvh, kcache.shape[2], window,
            ctypes.c_float(scale), ctypes.c_long(kcache.shape[0]), num_splits, _p(scratch), _p(pairs), _p(err), _stream()),
            "attention_decode_tma")
        return
    _check(L.vob_attention_decode(
        _p(q), ctypes.c_long(q_stride), _p(out), _p(kcache), _p(vcache), _p(block_tables), block_tables.shape[-1],
        _p(cu_q), _p(context_lens), num_requests, nh, kvh, kcache.shape[2], window, ctypes.c_float(scale),
        ctypes.c_long(kcache.shape[0]), num_splits, _p(scratch), _p(err), _stream()), "attention_decode")


def decode_pairs_counter(device) -> torch.Tensor:
    """The counter that `attention_decode(pairs=...)` draws (request, kv head) pairs from: one per caller whose launches
    do not overlap in time (the engine keeps one per attention layer)."""
    return torch.zeros(2, dtype=torch.int32, device=device)


def attention_prefill(q, q_stride, out, kcache, vcache, block_tables, cu_q, context_lens, num_requests, max_q, nh, kvh,
                      hd, window: int, scale: float, err, use_tma: bool = True, use_tc5: bool = True,
                      query_tiles: int = 2, tiles_by_tma: bool = True) -> None:
    """Requests that bring more than one token; the others are skipped.  Head sizes 64 and 128 run on the tcgen05
    tensor cores (`use_tc5`; `tiles_by_tma` False makes that kernel bring its query tiles in by cp.async and store its
    output row by row also where TMA could), other multiples of 64 on mma.sync with TMA copies (`use_tma`), the rest with
    cp.async."""
    _cuda(q, out, kcache, vcache, block_tables, cu_q, context_lens)
    assert q.dtype == torch.bfloat16 and kcache.dtype == torch.bfloat16
    L = attention_lib(hd)
    if use_tma and L.vob_attention_decode_has_tma() and kcache.is_contiguous() and vcache.is_contiguous():
        bs = kcache.shape[2]
        keys, slices = L.vob_attention_decode_box_keys(bs), L.vob_attention_decode_box_slices(bs)
        map_k, map_v = tensor_map(kcache.view(-1, hd), keys, slices), tensor_map(vcache.view(-1, hd), keys, slices)
        if use_tc5 and L.vob_attention_prefill_has_tc5() and q_stride % 8 == 0:
            # the query tiles come and whole output tiles leave by TMA too (a tile holds whole tokens: 128 // group of them)
            box_heads = L.vob_attention_prefill_q_box_heads(nh, kvh) if tiles_by_tma else 0
            map_q = tensor_map_heads(q, q_stride, nh, hd, box_heads, 128 // box_heads) if box_heads > 0 else None
            map_o = (tensor_map_heads(out, nh * hd, nh, hd, box_heads, 128 // box_heads)
                     if box_heads > 0 and out.is_contiguous() and out.data_ptr() % 16 == 0 else None)
            _check(L.vob_attention_prefill_tc5(
                map_k, map_v, map_q, map_o, _p(q), ctypes.c_long(q_stride), _p(out), _p(block_tables), block_tables.shape[-1], _p(cu_q),
                _p(context_lens), num_requests, max_q, nh, kvh, bs, window, ctypes.c_float(scale),
                ctypes.c_long(kcache.shape[0]), query_tiles, _p(err), _stream()), "attention_prefill_tc5")
            return
        _check(L.vob_attention_prefill_tma(
            map_k, map_v, _p(q), ctypes.c_long(q_stride), _p(out), _p(kcache), _p(vcache), _p(block_tables),
            block_tables.shape[-1], _p(cu_q), _p(context_lens), num_requests, max_q, nh, kvh, bs, window,
            ctypes.c_float(scale), ctypes.c_long(kcache.shape[0]), _p(err), _stream()), "attention_prefill_tma")
        return
    _check(L.vob_attention_prefill(
        _p(q), ctypes.c_long(q_stride), _p(out), _p(kcache), _p(vcache), _p(block_tables), block_tables.shape[-1],
        _p(cu_q), _p(context_lens), num_requests, max_q, nh, kvh, kcache.shape[2], window, ctypes.c_float(scale),
        ctypes.c_long(kcache.shape[0]), _p(err), _stream()), "attention_prefill")


def gemm_f32(a, w, out, bias=None) -> None:
    """out[M,N] = a[M,K] @ w[N,K]^T in true float32."""
    _cuda(a, w, out)
    assert a.dtype == w.dtype == out.dtype == torch.float32
    M, K = a.shape
    N = w.shape[0]
    assert w.shape[1] == K and out.shape[0] == M and out.shape[1] == N
    assert a.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
    _check(lib().vob_gemm_f32(_p(a), ctypes.c_long(a.stride(0)), _p(w), ctypes.c_long(w.stride(0)), _p(out),
                              ctypes.c_long(out.stride(0)), _p(bias), M, N, K, _stream()), "gemm_f32")


EPI_BF16, EPI_F32, EPI_SWIGLU, EPI_ADD = 0, 1, 2, 3
_tensor_maps = {}


def tensor_map(t: torch.Tensor, box_rows: int, box_slices: int):
    """A TMA descriptor (host memory, cached) of a row-major bfloat16 matrix whose width is a multiple of 64: one copy
    brings `box_slices` column slices (64 columns each) of `box_rows` rows."""
    key = (t.data_ptr(), t.shape[0], t.shape[1], t.stride(0), box_rows, box_slices)
    hit = _tensor_maps.get(key)
    if hit is None:
        raw = (ctypes.c_char * 256)()
        addr = (ctypes.addressof(raw) + 63) & ~63
        code = lib().vob_tensor_map_bf16_sliced(ctypes.c_void_p(addr), _p(t), ctypes.c_long(t.shape[0]),
                                                ctypes.c_long(t.shape[1]), ctypes.c_long(t.stride(0)), box_rows, box_slices)
        if code != 0:
            raise KernelError(f"tensor map for a [{t.shape[0]}, {t.shape[1]}] matrix: {lib().vob_error_string(code).decode()}")
        if len(_tensor_maps) > 4096:
            _tensor_maps.clear()
        hit = _tensor_maps[key] = (raw, ctypes.c_void_p(addr))
    return hit[1]


def tensor_map_heads(t: torch.Tensor, token_stride: int, heads: int, head_dim: int, box_heads: int, box_tokens: int):
    """A TMA descriptor (host memory, cached) of token rows that begin with `heads` heads of `head_dim` bfloat16 each: one
    copy brings a 64-column slice of `box_heads` heads for `box_tokens` tokens, as rows in the order (token, head)."""
    key = (t.data_ptr(), t.shape[0], token_stride, heads, head_dim, box_heads, box_tokens, "heads")
    hit = _tensor_maps.get(key)
    if hit is None:
        raw = (ctypes.c_char * 256)()
        addr = (ctypes.addressof(raw) + 63) & ~63
        code = lib().vob_tensor_map_bf16_heads(ctypes.c_void_p(addr), _p(t), ctypes.c_long(t.shape[0]), heads, head_dim,
                                               ctypes.c_long(token_stride), box_heads, box_tokens)
        if code != 0:
            raise KernelError(f"tensor map for {t.shape[0]} token rows of {heads} heads: {lib().vob_error_string(code).decode()}")
        if len(_tensor_maps) > 4096:
            _tensor_maps.clear()
        hit = _tensor_maps[key] = (raw, ctypes.c_void_p(addr))
    return hit[1]


def tensor_map_2d(t: torch.Tensor, box_rows: int):
    """A TMA descriptor (host memory, cached) of a row-major bfloat16 matrix with box [box_rows, 64 columns]."""
    key = (t.data_ptr(), t.shape[0], t.shape[1], t.stride(0), box_rows, "2d")
    hit = _tensor_maps.get(key)
    if hit is None:
        raw = (ctypes.c_char * 256)()
        addr = (ctypes.addressof(raw) + 63) & ~63
        code = lib().vob_tensor_map_bf16_2d(ctypes.c_void_p(addr), _p(t), ctypes.c_long(t.shape[0]), ctypes.c_long(t.shape[1]),
                                            ctypes.c_long(t.stride(0)), box_rows)
        if code != 0:
            raise KernelError(f"tensor map for a [{t.shape[0]}, {t.shape[1]}] matrix: {lib().vob_error_string(code).decode()}")
        if len(_tensor_maps) > 4096:
            _tensor_maps.clear()
        hit = _tensor_maps[key] = (raw, ctypes.c_void_p(addr))
    return hit[1]


def gemm_tc5_supported(x, w) -> bool:
    """Whether the tcgen05 product takes x[M,K] @ w[N,K]^T: bfloat16, at most 128 rows of x, K a multiple of 8,
    rows that start on 16-byte boundaries."""
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.dim() == 2 and 0 < x.shape[0] <= 128
            and x.shape[1] % 8 == 0 and x.stride(1) == 1 and w.stride(1) == 1 and (x.stride(0) * 2) % 16 == 0
            and (w.stride(0) * 2) % 16 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_tc5_cluster(x, w, epilogue: int) -> int:
    """The number of K ranges (blocks of a thread-block cluster) the tcgen05 product chooses for x @ w^T on this device."""
    L = lib()
    return int(L.vob_gemm_tc5_cluster(x.shape[0], ctypes.c_long(w.shape[0]), ctypes.c_long(w.shape[1]), epilogue))


def gemm_tc5(x, w, out, epilogue: int, err, cluster: int = 0) -> None:
    """out = x @ w^T on the tcgen05 tensor cores for at most 128 rows of x; epilogues as gemm_skinny.  The product
    is split along K over the blocks of a thread-block cluster where that fills the GPU better (`cluster` 0: chosen
    by the library; 1 to 8: that many K ranges); the partial tiles meet in shared memory, no scratch is needed."""
    _cuda(x, w, out)
    if not gemm_tc5_supported(x, w):
        raise KernelError("gemm_tc5: this product is not supported (bfloat16, at most 128 rows, K a multiple of 8, "
                          "16-byte aligned rows)")
    M, K = x.shape
    N = w.shape[0]
    assert w.shape[1] == K and out.stride(1) == 1 and out.shape[0] == M
    assert out.shape[1] == (N // 2 if epilogue == EPI_SWIGLU else N)
    assert out.dtype == (torch.float32 if epilogue == EPI_F32 else torch.bfloat16)
    L = lib()
    map_w = tensor_map_2d(w, 128)
    map_x = tensor_map_2d(x, int(L.vob_gemm_tc5_token_box(M)))
    _check(L.vob_gemm_tc5(map_w, map_x, _p(out), ctypes.c_long(out.stride(0)), M, N, K, epilogue, int(cluster),
                          _p(err), _stream()), "gemm_tc5")


def gemm_skinny_supported(x, w) -> bool:
    """Whether the weight-streaming kernel takes x[M,K] @ w[N,K]^T: bfloat16, M <= 16, K a multiple of 64 (the
    column slices of a TMA box), rows that start on 16-byte boundaries."""
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.dim() == 2 and 0 < x.shape[0] <= 16
            and x.shape[1] % 64 == 0
            and x.stride(1) == 1 and w.stride(1) == 1 and (x.stride(0) * 2) % 16 == 0 and (w.stride(0) * 2) % 16 == 0
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_skinny_weight_tiles(n_rows: int) -> int:
    """The number of row tiles the weight-streaming product cuts a matrix of `n_rows` rows into."""
    box = int(lib().vob_gemm_skinny_weight_box(ctypes.c_long(n_rows)))
    return (n_rows + box - 1) // box


def gemm_skinny(x, w, out, epilogue: int, err, norm_weight=None, eps: float = 0.0, emit=None, prenormed=None) -> None:
    """out = x @ w^T for at most 16 rows of x (see gemm_skinny_supported); epilogue EPI_BF16 (out bfloat16 [M,N]),
    EPI_F32 (out float32 [M,N], rounded to bfloat16 first), EPI_SWIGLU (the rows of w alternate in groups of
    eight between gate and up; out bfloat16 [M,N/2] = SiLU(gate) * up) or EPI_ADD (out bfloat16 [M,N] += the
    product rounded to bfloat16: out is the residual stream).  With `norm_weight` (float [K]; EPI_BF16 and EPI_SWIGLU)
    the product is that of RMSNorm(x) * norm_weight, the norm computed on the way.

    The same norm in two halves, for a chain of products: `emit=(weight, scaled, parts)` (EPI_ADD) makes the product
    leave bfloat16(out * weight) in `scaled` [M,N] and per-tile sums of the squares of the new `out` in `parts`
    (float, gemm_skinny_weight_tiles(N) * 16 entries are enough) for the norm that follows; `prenormed=parts` (EPI_BF16
    and EPI_SWIGLU, with `eps`) takes x to be such a `scaled` buffer and scales the product by 1/rms from the parts."""
    _cuda(x, w, out, norm_weight)
    if not gemm_skinny_supported(x, w):
        raise KernelError("gemm_skinny: this product is not supported (bfloat16, at most 16 rows, K a multiple of 64, 16-byte aligned rows)")
    M, K = x.shape
    N = w.shape[0]
    assert w.shape[1] == K and out.stride(1) == 1 and out.shape[0] == M
    assert out.shape[1] == (N // 2 if epilogue == EPI_SWIGLU else N)
    assert out.dtype == (torch.float32 if epilogue == EPI_F32 else torch.bfloat16)
    if norm_weight is not None:
        assert epilogue in (EPI_BF16, EPI_SWIGLU) and norm_weight.dtype == torch.float32 and norm_weight.numel() == K
    box_m = 8 if M <= 8 else 16
    ss_parts, ss_count = None, 0
    if prenormed is not None:
        assert norm_weight is None and epilogue in (EPI_BF16, EPI_SWIGLU) and prenormed.dtype == torch.float32
        ss_parts, ss_count = prenormed, gemm_skinny_weight_tiles(K)      # the product before wrote K outputs a token
        assert prenormed.numel() >= ss_count * box_m
    emit_w = emit_xn = emit_ss = None
    if emit is not None:
        emit_w, emit_xn, emit_ss = emit
        _cuda(emit_w, emit_xn, emit_ss)
        assert epilogue == EPI_ADD and emit_w.dtype == torch.float32 and emit_w.numel() == N
        assert emit_xn.dtype == torch.bfloat16 and emit_xn.is_contiguous() and emit_xn.shape == (M, N)
        assert emit_ss.dtype == torch.float32 and emit_ss.numel() >= gemm_skinny_weight_tiles(N) * box_m
    map_w = tensor_map(w, int(lib().vob_gemm_skinny_weight_box(ctypes.c_long(N))), 4)
    map_x = tensor_map(x, box_m, 4)
    _check(lib().vob_gemm_skinny(map_w, map_x, _p(out), ctypes.c_long(out.stride(0)), M, N, K, epilogue, _p(norm_weight),
                                 ctypes.c_float(eps), _p(ss_parts), ss_count, _p(emit_w), _p(emit_xn), _p(emit_ss),
                                 _p(err), _stream()), "gemm_skinny")


def gemm_skinny_set_wait_limit(tries: int, withhold_copies: bool = False) -> None:
    """For tests of the bounded waits: after `tries` attempts a pipeline wait of the weight-streaming product gives up
    (0 restores the default); with `withhold_copies` its producers issue no copy, so the waits are for something that
    never comes.  The kernel then sets the timeout bits of the error word and returns without writing."""
    torch.cuda.synchronize()
    code = lib().vob_gemm_skinny_set_wait_limit(ctypes.c_uint(tries), int(withhold_copies))
    if code != 0:
        raise KernelError(f"gemm_skinny_set_wait_limit: {lib().vob_error_string(code).decode()}")


def sample(logits, temperature, top_k, top_p, keys, out, num_rows: int) -> None:
    _cuda(logits, temperature, top_k, top_p, keys, out)
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    _check(lib().vob_sample(_p(logits), ctypes.c_long(logits.stride(0)), num_rows, logits.shape[1], _p(temperature),
                            _p(top_k), _p(top_p), _p(keys), _p(out), _stream()), "sample")


def apply_penalties(logits, row_of, token, count, presence, frequency, repetition, n: int) -> None:
    _cuda(logits, row_of, token, count)
    _check(lib().vob_apply_penalties(_p(logits), ctypes.c_long(logits.stride(0)), logits.shape[1], _p(row_of),
                                     _p(token), _p(count), _p(presence), _p(frequency), _p(repetition), n, _stream()),
           "apply_penalties")


def copy_pages(cache_plane, pairs, n_pairs: int) -> None:
    _cuda(cache_plane, pairs)
    page_elems = cache_plane[0].numel()
    _check(lib().vob_copy_pages(_p(cache_plane), _p(pairs), n_pairs, ctypes.c_long(page_elems),
                                _code(cache_plane.dtype), _stream()), "copy_pages")


if _os.environ.get("VOB_KERNEL_TIMERS", "") not in ("", "0"):
    enable_kernel_timers()
