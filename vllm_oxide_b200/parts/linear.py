"""y = x @ W^T with W stored [out, in], the one matrix product every part uses.

The reference calls a library product here (vllm-oxide, crates/vllm-oxide/src/layers/linear.rs:84-90:
`x.matmul(&weight.t())` through candle to cuBLAS).  On the bfloat16 path, steps of at most 16 tokens
(decoding) go to this package's weight-streaming kernel, larger ones to cuBLAS through torch.mm; both
accumulate in float and round to bfloat16 once.  On the 32-bit path it is this package's own float
kernel, which uses no tensor cores and no reduced-precision mode and gives every output element the
same chain of operations whatever the batch.
"""
from __future__ import annotations

import torch

from .. import kernels


def linear(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, ctx=None) -> torch.Tensor:
    if x.dtype == torch.float32:
        kernels.gemm_f32(x, weight, out)
    elif ctx is not None and kernels.gemm_skinny_supported(x, weight):
        kernels.gemm_skinny(x, weight, out, kernels.EPI_BF16, ctx.err)
    else:
        torch.mm(x, weight.t(), out=out)
    return out
