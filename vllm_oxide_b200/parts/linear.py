"""y = x @ W^T with W stored [out, in], the one matrix product every part uses.

The reference calls a library product here (vllm-oxide, crates/vllm-oxide/src/layers/linear.rs:84-90:
`x.matmul(&weight.t())` through candle to cuBLAS).  On the bfloat16 path this does the same
(cuBLAS through torch.mm, float accumulation, one rounding to bfloat16); on the 32-bit path it
is this package's own float kernel, which uses no tensor cores and no reduced-precision mode
and gives every output element the same chain of operations whatever the batch.
"""
from __future__ import annotations

import torch

from .. import kernels


def linear(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    if x.dtype == torch.float32:
        kernels.gemm_f32(x, weight, out)
    else:
        torch.mm(x, weight.t(), out=out)
    return out
