"""y = x @ W^T with W stored [out, in], the one matrix product every part uses.

The reference calls a library product here (vllm-oxide, crates/vllm-oxide/src/layers/linear.rs:84-90:
`x.matmul(&weight.t())` through candle to cuBLAS).  On the bfloat16 path, steps of at most 16 tokens
(decoding) go to this package's weight-streaming kernel, larger ones to cuBLAS through torch.mm (or, with
USE_TC5, steps of 17 to 128 tokens to this package's tcgen05 kernel with the accumulator in tensor memory);
all accumulate in float and round to bfloat16 once.  On the 32-bit path it is this package's own float
kernel, which uses no tensor cores and no reduced-precision mode and gives every output element the
same chain of operations whatever the batch.
"""
from __future__ import annotations

import torch

from .. import kernels

# The library's bfloat16 products may add the partial sums of a split along K in bfloat16 (torch's default allows it).
# A sum rounded to 8 bits at every partial is not the float accumulation the rest of the engine keeps: on a step of
# 6 tokens a logit of a tiny model came out 2.6 off where the plain bfloat16 implementation is 0.6 off.  Off, for
# every product this process runs.
torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False


# Steps of 17 to 128 tokens: this package's tcgen05 product (True) or the library's (False).  Off by default: at batch 64
# the decode step measures 6.79 ms with the library's product and 8.63 ms with this kernel (Qwen3-8B sizes).
USE_TC5 = False
# The output matrix is another matter: there the tcgen05 product is as fast as the library's (232 vs 225 us at 64
# rows) and writes float logits itself, which saves the conversion pass the library's bfloat16 result needs (27 us).
USE_TC5_LOGITS = True
# The gate|up product with the activation as its epilogue: 6.92 ms a decode step at batch 64 against 6.80 ms with the
# library's product followed by the activation kernel, so off as well.
USE_TC5_SWIGLU = False


def tc5_product(x, weight, out, epilogue: int, ctx) -> bool:
    """Runs x @ weight^T on the tcgen05 kernel if it takes the case (17 to 128 tokens); False if it does not."""
    on = USE_TC5_LOGITS if epilogue == kernels.EPI_F32 else (USE_TC5_SWIGLU if epilogue == kernels.EPI_SWIGLU else USE_TC5)
    if not (on and ctx is not None and 16 < x.shape[0] <= 128 and kernels.gemm_tc5_supported(x, weight)):
        return False
    kernels.gemm_tc5(x, weight, out, epilogue, ctx.err)
    return True


def linear(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, ctx=None) -> torch.Tensor:
    if x.dtype == torch.float32:
        kernels.gemm_f32(x, weight, out)
    elif ctx is not None and kernels.gemm_skinny_supported(x, weight):
        kernels.gemm_skinny(x, weight, out, kernels.EPI_BF16, ctx.err)
    elif not tc5_product(x, weight, out, kernels.EPI_BF16, ctx):
        torch.mm(x, weight.t(), out=out)
    return out


def linear_into_stream(x: torch.Tensor, weight: torch.Tensor, stream: torch.Tensor) -> None:
    """stream += x @ weight^T by the library's product with the stream as its addend (bfloat16 steps of more than 16
    tokens): the sum is made in float inside the product and rounded once, as the weight-streaming kernel's adding
    epilogue does for smaller steps, and the add+norm kernel that follows has one tensor less to read and none to
    write back."""
    torch.addmm(stream, x, weight.t(), out=stream)
