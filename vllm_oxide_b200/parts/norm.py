"""RMSNorm fused with the residual add (vllm-oxide, crates/vllm-oxide/src/layers/rmsnorm.rs:51-81)."""
from __future__ import annotations

from typing import Dict, List

import torch

from .. import kernels
from ..weights.loader import TensorSpec
from .base import Norm, register_part


class RMSNorm(Norm):
    graph_safe = True

    """(y, residual') = (RMSNorm(x + residual) * w, x + residual); with residual None, residual' = x.

    The residual buffer is updated in place.  With `rows` the norm is computed only for those
    source rows and the residual is left alone (the model's last norm, on the wanted rows)."""

    def __init__(self, size: int, eps: float, weight_name: str, **_):
        self.size, self.eps, self.weight_name = size, float(eps), weight_name
        self.weight = None

    def tensor_specs(self) -> List[TensorSpec]:
        return [TensorSpec(self.weight_name, (self.size,), "norm")]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors[self.weight_name].contiguous()

    def forward(self, x, residual, ctx, rows=None, n_rows=None, name="normed"):
        # x None: the part before has already added its output into the residual stream; the norm is of the stream
        # itself, which stays where it is (residual' = x, written onto itself)
        summed = x is None
        if summed:
            x, residual = residual, None
        n = x.shape[0] if rows is None else n_rows
        y = ctx.ws.get(name, n, self.size, x.dtype)
        has_residual = residual is not None
        if residual is None:
            residual = x if summed else ctx.ws.get("residual", x.shape[0], self.size, x.dtype)
        kernels.add_rmsnorm(x, residual, self.weight, y, self.eps, has_residual, ctx.err, rows=rows, n_out=n)
        return y, residual


register_part("norm", "rmsnorm", RMSNorm)
