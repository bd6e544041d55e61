"""RMSNorm fused with the residual add.

y = (x * (1 / sqrt(mean(x^2) + eps))) * w in float32, the order of operations of
crates/coheryn-engine/src/cpu.rs:49-57 (which sums the squares in float64; here the sum
is a float32 tree of fixed shape).  The weight has no bias and no "+1".
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import ops
from ..weights.spec import TensorSpec
from .base import Norm, NormedSum, PostNormed, Runtime, register_norm


class RMSNorm(Norm):
    accepts_partial_sums = True

    def __init__(self, runtime: Runtime, size: int, eps: float, tensor: str = "weight"):
        """``tensor``: the local name of the weight ("" when the checkpoint names the weight as it names the norm)."""
        super().__init__(runtime)
        self.size, self.eps, self.tensor = int(size), float(eps), str(tensor)
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {self.tensor: TensorSpec((self.size,), role="vector", init="norm")}

    def bind(self, tensors):
        self.weight = tensors[self.tensor]

    def forward(self, residual, delta, rows=None):
        """residual += delta (when given and no ``rows``); returns the normalised rows in
        the compute dtype.  With ``rows`` only those rows are produced."""
        n = residual.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, self.size), dtype=self.runtime.dtype, device=residual.device)
        if isinstance(delta, PostNormed):     # a summand that is normalised before it is added: one kernel for both norms
            apply_post_normed(residual, delta, self.weight, self.eps, out, rows)
            return out
        ops.add_rmsnorm(residual, delta, self.weight, self.eps, out, rows=rows)
        return out

    def post(self, residual, delta, alpha: float = 1.0, normed_summand: bool = False):
        """The norm AFTER the sum, in place on the float32 stream: residual <- (alpha residual + delta) / rms(..) * w; with
        ``normed_summand`` residual <- residual + delta / rms(delta) * w instead.  ``delta``: float32 [T, H] or a stack
        [P, T, H] of partial sums.  Returns the new stream in the compute dtype (the stream itself when that is float32)."""
        if delta.dtype != torch.float32:
            raise ValueError("a norm after the sum takes its summand in float32")
        cast = None if self.runtime.dtype == torch.float32 else torch.empty(residual.shape, dtype=self.runtime.dtype, device=residual.device)
        ops.scaled_add_norm(residual, delta, alpha, self.weight, self.eps, cast, normed_summand=normed_summand)
        return residual if cast is None else cast


def apply_post_normed(residual, delta: PostNormed, weight, eps: float, out, rows=None) -> None:
    """residual += delta.value / rms(delta.value) * delta.weight (without ``rows``); ``out`` = the normalised sum times
    ``weight`` (both may be None: the residual is only updated).  The two norms share one ``eps``."""
    if weight is not None and float(eps) != float(delta.eps):
        raise ValueError("a summand's norm and the norm that adds it are fused and must share their eps")
    v = delta.value
    if isinstance(v, NormedSum):
        if float(v.eps) != float(delta.eps):
            raise ValueError("the norms of a sum of normalised summands and the norm over it must share their eps")
        ops.add_normed_rmsnorm(residual, v.parts, v.weights, v.coef, delta.weight, weight, delta.eps, out, rows=rows)
    else:
        if v.dtype != torch.float32:
            v = v.float()
        ops.add_normed_rmsnorm(residual, v, None, 1.0, delta.weight, weight, delta.eps, out, rows=rows)


register_norm("rmsnorm", RMSNorm)
