"""RMSNorm fused with the residual sum: ``res += delta; x = res * rsqrt(mean(res^2) + eps) * w``
(inference_engine/kernels/rmsnorm.py:13-32,56-65, where the residual stays in the model dtype;
here the residual stream is float32 in both modes)."""
from __future__ import annotations

from ..kernels import ops
from ..weights.loader import TensorSpec
from .base import Part, StreamUpdated, register_part


class RMSNorm(Part):
    def __init__(self, size: int, eps: float):
        self.size = size
        self.eps = eps

    def tensor_specs(self):
        return {"weight": TensorSpec((self.size,), init="ones")}

    def bind(self, tensors, rt):
        self.rt = rt
        self.weight = rt.place(tensors["weight"])

    def kernel_sources(self):
        return {"norm"}

    def deferred_args(self):
        """Weight and eps, for a product that folds this norm into its neighbours' epilogues."""
        return self.weight, self.eps

    def __call__(self, delta, res, rows=None):
        if isinstance(delta, StreamUpdated):             # the part before added its output to the stream itself
            if delta.norm is self and delta.deferred is not None and rows is None:
                return delta.deferred                    # and left this norm's output, short of a factor, for the next product
            delta = None
        n_out = rows.numel() if rows is not None else res.shape[0]
        out = self.rt.empty(n_out, self.size)
        return ops.add_rmsnorm(delta, res, self.weight, self.eps, out, rows)


register_part("norm", "rmsnorm", RMSNorm)
