"""The matrix product y = x W^T (+ b) of every projection, by operand type.

* float32 activations (the true 32-bit mode), or a weight the checkpoint holds in 32 bits:
  the CUDA-core FMA kernel of ``csrc/gemm_simt.cu``.
* bfloat16 activations and weights: the tensor-core product.  The reference calls the vendor
  library for these (F.linear, inference_engine/model.py:172,178,180,181,185); ``LIBRARY`` is that
  product, and kernels of this package replace it where they are faster (see ``set_bf16_backend``).
"""
from __future__ import annotations

import torch

from . import ops

_bf16_backend = "library"


def set_bf16_backend(name: str) -> None:
    global _bf16_backend
    if name not in ("library", "simt", "tcgen05"):
        raise ValueError(name)
    _bf16_backend = name


def bf16_backend() -> str:
    return _bf16_backend


def linear(x: torch.Tensor, w: torch.Tensor, bias, out_dtype: torch.dtype) -> torch.Tensor:
    M = x.shape[0]
    N = w.shape[0]
    out = torch.empty(M, N, dtype=out_dtype, device=x.device)
    if M == 0:
        return out
    if x.dtype == torch.float32 or w.dtype == torch.float32 or _bf16_backend == "simt":
        return ops.gemm_simt(x, w, out, bias)
    if _bf16_backend == "tcgen05":
        from . import gemm_tc
        if gemm_tc.supports(x, w, out):
            return gemm_tc.gemm(x, w, out, bias)
    if not x.is_cuda:
        raise ops.KernelError("linear runs on CUDA tensors only")
    if out_dtype == torch.bfloat16:
        if bias is None:
            torch.mm(x, w.t(), out=out)
        else:
            torch.addmm(bias, x, w.t(), out=out)
        return out
    # bfloat16 operands, float32 result (the logits): the library rounds its float32 accumulator
    # to the output type, so ask for float32 directly
    out.copy_(torch.mm(x, w.t(), out_dtype=torch.float32))
    if bias is not None:
        out += bias
    return out
