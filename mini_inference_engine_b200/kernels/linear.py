"""The matrix product y = x W^T (+ b) of every projection, by operand type.

* float32 activations (the true 32-bit mode), or a weight the checkpoint holds in 32 bits:
  the CUDA-core FMA kernel of ``csrc/gemm_simt.cu``.
* bfloat16 activations and weights: a tensor-core product.  The reference calls the vendor library
  for these (F.linear, inference_engine/model.py:172,178,180,181,185).  ``auto`` (the default) uses
  this package's tcgen05 kernel (``csrc/gemm_tcgen05.cu``) where it is the faster one -- few tokens,
  i.e. decode steps, where it streams the weights, overlaps their fetch with the kernel before it
  and fuses SwiGLU -- its product on pairs of SMs (``csrc/gemm_pair_tc.cu``) for the gate/up projection
  of prompt-sized batches, where its 256 x 256 tiles fill the GPU's pairs evenly and SwiGLU rides in the
  epilogue, and the library product elsewhere; ``tcgen05`` and ``library`` force one.
"""
from __future__ import annotations

import torch

from . import gemm_tc, ops

_bf16_backend = "auto"
AUTO_MAX_TOKENS = 32          # up to this many tokens ``auto`` takes the tcgen05 kernel.  Whole decode step, TinyLlama-1.1B
                              # sizes on a B200: 24 tokens 1.057 ms against 1.098 ms with the library, 32 tokens 1.078 against
                              # 1.136 ms; with the 64-token tile (33 tokens and more) 1.417 / 1.510 / 1.575 ms at 33 / 48 / 64
                              # tokens against 1.18 / 1.22 ms with the library at 48 / 64 -- although blocks then own tokens
                              # and receive their partial sums as bulk copies (1.61 -> 1.51 ms at 48 tokens): three ring
                              # stages of 24 KB instead of five of 18 KB leave each block too little in flight


PAIR_MIN_TOKENS = 128         # from this many tokens on ``auto`` considers the product on pairs of SMs for gate/up with SwiGLU
PAIR_MIN_FILL = 0.7           # ... where the product fills at least this share of the 256 x 256 tiles that its rounds over the
                              # pairs of SMs offer.  Device time in a graph against the library's product and the SwiGLU
                              # kernel, TinyLlama-1.1B sizes at 512 / 768 / 1,024 / 2,048 / 8,192 tokens (shares 0.59 / 0.89 /
                              # 0.79 / 0.95 / 0.96): 26.8 / 28.2 / 37.1 / 61.4 / 234.4 us against 24.6 / 30.7 / 43.7 / 78.9 /
                              # 291.6 us; Llama-3-8B sizes at 256 / 384 / 512 / 2,048 tokens (0.76 / 0.57 / 0.76 / 0.93):
                              # 55.3 / 89.1 / 93.1 / 298.3 us against 60.2 / 78.1 / 104.4 / 344.8 us.  The other products stay
                              # with the library: plain, the paired kernel is 16.6 / 37.0 / 25.9 us for o / down / q|k|v at
                              # 2,048 tokens (64, 64 and 80 tiles: one or two rounds) against 14.1 / 33.7 / 17.4 us (at 8,192
                              # tokens 48.6 / 141.5 / 60.4 against 47.8 / 124.3 / 59.0 us), and its epilogue that adds to the
                              # residual stream and leaves the next norm's operand (a row of 256 float32 read, summed and
                              # written back per thread) costs more than the add + norm kernel it saves (o: + 23 us against
                              # 8.6 us)


def pair_fill(num_tokens: int, N: int) -> float:
    """The share of the 256 x 256 tiles offered by the paired product's rounds (every pair of SMs one tile a
    round) that a product of ``num_tokens`` x ``N`` outputs fills: partly empty tiles at the edges and pairs
    without a tile in the last round both count as offered and unused."""
    from .device import num_sms
    tiles = -(-num_tokens // 256) * -(-N // 256)
    pairs = max(1, num_sms() // 2)
    rounds = -(-tiles // pairs)
    return num_tokens * N / (rounds * pairs * 65536.0)


def takes_pair(num_tokens: int, w: torch.Tensor) -> bool:
    """Whether ``auto`` gives the gate/up product with these sizes to the kernel on pairs of SMs."""
    if _bf16_backend != "auto" or w.dtype != torch.bfloat16 or not w.is_cuda or num_tokens < PAIR_MIN_TOKENS:
        return False
    N, K = w.shape
    return (K % 8 == 0 and N % 8 == 0 and w.is_contiguous() and w.data_ptr() % 16 == 0
            and pair_fill(num_tokens, N) >= PAIR_MIN_FILL)


def set_bf16_backend(name: str) -> None:
    global _bf16_backend
    if name not in ("auto", "library", "simt", "tcgen05"):
        raise ValueError(name)
    _bf16_backend = name


def bf16_backend() -> str:
    return _bf16_backend


def uses_tcgen05(x: torch.Tensor, w: torch.Tensor, out_dtype=torch.bfloat16) -> bool:
    """Whether ``linear`` would run the tcgen05 kernel for these operands."""
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or _bf16_backend in ("library", "simt"):
        return False
    if _bf16_backend == "auto" and x.shape[0] > AUTO_MAX_TOKENS:
        return False
    K = x.shape[1]
    return K % 8 == 0 and w.shape[0] % 8 == 0 and x.is_contiguous() and w.is_contiguous()


def splits_k_on_tcgen05(num_tokens: int, w: torch.Tensor) -> bool:
    """Whether the product of ``num_tokens`` bfloat16 rows with ``w`` runs on the tcgen05 kernel with K
    split across a cluster -- the form that carries the residual and the norm-factor epilogues."""
    if w.dtype != torch.bfloat16 or _bf16_backend in ("library", "simt") or num_tokens < 1 or not w.is_cuda:
        return False
    if _bf16_backend == "auto" and num_tokens > AUTO_MAX_TOKENS:
        return False
    N, K = w.shape
    return K % 8 == 0 and N % 8 == 0 and w.is_contiguous() and w.data_ptr() % 16 == 0 and gemm_tc.splits_k(num_tokens, N, K)


def linear_into_stream(x, w: torch.Tensor, bias, res: torch.Tensor, norm_weight, eps: float):
    """res += x W^T (+ b) inside the product (``res`` float32, in place) and, for the RMSNorm with
    ``norm_weight`` that reads the stream next, the DeferredNorm for the product behind it.  Returns
    False where this product cannot do that (the caller then adds the product's output as before)."""
    if not splits_k_on_tcgen05(x.shape[0], w) or x.dtype != torch.bfloat16 or res.dtype != torch.float32:
        return False
    return gemm_tc.gemm_residual(x, w, res, bias, norm_weight, eps)


def linear(x, w: torch.Tensor, bias, out_dtype: torch.dtype) -> torch.Tensor:
    M = x.shape[0]
    N = w.shape[0]
    out = torch.empty(M, N, dtype=out_dtype, device=w.device)
    if M == 0:
        return out
    if isinstance(x, gemm_tc.DeferredNorm):          # only handed out where splits_k_on_tcgen05 said yes
        return gemm_tc.gemm(x, w, out, bias)
    if x.dtype == torch.float32 or w.dtype == torch.float32 or _bf16_backend == "simt":
        return ops.gemm_simt(x, w, out, bias)
    if uses_tcgen05(x, w, out_dtype) and gemm_tc.supports(x, w, out):
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


def linear_swiglu(x: torch.Tensor, w_interleaved: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """silu(x Wg^T) * (x Wu^T) for a weight whose rows alternate gate_i, up_i: fused into the
    tcgen05 product's epilogue where that kernel runs, else the product followed by the SwiGLU kernel."""
    M, inter = x.shape[0], w_interleaved.shape[0] // 2
    out = torch.empty(M, inter, dtype=out_dtype, device=w_interleaved.device)
    if M == 0:
        return out
    if isinstance(x, gemm_tc.DeferredNorm):
        if w_interleaved.shape[0] % 16 == 0:
            return gemm_tc.gemm(x, w_interleaved, out, swiglu=True)
        gu = gemm_tc.gemm(x, w_interleaved, torch.empty(M, 2 * inter, dtype=out_dtype, device=out.device))
        return ops.swiglu(gu, out, interleaved=True)       # the fused epilogue pairs rows within groups of 16
    if (takes_pair(M, w_interleaved) and w_interleaved.shape[0] % 16 == 0 and x.dtype == torch.bfloat16
            and out_dtype in (torch.bfloat16, torch.float32) and x.is_contiguous()):
        return gemm_tc.gemm_pair(x, w_interleaved, out, swiglu=True)
    if uses_tcgen05(x, w_interleaved) and w_interleaved.shape[0] % 16 == 0 and gemm_tc.supports(x, w_interleaved, out):
        return gemm_tc.gemm(x, w_interleaved, out, swiglu=True)
    gu = linear(x, w_interleaved, None, out_dtype)
    return ops.swiglu(gu, out, interleaved=True)
