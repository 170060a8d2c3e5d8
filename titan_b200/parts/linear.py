"""Matrix products of the parts: ``out = epilogue(x . w^T)``.

One function, so that which kernel runs is decided in one place.  float32
always takes the CUDA-core kernel (true 32-bit).  bfloat16 takes the tcgen05
tensor-core kernel when the shapes meet its alignment rules and the CUDA-core
kernel otherwise; ``ctx.options["gemm"] = "plain"`` forces the latter.
"""
from __future__ import annotations

import torch

from .. import kernels as K

EPI_STORE, EPI_F32, EPI_ADD, EPI_SWIGLU = K.EPI_STORE, K.EPI_F32, K.EPI_ADD, K.EPI_SWIGLU


def matmul(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epi: int, ctx) -> None:
    if w.dtype == torch.bfloat16 and ctx.options.get("gemm", "fast") != "plain":
        fast = getattr(K, "gemm_tc", None)
        if fast is not None and K.gemm_tc_accepts(x, w, out, epi):
            fast(x, w, out, epi, ctx.stream, ordered=bool(ctx.options.get("reproducible", False)))
            return
    K.gemm_simt(x, w, out, epi, ctx.stream)


def matmul_heads(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, heads: int, x_step: int, out_step: int, ctx) -> None:
    """One product per head, the heads side by side in the rows of ``x`` and ``out``:
    out[:, h * out_step : h * out_step + N] = x[:, h * x_step : h * x_step + K] . w[h]^T, with w [heads, N, K], in the
    compute dtype.  bfloat16 rows in numbers that fill the tensor-core kernel's tiles take that kernel head by head;
    everything else is one batched launch of the CUDA-core kernel."""
    N, K_ = w.shape[1], w.shape[2]
    if w.dtype == torch.bfloat16 and ctx.options.get("gemm", "fast") != "plain" and x.shape[0] >= 256:
        fast = getattr(K, "gemm_tc", None)
        views = [(x[:, h * x_step: h * x_step + K_], w[h], out[:, h * out_step: h * out_step + N]) for h in range(heads)]
        if fast is not None and all(K.gemm_tc_accepts(a, b, c, EPI_STORE) for a, b, c in views[:1] + views[-1:]):
            for a, b, c in views:
                fast(a, b, c, EPI_STORE, ctx.stream, ordered=bool(ctx.options.get("reproducible", False)))
            return
    K.gemm_simt_batched(x[:, :K_], w, out[:, :N], EPI_STORE, ctx.stream, heads, x_step, out_step)
