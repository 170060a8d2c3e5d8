"""Matrix products of the parts: ``out = epilogue(x . w^T)``.

One function, so that which kernel runs is decided in one place.  A few rows times a small matrix (a decode step's router,
a narrow gate) take the warp-per-output kernel in either dtype.  Otherwise float32
always takes the CUDA-core kernel (true 32-bit).  bfloat16 takes the tcgen05
tensor-core kernel when the shapes meet its alignment rules and the CUDA-core
kernel otherwise; ``ctx.options["gemm"] = "plain"`` forces the latter.
"""
from __future__ import annotations

import torch

from .. import kernels as K

EPI_STORE, EPI_F32, EPI_ADD, EPI_SWIGLU = K.EPI_STORE, K.EPI_F32, K.EPI_ADD, K.EPI_SWIGLU


# A product of at most this many rows with a matrix of at most this many elements runs a warp per output element: the fixed
# cost of a tensor-core launch (or, in float32, of 64 x 64 tiles with a few live rows) is more than such a product's work.
ROWS_MAX_M, ROWS_MAX_ELEMENTS = 8, 1 << 19


def matmul(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epi: int, ctx, gate: int = K.ACT_SILU, limit: float = 0.0) -> None:
    """``gate``, ``limit``: what the SWIGLU epilogue makes of a (gate, up) pair (``kernels.ACT_*``)."""
    if (x.shape[0] <= ROWS_MAX_M and w.shape[0] * w.shape[1] <= ROWS_MAX_ELEMENTS and epi in (EPI_STORE, EPI_F32, EPI_ADD)
            and ctx.options.get("small_products", True)):
        K.gemm_rows(x, w, out, epi, ctx.stream)
        return
    if w.dtype == torch.bfloat16 and ctx.options.get("gemm", "fast") != "plain":
        fast = getattr(K, "gemm_tc", None)
        if fast is not None and K.gemm_tc_accepts(x, w, out, epi):
            fast(x, w, out, epi, ctx.stream, ordered=bool(ctx.options.get("reproducible", False)), gate=gate, limit=limit)
            return
    K.gemm_simt(x, w, out, epi, ctx.stream, gate, limit)


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
