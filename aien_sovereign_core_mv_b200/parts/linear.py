"""Matrix products y = a . W^T with W in the checkpoint's [out, in] layout.

One entry point, :func:`linear`, chooses among the engine's own kernels by precision and by
the number of rows; all of them accumulate in float32.  The float32 engine always takes the
CUDA-core kernel whose per-row result does not depend on the batch.  ``AIEN_B200_GEMM`` can pin
the choice for debugging (``simple``, ``gemv``, ``tc``): it never selects a library routine.
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from .. import kernels as K
from .base import Prenormed, ResidualSink, StepContext

_FORCE = os.environ.get("AIEN_B200_GEMM", "").strip().lower()


def linear(ctx: StepContext, a: torch.Tensor, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
           out: Optional[torch.Tensor] = None, may_defer_sum: bool = False) -> torch.Tensor:
    """a [M, K] (row stride free), w [N, K] -> [M, N] taken from the step workspace.

    ``may_defer_sum``: the caller's consumer can add partial products, so the decode kernel may
    cut K across CTAs and return float32 partials [P, M, N] instead (the norm kernel, the q/k
    kernel and the row gather add them in order)."""
    M, N = a.shape[0], w.shape[0]
    if out is None and may_defer_sum and not _FORCE and M <= K.GEMV_ROUTE_ROWS and a.dtype == torch.bfloat16 \
            and w.dtype == torch.bfloat16:
        splits = K.gemv_splits(N, a.shape[1])
        if splits > 1:
            parts = ctx.workspace.take((splits, M, N), torch.float32)
            if K.gemv_supports(a, w, parts):
                K.gemv(a, w, parts)
                return parts
    if out is None and may_defer_sum and not _FORCE and M > K.GEMV_ROUTE_ROWS and a.dtype == torch.bfloat16 \
            and w.dtype == torch.bfloat16:
        splits = K.gemm_tc_splits(M, N, a.shape[1])
        if splits > 1:
            parts = ctx.workspace.take((splits, M, N), torch.float32)
            if K.gemm_tc_supports(a, w, parts[0]):
                K.gemm_tc(a, w, parts)
                return parts
    if out is None:
        out = ctx.workspace.take((M, N), out_dtype or a.dtype)
    choice = _FORCE or _choose(a, w, out, M)
    if choice == "gemv":
        K.gemv(a, w, out)
    elif choice == "tc":
        K.gemm_tc(a, w, out)
    else:
        K.gemm_simple(a, w, out)
    return out


def _choose(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, M: int) -> str:
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        return "simple"
    if M <= K.GEMV_ROUTE_ROWS and K.gemv_supports(a, w, out):
        return "gemv"
    if K.gemm_tc_supports(a, w, out):
        return "tc"
    return "simple"


def linear_prenormed(ctx: StepContext, h: Prenormed, w: torch.Tensor, epilogue: int = 0) -> Optional[torch.Tensor]:
    """(norm of the residual) . W^T from a Prenormed input: the streamed product multiplies its
    result rows by the norm's row factor.  ``epilogue`` 1: silu(gate)*up over rows of W interleaved
    in runs of 8.  None when the product cannot take it (the caller materialises the norm)."""
    if _FORCE or not K.gemv_stream_fusable(h.xw, w):
        return None
    M, N = h.xw.shape[0], w.shape[0]
    out = ctx.workspace.take((M, N // 2 if epilogue else N), torch.bfloat16)
    K.gemv_scaled(h.xw, w, out, h.ssq, h.parts, h.eps, epilogue)
    return out


def linear_into_residual(ctx: StepContext, a: torch.Tensor, w: torch.Tensor, sink: Optional[ResidualSink]) -> Optional[Prenormed]:
    """sink.x += a . W^T inside the product, which also leaves bfloat16(x * norm weight) and the
    partial sums of squares for the norm that follows.  None when there is no sink or the product
    cannot take it (the caller returns the branch output as a delta instead)."""
    if sink is None or _FORCE or not K.gemv_stream_fusable(a, w) or w.shape[0] != sink.x.shape[1]:
        return None
    M, N = a.shape[0], w.shape[0]
    xw = ctx.workspace.take((M, N), torch.bfloat16)
    ssq = ctx.workspace.take((K.gemv_stream_grid(N), 16), torch.float32)
    parts = K.gemv_residual(a, w, sink.x, sink.weight, xw, ssq)
    return Prenormed(xw, ssq, parts, sink.eps, sink.norm)
