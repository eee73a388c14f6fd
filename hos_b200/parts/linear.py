"""The matrix product that every part calls: y = x . W^T, W stored [out, in] as the
checkpoint has it (src/model.rs:179-180).  Chooses the kernel: in bfloat16, for up to 32
rows the register-streaming kernel, else the tcgen05/TMA kernel, when the sizes meet their
alignment rules; otherwise (and always in the 32-bit path) the plain CUDA-core kernel.  All
accumulate in 32-bit."""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops

_force_plain = False


def force_plain(on: bool) -> None:
    """Tests use this to compare the tensor-core kernel's results with the plain kernel's."""
    global _force_plain
    _force_plain = on


def plain_forced() -> bool:
    return _force_plain


def matmul(x: torch.Tensor, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
           epilogue: int = ops.EPI_NONE, cap: float = 0.0, act: int = 0,
           out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[M, N] = x[M, K] . w[N or 2N, K]^T (2N rows with the gated epilogue)."""
    m = x.shape[0]
    n = w.shape[0] // 2 if epilogue == ops.EPI_GATED else w.shape[0]
    if out is None:
        out = torch.empty((m, n), dtype=out_dtype or x.dtype, device=x.device)
    if m == 0:
        return out
    if (not _force_plain and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16):
        from . import gemm_skinny, gemm_tc
        if gemm_skinny.can_take(x, w, out, epilogue):
            gemm_skinny.matmul(x, w, out, epilogue, act)
            return out
        if gemm_tc.can_take(x, w, out, epilogue):
            gemm_tc.matmul(x, w, out, epilogue, cap, act)
            return out
    ops.gemm_plain(x, w, out, epilogue, cap, act)
    return out


def matmul_or_partials(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """x . w^T for a consumer that can add partial sums: either the product [M, N] in the
    activation type, or float32 partial sums [parts, M, N] when the tensor-core kernel splits K
    (few rows, few output tiles: decoding).  No epilogue."""
    if (not _force_plain and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[0] > 0):
        from . import gemm_skinny, gemm_tc
        if gemm_skinny.enabled and x.shape[0] <= gemm_skinny.MAX_ROWS:
            # a handful of rows: K is split over CTAs only when there are few output features
            if gemm_skinny.operands_ok(x, w):
                parts = gemm_skinny.matmul_partials(x, w)
                if parts is not None:
                    return parts
            return matmul(x, w)
        if gemm_tc.enabled and x.shape[1] % 8 == 0 and w.stride(1) == 1 and w.stride(0) % 8 == 0 \
                and x.is_contiguous() and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0:
            parts = gemm_tc.matmul_partials(x, w)
            if parts is not None:
                return parts
    return matmul(x, w)
