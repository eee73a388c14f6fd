"""Python face of the matrix product for up to 16 rows (csrc/gemm_skinny.cu): what decoding at
small batch runs.  bfloat16 operands, K a multiple of 8; epilogues none and gated."""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops

MAX_ROWS = 16
_lib: Optional[ops.Library] = None
enabled = True          # tests switch it off to compare with the other kernels


def lib() -> ops.Library:
    global _lib
    if _lib is None:
        _lib = ops.Library("gemm_skinny")
    return _lib


def can_take(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int) -> bool:
    if not enabled or x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or x.shape[0] > MAX_ROWS:
        return False
    if epilogue not in (ops.EPI_NONE, ops.EPI_GATED):
        return False
    k = x.shape[1]
    if k % 8 != 0 or x.stride(1) != 1 or w.stride(1) != 1 or x.stride(0) % 8 or w.stride(0) % 8:
        return False
    if x.data_ptr() % 16 or w.data_ptr() % 16 or not out.is_contiguous():
        return False
    if epilogue == ops.EPI_GATED:
        return out.dtype == torch.bfloat16
    return out.dtype in (torch.bfloat16, torch.float32)


def matmul(x, w, out, epilogue: int = ops.EPI_NONE, act: int = 0) -> None:
    m, k = x.shape
    n = out.shape[1]
    lib().call("hos_gemm_skinny", ops._ptr(x), ops._ptr(w), ops._ptr(out), ops.dtype_code(out.dtype), m, n, k,
               x.stride(0), w.stride(0), out.stride(0), epilogue, act, ops._stream())
