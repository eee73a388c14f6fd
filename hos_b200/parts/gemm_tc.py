"""Python face of the tcgen05/TMA matrix product (csrc/gemm_tc.cu)."""
from __future__ import annotations

import torch

from .. import ops

ENABLED = False     # switched on once the kernel is built and checked


def can_take(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int) -> bool:
    return False


def matmul(x, w, out, epilogue, cap, act) -> None:
    raise NotImplementedError
