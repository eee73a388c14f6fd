"""Python face of the matrix product for up to 32 rows (csrc/gemm_skinny.cu): what decoding at
small batch runs.  bfloat16 operands, K a multiple of 8; epilogues none and gated."""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops

MAX_ROWS = 32
_lib: Optional[ops.Library] = None
enabled = True          # tests switch it off to compare with the other kernels


def lib() -> ops.Library:
    global _lib
    if _lib is None:
        _lib = ops.Library("gemm_skinny")
    return _lib


def operands_ok(x: torch.Tensor, w: torch.Tensor) -> bool:
    if not enabled or x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or not 0 < x.shape[0] <= MAX_ROWS:
        return False
    if x.shape[1] % 8 or x.stride(1) != 1 or w.stride(1) != 1 or x.stride(0) % 8 or w.stride(0) % 8:
        return False
    return x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0


def can_take(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int) -> bool:
    if not operands_ok(x, w) or epilogue not in (ops.EPI_NONE, ops.EPI_GATED) or not out.is_contiguous():
        return False
    if epilogue == ops.EPI_GATED:
        return out.dtype == torch.bfloat16
    return out.dtype in (torch.bfloat16, torch.float32)


def matmul(x, w, out, epilogue: int = ops.EPI_NONE, act: int = 0) -> None:
    m, k = x.shape
    n = out.shape[1]
    lib().call("hos_gemm_skinny", ops._ptr(x), ops._ptr(w), ops._ptr(out), ops.dtype_code(out.dtype), m, n, k,
               x.stride(0), w.stride(0), out.stride(0), epilogue, act, 1, 1 if ops.take_room_left() else 0, ops._stream())


_MIN_K_PER_CTA = 4096      # below this a CTA's 8 warps have too few loads each to be worth another CTA


def k_splits_for(n: int, k: int) -> int:
    """CTAs own 16 output features each; with fewer of them than two per SM, K is split over
    more CTAs while each keeps enough of K to fill its loads."""
    ctas = (n + 15) // 16
    return max(1, min(2 * ops.sm_count() // ctas, k // _MIN_K_PER_CTA, 8))


def matmul_partials(x, w, k_splits: Optional[int] = None) -> Optional[torch.Tensor]:
    """x . w^T as float32 partial sums [parts, M, N] for a consumer that adds them, if K is worth
    splitting for these sizes; None if it is not (call `matmul` then)."""
    m, k = x.shape
    n = w.shape[0]
    if k_splits is None:
        k_splits = k_splits_for(n, k)
    if k_splits <= 1:
        return None
    parts = torch.empty((k_splits, m, n), dtype=torch.float32, device=x.device)
    lib().call("hos_gemm_skinny", ops._ptr(x), ops._ptr(w), ops._ptr(parts), ops.F32, m, n, k,
               x.stride(0), w.stride(0), n, ops.EPI_NONE, 0, k_splits, 1 if ops.take_room_left() else 0, ops._stream())
    return parts


def can_fuse_qkv_rope(x: torch.Tensor, w: torch.Tensor, head_dim: int, rotary_dim: int) -> bool:
    """Whether the projection of q, k, v with the rotary encoding and the cache write in its
    epilogue can run: the product's own rules, and head and rotary sizes in steps of 16."""
    return operands_ok(x, w) and head_dim % 16 == 0 and rotary_dim % 16 == 0


def qkv_rope(x, w, out, n_heads: int, n_kv_heads: int, head_dim: int, step, inv_freq, rotary_dim: int, style: int,
             cache) -> None:
    """out[M, (n_heads + 2 n_kv_heads) * head_dim] = x . w^T with q and k heads rotated and, if `cache` is
    given, keys and values stored at the tokens' places.  n_kv_heads = 0: q heads only."""
    m, k = x.shape
    lib().call("hos_qkv_rope_skinny", ops._ptr(x), ops._ptr(w), ops._ptr(out), m, k, x.stride(0), w.stride(0),
               out.stride(0), n_heads, n_kv_heads, head_dim, ops._ptr(step.token_pos), ops._ptr(step.token_seq),
               ops._ptr(step.seq_slot), ops._ptr(step.seq_len_after), ops._ptr(inv_freq) if inv_freq is not None else None,
               rotary_dim if inv_freq is not None else 0, style,
               ops._ptr(cache.k_pages) if cache else None, ops._ptr(cache.v_pages) if cache else None,
               ops._ptr(cache.page_table) if cache else None, cache.table_stride if cache else 0,
               cache.ring_pages if cache else 0, 1 if cache else 0, ops._stream())
