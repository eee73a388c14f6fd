"""Python face of the tcgen05/TMA matrix product (csrc/gemm_tc.cu): bfloat16 operands, both
K-major, 32-bit accumulation in tensor memory.  Up to 128 rows of activations run in the
swapped orientation (the weight tile is the 128-row operand), where K may be split over
CTAs when the output alone gives too few tiles to fill the GPU."""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from .. import ops

SWAP_MAX_ROWS = 128      # up to here the weight tile is the 128-row operand (csrc/gemm_tc.cu: kSwapMaxRows)
# From here on the product runs on pairs of SMs (everything above the swapped orientation's rows); a number no
# product reaches when HOS_GEMM_PAIR=0 keeps them on single SMs.
NEVER = 1 << 30
PAIR_MIN_ROWS = NEVER if os.environ.get("HOS_GEMM_PAIR", "1") == "0" else SWAP_MAX_ROWS + 1
_lib: Optional[ops.Library] = None
enabled = True          # tests switch it off to compare with the plain kernel


def lib() -> ops.Library:
    global _lib
    if _lib is None:
        _lib = ops.Library("gemm_tc")
    return _lib


def set_pair_min_rows(rows: int) -> None:
    """From how many rows on products run on pairs of SMs (0: never); tests compare the two kernels with it."""
    global PAIR_MIN_ROWS
    lib().call("hos_gemm_tc_pair_min_rows", int(rows))
    PAIR_MIN_ROWS = rows if rows > 0 else NEVER


def can_take(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int) -> bool:
    """bfloat16 operands, K a multiple of 8, rows 16-byte aligned; else the plain kernel runs."""
    if not enabled or x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        return False
    k = x.shape[1]
    if k % 8 != 0 or x.stride(1) != 1 or w.stride(1) != 1 or x.stride(0) % 8 or w.stride(0) % 8:
        return False
    if x.data_ptr() % 16 or w.data_ptr() % 16 or out.data_ptr() % 16 or not out.is_contiguous():
        return False
    if epilogue == ops.EPI_GATED and out.dtype != torch.bfloat16:
        return False
    if epilogue == ops.EPI_SOFTCAP and out.dtype != torch.float32:
        return False
    return out.dtype in (torch.bfloat16, torch.float32)


def k_splits_for(m: int, n: int, k: int, epilogue: int) -> int:
    """Swapped products whose output gives few tiles split K so that about every SM has work,
    keeping at least four 64-wide K blocks per share."""
    if epilogue != ops.EPI_NONE:
        return 1
    if m >= PAIR_MIN_ROWS:
        # pairs of SMs with tiles of 256 x 256: a prompt of some hundred tokens gives the o and down products
        # fewer tiles than there are pairs; K is then split so that most pairs have one, 8 blocks of 64 or more each
        tiles = ((m + 255) // 256) * ((n + 255) // 256)
        return max(1, min((ops.sm_count() // 2) // tiles, ((k + 63) // 64) // 8))
    if m > SWAP_MAX_ROWS:
        return 1
    tiles = (n + 127) // 128
    if tiles >= ops.sm_count() // 2:
        return 1
    k_blocks = (k + 63) // 64
    return max(1, min(ops.sm_count() // tiles, k_blocks // 4))      # tiles x splits stays within one wave


def matmul(x, w, out, epilogue: int = ops.EPI_NONE, cap: float = 0.0, act: int = 0,
           k_splits: Optional[int] = None) -> None:
    m, k = x.shape
    n = out.shape[1]
    if k_splits is None:
        k_splits = k_splits_for(m, n, k, epilogue)
    ws = None
    if k_splits > 1:
        ws = torch.empty(k_splits * m * n, dtype=torch.float32, device=x.device)
    lib().call("hos_gemm_tc", ops._ptr(x), ops._ptr(w), ops._ptr(out), ops.dtype_code(out.dtype), m, n, k,
               x.stride(0), w.stride(0), out.stride(0), epilogue, float(cap), act, k_splits, ops._ptr(ws),
               1, None, ops._stream())


def matmul_partials(x, w, k_splits: Optional[int] = None) -> Optional[torch.Tensor]:
    """x . w^T as partial sums [parts, M, N] (float32) for a consumer that adds them, if K is
    worth splitting for these sizes; None if it is not (call `matmul` then)."""
    m, k = x.shape
    n = w.shape[0]
    if k_splits is None:
        k_splits = k_splits_for(m, n, k, ops.EPI_NONE)
    if k_splits <= 1:
        return None
    ws = torch.empty((k_splits, m, n), dtype=torch.float32, device=x.device)
    used = ctypes.c_int(0)
    lib().call("hos_gemm_tc", ops._ptr(x), ops._ptr(w), None, ops.F32, m, n, k, x.stride(0), w.stride(0), n,
               ops.EPI_NONE, 0.0, 0, k_splits, ops._ptr(ws), 0, ctypes.byref(used), ops._stream())
    return ws[: used.value]


def wait_probe(limit_cycles: int = 1 << 20) -> None:
    """A tiny kernel that waits on a barrier nothing arrives at, gives up after `limit_cycles` (well
    under a millisecond by default) and records it as the product kernels do: for tests of what
    happens next."""
    lib().call("hos_gemm_tc_wait_probe", int(limit_cycles), ops._stream())


def gave_up() -> bool:
    """True if a launch since the last call left a bounded wait unfinished (synchronises)."""
    f = lib().lib.hos_gemm_tc_error
    f.restype = ctypes.c_int
    f.argtypes = []
    return bool(f())



def can_fuse_qkv_rope(x: torch.Tensor, w: torch.Tensor, head_dim: int, rotary_dim: int, style: int, inv_freq) -> bool:
    """Whether the q/k/v projection of many tokens can rotate q and k and store keys and values in its own
    epilogue: the product's rules, rows enough for the kernel on pairs of SMs, the whole head rotated with the rotate-half pairing,
    a head size that divides the tile's 256 columns."""
    if not enabled or x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or x.shape[0] < PAIR_MIN_ROWS:
        return False
    if inv_freq is None or rotary_dim != head_dim or style != 0 or head_dim not in (64, 128, 256):
        return False
    k = x.shape[1]
    if k % 8 != 0 or x.stride(1) != 1 or w.stride(1) != 1 or x.stride(0) % 8 or w.stride(0) % 8:
        return False
    return x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0


def step_angles(step, inv_freq: torch.Tensor) -> torch.Tensor:
    """(cos, sin) of every token's position times every inverse frequency, float32 [N, len(inv_freq), 2]:
    taken once per step and set of frequencies and kept on the step, so that all layers share it."""
    kept = getattr(step, "_angles", None)
    if kept is None:
        kept = {}
        try:
            step._angles = kept
        except AttributeError:
            pass
    key = (inv_freq.data_ptr(), inv_freq.shape[0])
    table = kept.get(key)
    if table is None or getattr(step, "replayed", False):
        table = kept[key] = ops.rope_table(step.token_pos, inv_freq)
    return table


def qkv_rope(x, w, out, n_heads: int, n_kv_heads: int, head_dim: int, step, inv_freq, cache) -> None:
    """out[M, (n_heads + 2 n_kv_heads) * head_dim] = x . w^T with q and k heads rotated and, if `cache` is given,
    keys and values stored at the tokens' places.  n_kv_heads = 0: q heads only."""
    m, k = x.shape
    angles = step_angles(step, inv_freq)
    lib().call("hos_gemm_tc_qkv_rope", ops._ptr(x), ops._ptr(w), ops._ptr(out), m, out.shape[1], k, x.stride(0),
               w.stride(0), out.stride(0), n_heads, n_kv_heads, head_dim, ops._ptr(step.token_pos),
               ops._ptr(step.token_seq), ops._ptr(step.seq_slot), ops._ptr(step.seq_len_after), ops._ptr(angles),
               ops._ptr(cache.k_pages) if cache else None, ops._ptr(cache.v_pages) if cache else None,
               ops._ptr(cache.page_table) if cache else None, cache.table_stride if cache else 0,
               cache.ring_pages if cache else 0, 1 if cache else 0, ops._stream())
