"""Python face of the tensor-core attention kernels (csrc/attention_decode.cu,
csrc/attention_prefill.cu).  They are compiled per head size (a multiple of 16, at most
256) as library `attn_hd<N>`; other head sizes are left to the plain kernel."""
from __future__ import annotations

import ctypes
import os
from typing import Dict, Optional

import torch

from .. import ops

MAX_HEAD_DIM = 256
MAX_SPLITS = 64

_libs: Dict[int, ops.Library] = {}
enabled = {"decode": True, "prefill": True, "prefill_tc": True, "chunk": True, "chunk_tc": True,
           "prefill_pair": os.environ.get("HOS_ATTN_PAIR", "1") != "0",
           "decode_cluster": os.environ.get("HOS_ATTN_CLUSTER", "1") != "0",
           "decode_even": os.environ.get("HOS_ATTN_EVEN", "1") != "0"}
_pair_state: Dict[int, bool] = {}
_cluster_state: Dict[int, bool] = {}     # tests switch a kernel off to compare with the plain one


def supports(head_dim: int) -> bool:
    return head_dim % 16 == 0 and 16 <= head_dim <= MAX_HEAD_DIM


def lib_for(head_dim: int) -> ops.Library:
    lib = _libs.get(head_dim)
    if lib is None:
        lib = _libs[head_dim] = ops.Library(f"attn_hd{head_dim}")
    return lib


def decode_splits(n_tokens: int, n_kv_heads: int, group: int, max_len: int, window: Optional[int],
                  min_live: int = 0, clusters_fit=None, max_live: int = 0, fill: float = 1.0) -> int:
    """How many shares the keys of one (token, kv head) are cut into.  The kernel's CTAs (one per
    SM) take items one after another; an item costs a fixed part (look-ups, first loads, the merge)
    and a part per page.  The number of shares is the one that makes the step shortest by that
    model (constants measured at head size 256), for all `n_tokens` rows live and, if the step is
    a replayed one whose last rows may be padding, for `min_live` live rows and half-way as well
    (`max_live`: no more than that many of the rows are live; 0: all may be).  `fill`: the sequences' lengths add
    up to at most this fraction of live rows x what the longest holds (in this layer: of its window, if it has one):
    equal shares follow the longest sequence whatever the others hold, even shares follow the sum.
    `clusters_fit(s)`: how many clusters of s CTAs of the kernel run at once (None: no cluster merge); with
    all of a step's clusters on the GPU at once the shares merge through shared memory, which is cheaper."""
    chunks = (group + 15) // 16
    span = min(max_len, window) if window else max_len
    pages = (span + ops.PAGE_TOKENS - 1) // ops.PAGE_TOKENS + (1 if window else 0)
    per_token = max(1, n_kv_heads * chunks)
    hi = max(1, min(n_tokens, max_live) if max_live else n_tokens)
    lo = min(max(1, min_live), hi) if min_live else hi
    lives = (lo, (lo + hi) // 2, hi, hi) if lo < hi else (hi,)      # fewest, middle and most live rows (a full batch counts twice)
    best, best_cost = 1, None
    sms = ops.sm_count()

    def merge_us(s: int) -> float:
        if s == 1:
            return 0.0
        if clusters_fit is not None and s <= CLUSTER_SHARES and hi * per_token * s <= sms \
                and clusters_fit(s) >= hi * per_token:
            return _CLUSTER_MERGE_US + _CLUSTER_MERGE_PER_SHARE_US * s      # the shares are one cluster
        return _MERGE_US + _MERGE_PER_SHARE_US * s

    for s in range(1, min(MAX_SPLITS, max(1, (pages + 1) // 2)) + 1):
        per_item = _ITEM_US + _PAGE_US * -(-pages // s) + merge_us(s)
        cost = sum(-(-live * per_token * s // sms) * per_item for live in lives)
        if best_cost is None or cost < 0.97 * best_cost:          # more shares only for a clear gain
            best, best_cost = s, cost
    # Even shares (0): every CTA the same number of pages, wherever the borders of the (token, kv head) fall.  They
    # cost a fixed part more (the running sums of the pages, a second piece of work per CTA, a merge of almost
    # every (token, kv head) through the workspace) and save the last round that equal items leave mostly empty.
    # Weighed with a model that knows that many CTAs at once share the memory's speed: a round of all SMs is
    # slower per page than a last round of a few.
    # Only while the longest (token, kv head) lies in at most EVEN_MOST_PARTS CTAs: the last CTA of each merges all
    # of its parts (one sequence at 32,768 keys in 37 parts: 1.90 ms a step against 1.75 ms in clusters).
    held = max(1.0, pages * fill)             # pages an average (token, kv head) holds in this layer
    if enabled["decode_even"] and n_tokens <= EVEN_MAX_ROWS and \
            pages <= EVEN_MOST_PARTS * max(1, -(-int(lo * per_token * held) // sms)):
        def page_us(active: int) -> float:
            return max(_PAGE_US, active * _PAGE_SHARED_US)
        share, equal, even = -(-pages // best), 0.0, 0.0
        for live in lives:
            full, rest = divmod(live * per_token * best, sms)      # rounds of all SMs, and what is left for a last one
            equal += full * (_ITEM_US + share * page_us(sms) + merge_us(best))
            if rest:
                equal += _ITEM_US + share * page_us(rest) + merge_us(best)
            equal += _ROUND_US * max(0, full + (1 if rest else 0) - 1)
            even += _EVEN_US + -(-int(live * per_token * held) // sms) * page_us(sms)
        if even < 0.95 * equal:
            return 0
    return best


# Fitted to measurements at head size 256, 8192 keys: one sequence takes 43.0 / 29.7 / 24.7 / 26.6 us with
# 4 / 8 / 16 / 32 shares (launch included), eight sequences 130 / 76 / 65.5 / 72.6 us with 1 / 2 / 4 / 9;
# at 64 sequences two shares instead of one cost 27 us more per layer.
_ITEM_US, _PAGE_US, _MERGE_US, _MERGE_PER_SHARE_US = 6.0, 0.9, 1.0, 0.275
# Up to 16 shares of at most one wave of items merge as a cluster through shared memory: 2.3 to 2.8 us less
# than through the workspace (one sequence, 8,192 keys, 16 shares: 17.4 -> 14.6 us; a window of 4,096: 13.5 -> 10.7).
CLUSTER_SHARES = 16
_CLUSTER_MERGE_US, _CLUSTER_MERGE_PER_SHARE_US = 0.3, 0.03
# Even shares against the best equal shares, a step of Gemma-2 2B sizes at 8,192 keys (ms): 20 sequences 3.63 / 3.81,
# 40: 5.80 / 6.92, 56: 7.28 / 8.15, 64: 8.04 / 8.02; but 8: 2.41 / 2.11, 16: 3.16 / 2.94, 32: 4.82 / 4.58.
# The model that fits these: 22 us more per launch than one round of equal shares, 8 us for every further round of
# equal shares, and a page costs a CTA 0.9 us alone but 0.0085 us times the number of CTAs that stream at once (64 KB
# per page at head size 256: 7.7 TB/s between them).  At Gemma-2 9B sizes, 16 sequences of 64 to 2,300 keys (0.64 of
# what 16 of the longest would hold) lose 0.15 ms a step with even shares: the model has to say no there.
# Sequences of unequal lengths (8,100 / 4,000 / 2,000 / 1,000 / 500 / 500 / 250 / 250 keys, repeated): equal shares
# take as long as the longest sequence's share, even shares follow the sum: 8 sequences 1.96 -> 1.86 ms a step, 16
# sequences 2.69 -> 2.22, 32 sequences 4.05 -> 3.00.
_EVEN_US = 22.0
_ROUND_US = 8.0
_PAGE_SHARED_US = 0.0085
EVEN_MAX_ROWS = 2048
EVEN_MOST_PARTS = 20


_fit_known: Dict[tuple, int] = {}


def clusters_fit(head_dim: int, n_heads: int, n_kv_heads: int, n_splits: int) -> int:
    """Clusters of n_splits CTAs of the decode kernel that run on the GPU at once (asked once per shape)."""
    key = (head_dim, n_heads, n_kv_heads, n_splits)
    n = _fit_known.get(key)
    if n is None:
        f = lib_for(head_dim).lib.hos_attn_decode_clusters
        f.restype, f.argtypes = ctypes.c_int, [ctypes.c_int, ctypes.c_int, ctypes.c_int]
        n = _fit_known[key] = int(f(n_heads, n_kv_heads, n_splits))
    return n


_ticket_store: Dict[object, list] = {}
_TICKETS_AT_LEAST = 1 << 16


def _tickets(device, n: int) -> torch.Tensor:
    """Zeroed counters that the kernel leaves zeroed, shared by all launches on a device.  Captured
    graphs keep the address they were given, so a buffer is never given up: if a launch needs more
    than the last one holds, another is made and the old ones stay."""
    held = _ticket_store.setdefault(device, [])
    if not held or held[-1].numel() < n:
        held.append(torch.zeros(max(n, _TICKETS_AT_LEAST), dtype=torch.int32, device=device))
    return held[-1]


def _clear_tickets() -> None:
    """After a kernel gave up: a share that left early took no ticket, so its counter is not at zero."""
    for held in _ticket_store.values():
        for t in held:
            t.zero_()


ops.on_give_up(_clear_tickets)


def decode(q: torch.Tensor, q_stride: int, out: torch.Tensor, token_pos, token_seq, seq_slot,
           cache: ops.PagedKVArgs, n_tokens: int, n_heads: int, scale: float, cap: float,
           window: Optional[int], max_len: int, n_splits: Optional[int] = None,
           max_new: Optional[int] = None, min_live: int = 0, token_slot=None, cluster: bool = True,
           max_live: int = 0, fill: float = 1.0) -> None:
    """Attention of n_tokens single queries over the paged cache (each token at its own
    position in its own sequence).  `max_new`: the most tokens any sequence brings in this step;
    the kernel may fetch keys that lie below them while the kernel before it (which writes the
    step's new keys) still runs.  None: it fetches nothing ahead.  `token_slot`: each token's cache slot
    (seq_slot[token_seq]) if the step has it: the kernel then finds its first page one look-up sooner.
    `cluster`: up to 16 shares of at most one wave of work items may run as clusters that merge through
    shared memory (False: always through the workspace)."""
    hd, nkv = cache.head_dim, cache.n_kv_heads
    lib = lib_for(hd)
    want = bool(cluster and enabled["decode_cluster"])
    if _cluster_state.get(hd) != want:
        lib.call("hos_attn_decode_cluster", 1 if want else 0)
        _cluster_state[hd] = want
    if n_splits is None:
        fit = (lambda s: clusters_fit(hd, n_heads, nkv, s)) if want else None
        n_splits = decode_splits(n_tokens, nkv, n_heads // nkv, max_len, window, min_live, fit, max_live, fill)
    ws = tickets = None
    if n_splits == 0:            # even shares: every CTA the same number of pages, two places per CTA for what is cut
        f = lib.lib.hos_attn_decode_even_workspace
        f.restype, f.argtypes = ctypes.c_longlong, [ctypes.c_int, ctypes.c_int]
        ws = torch.empty(int(f(n_heads, nkv)), dtype=torch.float32, device=q.device)
    elif n_splits > 1:
        ws = torch.empty(n_tokens * n_heads * n_splits * (hd + 2), dtype=torch.float32, device=q.device)
    if n_splits != 1:
        tickets = _tickets(q.device, n_tokens * nkv * ((n_heads // nkv + 15) // 16))
    lib.call("hos_attn_decode", ops._ptr(q), q_stride, ops._ptr(out), out.shape[1], ops._ptr(ws),
             ops._ptr(tickets), ops._ptr(token_pos), ops._ptr(token_seq), ops._ptr(seq_slot), ops._ptr(token_slot),
             ops._ptr(cache.k_pages),
             ops._ptr(cache.v_pages), ops._ptr(cache.page_table), cache.table_stride, cache.ring_pages,
             n_tokens, n_heads, nkv, hd, float(scale), float(cap), int(window) if window else 0,
             int(n_splits), int(max_new) if max_new else 1 << 30, ops._stream())
    # one or two sequences' worth of CTAs leave most SMs free: the product after this kernel may be placed beside it
    ctas = ops.sm_count() if n_splits == 0 else n_tokens * nkv * ((n_heads // nkv + 15) // 16) * n_splits
    ops.note_room_left(2 * ctas <= ops.sm_count())


def decode_gave_up(head_dim: int) -> bool:
    """True if a launch since the last call left a bounded wait unfinished (synchronises)."""
    lib = lib_for(head_dim)
    f = lib.lib.hos_attn_decode_error
    f.restype = ctypes.c_int
    f.argtypes = []
    return bool(f())


def has_tc_prefill(head_dim: int) -> bool:
    f = lib_for(head_dim).lib.hos_attn_prefill_tc_available
    f.restype, f.argtypes = ctypes.c_int, []
    return bool(f())


def prompt_blocks(step, block: int):
    """(sequences, blocks of `block` queries) a prompt kernel's grid has to cover.  From the host's
    lists when the step has them; for a replayed step an upper bound (the kernels skip blocks
    beyond the sequences' real ends, which they read on the device)."""
    if step.replayed or not step.cu_host:
        return step.n_seqs, (step.n_tokens + block - 1) // block + step.n_seqs
    cu = step.cu_host
    return len(cu) - 1, sum((cu[i + 1] - cu[i] + block - 1) // block for i in range(len(cu) - 1))


def prefill_tc(rows: torch.Tensor, out, cu_seqlens, n_seqs: int, blocks: int, n_heads, n_kv_heads, head_dim, scale, cap,
               window, pairs: bool = True) -> None:
    """Attention of whole prompts from position 0 on the tcgen05 tensor cores; `rows` is the
    fused projection output [N, (n_heads + 2 n_kv_heads) * head_dim] (head sizes 64, 128, 256).
    `blocks`: at least the sum over sequences of ceil(length / 128).  `pairs`: two query heads that
    share their keys may run as one pair of SMs (head sizes 128 and 256, an even group)."""
    lib = lib_for(head_dim)
    want = bool(pairs and enabled["prefill_pair"])
    if _pair_state.get(head_dim) != want:
        lib.call("hos_attn_prefill_pair", 1 if want else 0)
        _pair_state[head_dim] = want
    lib.call("hos_attn_prefill_tc", ops._ptr(rows), rows.shape[0], rows.shape[1], ops._ptr(out), out.shape[1],
             ops._ptr(cu_seqlens), n_seqs, blocks, n_heads, n_kv_heads, head_dim, float(scale), float(cap),
             int(window) if window else 0, ops._stream())


def prefill_tc_gave_up(head_dim: int) -> bool:
    f = lib_for(head_dim).lib.hos_attn_prefill_tc_error
    f.restype, f.argtypes = ctypes.c_int, []
    return bool(f())


def prefill(q, q_stride, k_rows, v_rows, kv_stride, out, cu_seqlens, n_seqs: int, blocks: int, n_heads, n_kv_heads,
            head_dim, scale, cap, window) -> None:
    """Attention of whole prompts from position 0 over their own packed rows (mma.sync kernel).
    `blocks`: at least the sum over sequences of ceil(length / 64)."""
    lib = lib_for(head_dim)
    lib.call("hos_attn_prefill", ops._ptr(q), q_stride, ops._ptr(k_rows), ops._ptr(v_rows), kv_stride,
             ops._ptr(out), out.shape[1], ops._ptr(cu_seqlens), n_seqs, blocks, n_heads, n_kv_heads, head_dim,
             float(scale), float(cap), int(window) if window else 0, ops._stream())


def chunk(q, q_stride, out, cu_seqlens, row_base: int, token_pos, seq_slot, n_seqs: int, blocks: int,
          cache: ops.PagedKVArgs, n_heads, scale, cap, window) -> None:
    """Attention of sequences that go on by many tokens over the paged cache (which holds the step's
    own keys already): sequence s has the rows cu_seqlens[s] - row_base .. of q and out, at consecutive
    positions from token_pos[its first row], and the page-table row seq_slot[s].  `blocks`: at least the
    sum over sequences of ceil(rows / 64)."""
    lib = lib_for(cache.head_dim)
    lib.call("hos_attn_chunk", ops._ptr(q), q_stride, ops._ptr(out), out.shape[1], ops._ptr(cu_seqlens), int(row_base),
             ops._ptr(token_pos), ops._ptr(seq_slot), n_seqs, blocks, ops._ptr(cache.k_pages), ops._ptr(cache.v_pages),
             ops._ptr(cache.page_table), cache.table_stride, cache.ring_pages, n_heads, cache.n_kv_heads,
             cache.head_dim, float(scale), float(cap), int(window) if window else 0, ops._stream())


def chunk_tc(q, out, cu_seqlens, row_base: int, token_pos, seq_slot, n_seqs: int, blocks: int,
             cache: ops.PagedKVArgs, n_heads, scale, cap, window) -> None:
    """As `chunk`, on the tcgen05 tensor cores (head sizes 64, 128, 256): q is [rows, stride] with the q heads
    first in a row; `blocks`: at least the sum over sequences of ceil(rows / 128)."""
    lib = lib_for(cache.head_dim)
    lib.call("hos_attn_chunk_tc", ops._ptr(q), q.shape[0], q.shape[1], ops._ptr(out), out.shape[1], ops._ptr(cu_seqlens),
             int(row_base), ops._ptr(token_pos), ops._ptr(seq_slot), n_seqs, blocks, ops._ptr(cache.k_pages),
             ops._ptr(cache.v_pages), cache.k_pages.shape[0], ops._ptr(cache.page_table), cache.table_stride,
             cache.ring_pages, n_heads, cache.n_kv_heads, cache.head_dim, float(scale), float(cap),
             int(window) if window else 0, ops._stream())


def attend_chunks(mixer, qkv, att, part, cache) -> bool:
    """The rows of `part` (sequences of a step that go on by many tokens; see StepInfo.rows) through
    a chunk kernel (the tcgen05 one where the head size has it); False if none takes the case."""
    if cache.k_pages.dtype != torch.bfloat16 or not supports(mixer.head_dim) or not enabled["chunk"]:
        return False
    if part.replayed:
        att.zero_()                          # which rows are padding is known on the device only: a defined output
    elif not part.cu_host:
        return False
    slots = part.seq_slot[part.seq_offset:]
    if enabled["chunk_tc"] and qkv.is_contiguous() and has_tc_prefill(mixer.head_dim):
        _, blocks = prompt_blocks(part, 128)
        chunk_tc(qkv, att, part.cu_seqlens, part.row_offset, part.token_pos, slots, part.n_seqs, blocks, cache,
                 mixer.n_heads, mixer.scale, mixer.softcap, mixer.window)
        return True
    _, blocks = prompt_blocks(part, 64)
    chunk(qkv, qkv.shape[1], att, part.cu_seqlens, part.row_offset, part.token_pos, slots, part.n_seqs, blocks, cache,
          mixer.n_heads, mixer.scale, mixer.softcap, mixer.window)
    return True


def attend(mixer, qkv, att, step, cache, packed: bool) -> bool:
    """Runs the tensor-core kernel if it takes the case; False hands it to the plain kernel."""
    if cache.k_pages.dtype != torch.bfloat16 or not supports(mixer.head_dim):
        return False
    if packed:
        if not enabled["prefill"]:
            return False
        if step.replayed or not step.cu_host:
            att.zero_()                          # which rows are padding is known on the device only
        elif step.n_tokens > step.cu_host[-1]:
            att[step.cu_host[-1]:].zero_()       # padding rows: a defined output
        if enabled["prefill_tc"] and qkv.is_contiguous() and has_tc_prefill(mixer.head_dim):
            n_seqs, blocks = prompt_blocks(step, 128)
            prefill_tc(qkv, att, step.cu_seqlens, n_seqs, blocks, mixer.n_heads, mixer.n_kv_heads, mixer.head_dim,
                       mixer.scale, mixer.softcap, mixer.window)
            return True
        n_seqs, blocks = prompt_blocks(step, 64)
        prefill(qkv, qkv.shape[1], qkv[:, mixer.q_dim:], qkv[:, mixer.q_dim + mixer.kv_dim:], qkv.shape[1],
                att, step.cu_seqlens, n_seqs, blocks, mixer.n_heads, mixer.n_kv_heads, mixer.head_dim,
                mixer.scale, mixer.softcap, mixer.window)
        return True
    if not enabled["decode"]:
        return False
    decode(qkv, qkv.shape[1], att, step.token_pos, step.token_seq, step.seq_slot, cache, step.n_tokens,
           mixer.n_heads, mixer.scale, mixer.softcap, mixer.window, step.max_len_after, max_new=step.max_new,
           min_live=getattr(step, "min_live", 0), token_slot=getattr(step, "token_slot", None),
           max_live=getattr(step, "max_live", 0),
           fill=step.fill_for(mixer.window) if hasattr(step, "fill_for") else 1.0)
    return True
