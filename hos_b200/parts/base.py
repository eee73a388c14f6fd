"""What a part is, and what it is handed when it runs.

A model is put together from parts of seven categories (see `hos_b200.registry`):

  embedding    tokens -> residual stream          forward(tokens, step) -> x  (float32 [N, width])
  norm         rows -> normalised rows            forward(x, out)
  position     encodes positions into q and k     (used by a mixer; see parts/rope.py)
  mixer        mixes information between tokens   forward(h, step, store) -> y
  feed_forward works on each token alone          forward(h, step) -> y
  arrangement  wires norms, mixer, feed-forward and the residual stream of one layer
               forward(x, step, store) -> None (x is updated in place)
  head         rows -> logits                     forward(h) -> float32 [n, vocab]

Every part is built from a `PartSpec` (its sizes and constants) and a `Runtime`
(device, compute dtype), says which tensors it wants (`weight_specs`), and
receives them once (`bind`).  No part knows which model it is in.

Data types: the residual stream is float32; what a part hands to the next matrix
product (`h`, `y`) has the runtime's compute dtype; logits are float32.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Mapping, Optional, Sequence, Tuple

import torch

from ..config.base import PartSpec


@dataclass(frozen=True)
class WeightSpec:
    """A tensor a part wants from the checkpoint."""
    name: str                        # checkpoint name
    shape: Tuple[int, ...]
    role: str                        # "matrix", "vector" or "table"
    init_std: float                  # standard deviation of the random-weights mode
    fallback: Optional[str] = None   # another tensor to use when this one is absent (tied head)


@dataclass(frozen=True)
class KVNeed:
    """A mixer's wish for keys and values per position.  Calls whose needs are equal
    share one group of the cache (one page table, storage of their own)."""
    n_kv_heads: int
    head_dim: int
    window: Optional[int]            # None: all keys; an int: the last `window` keys


@dataclass(frozen=True)
class StateNeed:
    """A mixer's wish for per-sequence state of fixed size, zeroed when a sequence starts."""
    name: str
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


class Runtime:
    """Where and in what precision a model runs."""

    def __init__(self, device: torch.device, dtype: torch.dtype):
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"compute dtype must be float32 or bfloat16, found {dtype}")
        self.device = torch.device(device)
        self.dtype = dtype

    @property
    def is_fp32(self) -> bool:
        return self.dtype == torch.float32

    def empty(self, *shape, dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        return torch.empty(shape, dtype=dtype or self.dtype, device=self.device)


FEW_TOKENS = 8      # a sequence that goes on by at most this many tokens counts among the step's "tail"


@dataclass
class StepInfo:
    """One step's batch as the kernels see it.  N tokens (rows) of B sequences, packed
    sequence after sequence.  A row with token_seq < 0 is padding: it is computed on
    but stores nothing and no other row reads it."""
    n_tokens: int
    n_seqs: int
    tokens: torch.Tensor          # int32 [N], -1 for padding
    token_pos: torch.Tensor       # int32 [N] position of each token in its sequence
    token_seq: torch.Tensor       # int32 [N] row of the batch, -1 for padding
    cu_seqlens: torch.Tensor      # int32 [B+1] first row of each sequence
    seq_slot: torch.Tensor        # int32 [B] cache slot of each sequence
    seq_len_after: torch.Tensor   # int32 [B] length of each sequence after this step
    from_zero: bool               # every sequence starts at position 0 in this step
    single_token: bool            # every sequence brings exactly one token
    max_new: int                  # most tokens any sequence brings
    max_len_after: int            # longest sequence after this step
    slots_host: Sequence[int] = ()   # the same as seq_slot, on the host
    cu_host: Sequence[int] = ()      # the same as cu_seqlens, on the host
    starts_host: Sequence[int] = ()  # each sequence's length before the step
    token_slot: Optional[torch.Tensor] = None   # int32 [N] seq_slot[token_seq] for every row (anything for padding), if at hand
    min_live: int = 0                # a replayed step's rows may be padding from this row on (0: none is)
    max_live: int = 0                # ... and at most this many of its rows are live (0: all may be)
    fill: float = 1.0                # the keys that the sequences hold add up to at most this fraction of (live rows x
                                     # the keys of the longest), for mixers that see all keys ...
    fills: tuple = ()                # ... and ((window, fraction), ...) for mixers that see a window of them: see fill_for
    replayed: bool = False           # the device arrays are refilled and the same launches replayed (a CUDA
                                     # graph): n_tokens and n_seqs are capacities, the host lists are empty
    fresh_seqs: int = 0              # a step that is not from_zero lists the sequences that start at position 0
    fresh_tokens: int = 0            # first: that many sequences, that many rows (0: every row continues)
    tail_seqs: int = 0               # and the sequences that go on by a few tokens only (FEW_TOKENS or fewer) last:
    tail_tokens: int = 0             # that many sequences, that many rows (a mixer may send them to another kernel)
    row_offset: int = 0              # of a part of a step (see rows()): its first row and its first sequence in the
    seq_offset: int = 0              # whole step, which cu_seqlens (rows) and token_seq, seq_slot (sequences) still count from

    def fill_for(self, window: Optional[int]) -> float:
        """How full of keys the step's sequences are for a mixer with this window (None: all keys): the sum over
        the sequences of the keys each holds, over (sequences x what the longest holds).  1.0 when they are all
        as long as the longest, or when nothing is known.  A kernel whose work follows the sum of the keys rather
        than the longest sequence plans with it."""
        if self.starts_host and self.cu_host:
            lens = [s + (self.cu_host[i + 1] - self.cu_host[i]) for i, s in enumerate(self.starts_host)]
            held = [min(n, window) if window else n for n in lens]
            return min(1.0, sum(held) / float(len(held) * max(held))) if held and max(held) > 0 else 1.0
        for w, f in self.fills:
            if w == (window or 0):
                return f
        return self.fill

    def rows(self, lo: int, hi: int, seq_lo: int, seq_hi: int) -> "StepInfo":
        """The step as seen by rows lo..hi-1 alone, which are the sequences seq_lo..seq_hi-1: what a
        mixer hands to a kernel that takes only a part of a step (the sequences that start at
        position 0 to one kernel, the ones that go on to another).  Row arrays are cut;
        `token_seq` keeps its values, so the per-sequence arrays `seq_slot` and `seq_len_after`
        stay whole (the part's first sequence is their entry `seq_offset`), while `cu_seqlens`
        is cut to the part's sequences and still counts rows from the whole step's first row
        (`row_offset` rows before the part's first); the host lists are cut and count from the
        part's first row."""
        import dataclasses
        cu = tuple(c - lo for c in self.cu_host[seq_lo:seq_hi + 1]) if self.cu_host else ()    # counted from the part's first row
        starts = tuple(self.starts_host[seq_lo:seq_hi]) if self.starts_host else ()
        news = [cu[i + 1] - cu[i] for i in range(len(cu) - 1)]
        fresh = seq_lo == 0 and seq_hi <= self.fresh_seqs
        return dataclasses.replace(
            self, n_tokens=hi - lo, n_seqs=seq_hi - seq_lo, tokens=self.tokens[lo:hi],
            token_pos=self.token_pos[lo:hi], token_seq=self.token_seq[lo:hi],
            cu_seqlens=self.cu_seqlens[seq_lo:seq_hi + 1],
            token_slot=self.token_slot[lo:hi] if self.token_slot is not None else None,
            from_zero=fresh or self.from_zero, single_token=bool(news) and all(k == 1 for k in news),
            max_new=max(news) if news else self.max_new,
            max_len_after=max((s + k for s, k in zip(starts, news)), default=self.max_len_after),
            slots_host=tuple(self.slots_host[seq_lo:seq_hi]) if self.slots_host else (), cu_host=cu,
            starts_host=starts, fresh_seqs=seq_hi - seq_lo if fresh else 0, fresh_tokens=hi - lo if fresh else 0,
            tail_seqs=max(0, min(seq_hi, self.n_seqs) - max(seq_lo, self.n_seqs - self.tail_seqs)),
            tail_tokens=max(0, min(hi, self.n_tokens) - max(lo, self.n_tokens - self.tail_tokens)),
            row_offset=self.row_offset + lo, seq_offset=self.seq_offset + seq_lo)


class CallStore:
    """The storage of one entry of the run order: its view of the paged cache (or
    of the cache of the entry it reads from) and its per-sequence state tensors."""

    def __init__(self, kv=None, owns_kv: bool = True, state: Optional[Dict[str, torch.Tensor]] = None):
        self.kv = kv                      # ops.PagedKVArgs or None
        self.owns_kv = owns_kv            # False: another entry writes this cache
        self.state = state or {}          # name -> tensor [n_slots, *shape]


class Part:
    """Base of every part."""

    # True if forward() only launches kernels on device data (no host reads of the step's
    # lists, no host-device synchronisation): single-token steps of a model whose parts all
    # say so are captured in a CUDA graph and replayed.  A part that loops over
    # `step.slots_host` or the like leaves it False and is run step by step.
    graph_safe = False

    def __init__(self, spec: PartSpec, rt: Runtime):
        self.spec = spec
        self.rt = rt

    def weight_specs(self) -> List[WeightSpec]:
        return []

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        """Receive the tensors named in weight_specs(), on the device, in their stored
        dtype (bfloat16 kept, 32-bit kept).  Convert or fuse them here, once."""

    # helpers -----------------------------------------------------------------------
    def _matrix(self, t: torch.Tensor) -> torch.Tensor:
        """A matrix as the products take it: float32 in the 32-bit path (an exact
        widening of bfloat16), else as stored (bfloat16, or 32-bit if it was so)."""
        if self.rt.is_fp32:
            return t.to(torch.float32).contiguous()
        if t.dtype == torch.float16:
            return t.to(torch.bfloat16).contiguous()
        return t.contiguous()

    @staticmethod
    def _vector32(t: torch.Tensor) -> torch.Tensor:
        return t.to(torch.float32).contiguous()


class Mixer(Part):
    def kv_need(self) -> Optional[KVNeed]:
        return None

    def state_needs(self) -> List[StateNeed]:
        return []

    def forward(self, h: torch.Tensor, step: StepInfo, store: CallStore) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, h: torch.Tensor, step: StepInfo) -> torch.Tensor:
        raise NotImplementedError


class Norm(Part):
    def forward(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        raise NotImplementedError

    def add_to(self, y: torch.Tensor, x: torch.Tensor, then: Optional["Norm"] = None) -> Optional[torch.Tensor]:
        """x += self(y).  If `then` is given, also return then(x).  The default does
        it in separate kernels; a norm may fuse them."""
        from .. import ops
        n = self.forward(y)
        ops.residual_add(n, x)
        return then.forward(x) if then is not None else None
