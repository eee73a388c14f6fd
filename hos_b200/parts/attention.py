"""Softmax attention with grouped queries: q, k, v projections (one fused product),
position encoding on q and k, keys and values kept in the paged cache, scores
(q.k) * scale, optional soft-cap c*tanh(s/c), causal mask with an optional window
of the last W keys, softmax, weighted values, output projection
(src/forward.rs:300-363; head map h // (heads / kv_heads), :340).

Every size and constant is a parameter: width, n_heads, n_kv_heads, head_dim,
scale, softcap (0 = off), window (None = all keys), and the position encoding
(a PartSpec of category "position").  The mixer asks the cache for keys and
values of [n_kv_heads, head_dim] per position, all of them or a window.

A sequence that starts at position 0 attends over its own freshly projected rows
and only stores to the cache; a sequence that goes on (by one token or by many)
stores first and then attends over the cache.  One step may hold both kinds: the
rows of the first kind come first and go to one kernel, the rest to another.  An entry of the run order that reads another entry's cache
projects q only and always attends over that cache.
"""
from __future__ import annotations

from typing import List, Mapping, Optional

import torch

from .. import ops
from ..errors import KernelError, SpecError
from ..registry import part_impl, register_part
from . import linear
from .base import CallStore, KVNeed, Mixer, StepInfo, WeightSpec


class SoftmaxAttention(Mixer):
    graph_safe = True

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        p = spec.params
        self.width = int(p["width"])
        self.n_heads = int(p["n_heads"])
        self.n_kv_heads = int(p["n_kv_heads"])
        self.head_dim = int(p["head_dim"])
        self.scale = float(p["scale"])
        self.softcap = float(p.get("softcap") or 0.0)
        self.window: Optional[int] = p.get("window")
        if self.n_heads % self.n_kv_heads != 0:
            raise SpecError(f"arch spec error: {self.n_heads} heads are not a multiple of "
                            f"{self.n_kv_heads} kv heads")
        pos_spec = p.get("position")
        self.position = part_impl("position", pos_spec.kind)(pos_spec, rt) if pos_spec else None
        self.q_dim = self.n_heads * self.head_dim
        self.kv_dim = self.n_kv_heads * self.head_dim
        self.w_qkv = self.w_q = self.w_o = None

    def weight_specs(self) -> List[WeightSpec]:
        w = self.spec.weights
        return [WeightSpec(w["q"], (self.q_dim, self.width), "matrix", 0.02),
                WeightSpec(w["k"], (self.kv_dim, self.width), "matrix", 0.02),
                WeightSpec(w["v"], (self.kv_dim, self.width), "matrix", 0.02),
                WeightSpec(w["o"], (self.width, self.q_dim), "matrix", 0.02)]

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        w = self.spec.weights
        q, k, v = (self._matrix(tensors[w[r]]) for r in ("q", "k", "v"))
        if not (q.dtype == k.dtype == v.dtype):
            q, k, v = q.float(), k.float(), v.float()
        self.w_qkv = torch.cat([q, k, v], dim=0).contiguous()    # one product for q, k and v
        self.w_q = self.w_qkv[: self.q_dim]                      # a view: rows of q alone
        self.w_o = self._matrix(tensors[w["o"]])

    def kv_need(self) -> KVNeed:
        return KVNeed(self.n_kv_heads, self.head_dim, self.window)

    def forward(self, h: torch.Tensor, step: StepInfo, store: CallStore) -> torch.Tensor:
        return self._run(h, step, store, False)

    def forward_partial(self, h: torch.Tensor, step: StepInfo, store: CallStore) -> torch.Tensor:
        """As forward, but the output projection may come back as float32 partial sums
        [parts, N, width] for a consumer that adds them (see linear.matmul_or_partials)."""
        return self._run(h, step, store, True)

    def _run(self, h: torch.Tensor, step: StepInfo, store: CallStore, partial_ok: bool) -> torch.Tensor:
        n = h.shape[0]
        cache = store.kv
        if cache is None:
            raise KernelError("attention needs a cache view")
        inv_freq, rotary_dim, style = self.position.kernel_args() if self.position else (None, 0, 0)
        w = self.w_qkv if store.owns_kv else self.w_q
        n_kv = self.n_kv_heads if store.owns_kv else 0
        from . import gemm_skinny, gemm_tc
        if not linear.plain_forced() and gemm_skinny.can_fuse_qkv_rope(h, w, self.head_dim, rotary_dim):
            # a handful of rows: projection, rotation and cache write in one kernel
            qkv = torch.empty((n, w.shape[0]), dtype=h.dtype, device=h.device)
            gemm_skinny.qkv_rope(h, w, qkv, self.n_heads, n_kv, self.head_dim, step, inv_freq, rotary_dim, style,
                                 cache if store.owns_kv else None)
        elif not linear.plain_forced() and gemm_tc.can_fuse_qkv_rope(h, w, self.head_dim, rotary_dim, style, inv_freq):
            # many rows: the same on the tensor cores (tiles of 256 columns hold whole heads)
            qkv = torch.empty((n, w.shape[0]), dtype=h.dtype, device=h.device)
            gemm_tc.qkv_rope(h, w, qkv, self.n_heads, n_kv, self.head_dim, step, inv_freq,
                             cache if store.owns_kv else None)
        elif store.owns_kv:
            qkv = linear.matmul_or_partials(h, w)
            parts = None
            if qkv.dim() == 3:       # partial sums: the rotate-and-store kernel adds them
                parts, qkv = qkv, torch.empty(qkv.shape[1:], dtype=h.dtype, device=h.device)
            ops.rope_kv_write(qkv, self.n_heads, step.token_pos, step.token_seq, step.seq_slot,
                              step.seq_len_after, inv_freq, rotary_dim, style, cache,
                              self.n_kv_heads, self.head_dim, partials=parts)
        else:
            qkv = linear.matmul(h, w)
            ops.rope_kv_write(qkv, self.n_heads, step.token_pos, step.token_seq, step.seq_slot,
                              step.seq_len_after, inv_freq, rotary_dim, style, None, 0, self.head_dim)
        att = torch.empty((n, self.q_dim), dtype=h.dtype, device=h.device)
        if step.from_zero and store.owns_kv:
            self._attend(qkv, att, step, cache, True)          # whole prompts: over the step's own rows
        else:
            # the sequences that start at position 0 come first and attend over their own rows;
            # every other row attends over the cache, which holds the step's keys already
            nf, sf = (step.fresh_tokens, step.fresh_seqs) if store.owns_kv else (0, 0)
            if nf > 0:
                self._attend(qkv[:nf], att[:nf], step.rows(0, nf, 0, sf), cache, True)
            if nf < n:
                rest = step if nf == 0 else step.rows(nf, n, sf, step.n_seqs)
                if cache.ring_pages > 0:
                    room = cache.ring_pages * ops.PAGE_TOKENS - int(self.window) + 1
                    if rest.max_new > room:
                        raise KernelError(
                            f"a step that continues sequences brings {rest.max_new} tokens to a layer that "
                            f"keeps a window of {self.window} keys in a ring of "
                            f"{cache.ring_pages * ops.PAGE_TOKENS}: at most {room} fit without overwriting "
                            f"keys that the step still reads")
                # sequences that bring many tokens: a kernel that takes 64 queries per key tile; the few-token
                # tail (decoding rows that share the step): the kernel that splits one query's keys over the GPU
                nt, st = rest.tail_tokens, rest.tail_seqs
                if rest.replayed and rest.single_token:
                    many = 0                 # a captured single-token step: the kernel that splits one query's keys
                elif rest.replayed:
                    # a captured step of several tokens per sequence (a short second turn): which rows are which is
                    # known on the device only; from 32 rows on all of them go to the kernel that takes many queries
                    # per key tile
                    nt, st = 0, 0
                    many = rest.n_tokens if rest.n_tokens >= 32 else 0
                else:
                    padded = not rest.cu_host or rest.cu_host[-1] != rest.n_tokens     # padding rows: one kernel takes all
                    many = 0 if padded else rest.n_tokens - nt
                if many > 0 and self._attend_chunks(qkv[nf:nf + many], att[nf:nf + many],
                                                    rest.rows(0, many, 0, rest.n_seqs - st), cache):
                    if nt > 0:
                        self._attend(qkv[nf + many:], att[nf + many:],
                                     rest.rows(many, rest.n_tokens, rest.n_seqs - st, rest.n_seqs), cache, False)
                else:
                    self._attend(qkv[nf:], att[nf:], rest, cache, False)
        return linear.matmul_or_partials(att, self.w_o) if partial_ok else linear.matmul(att, self.w_o)

    def _attend_chunks(self, qkv, att, part: StepInfo, cache) -> bool:
        """Sequences that go on by many tokens, over the cache, 64 queries at a time.  `part`: those
        rows of the step.  False: no such kernel for this case."""
        if self.rt.dtype != torch.bfloat16:
            return False
        from . import attention_fast
        return attention_fast.attend_chunks(self, qkv, att, part, cache)

    def _attend(self, qkv, att, step: StepInfo, cache, packed: bool) -> None:
        stride = qkv.shape[1]
        if self.rt.dtype == torch.bfloat16:
            from . import attention_fast
            if attention_fast.attend(self, qkv, att, step, cache, packed):
                return
        if packed:
            k_rows = qkv[:, self.q_dim:]
            v_rows = qkv[:, self.q_dim + self.kv_dim:]
            ops.attn_plain(qkv, stride, att, step.token_pos, step.token_seq, step.n_tokens,
                           self.n_heads, self.n_kv_heads, self.head_dim, self.scale, self.softcap,
                           self.window, k_rows=k_rows, v_rows=v_rows, kv_stride=stride,
                           cu_seqlens=step.cu_seqlens)
        else:
            ops.attn_plain(qkv, stride, att, step.token_pos, step.token_seq, step.n_tokens,
                           self.n_heads, self.n_kv_heads, self.head_dim, self.scale, self.softcap,
                           self.window, seq_slot=step.seq_slot, cache=cache)


register_part("mixer", "softmax_attention", SoftmaxAttention)
