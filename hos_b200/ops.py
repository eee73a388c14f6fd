"""Python faces of the CUDA kernels.

Every function here checks what it is given (device, dtype, contiguity, sizes),
passes raw pointers and the current stream to the `extern "C"` function of the
same purpose, and raises `KernelError` with the kernel's own message when that
refuses.  Nothing here computes: if the compiled library is missing and cannot be
built, loading it raises `ExtensionMissingError`.
"""
from __future__ import annotations

import ctypes
import os
import re
from dataclasses import dataclass
from typing import List, Optional

import torch

from .csrc import build
from .errors import KernelError

F32, BF16 = 0, 1
PAGE_TOKENS = 64
EPI_NONE, EPI_SOFTCAP, EPI_GATED = 0, 1, 2
ACT_GELU_TANH, ACT_SILU = 0, 1
ACTIVATIONS = {"gelu_tanh": ACT_GELU_TANH, "silu": ACT_SILU}
ROPE_STYLES = {"rotate_half": 0, "interleaved": 1}

_p, _i, _f, _l = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_longlong

_CT = {"p": _p, "i": _i, "f": _f, "l": _l}
_EXPORT = re.compile(r'extern\s+"C"\s+int\s+(\w+)\s*\(([^)]*)\)', re.S)


def _parse_signatures(sources) -> dict:
    """Argument types of every `extern "C" int f(...)` in the given .cu files, read
    from the sources themselves so that the Python side cannot drift from them."""
    sigs = {}
    for src in sources:
        with open(os.path.join(build.HERE, src)) as fh:
            text = fh.read()
        for name, args in _EXPORT.findall(text):
            sig = ""
            for a in args.split(","):
                a = a.strip()
                if not a:
                    continue
                if "*" in a or "cudaStream_t" in a:
                    sig += "p"
                elif "long long" in a:
                    sig += "l"
                elif a.startswith("float") or a.startswith("const float"):
                    sig += "f"
                else:
                    sig += "i"
            sigs[name] = sig
    return sigs


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return F32
    if dt == torch.bfloat16:
        return BF16
    raise KernelError(f"no kernel takes dtype {dt}")


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_device_index: Optional[int] = None


def _stream():
    """The current CUDA stream as a raw handle.  Asked for at every launch, so it goes the
    short way: one call into torch's C layer instead of building a Stream object."""
    global _device_index
    if _raw_stream is None:
        return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    if _device_index is None:
        _device_index = torch.cuda.current_device()
    return ctypes.c_void_p(_raw_stream(_device_index))


class Library:
    """A loaded CUDA library with typed entry points."""

    def __init__(self, name: str):
        self.name = name
        self.lib = build.load(name)
        self._signatures = _parse_signatures(build.library_spec(name)[0])
        self._fns = {}
        self._last_error = None
        if hasattr(self.lib, "hos_last_error"):
            self._last_error = self.lib.hos_last_error
            self._last_error.restype = ctypes.c_char_p
            self._last_error.argtypes = []
        # kernels whose bounded waits run out say so in one word of pinned host memory (check_errors)
        for setter in _ERROR_WORD_SETTERS:
            f = getattr(self.lib, setter, None)
            if f is not None and torch.cuda.is_available():
                f.restype, f.argtypes = ctypes.c_int, [ctypes.c_void_p]
                f(ctypes.c_void_p(_error_word().data_ptr()))
        self._set_pdl = getattr(self.lib, "hos_set_pdl", None)
        if self._set_pdl is not None:
            self._set_pdl.restype, self._set_pdl.argtypes = None, [ctypes.c_int]
            self._set_pdl(1 if _launch_ahead else 0)
        _libraries.append(self)

    def fn(self, name: str, signature: Optional[str] = None):
        f = self._fns.get(name)
        if f is None:
            try:
                f = getattr(self.lib, name)
            except AttributeError as e:
                raise KernelError(f"library {self.name} has no function {name}") from e
            sig = signature or self._signatures[name]
            f.argtypes = [_CT[c] for c in sig]
            f.restype = ctypes.c_int
            self._fns[name] = f
        return f

    def call(self, name: str, *args, signature: Optional[str] = None) -> None:
        global launch_count
        launch_count += 1
        rc = self.fn(name, signature)(*args)
        if rc != 0:
            msg = self._last_error() if self._last_error else b""
            raise KernelError((msg or b"").decode(errors="replace") or f"{name} failed with code {rc}")


_libraries: List["Library"] = []
_launch_ahead = False

_ERROR_WORD_SETTERS = ("hos_gemm_tc_set_error_word", "hos_attn_decode_set_error_word",
                       "hos_attn_prefill_tc_set_error_word")
GIVE_UP_CODES = {1: "the tcgen05 matrix product", 2: "the decode attention", 3: "the tcgen05 prompt attention"}
_error_word_tensor: Optional[torch.Tensor] = None
_after_give_up = []        # callables that put shared scratch state right after a kernel gave up


def _error_word() -> torch.Tensor:
    """One int32 in pinned host memory (the same address on the device): 0, or the code of the
    kernel whose bounded wait ran out last."""
    global _error_word_tensor
    if _error_word_tensor is None:
        _error_word_tensor = torch.zeros(1, dtype=torch.int32).pin_memory()
    return _error_word_tensor


def on_give_up(fn) -> None:
    """Register what has to be put right when a kernel gave up (counters it left behind)."""
    _after_give_up.append(fn)


def check_errors() -> None:
    """Call after a synchronisation, before a step's result is used: raises KernelError if a kernel of
    the steps that are complete by now gave up a bounded wait (its results are then not to be trusted).
    Costs a read of host memory."""
    w = _error_word_tensor
    if w is None:
        return
    code = int(w[0])
    if code == 0:
        return
    w[0] = 0
    for fn in _after_give_up:
        fn()
    raise KernelError(f"{GIVE_UP_CODES.get(code, 'a kernel')} gave up a wait that should have ended (about a second); "
                      f"the results of the steps since the last check are not valid")


_room_left = False


def note_room_left(left: bool) -> None:
    """A launcher's word about the kernel it has just launched: it leaves at least half of the SMs free (the decode
    attention of one sequence does: 64 CTAs).  The launcher of the next kernel may then place that kernel beside it,
    ahead of its end (`take_room_left`); with the SMs full, kernels that wait on them cost more than they hide."""
    global _room_left
    _room_left = bool(left)


def take_room_left() -> bool:
    """What the last launcher said (see note_room_left); the word holds for one launch."""
    global _room_left
    left, _room_left = _room_left, False
    return left


def set_launch_ahead(on: bool) -> None:
    """Whether kernels are launched so that they may be set up while the kernel before them still
    runs (programmatic dependent launch).  It pays for steps of many tokens, whose kernels are
    launched one by one, and costs for single-token steps; the runner switches it per step."""
    global _launch_ahead
    if on == _launch_ahead:
        return
    _launch_ahead = on
    for lib in _libraries:
        if lib._set_pdl is not None:
            lib._set_pdl(1 if on else 0)


_sm_count: Optional[int] = None


def sm_count() -> int:
    """Streaming multiprocessors of the current device (asked once).  Without a device, as the
    host-side choices are also exercised where there is none, the B200's 148."""
    global _sm_count
    if _sm_count is None:
        _sm_count = (torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
                     if torch.cuda.is_available() else 148)
    return _sm_count


_core: Optional[Library] = None
launch_count = 0        # calls into the CUDA libraries so far (each launches one kernel or more)


def core() -> Library:
    global _core
    if _core is None:
        _core = Library("core")
    return _core


def _check(t: torch.Tensor, what: str, dtype=None, dim=None) -> None:
    if not t.is_cuda:
        raise KernelError(f"{what} must be on the GPU")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{what} must be {dtype}, found {t.dtype}")
    if dim is not None and t.dim() != dim:
        raise KernelError(f"{what} must have {dim} dimensions, found {t.dim()}")
    if not t.is_contiguous():
        raise KernelError(f"{what} must be contiguous")


@dataclass
class PagedKVArgs:
    """One call's view of the paged cache, as the kernels take it."""
    k_pages: torch.Tensor        # [n_pages, n_kv_heads, 64, head_dim]
    v_pages: torch.Tensor
    page_table: torch.Tensor     # int32 [n_slots, table_stride]
    ring_pages: int              # 0: all keys kept; > 0: ring of that many pages
    n_kv_heads: int
    head_dim: int

    @property
    def table_stride(self) -> int:
        return self.page_table.shape[1]


# ---- element-wise and norms ------------------------------------------------------------

def embed(tokens: torch.Tensor, table: torch.Tensor, scale: float, out: torch.Tensor) -> None:
    _check(tokens, "tokens", torch.int32, 1)
    _check(table, "embedding table", None, 2)
    _check(out, "embedding output", torch.float32, 2)
    n, d = out.shape
    if tokens.shape[0] != n or table.shape[1] != d:
        raise KernelError("embed: sizes of tokens, table and output disagree")
    core().call("hos_embed", _ptr(tokens), _ptr(table), dtype_code(table.dtype), float(scale),
                _ptr(out), n, d, _stream())


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, add_one: bool, out: torch.Tensor) -> None:
    _check(x, "norm input", None, 2)
    _check(w, "norm weight", torch.float32, 1)
    _check(out, "norm output", None, 2)
    n, d = x.shape
    if out.shape != x.shape or w.shape[0] != d:
        raise KernelError("rmsnorm: sizes of input, weight and output disagree")
    core().call("hos_rmsnorm", _ptr(x), dtype_code(x.dtype), _ptr(w), float(eps), int(add_one),
                _ptr(out), dtype_code(out.dtype), n, d, _stream())


def norm_add_norm(y: torch.Tensor, w_post: torch.Tensor, eps_post: float, add_one_post: bool,
                  x: torch.Tensor, w_next: Optional[torch.Tensor] = None, eps_next: float = 0.0,
                  add_one_next: bool = False, h: Optional[torch.Tensor] = None) -> None:
    """x += RMSNorm(y; w_post); if h is given, h = RMSNorm(x; w_next).  y is [N, D], or
    [parts, N, D] float32 partial sums (of a matrix product that split K), added here."""
    _check(y, "norm input")
    _check(x, "residual stream", torch.float32, 2)
    _check(w_post, "norm weight", torch.float32, 1)
    n_parts = y.shape[0] if y.dim() == 3 else 1
    n, d = x.shape
    if tuple(y.shape[-2:]) != (n, d) or w_post.shape[0] != d or y.dim() not in (2, 3):
        raise KernelError("norm_add_norm: sizes disagree")
    if h is not None:
        _check(h, "next norm output", None, 2)
        _check(w_next, "next norm weight", torch.float32, 1)
        if h.shape != x.shape or w_next.shape[0] != d:
            raise KernelError("norm_add_norm: sizes of the next norm disagree")
    core().call("hos_norm_add_norm", _ptr(y), dtype_code(y.dtype), n_parts, _ptr(w_post), float(eps_post),
                int(add_one_post), _ptr(x), _ptr(w_next), float(eps_next), int(add_one_next),
                _ptr(h), dtype_code(h.dtype) if h is not None else 0, n, d, _stream())


def rope_table(token_pos: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    """float32 [N, len(inv_freq), 2]: (cos, sin) of position * inv_freq, taken in 32-bit."""
    _check(token_pos, "positions", torch.int32, 1)
    _check(inv_freq, "inverse frequencies", torch.float32, 1)
    out = torch.empty((token_pos.shape[0], inv_freq.shape[0], 2), dtype=torch.float32, device=token_pos.device)
    core().call("hos_rope_table", _ptr(token_pos), _ptr(inv_freq), _ptr(out), token_pos.shape[0], inv_freq.shape[0],
                _stream())
    return out


def residual_add(y: torch.Tensor, x: torch.Tensor) -> None:
    _check(y, "branch output")
    _check(x, "residual stream", torch.float32)
    if y.shape != x.shape:
        raise KernelError("residual_add: sizes disagree")
    core().call("hos_residual_add", _ptr(y), dtype_code(y.dtype), _ptr(x), x.numel(), _stream())


def rope_kv_write(qkv: torch.Tensor, n_heads: int, token_pos, token_seq, seq_slot, seq_len_after,
                  inv_freq: Optional[torch.Tensor], rotary_dim: int, style: int,
                  cache: Optional[PagedKVArgs], n_kv_heads: int, head_dim: int,
                  partials: Optional[torch.Tensor] = None) -> None:
    """Rotate the q and k heads of the fused projection rows `qkv` in place; if `cache` is
    given, store the rotated keys and the values at the tokens' places.  With `partials`
    ([parts, N, width] float32 partial sums of the projection) the rows are first formed from
    them and written to `qkv`."""
    _check(qkv, "qkv rows", None, 2)
    n, stride = qkv.shape
    if stride != (n_heads + 2 * n_kv_heads) * head_dim:
        raise KernelError("rope: row width does not match the head counts")
    if inv_freq is None:
        rotary_dim = 0
    else:
        _check(inv_freq, "inverse frequencies", torch.float32, 1)
        if inv_freq.shape[0] * 2 != rotary_dim:
            raise KernelError("rope: one inverse frequency per rotated pair is needed")
    if cache is not None and cache.k_pages.dtype != qkv.dtype:
        raise KernelError("rope: cache and activations differ in dtype")
    src, n_parts = qkv, 1
    if partials is not None:
        _check(partials, "partial sums", torch.float32, 3)
        if tuple(partials.shape[1:]) != (n, stride):
            raise KernelError("rope: partial sums and rows differ in size")
        src, n_parts = partials, partials.shape[0]
    core().call("hos_rope_kv_write", _ptr(src), dtype_code(src.dtype), n_parts, _ptr(qkv), dtype_code(qkv.dtype),
                stride, n_heads,
                _ptr(token_pos), _ptr(token_seq), _ptr(seq_slot), _ptr(seq_len_after),
                _ptr(inv_freq), rotary_dim, style,
                _ptr(cache.k_pages) if cache else None, _ptr(cache.v_pages) if cache else None,
                _ptr(cache.page_table) if cache else None, cache.table_stride if cache else 0,
                cache.ring_pages if cache else 0, n_kv_heads, head_dim, 1 if cache else 0, n,
                _stream())


def gated_act(gu: torch.Tensor, out: torch.Tensor, act: int) -> None:
    _check(gu, "gate|up rows", None, 2)
    _check(out, "activation output", gu.dtype, 2)
    n, f = out.shape
    if gu.shape != (n, 2 * f):
        raise KernelError("gated_act: sizes disagree")
    core().call("hos_gated_act", _ptr(gu), _ptr(out), dtype_code(gu.dtype), n, f, act, _stream())


def gather_rows(x: torch.Tensor, idx: torch.Tensor, out: torch.Tensor) -> None:
    _check(x, "rows", torch.float32, 2)
    _check(idx, "row indices", torch.int32, 1)
    _check(out, "gathered rows", torch.float32, 2)
    if out.shape != (idx.shape[0], x.shape[1]):
        raise KernelError("gather_rows: sizes disagree")
    core().call("hos_gather_rows", _ptr(x), _ptr(idx), _ptr(out), idx.shape[0], x.shape[1], _stream())


# ---- matrix product (plain) --------------------------------------------------------------

def gemm_plain(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int = EPI_NONE,
               cap: float = 0.0, act: int = 0) -> None:
    """out[M, N] = a[M, K] . w[N, K]^T with 32-bit accumulation on the CUDA cores.
    Gated epilogue: w has 2N rows (gate rows, then up rows), out = act(gate) * up."""
    _check(a, "left operand", None, 2)
    _check(w, "weight", None, 2)
    _check(out, "product", None, 2)
    m, k = a.shape
    n = out.shape[1]
    want_rows = 2 * n if epilogue == EPI_GATED else n
    if out.shape[0] != m or w.shape != (want_rows, k):
        raise KernelError(f"gemm: sizes disagree: a {tuple(a.shape)} w {tuple(w.shape)} out {tuple(out.shape)}")
    core().call("hos_gemm_plain", _ptr(a), dtype_code(a.dtype), _ptr(w), dtype_code(w.dtype),
                _ptr(out), dtype_code(out.dtype), m, n, k, k, k, n, epilogue, float(cap), act,
                _stream())


# ---- attention (plain) -------------------------------------------------------------------

def attn_plain(q: torch.Tensor, q_stride: int, out: torch.Tensor, token_pos, token_seq, n_tokens: int,
               n_heads: int, n_kv_heads: int, head_dim: int, scale: float, cap: float,
               window: Optional[int], *, k_rows=None, v_rows=None, kv_stride: int = 0,
               cu_seqlens=None, seq_slot=None, cache: Optional[PagedKVArgs] = None) -> None:
    """Either (k_rows, v_rows, cu_seqlens): keys of this step's own rows, sequences
    from position 0; or (cache, seq_slot): keys from the paged cache."""
    paged = cache is not None
    _check(out, "attention output", q.dtype, 2)
    core().call("hos_attn_plain", dtype_code(q.dtype), int(paged), _ptr(q), q_stride,
                _ptr(k_rows), _ptr(v_rows), kv_stride, _ptr(out), out.shape[1],
                _ptr(token_pos), _ptr(token_seq), _ptr(cu_seqlens), _ptr(seq_slot),
                _ptr(cache.k_pages) if paged else None, _ptr(cache.v_pages) if paged else None,
                _ptr(cache.page_table) if paged else None, cache.table_stride if paged else 0,
                cache.ring_pages if paged else 0, n_tokens, n_heads, n_kv_heads, head_dim,
                float(scale), float(cap), int(window) if window else 0, _stream())


# ---- sampling ----------------------------------------------------------------------------

_argmax_state = {}


def argmax(logits: torch.Tensor, out: torch.Tensor, rep_penalty: float = 1.0,
           recent: Optional[torch.Tensor] = None, recent_len: Optional[torch.Tensor] = None) -> None:
    """out[b] = the first maximum of row b.  With `recent` ([B, n] token ids, recent_len[b] of them
    valid) and a penalty other than 1 the sampler's repetition penalty is applied on the fly."""
    _check(logits, "logits", torch.float32, 2)
    _check(out, "tokens", torch.int32, 1)
    b, v = logits.shape
    stride = 0
    if recent is not None:
        _check(recent, "recent tokens", torch.int32, 2)
        _check(recent_len, "recent counts", torch.int32, 1)
        if recent.shape[0] != b or recent_len.shape[0] != b:
            raise KernelError("argmax: one row of recent tokens per row of logits is needed")
        stride = recent.shape[1]
    lib = core()
    f = lib.lib.hos_argmax_chunks
    f.restype, f.argtypes = ctypes.c_int, [ctypes.c_int]
    chunks = f(v)
    key = (logits.device, b, chunks)
    st = _argmax_state.get(key)
    if st is None:       # partial maxima and ids, and the tickets (zero between launches)
        st = _argmax_state[key] = (torch.empty(2 * b * chunks, dtype=torch.float32, device=logits.device),
                                   torch.zeros(b, dtype=torch.int32, device=logits.device))
    lib.call("hos_argmax", _ptr(logits), v, b, v, _ptr(out), _ptr(st[0]), _ptr(st[1]), _ptr(recent), stride,
             _ptr(recent_len), float(rep_penalty), _stream())


def sample(logits: torch.Tensor, uniforms: torch.Tensor, out: torch.Tensor, temp: float, top_k: int,
           top_p: float, rep_penalty: float = 1.0, recent: Optional[torch.Tensor] = None,
           recent_len: Optional[torch.Tensor] = None) -> None:
    _check(logits, "logits", torch.float32, 2)
    _check(uniforms, "uniform draws", torch.float32, 1)
    _check(out, "tokens", torch.int32, 1)
    b, v = logits.shape
    if recent is not None:
        _check(recent, "recent tokens", torch.int32, 2)
        _check(recent_len, "recent lengths", torch.int32, 1)
    core().call("hos_sample", _ptr(logits), v, b, v, _ptr(uniforms), _ptr(recent),
                recent.shape[1] if recent is not None else 0, _ptr(recent_len), float(temp),
                int(top_k), float(top_p), float(rep_penalty), _ptr(out), _stream())


# ---- the per-slot record (csrc/slot_state.cu) ----------------------------------------------
SLOT_WORDS, RECENT_MAX, MAX_STOPS = 8, 256, 16
SLOT_POS, SLOT_LAST, SLOT_FLAGS, SLOT_COUNT, SLOT_RNG_LO, SLOT_RNG_HI, SLOT_LIMIT = range(7)
BEGIN_ADVANCE, BEGIN_TOKEN_FROM_RECORD, BEGIN_UNIFORM, BEGIN_RECENT, BEGIN_SKIP_FINISHED = 1, 2, 4, 8, 16


def slot_begin(record, ring, slots, meta, b: int, flags: int, tokens, pos, after, seq, cu, uniforms=None,
               recent=None, recent_len=None) -> None:
    """The start of a single-token step of up to b rows (meta[0] of them live): row i belongs to slot
    slots[i]; positions come from the record and move on by one; the input token comes from the
    record (or stays the caller's); for sampling, the next draw of each sequence's generator and its
    recent tokens."""
    core().call("hos_slot_begin", _ptr(record), _ptr(ring), _ptr(slots), _ptr(meta), int(b), int(flags), _ptr(tokens),
                _ptr(pos), _ptr(after), _ptr(seq), _ptr(cu), _ptr(uniforms), _ptr(recent), _ptr(recent_len),
                recent.shape[1] if recent is not None else 0, _stream())


def slot_end(record, ring, slots, meta, b: int, sampled) -> None:
    """After sampling: the tokens go into the records (last token, recent tokens, count, finished)."""
    core().call("hos_slot_end", _ptr(record), _ptr(ring), _ptr(slots), _ptr(meta), int(b), _ptr(sampled), _stream())


def slot_set_pos(record, seq_slot, seq_len_after, cu_seqlens, n_seqs: int) -> None:
    core().call("hos_slot_set_pos", _ptr(record), _ptr(seq_slot), _ptr(seq_len_after), _ptr(cu_seqlens), int(n_seqs),
                _stream())


def slot_write(record, slots, values, word_mask: int) -> None:
    """record[slots[i]][w] = values[i][w] for the words w whose bit is set in word_mask."""
    _check(values, "record values", torch.int32, 2)
    core().call("hos_slot_write", _ptr(record), _ptr(slots), _ptr(values), int(word_mask), values.shape[0], _stream())


def decode_advance(tokens, token_pos, seq_len_after, token_seq, sampled) -> None:
    core().call("hos_decode_advance", _ptr(tokens), _ptr(token_pos), _ptr(seq_len_after), _ptr(token_seq),
                _ptr(sampled), tokens.shape[0], _stream())
