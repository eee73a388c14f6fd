"""Each CUDA kernel alone against a plain float32 PyTorch statement of the same operation,
at sizes other than the engine's (widths and vocabularies that are no power of two, odd
head counts, head sizes in steps of 16)."""
import math
import random

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def tol(dtype):
    return dict(atol=1e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)


def close(a, b, dtype, scale=1.0):
    t = tol(dtype)
    torch.testing.assert_close(a.float().cpu(), b.float().cpu(), atol=t["atol"] * scale, rtol=t["rtol"] * scale)


def test_missing_library_fails_loudly(monkeypatch):
    from hos_b200.csrc import build
    from hos_b200.errors import ExtensionMissingError
    with pytest.raises(ExtensionMissingError):
        build.load("no_such_library")


@pytest.mark.parametrize("table_dtype", ["float32", "bfloat16"])
def test_embed(table_dtype):
    from hos_b200 import ops
    V, D = 1003, 200
    table = torch.randn(V, D, device=DEV).to(DT[table_dtype])
    toks = torch.tensor([0, 1002, 7, -1, 500], dtype=torch.int32, device=DEV)
    out = torch.full((5, D), 9.0, device=DEV)
    ops.embed(toks, table, 14.142135, out)
    want = table.float()[toks.clamp(min=0).long()] * torch.tensor(14.142135)
    want[3] = 0
    assert torch.equal(out, want)


@pytest.mark.parametrize("out_dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("D", [1, 80, 1000, 2304, 13000])
def test_rmsnorm(D, out_dtype):
    from hos_b200 import ops
    x = torch.randn(7, D, device=DEV) * 3
    w = torch.randn(D, device=DEV) * 0.1
    out = torch.empty(7, D, device=DEV, dtype=DT[out_dtype])
    ops.rmsnorm(x, w, 1e-6, True, out)
    want = x / torch.sqrt((x * x).mean(-1, keepdim=True) + 1e-6) * (1 + w)
    close(out, want.to(DT[out_dtype]), DT[out_dtype])
    ops.rmsnorm(x, w, 1e-3, False, out)
    want = x / torch.sqrt((x * x).mean(-1, keepdim=True) + 1e-3) * w
    close(out, want.to(DT[out_dtype]), DT[out_dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", [(5, 328), (3, 30), (700, 328), (300, 2304), (257, 72)])
def test_norm_add_norm(dtype, shape):
    """Few rows (a block per row; width 30 is no multiple of 4: the shared-memory kernel) and many
    rows (blocks that walk over rows, 8 columns per thread; 328/8 = 41 threads fill no warp)."""
    from hos_b200 import ops
    dt = DT[dtype]
    N, D = shape
    y = (torch.randn(N, D, device=DEV) * 2).to(dt)
    x0 = torch.randn(N, D, device=DEV)
    w1, w2 = torch.randn(D, device=DEV) * 0.1, torch.randn(D, device=DEV) * 0.1

    def norm(v, w, eps):
        return v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps) * (1 + w)
    x = x0.clone()
    h = torch.empty(N, D, device=DEV, dtype=dt)
    ops.norm_add_norm(y, w1, 1e-6, True, x, w2, 1e-5, True, h)
    want_x = x0 + norm(y.float(), w1, 1e-6)
    close(x, want_x, torch.float32)                       # the residual sum is 32-bit in both paths
    close(h, norm(want_x, w2, 1e-5).to(dt), dt)
    x = x0.clone()
    ops.norm_add_norm(y, w1, 1e-6, True, x)
    close(x, want_x, torch.float32)
    x = x0.clone()
    ops.residual_add(y, x)
    close(x, x0 + y.float(), torch.float32)
    if D % 4 == 0:                                        # 32-bit partial sums of the branch output
        parts = torch.randn(3, N, D, device=DEV)
        x = x0.clone()
        ops.norm_add_norm(parts, w1, 1e-6, True, x, w2, 1e-5, True, h)
        want_x = x0 + norm(parts.sum(0), w1, 1e-6)
        close(x, want_x, torch.float32, scale=2)
        close(h, norm(want_x, w2, 1e-5).to(dt), dt)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("act", ["gelu_tanh", "silu"])
def test_gated_act(dtype, act):
    from hos_b200 import ops
    dt = DT[dtype]
    gu = (torch.randn(6, 2 * 136, device=DEV) * 2).to(dt)
    out = torch.empty(6, 136, device=DEV, dtype=dt)
    ops.gated_act(gu, out, ops.ACTIVATIONS[act])
    g, u = gu.float()[:, :136], gu.float()[:, 136:]
    a = torch.nn.functional.gelu(g, approximate="tanh") if act == "gelu_tanh" else torch.nn.functional.silu(g)
    close(out, (a * u).to(dt), dt)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", [(1, 1, 1), (3, 70, 33), (65, 129, 200), (130, 64, 17), (8, 1003, 96)])
def test_gemm_plain(shape, dtype):
    from hos_b200 import ops
    dt = DT[dtype]
    M, N, K = shape
    a = torch.randn(M, K, device=DEV).to(dt)
    w = (torch.randn(2 * N, K, device=DEV) / math.sqrt(K)).to(dt)
    out = torch.empty(M, N, device=DEV, dtype=dt)
    ops.gemm_plain(a, w[:N].contiguous(), out)
    ref = a.double() @ w[:N].double().T
    close(out, ref.to(dt), dt)
    out32 = torch.empty(M, N, device=DEV)
    ops.gemm_plain(a, w[:N].contiguous(), out32, ops.EPI_SOFTCAP, cap=0.7)
    close(out32, 0.7 * torch.tanh(ref / 0.7), torch.float32)
    ops.gemm_plain(a, w, out, ops.EPI_GATED, act=ops.ACT_GELU_TANH)
    g, u = a.double() @ w[:N].double().T, a.double() @ w[N:].double().T
    close(out, (torch.nn.functional.gelu(g, approximate="tanh") * u).to(dt), dt)


def _fill_cache(k_rows, v_rows, seq_lens, n_kv, hd, ring_pages, dtype, n_slots=4, scatter_seed=0,
                fill=float("nan")):
    """Put per-sequence keys/values [len, n_kv, hd] into a paged cache with scattered pages,
    through the library's own write kernel (rope off)."""
    from hos_b200 import ops
    rng = random.Random(scatter_seed)
    pages_per = [(min(l, ring_pages * 64) if ring_pages else l) for l in seq_lens]
    pages_per = [(p + 63) // 64 for p in pages_per]
    stride = max(pages_per)
    n_pages = sum(pages_per) + 3
    ids = list(range(n_pages))
    rng.shuffle(ids)
    table = torch.zeros(n_slots, stride, dtype=torch.int32)
    slots = rng.sample(range(n_slots), len(seq_lens))
    it = iter(ids)
    for s, npg in zip(slots, pages_per):
        for e in range(npg):
            table[s, e] = next(it)
    kp = torch.full((n_pages, n_kv, 64, hd), fill, device=DEV).to(dtype)
    vp = torch.full((n_pages, n_kv, 64, hd), fill, device=DEV).to(dtype)
    cache = ops.PagedKVArgs(kp, vp, table.to(DEV), ring_pages, n_kv, hd)
    # rows: [q(0 heads) | k | v]
    rows = torch.cat([torch.cat([k.reshape(len(k), -1), v.reshape(len(v), -1)], 1) for k, v in zip(k_rows, v_rows)])
    pos = torch.cat([torch.arange(l) for l in seq_lens]).int().to(DEV)
    seq = torch.cat([torch.full((l,), i) for i, l in enumerate(seq_lens)]).int().to(DEV)
    ops.rope_kv_write(rows.to(dtype).contiguous(), 0, pos, seq, torch.tensor(slots, dtype=torch.int32, device=DEV),
                      torch.tensor(seq_lens, dtype=torch.int32, device=DEV), None, 0, 0, cache, n_kv, hd)
    return cache, slots


def _ref_attention(q, k, v, pos, scale, cap, window):
    """q [nh, hd] at position pos; k, v [len, nkv, hd] -> [nh, hd] (float64)."""
    nh, nkv = q.shape[0], k.shape[1]
    lo = max(0, pos + 1 - window) if window else 0
    out = torch.empty_like(q, dtype=torch.float64)
    for h in range(nh):
        kh, vh = k[lo:pos + 1, h // (nh // nkv)].double(), v[lo:pos + 1, h // (nh // nkv)].double()
        s = (kh @ q[h].double()) * scale
        if cap > 0:
            s = cap * torch.tanh(s / cap)
        out[h] = torch.softmax(s, 0) @ vh
    return out


@pytest.mark.parametrize("cfg", [dict(nh=4, nkv=2, hd=16, window=8, cap=50.0, slack=40),
                                 dict(nh=6, nkv=1, hd=48, window=37, cap=20.0, slack=100),
                                 dict(nh=3, nkv=1, hd=64, window=None, cap=0.0, slack=0),
                                 dict(nh=10, nkv=5, hd=80, window=130, cap=9.0, slack=70),
                                 dict(nh=4, nkv=2, hd=128, window=70, cap=50.0, slack=130),
                                 dict(nh=8, nkv=4, hd=256, window=200, cap=50.0, slack=120),
                                 dict(nh=2, nkv=1, hd=256, window=None, cap=50.0, slack=0)])
def test_attention_chunk_kernel(cfg):
    """Sequences that go on by many tokens, over a scattered paged cache that holds their keys
    already, through the mma.sync kernel and (head sizes 64, 128, 256) the tcgen05 kernel, which takes
    the cache's tiles as they lie: pieces of 1, 64, 65 and 100-odd tokens that begin inside a page, rings that have
    wrapped and are as long as the window plus the piece needs, a key at the window's edge that
    stands out (and the one before it, which must not be seen), rows of other sequences before
    the first piece (the row base)."""
    from hos_b200.parts import attention_fast as af
    dt = torch.bfloat16
    nh, nkv, hd, window, cap, slack = (cfg[k] for k in ("nh", "nkv", "hd", "window", "cap", "slack"))
    torch.manual_seed(4)
    seq_lens = [77, 64, 300, 517, 130]                      # lengths after the step
    news = [1, 64, min(slack, 65) if window else 65, min(slack, 110) if window else 110,
            min(slack, 100) if window else 100]      # a ring has room for `slack` tokens per step
    ks = [torch.randn(l, nkv, hd).to(dt).float() for l in seq_lens]
    vs = [torch.randn(l, nkv, hd).to(dt).float() for l in seq_lens]
    qs = [torch.randn(l, nh, hd).to(dt).float() for l in seq_lens]
    g = nh // nkv
    if window:
        p = 517 - 3                                         # a query of the long sequence's piece
        lo = p + 1 - window
        ks[3][lo] = qs[3][p, 0::g][:nkv] * 3.0
        ks[3][lo - 1] = qs[3][p, 0::g][:nkv] * 6.0
    scale = 0.9 / math.sqrt(hd)
    ring = (window + slack - 1 + 63) // 64 if window else 0
    cache, slots = _fill_cache([k.to(DEV) for k in ks], [v.to(DEV) for v in vs], seq_lens, nkv, hd, ring, dt,
                               n_slots=9, scatter_seed=5, fill=0.0)
    base = 3                                                # rows of other sequences come first
    rows, pos, cu = [torch.zeros(base, nh * hd)], [torch.zeros(base, dtype=torch.int32)], [base]
    for i, (l, n) in enumerate(zip(seq_lens, news)):
        rows.append(qs[i][l - n:].reshape(n, nh * hd))
        pos.append(torch.arange(l - n, l, dtype=torch.int32))
        cu.append(cu[-1] + n)
    q = torch.cat(rows).to(DEV).to(dt).contiguous()
    out = torch.full_like(q, 7.0)
    pos_t = torch.cat(pos).to(DEV)
    seq_slot = torch.tensor([0, 0] + slots, dtype=torch.int32, device=DEV)      # two other sequences before them
    cu_t = torch.tensor(cu, dtype=torch.int32, device=DEV)
    kernels = ["mma.sync"] + (["tcgen05"] if af.has_tc_prefill(hd) else [])
    for kernel in kernels:
        out = torch.full_like(q, 7.0)
        if kernel == "mma.sync":
            af.chunk(q[base:], nh * hd, out[base:], cu_t, base, pos_t[base:], seq_slot[2:], len(news),
                     sum((n + 63) // 64 for n in news) + 2, cache, nh, scale, cap, window)
        else:
            af.chunk_tc(q[base:], out[base:], cu_t, base, pos_t[base:], seq_slot[2:], len(news),
                        sum((n + 127) // 128 for n in news) + 2, cache, nh, scale, cap, window)
            assert not af.prefill_tc_gave_up(hd)
        torch.cuda.synchronize()
        assert float((out[:base] - 7.0).abs().sum()) == 0.0     # rows before the base are not touched
        at = base
        for i, (l, n) in enumerate(zip(seq_lens, news)):
            for j in range(n):
                p = l - n + j
                want = _ref_attention(qs[i][p], ks[i], vs[i], p, scale, cap, window)
                close(out[at + j].reshape(nh, hd), want.to(dt), dt)
            at += n


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("cfg", [dict(nh=4, nkv=2, hd=16, window=None, cap=0.0),
                                 dict(nh=6, nkv=1, hd=48, window=37, cap=20.0),
                                 dict(nh=3, nkv=3, hd=64, window=64, cap=50.0),
                                 dict(nh=8, nkv=4, hd=256, window=100, cap=30.0),
                                 dict(nh=2, nkv=1, hd=128, window=None, cap=50.0)])
def test_attention_plain_over_the_cache_and_over_packed_rows(cfg, dtype):
    """One query per sequence at its last position over a scattered paged cache (with a
    ring for windowed layers, wrapped), and whole prompts over their own packed rows."""
    from hos_b200 import ops
    dt = DT[dtype]
    nh, nkv, hd, window, cap = cfg["nh"], cfg["nkv"], cfg["hd"], cfg["window"], cfg["cap"]
    torch.manual_seed(1)
    seq_lens = [1, 63, 64, 65, 300]
    ks = [torch.randn(l, nkv, hd).to(dt).float() for l in seq_lens]
    vs = [torch.randn(l, nkv, hd).to(dt).float() for l in seq_lens]
    qs = [torch.randn(l, nh, hd).to(dt).float() for l in seq_lens]
    # a far key that matters: in the longest sequence one early key is made to stand out
    far = 300 - (window - 1 if window else 290)
    ks[4][far] = qs[4][299, 0::max(1, nh // nkv)][: nkv] * 3.0
    scale = 1.0 / math.sqrt(hd)
    ring = (window + 63) // 64 if window else 0
    # --- decode: one query per sequence over the cache ---
    cache, slots = _fill_cache([k.to(DEV) for k in ks], [v.to(DEV) for v in vs], seq_lens, nkv, hd, ring, dt,
                               n_slots=7)
    q_last = torch.stack([q[-1] for q in qs]).reshape(len(seq_lens), nh * hd).to(DEV).to(dt).contiguous()
    out = torch.empty_like(q_last)
    pos = torch.tensor([l - 1 for l in seq_lens], dtype=torch.int32, device=DEV)
    seq = torch.arange(len(seq_lens), dtype=torch.int32, device=DEV)
    ops.attn_plain(q_last, nh * hd, out, pos, seq, len(seq_lens), nh, nkv, hd, scale, cap, window,
                   seq_slot=torch.tensor(slots, dtype=torch.int32, device=DEV), cache=cache)
    for i, l in enumerate(seq_lens):
        want = _ref_attention(qs[i][-1], ks[i], vs[i], l - 1, scale, cap, window)
        close(out[i].reshape(nh, hd), want.to(dt), dt)
    # --- prompts: all positions over the step's own rows ---
    rows = torch.cat([torch.cat([q.reshape(len(q), -1), k.reshape(len(k), -1), v.reshape(len(v), -1)], 1)
                      for q, k, v in zip(qs, ks, vs)]).to(DEV).to(dt).contiguous()
    N = rows.shape[0]
    out = torch.empty(N, nh * hd, device=DEV, dtype=dt)
    pos = torch.cat([torch.arange(l) for l in seq_lens]).int().to(DEV)
    seq = torch.cat([torch.full((l,), i) for i, l in enumerate(seq_lens)]).int().to(DEV)
    cu = torch.tensor([0] + list(torch.tensor(seq_lens).cumsum(0)), dtype=torch.int32, device=DEV)
    stride = rows.shape[1]
    ops.attn_plain(rows, stride, out, pos, seq, N, nh, nkv, hd, scale, cap, window,
                   k_rows=rows[:, nh * hd:], v_rows=rows[:, (nh + nkv) * hd:], kv_stride=stride, cu_seqlens=cu)
    base = 0
    for i, l in enumerate(seq_lens):
        for p in sorted({0, min(1, l - 1), l // 2, l - 1}):
            want = _ref_attention(qs[i][p], ks[i], vs[i], p, scale, cap, window)
            close(out[base + p].reshape(nh, hd), want.to(dt), dt)
        base += l


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("style", ["rotate_half", "interleaved"])
@pytest.mark.parametrize("rot", [24, 16, 32])
def test_rope_and_cache_write(dtype, style, rot):
    """Rotation in place and the store into the paged cache, for both pairings, with all and
    with a part of the head rotated (24 of 32 is no multiple of 16: the one-element-at-a-time
    kernel; 16 and 32: the 16-bytes-at-a-time kernel in bfloat16)."""
    from hos_b200 import ops
    dt = DT[dtype]
    nh, nkv, hd, theta = 3, 2, 32, 5000.0
    N = 70
    rows0 = torch.randn(N, (nh + 2 * nkv) * hd, device=DEV).to(dt)
    rows = rows0.clone()
    pos = torch.arange(N, dtype=torch.int32, device=DEV) + 1000
    seq = torch.zeros(N, dtype=torch.int32, device=DEV)
    seq[5] = -1                                              # a padding row: untouched, not stored
    inv = (1.0 / torch.pow(torch.tensor(theta), 2.0 * torch.arange(rot // 2).float() / rot)).to(DEV)
    table = torch.tensor([[9] + [0] * 16, list(range(16, 33))], dtype=torch.int32, device=DEV)
    kp = torch.zeros(40, nkv, 64, hd, device=DEV, dtype=dt)
    vp = torch.zeros_like(kp)
    cache = ops.PagedKVArgs(kp, vp, table, 0, nkv, hd)
    ops.rope_kv_write(rows, nh, pos, seq, torch.tensor([1], dtype=torch.int32, device=DEV),
                      torch.tensor([1000 + N], dtype=torch.int32, device=DEV), inv, rot, ops.ROPE_STYLES[style],
                      cache, nkv, hd)
    x = rows0.float().view(N, nh + 2 * nkv, hd).clone()
    ang = pos.float()[:, None] * inv[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    want = x.clone()
    if style == "rotate_half":
        a, b = x[:, :nh + nkv, :rot // 2], x[:, :nh + nkv, rot // 2:rot]
        want[:, :nh + nkv, :rot // 2], want[:, :nh + nkv, rot // 2:rot] = a * c - b * s, a * s + b * c
    else:
        a, b = x[:, :nh + nkv, 0:rot:2], x[:, :nh + nkv, 1:rot:2]
        want[:, :nh + nkv, 0:rot:2], want[:, :nh + nkv, 1:rot:2] = a * c - b * s, a * s + b * c
    want[5] = x[5]
    close(rows.view(N, -1, hd), want.to(dt), dt)
    # the cache holds the rotated keys and the values at (page of position, row of position)
    for n in (0, 23, 24, 69):
        p = 1000 + n
        page = int(table[1, p // 64])
        got_k = torch.stack([kp[page, :, p % 64, :]])[0]
        assert torch.equal(got_k, rows.view(N, -1, hd)[n, nh:nh + nkv])
        assert torch.equal(vp[page, :, p % 64, :], rows.view(N, -1, hd)[n, nh + nkv:])
    assert float(kp[int(table[1, 1005 // 64]), :, 1005 % 64].abs().sum()) == 0      # the padding row stored nothing


def test_cache_write_skips_ring_positions_that_the_same_step_overwrites():
    from hos_b200 import ops
    nkv, hd, N = 1, 16, 200                                   # ring of 2 pages = 128 positions
    rows = torch.arange(N, device=DEV).float()[:, None].repeat(1, 2 * nkv * hd).contiguous()
    kp = torch.full((4, nkv, 64, hd), -1.0, device=DEV)
    vp = kp.clone()
    table = torch.tensor([[2, 1]], dtype=torch.int32, device=DEV)
    cache = ops.PagedKVArgs(kp, vp, table, 2, nkv, hd)
    pos = torch.arange(N, dtype=torch.int32, device=DEV)
    ops.rope_kv_write(rows, 0, pos, torch.zeros(N, dtype=torch.int32, device=DEV),
                      torch.zeros(1, dtype=torch.int32, device=DEV), torch.tensor([N], dtype=torch.int32, device=DEV),
                      None, 0, 0, cache, nkv, hd)
    for p in range(N - 128, N):                               # the last 128 positions are there
        page = [2, 1][(p // 64) % 2]
        assert float(kp[page, 0, p % 64, 0]) == p
    assert float(kp[0].max()) == -1 and float(kp[3].max()) == -1


def test_argmax_first_maximum_wins():
    from hos_b200 import ops
    V = 256000 + 37
    logits = torch.randn(5, V, device=DEV)
    logits[0, 77] = logits[0, 200000] = 9.0
    logits[1, V - 1] = 9.0
    logits[2, :] = 1.5                                        # all equal: token 0
    logits[3, 0] = 9.0
    out = torch.empty(5, dtype=torch.int32, device=DEV)
    ops.argmax(logits, out)
    assert out.tolist()[:4] == [77, V - 1, 0, 0]
    assert out.tolist()[4] == int(logits[4].argmax())


@pytest.mark.parametrize("rep", [1.5, 0.7])
def test_argmax_with_the_repetition_penalty_on_the_fly(rep):
    """Greedy choice under the sampler's penalty (once per occurrence of a recent token, logits
    untouched): against the plain sampler, with recent tokens that repeat, that hold the maximum,
    that have negative logits, that crowd into one chunk, and ids outside the vocabulary."""
    from plain import gemma2_plain as P
    from hos_b200 import ops
    V, B = 20011, 9
    g = torch.Generator().manual_seed(3)
    logits = torch.randn(B, V, generator=g) * 2.0
    recent = []
    for b in range(B):
        top = [int(t) for t in logits[b].topk(6).indices]
        r = top[:4] + [top[0]] * 2 + [int(x) for x in torch.randint(0, V, (5,), generator=g)]
        if b == 2:
            r = list(range(300, 311))                        # eleven neighbours: one chunk holds them all
            logits[b, 300:311] = 9.0
        recent.append(r[:11])
    want = [_plain_sample_with_u(P, logits[b], dict(temp=0.0, top_k=0, top_p=1.0, rep=rep), recent[b], 0.0)[0]
            for b in range(B)]
    rt = torch.tensor([r + [V + 5] for r in recent], dtype=torch.int32, device=DEV)     # a 12th entry beyond the count
    dl = logits.to(DEV).contiguous()
    keep = dl.clone()
    out = torch.empty(B, dtype=torch.int32, device=DEV)
    ops.argmax(dl, out, rep, rt, torch.full((B,), 11, dtype=torch.int32, device=DEV))
    assert out.tolist() == want
    assert torch.equal(dl, keep)
    if rep > 1:
        assert out.tolist() != [int(t) for t in logits.argmax(-1)]          # the penalty did change choices


@pytest.mark.parametrize("params", [dict(temp=1.0, top_k=0, top_p=1.0, rep=1.0),
                                    dict(temp=0.7, top_k=5, top_p=1.0, rep=1.0),
                                    dict(temp=1.3, top_k=0, top_p=0.8, rep=1.0),
                                    dict(temp=0.9, top_k=50, top_p=0.6, rep=1.4),
                                    dict(temp=0.0, top_k=40, top_p=0.95, rep=1.5),
                                    dict(temp=2.0, top_k=1, top_p=1.0, rep=1.0)])
@pytest.mark.parametrize("kernel", ["cluster", "one_cta"])
def test_sampling_kernel_follows_the_plain_sampler(params, kernel):
    """Same logits, same uniform draw -> the same token as the plain restatement of the
    reference's sampler, ties and repeated 'recent' tokens included.  Temperature sampling from
    a top_k of up to 1024 runs as a cluster of 8 CTAs per row unless that is switched off; both
    kernels go through every case."""
    from plain import gemma2_plain as P
    from hos_b200 import ops
    _use_cluster_sampler(kernel == "cluster")
    V, B = 1003, 24
    g = torch.Generator().manual_seed(11)
    logits = torch.randn(B, V, generator=g) * 2.0
    logits[:, 100:110] = logits[:, 100:101]                  # ten exactly equal logits per row
    logits[3, :] = 0.25                                       # a row where everything ties
    logits[4, 500:520] = 6.0                                  # a tie at the top
    recent = [[int(x) for x in torch.randint(0, V, (6,), generator=g)] + [int(logits[b].argmax())] * 2
              for b in range(B)]
    state = 0x9E3779B97F4A7C15
    us = []
    for b in range(B):
        state, u = P.next_rand(state)
        us.append(u)
    us[5] = 0.0
    want = []
    for b in range(B):
        class Fixed:                                          # make P.sample draw exactly us[b]
            pass
        tok, _ = _plain_sample_with_u(P, logits[b], params, recent[b], us[b])
        want.append(tok)
    dl = logits.to(DEV).contiguous()
    keep = dl.clone()
    out = torch.empty(B, dtype=torch.int32, device=DEV)
    ops.sample(dl, torch.tensor(us, device=DEV), out, params["temp"], params["top_k"], params["top_p"],
               params["rep"], torch.tensor(recent, dtype=torch.int32, device=DEV),
               torch.full((B,), 8, dtype=torch.int32, device=DEV))
    _use_cluster_sampler(True)
    assert out.tolist() == want
    assert torch.equal(dl, keep)                              # the logits are handed back unchanged


def _use_cluster_sampler(on: bool) -> None:
    import ctypes
    from hos_b200 import ops
    f = ops.core().lib.hos_sample_use_cluster
    f.restype, f.argtypes = None, [ctypes.c_int]
    f(1 if on else 0)


def test_cluster_sampler_on_a_large_vocabulary():
    """256,000 logits per row (an eighth of a row per CTA, the vocabulary no multiple of 8 CTAs x 4):
    the cluster kernel and the one-CTA kernel choose the same tokens, with a penalty on recent
    tokens that lie in different CTAs' parts, a tie across the top_k cut, a top_k of 1024, and
    without top_k (the whole row, and its top_p prefix: selection by probability mass)."""
    from hos_b200 import ops
    V, B = 255999, 12
    g = torch.Generator().manual_seed(5)
    logits = (torch.randn(B, V, generator=g) * 3.0).to(DEV)
    logits[1, 70000] = logits[1, 200000] = logits[1, 5] = float(logits[1].topk(40).values[-1])   # ties at the 40th place
    recent = torch.stack([torch.randint(0, V, (8,), generator=g) for _ in range(B)]).to(torch.int32)
    recent[:, 0] = logits.argmax(-1).cpu().to(torch.int32)                  # the best token is penalised
    us = torch.rand(B, generator=g).to(DEV)
    rlen = torch.full((B,), 8, dtype=torch.int32, device=DEV)
    for top_k, top_p, temp, rep in [(40, 0.95, 0.8, 1.1), (1024, 1.0, 1.5, 1.0), (1, 0.5, 0.3, 2.0), (40, 0.2, 1.0, 1.3),
                                    (0, 1.0, 1.0, 1.0), (0, 0.9, 0.7, 1.2), (0, 0.3, 2.0, 1.0)]:
        outs = []
        for cluster in (True, False):
            _use_cluster_sampler(cluster)
            out = torch.empty(B, dtype=torch.int32, device=DEV)
            ops.sample(logits.clone(), us, out, temp, top_k, top_p, rep, recent.to(DEV), rlen)
            outs.append(out.tolist())
        _use_cluster_sampler(True)
        assert outs[0] == outs[1], (top_k, top_p, temp, rep)
        assert all(0 <= t < V for t in outs[0])


def _plain_sample_with_u(P, logits, params, recent, u):
    """P.sample with its generator replaced by a fixed draw u."""
    orig = P.next_rand
    P.next_rand = lambda s: (s, u)
    try:
        return P.sample(logits, params["temp"], params["top_k"], params["top_p"], params["rep"], recent, 1)
    finally:
        P.next_rand = orig


def test_a_wait_that_runs_out_is_reported_to_the_host():
    """The give-up path in its harmless form: one thread waits half a millisecond on a barrier that
    nothing arrives at, gives up and records it exactly as the product kernels do; the kernel ends
    normally.  The host sees it without asking the device (a word in pinned memory), raises, puts
    the shared counters right, and the next launches work."""
    from hos_b200 import ops
    from hos_b200.errors import KernelError
    from hos_b200.parts import attention_fast as af, gemm_tc
    ops.check_errors()                                   # nothing pending
    tickets = af._tickets(torch.device(DEV, torch.cuda.current_device()), 16)
    tickets[3] = 2                                       # as a share that left early would leave it
    gemm_tc.wait_probe()
    torch.cuda.synchronize()
    assert gemm_tc.gave_up()                             # the device flag (reading it clears it)
    assert not gemm_tc.gave_up()
    with pytest.raises(KernelError, match="gave up a wait"):
        ops.check_errors()
    assert int(tickets.abs().sum()) == 0                 # the counters are clean again
    ops.check_errors()                                   # and the word is cleared
    x = torch.randn(70, 64, device=DEV).to(torch.bfloat16)
    w = torch.randn(128, 64, device=DEV).to(torch.bfloat16)
    out = torch.empty(70, 128, device=DEV, dtype=torch.bfloat16)
    gemm_tc.matmul(x, w, out)
    torch.cuda.synchronize()
    ops.check_errors()
    assert not gemm_tc.gave_up()
    close(out, x.float() @ w.float().T, torch.bfloat16)


def test_slot_record_kernels():
    """The per-slot record on the device against a few lines of Python: positions handed out and moved on,
    the input token from the record or from the caller, the xorshift64 draws (the host's `next_rand`), the
    recent tokens in order, also after the ring of 256 has wrapped, the finished flag on a stop id and at the
    limit, finished rows turned into padding, rows beyond the live ones left as padding."""
    from hos_b200 import ops
    from hos_b200.sampling import next_rand
    n_slots, B = 7, 6
    dev = torch.device(DEV)
    record = torch.zeros((n_slots, ops.SLOT_WORDS), dtype=torch.int32, device=dev)
    ring = torch.zeros((n_slots, ops.RECENT_MAX), dtype=torch.int32, device=dev)
    slots = [5, 2, 6, 0]                                        # four live rows of a step of up to six
    seeds = [42, 0x9E3779B97F4A7C15, 7, (1 << 63) + 12345]
    starts = [10, 0, 300, 77]
    vals = torch.zeros((4, ops.SLOT_WORDS), dtype=torch.int32)
    for i in range(4):
        vals[i, ops.SLOT_POS] = starts[i]
        vals[i, ops.SLOT_LAST] = 1000 + i
        lo, hi = seeds[i] & 0xffffffff, seeds[i] >> 32
        vals[i, ops.SLOT_RNG_LO] = lo - (1 << 32) if lo >= 1 << 31 else lo
        vals[i, ops.SLOT_RNG_HI] = hi - (1 << 32) if hi >= 1 << 31 else hi
        vals[i, ops.SLOT_LIMIT] = [0, 3, 0, 0][i]
    slots_t = torch.tensor(slots + [0, 0], dtype=torch.int32, device=dev)
    ops.slot_write(record, slots_t[:4].contiguous(), vals.to(dev), 0xff)
    meta = torch.zeros(2 + ops.MAX_STOPS, dtype=torch.int32, device=dev)
    meta[0], meta[1], meta[2], meta[3] = 4, 2, 555, 777           # live rows; two stop ids
    out = {k: torch.full((B,), -9, dtype=torch.int32, device=dev) for k in ("tokens", "pos", "after", "seq")}
    cu = torch.full((B + 1,), -9, dtype=torch.int32, device=dev)
    uniforms = torch.full((B,), -1.0, device=dev)
    n_rec = 5
    recent = torch.full((B, n_rec), -9, dtype=torch.int32, device=dev)
    recent_len = torch.full((B,), -9, dtype=torch.int32, device=dev)
    flags = (ops.BEGIN_ADVANCE | ops.BEGIN_TOKEN_FROM_RECORD | ops.BEGIN_UNIFORM | ops.BEGIN_RECENT |
             ops.BEGIN_SKIP_FINISHED)
    rng = list(seeds)
    sampled_history = [[] for _ in range(4)]
    finished = [False] * 4
    pos = list(starts)
    last = [1000 + i for i in range(4)]
    for step in range(270):                                      # the ring of 256 wraps
        ops.slot_begin(record, ring, slots_t, meta, B, flags, out["tokens"], out["pos"], out["after"], out["seq"], cu,
                       uniforms, recent, recent_len)
        tk, ps, af_, sq, cu_h, un, rc, rl = (t.cpu() for t in (out["tokens"], out["pos"], out["after"], out["seq"], cu,
                                                               uniforms, recent, recent_len))
        assert cu_h.tolist() == [0, 1, 2, 3, 4, 4, 4]
        assert sq[4:].tolist() == [-1, -1] and tk[4:].tolist() == [-1, -1]          # padding rows
        for i in range(4):
            assert int(ps[i]) == pos[i] and int(af_[i]) == pos[i] + 1 and int(tk[i]) == last[i]
            assert int(sq[i]) == (-1 if finished[i] else i)
            new_state, u = next_rand(rng[i])
            assert abs(float(un[i]) - u) < 1e-9, (step, i)
            h = sampled_history[i][-n_rec:]
            assert int(rl[i]) == len(h) and rc[i, :len(h)].tolist() == h
            if not finished[i]:
                pos[i] += 1
                rng[i] = new_state
        # what the step "samples": stop ids now and then; slot 2 (limit 3) ends after three tokens
        toks = [(step * 7 + i) % 1000 + 2000 for i in range(4)]
        if step == 20:
            toks[0] = 777                                        # a stop id for the first row
        sampled = torch.tensor(toks + [0, 0], dtype=torch.int32, device=dev)
        ops.slot_end(record, ring, slots_t, meta, B, sampled)
        for i in range(4):
            if finished[i]:
                continue
            last[i] = toks[i]
            sampled_history[i].append(toks[i])
            if toks[i] in (555, 777) or (i == 1 and len(sampled_history[i]) >= 3):
                finished[i] = True
    rec = record.cpu()
    assert finished == [True, True, False, False]
    for i, s in enumerate(slots):
        assert int(rec[s, ops.SLOT_POS]) == pos[i] and int(rec[s, ops.SLOT_COUNT]) == len(sampled_history[i])
        assert (int(rec[s, ops.SLOT_FLAGS]) & 1) == int(finished[i]) and int(rec[s, ops.SLOT_LAST]) == last[i]
    assert len(sampled_history[2]) == 270 and pos[0] == starts[0] + 21 and pos[1] == 3
    assert int(rec[1].abs().sum()) == 0 and int(rec[3].abs().sum()) == 0      # slots that took no part are untouched
    # a step of many tokens tells the records the new lengths; sequences that brought nothing are left alone
    seq_slot = torch.tensor([5, 2, 6], dtype=torch.int32, device=dev)
    after = torch.tensor([40, 9, 999], dtype=torch.int32, device=dev)
    cu3 = torch.tensor([0, 30, 30, 31], dtype=torch.int32, device=dev)       # the second one brought no token
    ops.slot_set_pos(record, seq_slot, after, cu3, 3)
    rec = record.cpu()
    assert int(rec[5, ops.SLOT_POS]) == 40 and int(rec[2, ops.SLOT_POS]) == pos[1] and int(rec[6, ops.SLOT_POS]) == 999


def test_gather_rows():
    from hos_b200 import ops
    x = torch.randn(50, 331, device=DEV)
    idx = torch.tensor([49, 0, 7, 7], dtype=torch.int32, device=DEV)
    out = torch.empty(4, 331, device=DEV)
    ops.gather_rows(x, idx, out)
    assert torch.equal(out, x[idx.long()])


@pytest.mark.parametrize("cfg", [dict(nh=4, nkv=2, hd=16, window=8, cap=50.0),
                                 dict(nh=6, nkv=1, hd=32, window=16, cap=20.0),
                                 dict(nh=5, nkv=5, hd=48, window=40, cap=30.0),
                                 dict(nh=3, nkv=1, hd=64, window=None, cap=0.0),
                                 dict(nh=40, nkv=2, hd=80, window=130, cap=9.0),
                                 dict(nh=4, nkv=2, hd=128, window=None, cap=50.0),
                                 dict(nh=8, nkv=4, hd=256, window=200, cap=50.0),
                                 dict(nh=2, nkv=1, hd=256, window=None, cap=50.0)])
@pytest.mark.parametrize("n_splits", [0, 1, 3, 8, 64])      # 0: even shares
def test_attention_decode_kernel(cfg, n_splits):
    """The tensor-core decode kernel over a scattered paged cache: rings that have wrapped,
    a key at the window's edge that stands out, sequences of 1 token and of several pages,
    more splits than pages, 20 heads on one kv head (two MMA tiles), a padding row, and
    several tokens of one sequence in one launch."""
    from hos_b200 import ops
    from hos_b200.parts import attention_fast as af
    dt = torch.bfloat16
    nh, nkv, hd, window, cap = cfg["nh"], cfg["nkv"], cfg["hd"], cfg["window"], cfg["cap"]
    torch.manual_seed(2)
    seq_lens = [1, 64, 65, 130, 517]
    ks = [torch.randn(l, nkv, hd).to(dt).float() for l in seq_lens]
    vs = [torch.randn(l, nkv, hd).to(dt).float() for l in seq_lens]
    qs = [torch.randn(l, nh, hd).to(dt).float() for l in seq_lens]
    g = nh // nkv
    lo = max(0, 517 - window) if window else 0
    ks[4][lo] = qs[4][516, 0::g][:nkv] * 3.0           # the oldest visible key stands out
    if lo > 0:
        ks[4][lo - 1] = qs[4][516, 0::g][:nkv] * 6.0   # and the newest invisible one would even more
    scale = 0.9 / math.sqrt(hd)
    ring = (window + 63) // 64 if window else 0
    cache, slots = _fill_cache([k.to(DEV) for k in ks], [v.to(DEV) for v in vs], seq_lens, nkv, hd, ring, dt,
                               n_slots=9, scatter_seed=3, fill=0.0)
    # queries: the last position of every sequence, a padding row, and three earlier positions
    # of the longest sequence that are still answerable from what the cache holds
    items = [(i, l - 1) for i, l in enumerate(seq_lens)] + [(-1, 0)]
    keep_from = 517 - ring * 64 if ring else 0             # oldest position still stored
    for p in (516 - 1, 516 - 7, 450):
        if (max(0, p + 1 - window) if window else 0) >= keep_from:
            items.append((4, p))
    q = torch.stack([qs[i][p] if i >= 0 else torch.zeros(nh, hd) for i, p in items]).reshape(len(items), nh * hd)
    q = q.to(DEV).to(dt).contiguous()
    out = torch.full_like(q, 7.0)
    pos = torch.tensor([p for _, p in items], dtype=torch.int32, device=DEV)
    seq = torch.tensor([i for i, _ in items], dtype=torch.int32, device=DEV)
    af.decode(q, nh * hd, out, pos, seq, torch.tensor(slots, dtype=torch.int32, device=DEV), cache, len(items),
              nh, scale, cap, window, 517, n_splits=n_splits)
    assert not af.decode_gave_up(hd)
    for j, (i, p) in enumerate(items):
        if i < 0:
            assert float(out[j].abs().sum()) == 0.0
            continue
        want = _ref_attention(qs[i][p], ks[i], vs[i], p, scale, cap, window)
        close(out[j].reshape(nh, hd), want.to(dt), dt)
    # the heuristic's own choice of splits gives the same, and so does fetching ahead of the kernel before
    # (here nothing is being written, so every page may be fetched ahead)
    out2 = torch.empty_like(q)
    af.decode(q, nh * hd, out2, pos, seq, torch.tensor(slots, dtype=torch.int32, device=DEV), cache, len(items),
              nh, scale, cap, window, 517, max_new=1)
    close(out2, out, dt)
    # shares that merge through the workspace and a ticket (what runs when the clusters would not fit at once)
    out3 = torch.empty_like(q)
    af.decode(q, nh * hd, out3, pos, seq, torch.tensor(slots, dtype=torch.int32, device=DEV), cache, len(items),
              nh, scale, cap, window, 517, n_splits=n_splits, cluster=False)
    assert not af.decode_gave_up(hd)
    close(out3, out, dt)


@pytest.mark.parametrize("hd,nh,nkv", [(64, 4, 2), (256, 2, 1)])
def test_attention_decode_even_shares_one_long_sequence_among_short_ones(hd, nh, nkv):
    """Even shares where they are hardest: one sequence of 40,000 keys (625 pages: more than 32 CTAs' fair
    shares, so the CTAs' shares grow until it lies in at most 32 of them) beside sequences of 1 to 3 pages and
    padding rows at the front, in the middle and at the end; one key far back in the long sequence stands out.
    Twice in a row (the counters must be back at zero), against float64."""
    from hos_b200.parts import attention_fast as af
    dt = torch.bfloat16
    torch.manual_seed(8)
    seq_lens = [40000, 3, 70, 129, 64]
    ks = [torch.randn(l, nkv, hd).to(dt).float() for l in seq_lens]
    vs = [torch.randn(l, nkv, hd).to(dt).float() for l in seq_lens]
    qs = [torch.randn(nh, hd).to(dt).float() for _ in seq_lens]
    g = nh // nkv
    ks[0][1234] = qs[0][0::g][:nkv] * 4.0                    # a far key that takes most of the weight
    scale = 1.0 / math.sqrt(hd)
    cache, slots = _fill_cache([k.to(DEV) for k in ks], [v.to(DEV) for v in vs], seq_lens, nkv, hd, 0, dt,
                               n_slots=7, scatter_seed=5, fill=0.0)
    items = [(-1, 0), (0, 39999), (1, 2), (-1, 0), (2, 69), (3, 128), (4, 63), (-1, 0)]
    q = torch.stack([qs[i] if i >= 0 else torch.zeros(nh, hd) for i, _ in items]).reshape(len(items), nh * hd)
    q = q.to(DEV).to(dt).contiguous()
    pos = torch.tensor([p for _, p in items], dtype=torch.int32, device=DEV)
    seq = torch.tensor([i for i, _ in items], dtype=torch.int32, device=DEV)
    slot_t = torch.tensor(slots, dtype=torch.int32, device=DEV)
    for _ in range(2):
        out = torch.full_like(q, 7.0)
        af.decode(q, nh * hd, out, pos, seq, slot_t, cache, len(items), nh, scale, 0.0, None, 40000, n_splits=0)
        assert not af.decode_gave_up(hd)
        for j, (i, p) in enumerate(items):
            if i < 0:
                assert float(out[j].abs().sum()) == 0.0
                continue
            close(out[j].reshape(nh, hd), _ref_attention(qs[i], ks[i], vs[i], p, scale, 0.0, None).to(dt), dt)


@pytest.mark.parametrize("cfg", [dict(nh=4, nkv=2, hd=16, window=8, cap=50.0),
                                 dict(nh=6, nkv=1, hd=32, window=16, cap=20.0),
                                 dict(nh=5, nkv=5, hd=48, window=40, cap=30.0),
                                 dict(nh=3, nkv=1, hd=64, window=None, cap=0.0),
                                 dict(nh=4, nkv=2, hd=128, window=100, cap=50.0),
                                 dict(nh=8, nkv=4, hd=256, window=200, cap=50.0),
                                 dict(nh=2, nkv=2, hd=256, window=None, cap=50.0)])
def test_attention_prefill_kernel(cfg):
    """The tensor-core prompt kernel over packed rows of unequal sequences (1, 63, 64, 65, 130
    and 517 tokens): every position, causal and windowed, against float64."""
    from hos_b200.parts import attention_fast as af
    dt = torch.bfloat16
    nh, nkv, hd, window, cap = cfg["nh"], cfg["nkv"], cfg["hd"], cfg["window"], cfg["cap"]
    torch.manual_seed(3)
    seq_lens = [1, 63, 64, 65, 130, 517]
    ks = [torch.randn(l, nkv, hd).to(dt).float() for l in seq_lens]
    vs = [torch.randn(l, nkv, hd).to(dt).float() for l in seq_lens]
    qs = [torch.randn(l, nh, hd).to(dt).float() for l in seq_lens]
    g = nh // nkv
    if window:
        ks[5][517 - window] = qs[5][516, 0::g][:nkv] * 3.0       # the window's oldest key stands out
        ks[5][517 - window - 1] = qs[5][516, 0::g][:nkv] * 6.0   # just outside: must not be seen
    scale = 0.9 / math.sqrt(hd)
    rows = torch.cat([torch.cat([q.reshape(len(q), -1), k.reshape(len(k), -1), v.reshape(len(v), -1)], 1)
                      for q, k, v in zip(qs, ks, vs)]).to(DEV).to(dt)
    rows = torch.cat([rows, torch.full((5, rows.shape[1]), float("nan"), device=DEV, dtype=dt)]).contiguous()
    N, stride = rows.shape
    cu_host = [0]
    for l in seq_lens:
        cu_host.append(cu_host[-1] + l)
    cu = torch.tensor(cu_host, dtype=torch.int32, device=DEV)
    out = torch.full((N, nh * hd), 7.0, device=DEV, dtype=dt)
    blocks = sum((l + 63) // 64 for l in seq_lens) + 3          # a grid larger than needed: the extra blocks leave at once
    af.prefill(rows, stride, rows[:, nh * hd:], rows[:, (nh + nkv) * hd:], stride, out, cu, len(seq_lens), blocks, nh, nkv, hd,
               scale, cap, window)
    assert float((out[cu_host[-1]:] - 7.0).abs().sum()) == 0.0      # padding rows are not touched
    base = 0
    for i, l in enumerate(seq_lens):
        q, k, v = qs[i].double(), ks[i].double(), vs[i].double()
        pos = torch.arange(l)
        vis = pos[None, :] <= pos[:, None]
        if window:
            vis &= pos[None, :] > pos[:, None] - window
        for h in range(nh):
            s = (q[:, h] @ k[:, h // g].T) * scale
            if cap > 0:
                s = cap * torch.tanh(s / cap)
            want = torch.softmax(s.masked_fill(~vis, float("-inf")), -1) @ v[:, h // g]
            close(out[base:base + l, h * hd:(h + 1) * hd], want.to(dt), dt)
        base += l


@pytest.mark.parametrize("shape", [(128, 256, 64), (200, 300, 136), (257, 520, 2304), (1, 128, 64), (8, 1000, 200),
                                   (16, 512, 72), (17, 264, 640), (33, 2304, 96), (64, 384, 192), (65, 136, 80), (100, 2304, 264), (129, 200, 72),
                                   (512, 256, 64), (700, 520, 136), (1100, 2304, 200), (2048, 1000, 2304),
                                   (600, 1001, 72), (513, 260, 64)])     # rows of a width that no 16-byte store fits
@pytest.mark.parametrize("variant", ["plain_out", "f32_out", "softcap", "gated_gelu", "gated_silu", "split_k"])
def test_gemm_tensor_core(shape, variant):
    """The tcgen05/TMA product against float64, in both orientations (up to 128 rows: the weight
    tile is the 128-row operand and the tokens are 16, 32, 64 or 128 columns; more: pairs of SMs with
    tiles of 256 x 256, cta_group::2), with row and column counts and a K that fill no tile, and
    every epilogue; and against the plain kernel."""
    from hos_b200 import ops
    from hos_b200.parts import gemm_tc
    M, N, K = shape
    torch.manual_seed(5)
    a = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    gated = variant.startswith("gated")
    w = (torch.randn(2 * N if gated else N, K, device=DEV) / math.sqrt(K)).to(torch.bfloat16)
    ref = a.double() @ w[:N].double().T
    if variant == "plain_out":
        out = torch.full((M, N), 7.0, device=DEV, dtype=torch.bfloat16)
        gemm_tc.matmul(a, w, out)
        close(out, ref.to(torch.bfloat16), torch.bfloat16)
        plain = torch.empty_like(out)
        ops.gemm_plain(a, w, plain)
        close(out, plain, torch.bfloat16)
    elif variant == "f32_out":
        out = torch.empty((M, N), device=DEV)
        gemm_tc.matmul(a, w, out)
        close(out, ref, torch.float32, scale=3)
    elif variant == "softcap":
        out = torch.empty((M, N), device=DEV)
        gemm_tc.matmul(a, w, out, ops.EPI_SOFTCAP, cap=0.6)
        close(out, 0.6 * torch.tanh(ref / 0.6), torch.float32, scale=3)
    elif gated:
        act = "gelu_tanh" if variant == "gated_gelu" else "silu"
        out = torch.empty((M, N), device=DEV, dtype=torch.bfloat16)
        gemm_tc.matmul(a, w, out, ops.EPI_GATED, act=ops.ACTIVATIONS[act])
        g, u = ref, a.double() @ w[N:].double().T
        af = torch.nn.functional.gelu(g, approximate="tanh") if act == "gelu_tanh" else torch.nn.functional.silu(g)
        close(out, (af * u).to(torch.bfloat16), torch.bfloat16)
    else:
        if M > 128:
            pytest.skip("K is split in the swapped orientation only")
        for ks in (2, 3, 100):
            out = torch.empty((M, N), device=DEV, dtype=torch.bfloat16)
            gemm_tc.matmul(a, w, out, k_splits=ks)
            close(out, ref.to(torch.bfloat16), torch.bfloat16)
    assert not gemm_tc.gave_up()


@pytest.mark.parametrize("shape", [(129, 136, 80), (200, 300, 136), (700, 520, 136), (1100, 2304, 200)])
@pytest.mark.parametrize("variant", ["plain_out", "f32_out", "softcap", "gated_gelu", "gated_silu"])
def test_gemm_tensor_core_on_single_sms(shape, variant):
    """The kernel that runs when products are kept off the pairs of SMs (HOS_GEMM_PAIR=0): tiles of 128 x 256 on
    one SM each, every epilogue, against float64."""
    from hos_b200 import ops
    from hos_b200.parts import gemm_tc
    M, N, K = shape
    torch.manual_seed(6)
    a = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    gated = variant.startswith("gated")
    w = (torch.randn(2 * N if gated else N, K, device=DEV) / math.sqrt(K)).to(torch.bfloat16)
    ref = a.double() @ w[:N].double().T
    was = gemm_tc.PAIR_MIN_ROWS
    gemm_tc.set_pair_min_rows(0)
    try:
        assert gemm_tc.k_splits_for(M, N, K, ops.EPI_NONE) == 1
        if variant == "plain_out":
            out = torch.full((M, N), 7.0, device=DEV, dtype=torch.bfloat16)
            gemm_tc.matmul(a, w, out)
            close(out, ref.to(torch.bfloat16), torch.bfloat16)
        elif variant == "f32_out":
            out = torch.empty((M, N), device=DEV)
            gemm_tc.matmul(a, w, out)
            close(out, ref, torch.float32, scale=3)
        elif variant == "softcap":
            out = torch.empty((M, N), device=DEV)
            gemm_tc.matmul(a, w, out, ops.EPI_SOFTCAP, cap=0.6)
            close(out, 0.6 * torch.tanh(ref / 0.6), torch.float32, scale=3)
        else:
            act = "gelu_tanh" if variant == "gated_gelu" else "silu"
            out = torch.empty((M, N), device=DEV, dtype=torch.bfloat16)
            gemm_tc.matmul(a, w, out, ops.EPI_GATED, act=ops.ACTIVATIONS[act])
            g, u = ref, a.double() @ w[N:].double().T
            af = torch.nn.functional.gelu(g, approximate="tanh") if act == "gelu_tanh" else torch.nn.functional.silu(g)
            close(out, (af * u).to(torch.bfloat16), torch.bfloat16)
        assert not gemm_tc.gave_up()
    finally:
        gemm_tc.set_pair_min_rows(was if was != gemm_tc.NEVER else 0)


def test_gemm_tensor_core_refuses_what_it_cannot_take():
    from hos_b200 import ops
    from hos_b200.parts import gemm_tc, linear
    a = torch.randn(4, 100, device=DEV).to(torch.bfloat16)          # K = 100 is no multiple of 8
    w = torch.randn(24, 100, device=DEV).to(torch.bfloat16)
    out = torch.empty(4, 24, device=DEV, dtype=torch.bfloat16)
    assert not gemm_tc.can_take(a, w, out, ops.EPI_NONE)
    from hos_b200.errors import KernelError
    with pytest.raises(KernelError, match="multiples of 8"):
        gemm_tc.matmul(a, w, out)
    got = linear.matmul(a, w)                                        # the dispatcher falls back to the plain kernel
    close(got, (a.double() @ w.double().T).to(torch.bfloat16), torch.bfloat16)


def test_consumers_add_partial_sums():
    """What a K-split product leaves ([parts, rows, width] float32) is added by its consumers:
    the norm-and-residual kernel and the rotate-and-store kernel give what they give on the sum."""
    from hos_b200 import ops
    torch.manual_seed(9)
    N, D = 5, 328
    parts = torch.randn(3, N, D, device=DEV)
    total = parts.sum(0)
    x0 = torch.randn(N, D, device=DEV)
    w1, w2 = torch.randn(D, device=DEV) * 0.1, torch.randn(D, device=DEV) * 0.1
    xa, xb = x0.clone(), x0.clone()
    ha = torch.empty(N, D, device=DEV, dtype=torch.bfloat16)
    hb = torch.empty_like(ha)
    ops.norm_add_norm(parts, w1, 1e-6, True, xa, w2, 1e-6, True, ha)
    ops.norm_add_norm(total, w1, 1e-6, True, xb, w2, 1e-6, True, hb)
    close(xa, xb, torch.float32)
    close(ha, hb, torch.bfloat16)
    # rope: rows formed from partial sums, rotated, stored
    nh, nkv, hd = 3, 1, 32
    width = (nh + 2 * nkv) * hd
    parts = torch.randn(4, N, width, device=DEV)
    rows_ref = parts.sum(0).to(torch.bfloat16)
    rows_out = torch.full((N, width), 7.0, device=DEV, dtype=torch.bfloat16)
    pos = torch.arange(N, dtype=torch.int32, device=DEV) + 3
    seq = torch.zeros(N, dtype=torch.int32, device=DEV)
    inv = (1.0 / torch.pow(torch.tensor(100.0), 2.0 * torch.arange(8).float() / 16)).to(DEV)
    slot = torch.zeros(1, dtype=torch.int32, device=DEV)
    after = torch.tensor([3 + N], dtype=torch.int32, device=DEV)
    def cache():
        return ops.PagedKVArgs(torch.zeros(2, nkv, 64, hd, device=DEV, dtype=torch.bfloat16),
                               torch.zeros(2, nkv, 64, hd, device=DEV, dtype=torch.bfloat16),
                               torch.tensor([[1]], dtype=torch.int32, device=DEV), 0, nkv, hd)
    ca, cb = cache(), cache()
    ops.rope_kv_write(rows_out, nh, pos, seq, slot, after, inv, 16, 0, ca, nkv, hd, partials=parts)
    ops.rope_kv_write(rows_ref, nh, pos, seq, slot, after, inv, 16, 0, cb, nkv, hd)
    close(rows_out, rows_ref, torch.bfloat16)
    close(ca.k_pages, cb.k_pages, torch.bfloat16)
    close(ca.v_pages, cb.v_pages, torch.bfloat16)
    assert float(cb.k_pages[1, 0, 3:3 + N].abs().sum()) > 0


@pytest.mark.parametrize("shape", [(1, 16, 32), (3, 40, 72), (8, 2304, 2048), (8, 1000, 200), (9, 136, 264),
                                   (16, 520, 2304), (5, 2304, 9216), (17, 136, 520), (24, 2304, 2048),
                                   (25, 40, 72), (32, 520, 2304)])
@pytest.mark.parametrize("variant", ["bf16_out", "f32_out", "gated_gelu", "gated_silu", "k_split"])
def test_gemm_skinny(shape, variant):
    """The product for up to 32 rows against float64: row counts on both sides of every token
    tile of 8, feature counts and K that fill no tile, both epilogues."""
    from hos_b200 import ops
    from hos_b200.parts import gemm_skinny
    M, N, K = shape
    torch.manual_seed(6)
    a = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    gated = variant.startswith("gated")
    w = (torch.randn(2 * N if gated else N, K, device=DEV) / math.sqrt(K)).to(torch.bfloat16)
    ref = a.double() @ w[:N].double().T
    if variant == "bf16_out":
        out = torch.full((M, N), 7.0, device=DEV, dtype=torch.bfloat16)
        assert gemm_skinny.can_take(a, w, out, ops.EPI_NONE)
        gemm_skinny.matmul(a, w, out)
        close(out, ref.to(torch.bfloat16), torch.bfloat16)
    elif variant == "f32_out":
        out = torch.empty((M, N), device=DEV)
        gemm_skinny.matmul(a, w, out)
        close(out, ref, torch.float32, scale=3)
    elif variant == "k_split":
        # partial sums over shares of K that do not divide it, more shares than k-blocks included
        for splits in (2, 3, 7):
            parts = gemm_skinny.matmul_partials(a, w, k_splits=splits)
            assert parts.shape == (splits, M, N) and parts.dtype == torch.float32
            close(parts.sum(0), ref, torch.float32, scale=3)
        assert gemm_skinny.k_splits_for(2304, 9216) == 2 and gemm_skinny.k_splits_for(2304, 2048) == 1
        assert gemm_skinny.k_splits_for(18432, 2304) == 1
    else:
        act = "gelu_tanh" if variant == "gated_gelu" else "silu"
        out = torch.empty((M, N), device=DEV, dtype=torch.bfloat16)
        gemm_skinny.matmul(a, w, out, ops.EPI_GATED, act=ops.ACTIVATIONS[act])
        g, u = ref, a.double() @ w[N:].double().T
        af = torch.nn.functional.gelu(g, approximate="tanh") if act == "gelu_tanh" else torch.nn.functional.silu(g)
        close(out, (af * u).to(torch.bfloat16), torch.bfloat16)
    big = torch.empty((33, N), device=DEV, dtype=torch.bfloat16)
    assert not gemm_skinny.can_take(torch.zeros(33, K, device=DEV, dtype=torch.bfloat16), w, big, ops.EPI_NONE)


@pytest.mark.parametrize("cfg", [dict(M=1, nh=3, nkv=1, hd=48, rot=48, style="rotate_half", K=72, ring=0),
                                 dict(M=7, nh=2, nkv=2, hd=64, rot=32, style="rotate_half", K=200, ring=2),
                                 dict(M=9, nh=4, nkv=2, hd=64, rot=64, style="interleaved", K=136, ring=0),
                                 dict(M=16, nh=8, nkv=4, hd=256, rot=256, style="rotate_half", K=2304, ring=0),
                                 dict(M=23, nh=2, nkv=1, hd=64, rot=64, style="interleaved", K=72, ring=0),
                                 dict(M=32, nh=4, nkv=2, hd=128, rot=128, style="rotate_half", K=520, ring=2),
                                 dict(M=5, nh=2, nkv=1, hd=32, rot=0, style="rotate_half", K=64, ring=0),
                                 dict(M=4, nh=3, nkv=0, hd=32, rot=16, style="interleaved", K=96, ring=0)])
def test_qkv_projection_with_rotation_and_cache_write_fused(cfg):
    """The one-kernel q/k/v projection of a handful of tokens against a float64 product and
    rotation, and its cache against the separate rotate-and-store kernel given the same rows:
    head sizes that are and are not permuted in the cache, a part of the head rotated, both
    pairings, a ring, padding rows, q heads alone."""
    from types import SimpleNamespace
    from hos_b200 import ops
    from hos_b200.parts import gemm_skinny
    M, nh, nkv, hd, rot, style, K, ring = (cfg[k] for k in ("M", "nh", "nkv", "hd", "rot", "style", "K", "ring"))
    torch.manual_seed(11)
    width = (nh + 2 * nkv) * hd
    x = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    w = (torch.randn(width, K, device=DEV) / math.sqrt(K)).to(torch.bfloat16)
    # tokens of two sequences at far positions; one padding row if there is room
    pos = torch.tensor([700 + 3 * i for i in range(M)], dtype=torch.int32, device=DEV)
    seq = torch.tensor([i % 2 for i in range(M)], dtype=torch.int32, device=DEV)
    if M > 2:
        seq[2] = -1
    slot = torch.tensor([2, 0], dtype=torch.int32, device=DEV)
    # in a ring, sequence 0's tokens are overwritten later in the same step and must not be stored
    len_after = torch.tensor([850 if ring else 760, 760], dtype=torch.int32, device=DEV)
    inv = (1.0 / torch.pow(torch.tensor(5000.0), 2.0 * torch.arange(rot // 2).float() / max(rot, 1))).to(DEV) if rot else None
    n_entries = ring if ring else 16
    table = (torch.randperm(3 * n_entries, device=DEV)[: 3 * n_entries].view(3, n_entries)).to(torch.int32)
    step = SimpleNamespace(token_pos=pos, token_seq=seq, seq_slot=slot, seq_len_after=len_after)

    def caches():
        kp = torch.zeros(3 * n_entries, max(nkv, 1), 64, hd, device=DEV, dtype=torch.bfloat16)
        return ops.PagedKVArgs(kp, torch.zeros_like(kp), table, ring, max(nkv, 1), hd)

    assert gemm_skinny.can_fuse_qkv_rope(x, w, hd, rot)
    out = torch.full((M, width), 7.0, device=DEV, dtype=torch.bfloat16)
    ca = caches()
    gemm_skinny.qkv_rope(x, w, out, nh, nkv, hd, step, inv, rot, ops.ROPE_STYLES[style], ca if nkv else None)
    # float64 product, rotation in float64
    y = (x.double() @ w.double().T).view(M, nh + 2 * nkv, hd)
    want = y.clone()
    if rot:
        ang = pos.double()[:, None] * inv.double()[None, :]
        c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
        if style == "rotate_half":
            a, b = y[:, :nh + nkv, :rot // 2], y[:, :nh + nkv, rot // 2:rot]
            want[:, :nh + nkv, :rot // 2], want[:, :nh + nkv, rot // 2:rot] = a * c - b * s, a * s + b * c
        else:
            a, b = y[:, :nh + nkv, 0:rot:2], y[:, :nh + nkv, 1:rot:2]
            want[:, :nh + nkv, 0:rot:2], want[:, :nh + nkv, 1:rot:2] = a * c - b * s, a * s + b * c
    live = seq >= 0
    close(out.view(M, -1, hd)[live], want.to(torch.bfloat16)[live], torch.bfloat16)
    if nkv:
        # the separate kernel stores the fused kernel's own rows: the caches must be equal bit for bit
        cb = caches()
        rows = out.clone()
        rows[~live] = 0
        ops.rope_kv_write(rows, nh, pos, seq, slot, len_after, None, 0, 0, cb, nkv, hd)   # no rotation: store only
        assert torch.equal(ca.k_pages, cb.k_pages) and torch.equal(ca.v_pages, cb.v_pages)
        assert float(ca.k_pages.abs().sum()) > 0


@pytest.mark.parametrize("cfg", [dict(nh=3, nkv=1, hd=64, K=264, ring=0),
                                 dict(nh=4, nkv=2, hd=128, K=520, ring=3),
                                 dict(nh=2, nkv=1, hd=256, K=136, ring=0),
                                 dict(nh=5, nkv=0, hd=64, K=72, ring=0)])
def test_qkv_projection_of_many_tokens_with_rotation_and_cache_write_fused(cfg):
    """The tensor-core q/k/v projection of 600 tokens that rotates and stores in its epilogue, against a
    float64 product and rotation, and its cache against the separate rotate-and-store kernel given the
    same rows: tiles that hold four, two and one head and a last tile that is partly empty, three
    sequences at far positions, a ring whose oldest tokens must not be stored, padding rows, q heads alone."""
    from types import SimpleNamespace
    from hos_b200 import ops
    from hos_b200.parts import gemm_tc
    nh, nkv, hd, K, ring = (cfg[k] for k in ("nh", "nkv", "hd", "K", "ring"))
    M = 600
    torch.manual_seed(13)
    width = (nh + 2 * nkv) * hd
    x = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    w = (torch.randn(width, K, device=DEV) / math.sqrt(K)).to(torch.bfloat16)
    lens = [250, 200, 140]                      # 590 real rows, 10 padding rows
    starts = [0, 3000, 100]
    pos = torch.cat([torch.arange(s, s + l) for s, l in zip(starts, lens)] + [torch.zeros(10, dtype=torch.long)]).to(torch.int32).to(DEV)
    seq = torch.cat([torch.full((l,), i) for i, l in enumerate(lens)] + [torch.full((10,), -1)]).to(torch.int32).to(DEV)
    slot = torch.tensor([2, 0, 1], dtype=torch.int32, device=DEV)
    len_after = torch.tensor([s + l for s, l in zip(starts, lens)], dtype=torch.int32, device=DEV)
    inv = (1.0 / torch.pow(torch.tensor(5000.0), 2.0 * torch.arange(hd // 2).float() / hd)).to(DEV)
    n_entries = ring if ring else 64
    table = torch.randperm(3 * n_entries, device=DEV).view(3, n_entries).to(torch.int32)
    step = SimpleNamespace(token_pos=pos, token_seq=seq, seq_slot=slot, seq_len_after=len_after)

    def caches():
        kp = torch.zeros(3 * n_entries, max(nkv, 1), 64, hd, device=DEV, dtype=torch.bfloat16)
        return ops.PagedKVArgs(kp, torch.zeros_like(kp), table, ring, max(nkv, 1), hd)

    assert gemm_tc.can_fuse_qkv_rope(x, w, hd, hd, 0, inv)
    out = torch.full((M, width), 7.0, device=DEV, dtype=torch.bfloat16)
    ca = caches()
    gemm_tc.qkv_rope(x, w, out, nh, nkv, hd, step, inv, ca if nkv else None)
    assert not gemm_tc.gave_up()
    y = (x.double() @ w.double().T).view(M, nh + 2 * nkv, hd)
    want = y.clone()
    ang = pos.double()[:, None] * inv.double()[None, :]
    c, sn = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = y[:, :nh + nkv, :hd // 2], y[:, :nh + nkv, hd // 2:]
    want[:, :nh + nkv, :hd // 2], want[:, :nh + nkv, hd // 2:] = a * c - b * sn, a * sn + b * c
    live = seq >= 0
    close(out.view(M, -1, hd)[live], want.to(torch.bfloat16)[live], torch.bfloat16)
    assert bool(torch.isfinite(out.float()).all())            # padding rows hold the plain product
    close(out.view(M, -1, hd)[~live], y.to(torch.bfloat16)[~live], torch.bfloat16)
    if nkv:
        # the separate kernel stores the fused kernel's own rows: the caches must be equal bit for bit
        cb = caches()
        rows = out.clone()
        rows[~live] = 0
        ops.rope_kv_write(rows, nh, pos, seq, slot, len_after, None, 0, 0, cb, nkv, hd)   # no rotation: store only
        assert torch.equal(ca.k_pages, cb.k_pages) and torch.equal(ca.v_pages, cb.v_pages)
        assert float(ca.k_pages.abs().sum()) > 0


@pytest.mark.parametrize("cfg", [dict(nh=3, nkv=1, hd=64, window=None, cap=0.0),
                                 dict(nh=2, nkv=2, hd=64, window=70, cap=30.0),
                                 dict(nh=4, nkv=2, hd=128, window=100, cap=50.0),
                                 dict(nh=8, nkv=4, hd=256, window=200, cap=50.0),
                                 dict(nh=2, nkv=1, hd=256, window=None, cap=50.0),
                                 dict(nh=8, nkv=2, hd=128, window=None, cap=0.0)])
@pytest.mark.parametrize("pairs", [True, False])
def test_attention_prefill_tensor_core_kernel(cfg, pairs):
    """The tcgen05 prompt kernels over packed rows of unequal sequences (1 to 517 tokens; blocks
    of 128 queries that are full, partial, and cut by the window), every position against
    float64.  One logit is made large early in a sequence so that the running maximum has to
    be raised, and O rescaled, in the middle of a walk.  `pairs`: the kernel on pairs of SMs
    (head sizes 128 and 256 with an even number of query heads per kv head) or the one-CTA kernel."""
    from hos_b200.parts import attention_fast as af
    dt = torch.bfloat16
    nh, nkv, hd, window, cap = cfg["nh"], cfg["nkv"], cfg["hd"], cfg["window"], cfg["cap"]
    assert af.has_tc_prefill(hd)
    torch.manual_seed(4)
    seq_lens = [1, 127, 128, 129, 300, 517]
    ks = [torch.randn(l, nkv, hd).to(dt).float() for l in seq_lens]
    vs = [torch.randn(l, nkv, hd).to(dt).float() for l in seq_lens]
    qs = [torch.randn(l, nh, hd).to(dt).float() * 0.5 for l in seq_lens]
    g = nh // nkv
    ks[5][400] = qs[5][516, 0::g][:nkv] * 4.0          # a late key that dwarfs the earlier maxima
    if window:
        ks[5][517 - window] = qs[5][516, 0::g][:nkv] * 3.0
        ks[5][517 - window - 1] = qs[5][516, 0::g][:nkv] * 8.0       # just outside the window: must not be seen
    scale = 0.9 / math.sqrt(hd)
    rows = torch.cat([torch.cat([q.reshape(len(q), -1), k.reshape(len(k), -1), v.reshape(len(v), -1)], 1)
                      for q, k, v in zip(qs, ks, vs)]).to(DEV).to(dt)
    rows = torch.cat([rows, torch.full((5, rows.shape[1]), 1e4, device=DEV, dtype=dt)]).contiguous()   # padding rows
    N = rows.shape[0]
    cu_host = [0]
    for l in seq_lens:
        cu_host.append(cu_host[-1] + l)
    cu = torch.tensor(cu_host, dtype=torch.int32, device=DEV)
    out = torch.full((N, nh * hd), 7.0, device=DEV, dtype=dt)
    blocks = sum((l + 127) // 128 for l in seq_lens) + 2        # a grid larger than needed: the extra blocks leave at once
    af.prefill_tc(rows, out, cu, len(seq_lens), blocks, nh, nkv, hd, scale, cap, window, pairs=pairs)
    assert not af.prefill_tc_gave_up(hd)
    assert float((out[cu_host[-1]:] - 7.0).abs().sum()) == 0.0      # padding rows are not touched
    base = 0
    for i, l in enumerate(seq_lens):
        q, k, v = qs[i].double(), ks[i].double(), vs[i].double()
        pos = torch.arange(l)
        vis = pos[None, :] <= pos[:, None]
        if window:
            vis &= pos[None, :] > pos[:, None] - window
        for h in range(nh):
            s = (q[:, h] @ k[:, h // g].T) * scale
            if cap > 0:
                s = cap * torch.tanh(s / cap)
            want = torch.softmax(s.masked_fill(~vis, float("-inf")), -1) @ v[:, h // g]
            close(out[base:base + l, h * hd:(h + 1) * hd], want.to(dt), dt)
        base += l


@pytest.mark.parametrize("shape", [(600, 264, 1104, 3), (512, 2304, 2048, 4), (1030, 520, 4104, 2)])
def test_product_on_pairs_of_sms_with_k_split(shape):
    """A prompt of some hundred tokens: the product on pairs of SMs with K split over tiles, as 32-bit
    partial sums for a consumer that adds them and reduced in place, against float64 (K that does not
    divide evenly, a last tile of rows and of columns that is partly empty)."""
    from hos_b200 import ops
    from hos_b200.parts import gemm_tc
    M, N, K, splits = shape
    torch.manual_seed(21)
    x = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    w = (torch.randn(N, K, device=DEV) / math.sqrt(K)).to(torch.bfloat16)
    want = x.double() @ w.double().T
    parts = gemm_tc.matmul_partials(x, w, k_splits=splits)
    assert parts is not None and parts.shape[1:] == (M, N) and 2 <= parts.shape[0] <= splits
    close(parts.sum(0), want.float(), torch.float32, scale=100.0)      # bf16 products, 32-bit sums: 1e-3
    out = torch.full((M, N), 7.0, device=DEV, dtype=torch.bfloat16)
    gemm_tc.matmul(x, w, out, k_splits=splits)
    close(out, want.to(torch.bfloat16), torch.bfloat16)
    assert not gemm_tc.gave_up()
    assert gemm_tc.k_splits_for(512, 2304, 9216, ops.EPI_NONE) > 1 and gemm_tc.k_splits_for(2048, 2304, 9216, ops.EPI_NONE) == 1
