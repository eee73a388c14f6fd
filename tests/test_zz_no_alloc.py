"""The entry point that allocates nothing, `hos_attn_decode_noalloc` (csrc/attn_decode_noalloc.h).

It is for embedders that may not allocate device memory while a step runs: a serving loop
whose memory all belongs to its own pool, or a plugin inside another framework's memory allowance.
The test calls it through its exported C symbol, as such a caller would, with buffers the
caller owns, twice in a row (the second call finds the first call's partial results in the
library's built-in scratch), and checks each result against a float64 restatement of the
attention and against the ordinary entry point, which takes its workspace from the caller.
It also checks that device memory is not taken and that sizes beyond the built-in scratch or
its counters are refused with a message.

This file is collected last on purpose: a run that stops at the first failure has then run
every other test.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"
HD, NH, NKV = 64, 6, 2


def _load():
    from hos_b200.csrc import build
    lib = ctypes.CDLL(build.library_path(f"attn_hd{HD}"))
    p, i, f = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    lib.hos_attn_decode_noalloc.restype = i
    lib.hos_attn_decode_noalloc.argtypes = [p, i, p, i, p, p, p, p, p, p, i, i, i, i, i, i, f, f, i, i, p]
    lib.hos_last_error.restype = ctypes.c_char_p
    return lib


def _case(seed, lens, window):
    """A paged cache with scattered pages, one query per sequence at its last position."""
    g = torch.Generator().manual_seed(seed)
    n_seq = len(lens)
    ring = (window + 63) // 64 if window else 0
    per = [min((l + 63) // 64, ring) if ring else (l + 63) // 64 for l in lens]
    n_pages = sum(per) + 2
    kp = (torch.randn(n_pages, NKV, 64, HD, generator=g)).to(torch.bfloat16).to(DEV)
    vp = (torch.randn(n_pages, NKV, 64, HD, generator=g)).to(torch.bfloat16).to(DEV)
    order = torch.randperm(n_pages - 1, generator=g) + 1
    table = torch.zeros(n_seq, max(per), dtype=torch.int32)
    k = 0
    for s, n in enumerate(per):
        for e in range(n):
            table[s, e] = int(order[k]); k += 1
    q = torch.randn(n_seq, NH * HD, generator=g).to(torch.bfloat16).to(DEV)
    pos = torch.tensor([l - 1 for l in lens], dtype=torch.int32, device=DEV)
    seq = torch.arange(n_seq, dtype=torch.int32, device=DEV)
    return q, kp, vp, table.to(DEV), ring, pos, seq


def _call_noalloc(lib, q, kp, vp, table, ring, pos, seq, window, n_splits):
    out = torch.full_like(q, 7.0)
    ptr = lambda t: ctypes.c_void_p(t.data_ptr())
    rc = lib.hos_attn_decode_noalloc(ptr(q), q.shape[1], ptr(out), out.shape[1], ptr(pos), ptr(seq), ptr(seq),
                                     ptr(kp), ptr(vp), ptr(table), table.shape[1], ring, q.shape[0], NH, NKV, HD,
                                     1.0 / math.sqrt(HD), 30.0, window or 0, n_splits,
                                     ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    return rc, out


def _reference(q, kp, vp, table, ring, pos, window, cap=30.0):
    """float64 attention of each query over its sequence's pages, read straight from the cache's
    layout (csrc/kv_layout.cuh): position t of sequence s is row t % 64 of page
    table[s, (t // 64) % ring or t // 64], and 16-byte groups of a row are XOR-permuted by (row & 7)."""
    q, kp, vp, table, pos = q.float().cpu(), kp.float().cpu(), vp.float().cpu(), table.cpu(), pos.cpu()
    n = q.shape[0]
    d = torch.arange(HD)
    out = torch.empty(n, NH, HD, dtype=torch.float64)
    for i in range(n):
        p = int(pos[i])
        lo = max(0, p + 1 - window) if window else 0
        t = torch.arange(lo, p + 1)
        lp, row = t // 64, t % 64
        page = table[i, (lp % ring) if ring else lp].long()
        col = (((d[None, :] >> 3) ^ (row[:, None] & 7)) << 3) + (d[None, :] & 7)        # where element d of a row lies
        for h in range(NH):
            kvh = h // (NH // NKV)
            k = kp[page, kvh, row].gather(1, col).double()
            v = vp[page, kvh, row].gather(1, col).double()
            sc = (k @ q[i, h * HD:(h + 1) * HD].double()) / math.sqrt(HD)
            sc = cap * torch.tanh(sc / cap)
            out[i, h] = torch.softmax(sc, 0) @ v
    return out.reshape(n, NH * HD)


def _cluster_merge(lib, on: bool) -> None:
    lib.hos_attn_decode_cluster.restype, lib.hos_attn_decode_cluster.argtypes = ctypes.c_int, [ctypes.c_int]
    lib.hos_attn_decode_cluster(1 if on else 0)


@pytest.mark.parametrize("through_scratch", [True, False])
def test_no_alloc_entry_point_twice_in_a_row_against_a_float64_reference(through_scratch):
    """Two calls in a row with other lengths and another number of shares, so that the second finds
    the first one's partial results and counters in the built-in scratch.  With `through_scratch` the
    cluster merge is switched off, so every share does go through the scratch array and a counter;
    the second case has more work items than the GPU has SMs, which takes that way in any case."""
    from hos_b200.parts import attention_fast as af
    lib = _load()
    _cluster_merge(lib, not through_scratch)
    af._cluster_state.pop(HD, None)                # the library's switch no longer is what the Python face remembers
    try:
        results = []
        cases = [(1, [700, 64, 1, 333], None, 5),
                 (2, [129, 512, 40, 900] + [65 + 7 * i for i in range(36)], 200, 3)]
        for seed, lens, window, n_splits in cases:
            q, kp, vp, table, ring, pos, seq = _case(seed, lens, window)
            want = _reference(q, kp, vp, table, ring, pos, window)
            out_probe = torch.full_like(q, 7.0)            # the output's memory exists before the count is taken
            del out_probe
            torch.cuda.synchronize()
            free_before = torch.cuda.mem_get_info()[0] if results else None      # after the first call's set-up
            rc, got = _call_noalloc(lib, q, kp, vp, table, ring, pos, seq, window, n_splits)
            assert rc == 0, lib.hos_last_error().decode()
            torch.cuda.synchronize()
            if free_before is not None:
                assert torch.cuda.mem_get_info()[0] == free_before                # no device memory was taken
            torch.testing.assert_close(got.float().cpu(), want.to(torch.bfloat16).float(), atol=2e-2, rtol=2e-2)
            assert float(got.float().abs().sum()) > 0
            results.append(got)
            # and the ordinary entry point, which takes its workspace from the caller, agrees
            from hos_b200 import ops
            same = torch.empty_like(q)
            cache = ops.PagedKVArgs(kp, vp, table, ring, NKV, HD)
            af.decode(q, q.shape[1], same, pos, seq, seq, cache, len(lens), NH, 1.0 / math.sqrt(HD), 30.0, window,
                      max(lens), n_splits=n_splits, cluster=not through_scratch)
            torch.testing.assert_close(got.float().cpu(), same.float().cpu(), atol=2e-2, rtol=2e-2)
        assert results[0].shape != results[1].shape
    finally:
        _cluster_merge(lib, True)
        af._cluster_state.pop(HD, None)


def test_no_alloc_entry_point_refuses_what_its_scratch_cannot_hold():
    lib = _load()
    q, kp, vp, table, ring, pos, seq = _case(3, [100], None)
    big = 2200                                    # 2200 tokens x 6 heads x 10 splits x 66 floats > 8 MiB
    qb = q.repeat(big, 1).contiguous()
    posb, seqb = pos.repeat(big), torch.zeros(big, dtype=torch.int32, device=DEV)
    rc, _ = _call_noalloc(lib, qb, kp, vp, table, ring, posb, seqb, None, 10)
    assert rc != 0 and b"built-in scratch holds" in lib.hos_last_error()
    # 2100 tokens x 2 kv heads are more (token, kv head) pairs than the 4096 built-in counters
    rc, _ = _call_noalloc(lib, qb[:2100], kp, vp, table, ring, posb[:2100], seqb[:2100], None, 2)
    assert rc != 0 and b"built-in counters hold" in lib.hos_last_error()
