"""The choice of how many shares the decode attention cuts a sequence's keys into
(hos_b200/parts/attention_fast.py: decode_splits): pure arithmetic, checked without a GPU."""
import pytest

from hos_b200.parts import attention_fast as af


@pytest.mark.parametrize("window", [None, 4096, 100])
@pytest.mark.parametrize("n_tokens", [1, 2, 3, 8, 17, 64, 200])
@pytest.mark.parametrize("max_len", [1, 64, 65, 1000, 8192, 100000])
def test_shares_are_within_bounds(n_tokens, max_len, window):
    for fit in (None, lambda s: 0, lambda s: 1000):
        s = af.decode_splits(n_tokens, 4, 2, max_len, window, 0, fit)
        span = min(max_len, window) if window else max_len
        pages = (span + 63) // 64 + (1 if window else 0)
        assert 0 <= s <= af.MAX_SPLITS                # 0: even shares
        assert s <= max(1, (pages + 1) // 2)          # a share holds two pages or more (or there is one share)


def test_one_page_is_never_cut():
    assert af.decode_splits(1, 4, 2, 60, None) == 1
    assert af.decode_splits(64, 1, 8, 64, None) == 1


def test_few_sequences_are_cut_finely_and_many_not_at_all():
    # (in between the choice follows how the items fill waves of 148 CTAs, so it need not fall steadily)
    assert af.decode_splits(1, 4, 2, 8192, None) >= 8
    assert 2 <= af.decode_splits(8, 4, 2, 8192, None) <= 8
    assert af.decode_splits(32, 4, 2, 8192, None) == 1         # 128 items: one wave as they are
    assert af.decode_splits(64, 4, 2, 8192, None) == 1


def test_even_shares_where_equal_ones_leave_a_round_mostly_empty():
    assert af.decode_splits(40, 4, 2, 8192, None) == 0         # 160 items on 148 SMs
    assert af.decode_splits(40, 4, 2, 8192, 4096) == 0
    assert af.decode_splits(56, 4, 2, 8192, None) == 0
    assert af.decode_splits(48, 4, 2, 8192, None, 37, None, 40) == 0       # a bucket of 48 rows, 37 to 40 of them live
    for n in (1, 2, 4, 8, 16, 32):                              # whole rounds (or clusters): nothing to gain
        assert af.decode_splits(n, 4, 2, 8192, None, 0, lambda s: 1000) >= 1
    was = af.enabled["decode_even"]
    af.enabled["decode_even"] = False
    try:
        assert af.decode_splits(40, 4, 2, 8192, None) >= 1
    finally:
        af.enabled["decode_even"] = was
    assert af.decode_splits(af.EVEN_MAX_ROWS + 1, 4, 2, 8192, None) >= 1   # more rows than the kernel's running sums hold


def test_sequences_of_unequal_lengths_argue_for_even_shares():
    """Equal shares take as long as the longest sequence's share whatever the others hold; even shares follow the
    sum of the keys.  `fill`: that sum over (sequences x the longest's keys)."""
    fit = lambda s: 148 // s
    assert af.decode_splits(16, 4, 2, 8192, None, 16, fit, 16, 1.0) >= 1       # sixteen sequences, all long: clusters
    assert af.decode_splits(16, 4, 2, 8192, None, 16, fit, 16, 0.5) == 0       # half as many keys: even shares
    assert af.decode_splits(32, 4, 2, 8192, 4096, 32, fit, 32, 0.25) == 0
    assert af.decode_splits(1, 4, 2, 8192, None, 1, fit, 1, 0.125) >= 1        # one sequence is as long as itself
    assert af.decode_splits(4, 4, 2, 8192, None, 4, fit, 4, 0.5) >= 1          # few sequences: clusters are cheaper
    assert af.decode_splits(16, 8, 2, 2049, None, 16, fit, 16, 0.64) >= 1      # 16 of 64 to 2,049 keys, 8 kv heads: little to gain


def test_how_full_of_keys_a_step_is():
    from hos_b200.engine.decode import fill_class
    from hos_b200.parts.base import StepInfo
    assert fill_class(None, 8, 8192) == 1.0 and fill_class(8 * 8192, 8, 8192) == 1.0
    assert fill_class(16600, 8, 8192) == 0.5 and fill_class(8 * 1000, 8, 8192) == 0.125 and fill_class(5, 8, 8192) == 0.125
    kw = dict(n_tokens=3, n_seqs=3, tokens=None, token_pos=None, token_seq=None, cu_seqlens=None, seq_slot=None,
              seq_len_after=None, from_zero=False, single_token=True, max_new=1, max_len_after=1000)
    step = StepInfo(**kw, cu_host=(0, 1, 2, 3), starts_host=(999, 499, 99))
    assert abs(step.fill_for(None) - 1600 / 3000) < 1e-9                    # from the host's lists, exactly
    assert abs(step.fill_for(200) - 500 / 600) < 1e-9                       # a window of 200 keys: 200 + 200 + 100
    replayed = StepInfo(**kw, replayed=True, fills=((0, 0.5), (200, 0.25)))
    assert replayed.fill_for(None) == 0.5 and replayed.fill_for(200) == 0.25 and replayed.fill_for(64) == 1.0


def test_clusters_that_do_not_fit_change_nothing():
    for n in (1, 2, 4, 8):
        for window in (None, 4096):
            assert af.decode_splits(n, 4, 2, 8192, window, 0, lambda s: 0) == af.decode_splits(n, 4, 2, 8192, window)


def test_a_cluster_is_preferred_only_where_it_fits():
    # one sequence, four kv heads: 4 s CTAs.  With room for every cluster the cheaper merge allows up to 16 shares;
    # with room for clusters of at most 8 CTAs the choice stays at a size that fits or goes back to the workspace.
    roomy = af.decode_splits(1, 4, 2, 8192, None, 0, lambda s: 1000)
    assert 8 <= roomy <= af.CLUSTER_SHARES
    asked = []
    tight = af.decode_splits(1, 4, 2, 8192, None, 0, lambda s: (asked.append(s), 4 if s <= 8 else 0)[1])
    assert asked and max(asked) <= af.CLUSTER_SHARES          # never asks about clusters that cannot exist
    assert tight >= 8


def test_a_replayed_step_weighs_fewer_live_rows_too():
    full = af.decode_splits(12, 4, 2, 8192, None, 0)
    part = af.decode_splits(12, 4, 2, 8192, None, 9)
    assert part >= full                                # fewer live rows never argue for fewer shares


def test_k_splits_of_the_products():
    """How many shares of K the tensor-core product takes (hos_b200/parts/gemm_tc.py: k_splits_for): only
    without an epilogue; few rows (the weights are the M operand) when the output gives few tiles; many
    rows on pairs of SMs when a prompt of some hundred tokens gives fewer tiles than pairs; never
    shares of fewer than a few blocks of K."""
    from hos_b200 import ops
    from hos_b200.parts import gemm_tc
    none, gated = ops.EPI_NONE, ops.EPI_GATED
    assert gemm_tc.k_splits_for(8, 2304, 9216, gated) == 1 and gemm_tc.k_splits_for(600, 2304, 9216, gated) == 1
    assert gemm_tc.k_splits_for(40, 2304, 9216, none) > 1              # 18 tiles of 128 features
    assert gemm_tc.k_splits_for(40, 256000, 2304, none) == 1           # the head: tiles enough
    assert gemm_tc.k_splits_for(100, 2304, 9216, none) == 8            # up to 128 rows: the weights are the M operand, 18 tiles
    assert gemm_tc.k_splits_for(200, 2304, 9216, none) == 8            # from 129 rows on: pairs of SMs, 9 tiles for 74 pairs
    assert gemm_tc.k_splits_for(512, 2304, 9216, none) == 4 and gemm_tc.k_splits_for(512, 2304, 2048, none) == 4
    assert gemm_tc.k_splits_for(1024, 2304, 9216, none) == 2
    assert gemm_tc.k_splits_for(2048, 2304, 9216, none) == 1 and gemm_tc.k_splits_for(8192, 2304, 2048, none) == 1
    assert gemm_tc.k_splits_for(512, 2304, 512, none) == 1             # eight blocks of 64 are one share
    for m in (512, 700, 1024, 1500):
        for n, k in ((2304, 2048), (2304, 9216), (4608, 36864), (3584, 14336)):
            s = gemm_tc.k_splits_for(m, n, k, none)
            tiles = ((m + 255) // 256) * ((n + 255) // 256)
            assert 1 <= s and tiles * s <= 74 or s == 1                 # at most one tile per pair of SMs
            assert s == 1 or (k + 63) // 64 // s >= 8


def test_replayed_steps_are_planned_for_the_class_above_the_longest_sequence():
    from hos_b200.engine.decode import MIN_LENGTH_CLASS, length_class
    assert length_class(None, 8192) == 8192                  # not known: the longest the cache holds
    assert length_class(1, 8192) == MIN_LENGTH_CLASS
    assert length_class(512, 8192) == 512 and length_class(513, 8192) == 768 and length_class(769, 8192) == 1024
    assert length_class(1025, 8192) == 1536 and length_class(2304, 8192) == 3072 and length_class(5000, 8192) == 6144
    assert length_class(6145, 8192) == 8192 and length_class(9000, 8192) == 8192 and length_class(3000, 3500) == 3072
    assert length_class(3100, 3500) == 3500
    # the class never lies below the sequence: a share of the keys is never planned away
    for n in range(1, 9000, 37):
        assert length_class(n, 8192) >= min(n, 8192)
