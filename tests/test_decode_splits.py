"""The host-side choice of how many slices a decoded token's context is cut into
(gollmgo_b200/parts/attention.py::decode_splits): a pure function of the batch, the
heads and what the device holds at once.  No GPU."""
import importlib

import pytest

A = importlib.import_module("gollmgo_b200.parts.attention")

# clusters of s slices that a B200 holds at once for head size 128 (measured; index = s)
CAPACITY = [0, 444, 222, 142, 104, 82, 71, 56, 48]
SMS = 148


def splits(n, tiles=32, capacity=CAPACITY, ctas_per_split=8, tile_bytes=32768):
    return A.decode_splits(n, ctas_per_split, SMS, capacity, tiles, tile_bytes)


def test_the_count_stays_within_its_bounds_and_depends_on_nothing_else():
    for n in range(1, 300):
        for tiles in (1, 8, 32, 128, 512):
            s = splits(n, tiles)
            many = tiles >= A.MANY_SLICES_FROM_TILES
            assert 1 <= s <= (A.MAX_SPLITS_MANY if many else A.MAX_SPLITS)
            assert s == splits(n, tiles)                    # same batch and context size, same answer


def test_contexts_are_rounded_up_to_a_power_of_two_of_tiles():
    assert [A.context_tiles(c) for c in (1, 64, 65, 128, 129, 2048, 2049, 10 ** 7)] == [1, 1, 2, 2, 4, 32, 64, A.MAX_TILES]
    assert A.context_tiles(5000, window=100) == 4           # a window bounds what a query reads: 164 keys at most
    assert A.context_tiles(90, window=100) == 2


def test_short_contexts_are_cut_less_and_small_heads_too():
    assert splits(1, 1) == 1 and splits(8, 2) <= 2           # nothing to cut in one or two tiles
    assert splits(1, 4) <= splits(1, 32) <= splits(1, 512)
    assert splits(8, 8) <= splits(8, 32)
    # a head size of 64 halves a tile's bytes: the fixed costs weigh more, never more slices than for 128
    for n in (1, 2, 4, 8, 16):
        assert splits(n, 32, tile_bytes=16384) <= splits(n, 32)


def test_few_sequences_are_cut_into_many_slices_and_many_sequences_are_not():
    assert splits(1) == 8                                   # the largest cluster
    assert splits(8) == 5                                   # 64 clusters of 6 would need every place of 71
    assert splits(1) >= splits(8) >= splits(16) >= splits(48)
    assert splits(48) == 1 and splits(256) == 1


def test_a_single_round_does_not_count_on_the_last_places():
    # 64 pairs: six slices would be 64 clusters of the 71 that fit, more than the share to count on
    assert 64 > CAPACITY[6] * A.CLUSTER_FILL
    assert splits(8) != 6
    # with room to spare six slices are taken
    roomy = list(CAPACITY)
    roomy[6] = 100
    assert splits(8, capacity=roomy) == 6


def test_a_launch_of_several_rounds_fills_every_place():
    # 256 pairs: three slices are 256 clusters in two rounds of 142, not three rounds of 127
    assert splits(32) == 3
    tight = list(CAPACITY)
    tight[3] = 127                                          # then it would be three rounds: whole contexts win
    assert splits(32, capacity=tight) != 3


def test_long_contexts_of_few_sequences_are_cut_beyond_a_cluster():
    for n in range(1, 300):
        if n * 8 * 8 >= A.CTAS_PER_SM * SMS:
            assert splits(n, 256) <= A.MAX_SPLITS            # enough pairs to fill the device: no merge kernel needed
    assert splits(1, 256) > 8 and splits(2, 256) > 8 and splits(4, 256) > 8
    assert splits(1, 256) * 8 <= A.CTAS_PER_SM * SMS        # one round of CTAs
    assert splits(1, 256) >= splits(2, 256) >= splits(4, 256)


def test_without_clusters_the_merge_kernel_is_paid_for():
    none = [0] * 9
    assert splits(1, capacity=none) > 8                     # nothing special about eight any more
    assert splits(55, capacity=none) == 1                   # 440 CTAs: one round of whole contexts
    assert splits(200, capacity=none) == 1


@pytest.mark.parametrize("forced", [1, 3, 11])
def test_a_fixed_count_for_measurements(monkeypatch, forced):
    monkeypatch.setattr(A, "FORCED_SPLITS", forced)
    assert splits(1) == forced and splits(200, 256) == forced
