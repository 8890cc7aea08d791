"""The host's choice of key splits for decode attention (no GPU needed): it is a pure function of the batch's shape."""

import pytest

from ampere_kv_engine_b200.kernels.ops import choose_splits


@pytest.mark.parametrize("batch,keys,expected", [
    (1, 1088, 8), (8, 1088, 8), (12, 1088, 4), (16, 1088, 4), (24, 1088, 2), (32, 1088, 2), (48, 1088, 1),
    (64, 1088, 1), (24, 2048, 2), (12, 4096, 4), (32, 4096, 2), (48, 4096, 4), (64, 4096, 1), (64, 8192, 1),
])
def test_equal_lengths_follow_the_measured_table(batch, keys, expected):
    """For each of these shapes the expected count was the fastest, or within 10 % of it, on a B200."""
    assert choose_splits(batch, 8, 4, keys, True) == expected
    assert choose_splits(batch, 8, 4, keys, True, mean_context=keys) == expected


@pytest.mark.parametrize("batch,longest,mean,expected", [
    (64, 4585, 2506, 2), (40, 4560, 2467, 4), (20, 4569, 2400, 8), (12, 4600, 2272, 8), (64, 1197, 1097, 1),
    (64, 1964, 1160, 2), (64, 7838, 4465, 2),
])
def test_one_long_sequence_among_short_ones_is_split(batch, longest, mean, expected):
    """Mixed lengths: a count chosen for the mean alone leaves the longest sequence to one CTA (batch 64 with 300
    to 4,600 keys, longest first: 171 us unsplit, 110 us in two splits)."""
    assert choose_splits(batch, 8, 4, longest, True, mean_context=mean) == expected


def test_short_contexts_are_not_split_below_two_blocks():
    assert choose_splits(1, 8, 4, 32, True) == 1
    assert choose_splits(1, 8, 4, 64, True) == 1
    assert choose_splits(1, 8, 4, 512, True) == 8
    assert choose_splits(64, 8, 4, 100, True, mean_context=3) == 1


@pytest.mark.parametrize("tensor_core", [False, True])
def test_split_counts_are_ones_the_kernels_take(tensor_core):
    for batch in (1, 3, 8, 17, 64, 200, 512):
        for kv_heads in (1, 2, 8, 16):
            for keys in (1, 17, 100, 1000, 5000, 40000):
                for mean in (None, 1, keys // 3 + 1, keys, 10 * keys):
                    s = choose_splits(batch, kv_heads, 4, keys, tensor_core, mean_context=mean)
                    assert 1 <= s <= 64 and (not tensor_core or s in (1, 2, 4, 8))
