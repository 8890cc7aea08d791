"""The host's choice of key splits for decode attention (no GPU needed): it is a pure function of the batch's shape."""

import pytest

from ampere_kv_engine_b200.kernels.ops import choose_splits


@pytest.mark.parametrize("batch,keys,expected", [
    (1, 1088, 8), (8, 1088, 8), (12, 1088, 4), (16, 1088, 4), (24, 1088, 2), (32, 1088, 2), (48, 1088, 1),
    (64, 1088, 1), (24, 2048, 2), (48, 2048, 4), (24, 4096, 8), (48, 4096, 4), (64, 4096, 1), (64, 8192, 1),
])
def test_tensor_core_decode_splits_follow_the_measured_table(batch, keys, expected):
    assert choose_splits(batch, 8, 4, keys, True) == expected


def test_short_contexts_are_not_split_below_two_blocks():
    assert choose_splits(1, 8, 4, 32, True) == 1
    assert choose_splits(1, 8, 4, 64, True) == 1
    assert choose_splits(1, 8, 4, 128, True) == 2
    assert choose_splits(1, 8, 4, 512, True) == 8


@pytest.mark.parametrize("tensor_core", [False, True])
def test_split_counts_are_ones_the_kernels_take(tensor_core):
    for batch in (1, 3, 8, 17, 64, 200, 512):
        for kv_heads in (1, 2, 8, 16):
            for keys in (1, 17, 100, 1000, 5000, 40000):
                s = choose_splits(batch, kv_heads, 4, keys, tensor_core)
                assert 1 <= s <= 64 and (not tensor_core or s in (1, 2, 4, 8))
