"""Host side of sampling: the per-(seed, request, step) uniform is the plain implementation's."""

import pytest

from ampere_kv_engine_b200.sampling.sampler import SamplingParams, uniform_for
from plain import qwen3_plain as plain


def test_uniform_matches_the_plain_generator():
    for seed, stream, step in [(0, 0, 0), (1234, 2, 7), (2 ** 40 + 3, 99, 10 ** 6), (7, 1, 0)]:
        assert uniform_for(seed, stream, step) == plain.uniform_from_key(seed, stream, step)


def test_negative_temperature_is_refused():
    with pytest.raises(ValueError):
        SamplingParams(temperature=-0.1)
