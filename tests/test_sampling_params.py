"""Sampling options and the seeded stream, without a GPU."""
import pytest

from vllm_lite_b200.sampling import SamplingParams, seeded_uniform, splitmix64


def test_defaults_are_the_reference_defaults_and_greedy():
    p = SamplingParams().validate()
    assert (p.temperature, p.top_k, p.top_p, p.repeat_penalty, p.presence_penalty) == (0.0, 0, 1.0, 1.0, 0.0)
    assert p.seed is None and p.logit_bias is None and p.stop_token_sequences is None
    assert not p.needs_penalties
    assert SamplingParams(repeat_penalty=1.1).needs_penalties and SamplingParams(presence_penalty=0.2).needs_penalties
    assert SamplingParams(logit_bias={3: 1.0}).needs_penalties and not SamplingParams(logit_bias={}).needs_penalties


@pytest.mark.parametrize("bad", [dict(temperature=-0.1), dict(temperature=float("nan")), dict(top_k=-1),
                                 dict(top_p=0.0), dict(top_p=1.5), dict(repeat_penalty=0.0)])
def test_options_out_of_range_are_refused(bad):
    with pytest.raises(ValueError):
        SamplingParams(**bad).validate()


def test_splitmix64_is_the_published_bijection():
    # first outputs of the generator of that name started at 0 (state advanced by the golden-ratio increment)
    assert splitmix64(0) == 0xE220A8397B1DCDAF
    assert splitmix64(0x9E3779B97F4A7C15) == 0x6E789E6AA1B965F4
    assert len({splitmix64(i) for i in range(1000)}) == 1000


def test_seeded_stream_is_reproducible_and_spread():
    a = [seeded_uniform(1234, s) for s in range(2000)]
    assert a == [seeded_uniform(1234, s) for s in range(2000)]
    assert a != [seeded_uniform(1235, s) for s in range(2000)]
    assert all(0.0 <= u < 1.0 for u in a)
    assert abs(sum(a) / len(a) - 0.5) < 0.03
    assert min(a) < 0.01 and max(a) > 0.99
    assert seeded_uniform(-1, 5) == seeded_uniform((1 << 64) - 1, 5)      # seeds are taken modulo 2^64
