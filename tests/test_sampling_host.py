"""The caller-side sampler against the cases of the reference's own tests (crates/onyxia-cli/src/sampling.rs:186-279)
and against its arithmetic on hand-made draws."""
import numpy as np
import pytest

from onyxia_b200 import sampling
from onyxia_b200.sampling import Rng, SamplingConfig


class FixedRng:
    def __init__(self, *values):
        self.values = list(values)

    def next_u32(self):
        return self.values.pop(0)


def test_sample_greedy_cases():
    assert sampling.sample_greedy(np.array([0.1, 0.5, 0.8, 0.3], np.float32)) == 2
    assert sampling.sample_greedy(np.array([-1.0, -0.1, -0.5], np.float32)) == 1
    assert sampling.sample_greedy(np.array([-10.0, -5.0, -1.0, -20.0], np.float32)) == 2
    assert sampling.sample_greedy(np.array([3.0, 3.0, 1.0], np.float32)) == 1  # the last of equal maxima (Iterator::max_by)


def test_temperature_zero_is_greedy_and_positive_temperature_draws():
    logits = np.array([1.0, 2.0, 3.0], np.float32)
    rng = Rng(42)
    assert sampling.sample(logits, SamplingConfig(temperature=0.0), rng) == 2
    assert sampling.sample(logits, SamplingConfig(temperature=5e-7), rng) == 2
    assert sampling.sample(logits, SamplingConfig(temperature=2.0), rng) <= 2


def test_top_k_keeps_the_k_highest():
    rng = Rng(42)
    for _ in range(50):
        assert sampling.sample_top_k(np.array([0.1, 0.5, 0.8, 0.3, 0.2], np.float32), 2, rng) in (1, 2)
    assert sampling.sample_top_k(np.array([0.1, 0.5], np.float32), 5, FixedRng(0)) == 0  # k ≥ vocabulary: everything stays


def test_top_p_keeps_the_smallest_covering_set():
    rng = Rng(42)
    for _ in range(50):
        assert sampling.sample_top_p(np.array([1.0, 0.5, 0.1, 0.05], np.float32), 0.5, rng) <= 1
    # probabilities ≈ 0.42, 0.26, 0.17, 0.16: p = 0.4 is reached by the first alone, even at the largest random number
    assert sampling.sample_top_p(np.array([1.0, 0.5, 0.1, 0.05], np.float32), 0.4, FixedRng(0xFFFFFFFF)) == 0


def test_same_seed_same_token_and_valid_range():
    logits = np.array([1.0, 2.0, 1.5, 0.5], np.float32)
    cfg = SamplingConfig(temperature=1.0, seed=12345)
    assert [sampling.sample(logits, cfg, Rng(12345)) for _ in range(3)] == [sampling.sample(logits, cfg, Rng(12345)) for _ in range(3)]
    rng = Rng(999)
    assert all(sampling.sample_from_distribution(np.array([0.0, 1.0, 2.0], np.float32), rng) <= 2 for _ in range(100))


def test_the_draw_walks_the_running_sum():
    # e = exp(x − 2) = 0.1353, 0.3679, 1 (sum 1.5032): u·Σ picks the first index whose running sum reaches it
    x = np.array([0.0, 1.0, 2.0], np.float32)
    assert sampling.sample_from_distribution(x, FixedRng(0)) == 0
    assert sampling.sample_from_distribution(x, FixedRng(int(0.08 * 0xFFFFFFFF))) == 0   # 0.12 ≤ 0.1353
    assert sampling.sample_from_distribution(x, FixedRng(int(0.2 * 0xFFFFFFFF))) == 1    # 0.30 ≤ 0.5032
    assert sampling.sample_from_distribution(x, FixedRng(int(0.5 * 0xFFFFFFFF))) == 2
    assert sampling.sample_from_distribution(x, FixedRng(0xFFFFFFFF)) == 2
    # non-finite entries carry no weight
    holes = np.array([-np.inf, 1.0, np.nan, 1.0, -np.inf], np.float32)
    assert sampling.sample_from_distribution(holes, FixedRng(int(0.75 * 0xFFFFFFFF))) == 3
    assert sampling.sample_from_distribution(holes, FixedRng(int(0.25 * 0xFFFFFFFF))) == 1


def test_empty_and_non_finite_logits_are_errors():
    with pytest.raises(ValueError, match="empty"):
        sampling.sample(np.array([], np.float32), SamplingConfig(), Rng(0))
    with pytest.raises(ValueError, match="NaN or Inf"):
        sampling.sample(np.array([np.nan, np.inf], np.float32), SamplingConfig(), Rng(0))


def test_device_sampler_passes_the_configuration_and_the_uniform_number():
    calls = []

    class FakeSession:
        def step_greedy(self, ids):
            calls.append(("greedy", list(ids)))
            return 7

        def step_sampled(self, ids, temperature, top_k, top_p, uniform):
            calls.append(("sampled", list(ids), temperature, top_k, top_p, uniform))
            return 3

    assert sampling.DeviceSampler(FakeSession(), SamplingConfig(temperature=0.0)).step([1, 2]) == 7
    s = sampling.DeviceSampler(FakeSession(), SamplingConfig(temperature=0.8, top_k=40, top_p=0.0, seed=5))
    assert s.step([9]) == 3
    kind, ids, t, k, p, u = calls[-1]
    assert (kind, ids, k, p) == ("sampled", [9], 40, 0.0) and abs(t - 0.8) < 1e-9 and 0.0 <= u <= 1.0
    assert u == Rng(5).uniform()  # the seed of the configuration drives the generator
