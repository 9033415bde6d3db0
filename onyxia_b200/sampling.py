"""Token sampling on the caller's side: the interface of ``crates/onyxia-cli/src/sampling.rs`` (``SamplingConfig``,
``sample``, ``sample_greedy``, ``sample_top_k``, ``sample_top_p``) over logits that are already on the host, and
``DeviceSampler``, which draws the same way without moving the logits (``ox_llm_step_sampled``: the caller supplies
only the uniform number).

Arithmetic follows the reference: everything in f32, running sums added one element after the other, the random number
``next_u32() / u32::MAX`` scaled by the sum of the exponentials, the first index whose running sum reaches it. The
reference's generator (``rand::StdRng``) is not restated: any object with ``next_u32()`` serves (``Rng`` wraps
numpy's), so a fixed seed gives a reproducible sequence, though not the reference's own."""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from .llm import sample_greedy

__all__ = ["SamplingConfig", "Rng", "sample", "sample_greedy", "sample_top_k", "sample_top_p", "sample_from_distribution",
           "DeviceSampler"]

_F32 = np.float32
_U32_MAX = _F32(4294967295.0)


@dataclass
class SamplingConfig:
    """sampling.rs:9-30: temperature 0 = greedy; top_k 0 = off; top_p 0 or 1 = off; seed None = entropy."""
    temperature: float = 1.0
    top_k: int = 0
    top_p: float = 0.0
    seed: int | None = None


class Rng:
    """A source of ``next_u32()`` (numpy's PCG64 underneath)."""

    def __init__(self, seed: int | None = None):
        self._g = np.random.default_rng(seed)

    def next_u32(self) -> int:
        return int(self._g.integers(0, 1 << 32, dtype=np.uint64))

    def uniform(self) -> float:
        """The number the samplers scale the sum by: next_u32() / u32::MAX in f32."""
        return float(_F32(self.next_u32()) / _U32_MAX)


def sample_from_distribution(logits, rng) -> int:
    """Softmax and one draw (sampling.rs:156-184): non-finite logits carry no weight; the fallback is the last index."""
    x = np.asarray(logits, _F32)
    finite = np.isfinite(x)
    mx = _F32(np.max(np.where(np.isnan(x), -np.inf, x))) if x.size else _F32(-np.inf)  # f32::max ignores NaN
    with np.errstate(invalid="ignore", over="ignore"):
        e = np.where(finite, np.exp((x - mx).astype(_F32)).astype(_F32), _F32(0)).astype(_F32)
    cum = np.cumsum(e, dtype=_F32)  # one element after the other, in f32
    total = cum[-1] if cum.size else _F32(0)
    rand_val = _F32(_F32(rng.next_u32()) / _U32_MAX) * total
    hit = np.nonzero(cum >= rand_val)[0]
    return int(hit[0]) if hit.size else int(x.size - 1)


def sample_top_k(logits, k: int, rng) -> int:
    """Among the k highest logits (sampling.rs:84-106); the others are masked to −inf. Which of several equal logits at
    the k-th place stay is not specified by the reference's partial sort; here the earlier index stays."""
    x = np.asarray(logits, _F32)
    if k >= x.size:
        return sample_from_distribution(x, rng)
    order = np.argsort(-x, kind="stable")
    filtered = np.full(x.shape, -np.inf, _F32)
    filtered[order[:k]] = x[order[:k]]
    return sample_from_distribution(filtered, rng)


def sample_top_p(logits, p: float, rng) -> int:
    """Within the smallest set of tokens, taken in descending order, whose probability reaches p (sampling.rs:111-152)."""
    x = np.asarray(logits, _F32)
    order = np.argsort(-x, kind="stable")
    s = x[order]
    e = np.exp((s - s[0]).astype(_F32)).astype(_F32)
    total = np.cumsum(e, dtype=_F32)[-1]
    probs = (e / total).astype(_F32)
    cum = np.cumsum(probs, dtype=_F32)
    hit = np.nonzero(cum >= _F32(p))[0]
    cutoff = int(hit[0]) + 1 if hit.size else x.size
    filtered = np.full(x.shape, -np.inf, _F32)
    filtered[order[:cutoff]] = x[order[:cutoff]]
    return sample_from_distribution(filtered, rng)


def sample(logits, config: SamplingConfig, rng) -> int:
    """sampling.rs:36-65: greedy at temperature ≤ 1e-6, else temperature scaling, then top-k, or top-p, or the whole
    distribution. Empty logits or logits without a finite value are an error."""
    x = np.asarray(logits, _F32)
    if x.size == 0:
        raise ValueError("Cannot sample from empty logits")
    if not np.isfinite(x).any():
        raise ValueError("All logits are NaN or Inf, cannot sample")
    if config.temperature <= 0.0 or config.temperature < 1e-6:
        return sample_greedy(x)
    scaled = (x / _F32(config.temperature)).astype(_F32)
    if config.top_k > 0:
        return sample_top_k(scaled, config.top_k, rng)
    if 0.0 < config.top_p < 1.0:
        return sample_top_p(scaled, config.top_p, rng)
    return sample_from_distribution(scaled, rng)


class DeviceSampler:
    """The same draw on the device: one step of a `NativeLlmSession` whose next token is picked by the library's
    sampling kernel from the step's own last-position logits; only the uniform number comes from here."""

    def __init__(self, session, config: SamplingConfig, rng=None):
        self.session, self.config = session, config
        self.rng = rng if rng is not None else Rng(config.seed)

    def step(self, ids) -> int:
        c = self.config
        if c.temperature <= 0.0 or c.temperature < 1e-6:
            return self.session.step_greedy(ids)
        u = self.rng.uniform() if hasattr(self.rng, "uniform") else float(_F32(self.rng.next_u32()) / _U32_MAX)
        return self.session.step_sampled(ids, c.temperature, c.top_k, c.top_p, u)
