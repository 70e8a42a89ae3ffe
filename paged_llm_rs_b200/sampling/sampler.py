"""Choosing the next token (crates/pagedllm/src/sampler.rs).

``SamplingParams`` validates like the reference (sampler.rs:72-95): temperature
finite and not negative, top_k not 0, top_p in (0, 1].  ``Rng`` is its splitmix64
(sampler.rs:23-43), one per request.  ``sample_host`` restates its sampler
(sampler.rs:113-183) with one thing pinned down that the reference leaves open:
equal logits are ordered by token id.  Greedy takes the first maximum and does
not touch the generator (sampler.rs:119-121, 186-194).

On the serving path greedy and plain temperature requests are drawn on the
device by the sampling kernel (one uniform number per row comes from the
request's generator); requests with top-k or top-p take the host sampler.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional, Sequence

import numpy as np

from ..errors import ConfigError

_MASK = (1 << 64) - 1


class Rng:
    def __init__(self, seed: int):
        self.state = int(seed) & _MASK

    def next_u64(self) -> int:
        self.state = (self.state + 0x9E3779B97F4A7C15) & _MASK
        z = self.state
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
        return z ^ (z >> 31)

    def next_f32(self) -> float:
        """A number in [0, 1) from the top 24 bits."""
        return (self.next_u64() >> 40) / 16777216.0


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0
    top_k: Optional[int] = None
    top_p: Optional[float] = None
    # True: a plain temperature request is drawn on the host too, in the reference's order (falling
    # probability, sampler.rs:143-183), so that a seed gives the reference's tokens; the device walks
    # token ids upward: the same distribution, another token for the same uniform number
    reference_order: bool = False

    def __post_init__(self):
        t = self.temperature
        if not isinstance(t, (int, float)) or not math.isfinite(t) or t < 0:
            raise ConfigError(f"temperature {t}, which has to be zero or above")
        if self.top_k is not None and self.top_k <= 0:
            raise ConfigError(f"top_k {self.top_k}, which would leave no token to choose from")
        p = self.top_p
        if p is not None and (not math.isfinite(p) or p <= 0.0 or p > 1.0):
            raise ConfigError(f"top_p {p}, which has to sit in (0, 1]")

    @classmethod
    def greedy(cls) -> "SamplingParams":
        return cls(0.0, None, None)

    @property
    def is_greedy(self) -> bool:
        return self.temperature <= 0.0

    @property
    def on_device(self) -> bool:
        """Greedy and plain temperature are drawn by the kernel."""
        if self.is_greedy:
            return True
        return not self.reference_order and self.top_k is None and (self.top_p is None or self.top_p >= 1.0)


def argmax_first(logits: np.ndarray) -> int:
    return int(np.argmax(logits))  # numpy returns the first maximum


def sample_host(logits: Sequence[float], params: SamplingParams, rng: Rng) -> int:
    logits = np.asarray(logits, dtype=np.float32)
    if logits.size == 0:
        raise ConfigError("cannot sample from an empty logit vector")
    if params.is_greedy:
        return argmax_first(logits)
    scaled = logits * (np.float32(1.0) / np.float32(params.temperature))
    ids = np.arange(scaled.size)
    if params.top_k is not None and params.top_k < scaled.size:
        # the k largest, ties broken by id
        order = np.lexsort((ids, -scaled))[: params.top_k]
    else:
        order = np.lexsort((ids, -scaled))
    vals = scaled[order]
    weights = np.exp(vals - vals[0], dtype=np.float32)
    # sums run in float32 in the order of the candidates, as the reference's loop does
    running = np.cumsum(weights, dtype=np.float32)
    total = running[-1]
    if params.top_p is not None and params.top_p < 1.0:
        target = np.float32(params.top_p) * total
        keep = int(np.searchsorted(running, target, side="left")) + 1  # the crossing token is kept
        keep = min(keep, order.size)
        order, weights = order[:keep], weights[:keep]
        running = np.cumsum(weights, dtype=np.float32)
        total = running[-1]
    point = np.float32(rng.next_f32()) * total
    # walk down the weights until the point is used up
    for i, w in zip(order, weights):
        point = np.float32(point - w)
        if point <= 0.0:
            return int(i)
    return int(order[-1])
