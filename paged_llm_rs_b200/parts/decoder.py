"""The generic decoder: a ModelSpec built from the part registries.

Runs the schedule entry by entry (crates/pagedllm/src/model/mod.rs:315-352 is
the fixed-order original): embedding, each scheduled layer with the cache the
cache manager made for that entry, then the final norm on the wanted rows only
and the head (mod.rs:340-351).
"""

from __future__ import annotations

from typing import Dict, List, Optional

import torch

from . import attention, block, embedding, feed_forward, norm, position  # noqa: F401  (register the parts)
from .base import (BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITION_ENCODINGS, Runtime, StepState,
                   make)
from .spec import ModelSpec, TensorSpec


class DecoderModel:
    def __init__(self, spec: ModelSpec, rt: Runtime):
        spec.validate()
        self.spec, self.rt = spec, rt
        self.position_encodings = {name: make(POSITION_ENCODINGS, "position encoding", ps, rt)
                                   for name, ps in spec.position_encodings.items()}
        self.embedding = make(EMBEDDINGS, "embedding", spec.embedding, rt)
        self.blocks = []
        for ls in spec.layers:
            mixer = make(MIXERS, "mixer", ls.mixer, rt, position_encodings=self.position_encodings)
            ff = make(FEED_FORWARDS, "feed-forward", ls.feed_forward, rt)
            norms = {k: make(NORMS, "norm", ns, rt) for k, ns in ls.norms.items()}
            if ls.block not in BLOCKS:
                raise KeyError(f"no block arrangement {ls.block!r} is registered; known: {sorted(BLOCKS)}")
            self.blocks.append(BLOCKS[ls.block](mixer, ff, norms))
            self.blocks[-1].prefix = ls.prefix
        self.final_norm = make(NORMS, "norm", spec.final_norm, rt)
        self.head = make(HEADS, "head", spec.head, rt)
        self.schedule = list(spec.schedule)

    def parts(self):
        yield from self.position_encodings.values()
        yield self.embedding
        for b in self.blocks:
            yield b.mixer
            yield b.feed_forward
            yield from b.norms.values()
        yield self.final_norm
        yield self.head

    def tensor_specs(self) -> List[TensorSpec]:
        return [t for p in self.parts() for t in p.tensors()]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        for p in self.parts():
            p.bind(tensors)

    def cache_needs(self) -> List[Optional[object]]:
        """Per schedule entry what its mixer needs of the cache manager; None for
        an entry that reads another entry's cache or needs nothing."""
        return [None if e.reads_cache_of is not None else self.blocks[e.layer].mixer.cache_need()
                for e in self.schedule]

    def capturable(self) -> bool:
        """Whether a step of this model can be captured and replayed: every mixer either launches
        fixed kernels only (``graph_safe``) or sits in a block that can be run in halves around it."""
        return all(getattr(b.mixer, "graph_safe", False) or (b.pre_mixer is not None and b.post_mixer is not None)
                   for b in self.blocks)

    def forward(self, step: StepState, caches: List[object], outside=None) -> torch.Tensor:
        """Run the step's tokens; return float32 logits [step.n_wanted, vocab].  ``outside``
        (for a step that is being captured): called as outside(fn, like) for every mixer that is
        not ``graph_safe``; it runs fn() outside the capture, now and at every replay, and returns
        a tensor shaped like ``like`` that holds fn()'s result each time."""
        residual = self.embedding.forward(step.tokens)
        for encoding in self.position_encodings.values():
            residual = encoding.at_embedding(residual, step)
        delta = None
        for i, e in enumerate(self.schedule):
            own = e.reads_cache_of is None
            blk, cache = self.blocks[e.layer], caches[i if own else e.reads_cache_of]
            if outside is not None and not getattr(blk.mixer, "graph_safe", False):
                h = blk.pre_mixer(residual, delta)
                a = outside(lambda blk=blk, h=h, cache=cache, own=own: blk.mixer.forward(h, step, cache, own), h)
                residual, delta = blk.post_mixer(residual, a, step)
                continue
            residual, delta = blk.forward(residual, delta, step, cache, own)
        if step.n_wanted == 0:
            # A portion in the middle of a prompt runs only to fill the cache (mod.rs:336-346).
            return torch.zeros((0, self.spec.vocab_size), dtype=torch.float32, device=self.rt.device)
        h = self.final_norm.add_norm(residual, delta, rows=step.logit_rows)
        logits = self.head.forward(h)
        self.rt.record("logits", logits)
        return logits


def tensor_specs_of(spec: ModelSpec) -> List[TensorSpec]:
    """The tensors a model of this description reads, without building anything
    on a device (used by the random-weights writer and by weight checks)."""
    return DecoderModel(spec, Runtime(torch.device("cpu"), torch.float32)).tensor_specs()
