"""The model on the device with its cache, and the one step function.

``ModelRunner.step`` is the engine's only forward pass
(crates/pagedllm/src/model/mod.rs:315-352 in the reference): it runs exactly the
tokens it is given, as one batch, from the cache that earlier steps left, writes
their keys and values, and returns the logits at the wanted places.  It does not
advance any length: whoever asked for the step commits it afterwards
(mod.rs:312-314), so a failed step leaves the bookkeeping untouched.
Generation, the scheduler and trace replay all go through it.
"""

from __future__ import annotations

import gc
import os
from typing import List, Optional, Sequence

import numpy as np
import torch

from .. import models  # noqa: F401  (registers the architectures)
from ..cache.manager import CacheManager
from ..config.registry import load_config
from ..errors import ConfigError, KernelError
from ..kernels import attention_plan, ops
from ..parts.base import PagedNeed, Runtime
from ..parts.decoder import DecoderModel
from ..weights.loader import load_weights
from .step import GroupPlanConfig, NativeDecodePacker, StepCaps, StepEntry, StepPacker

DTYPES = {"float32": torch.float32, "f32": torch.float32, "fp32": torch.float32,
          "bfloat16": torch.bfloat16, "bf16": torch.bfloat16}


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name not in (torch.float32, torch.bfloat16):
            raise ConfigError(f"dtype {name} is not served; float32 and bfloat16 are")
        return name
    try:
        return DTYPES[str(name).lower()]
    except KeyError:
        raise ConfigError(f"dtype {name!r} is not served; float32 and bfloat16 are") from None


class _DecodeGraph:
    """One captured step.  The decode form: up to ``B`` requests, one token each, block
    tables at most ``W`` pages wide.  The general form (``segments`` given): up to ``B``
    tokens in up to ``segments`` requests, portions of prompts beside decoded tokens.
    Every launch argument is fixed: the step's data (token ids, positions, slots,
    tables, work items, sampling numbers) lives in one device buffer that each replay
    overwrites; what does not fill the capacities is padding that writes nothing
    (slot -1) and attends to nothing (no work item)."""

    def __init__(self, runner: "ModelRunner", B: int, W: int, segments: Optional[int] = None):
        self.runner, self.B, self.W = runner, B, W
        pk = runner.packer
        self.decode = segments is None
        n_seg = B if self.decode else segments
        self.caps = StepCaps(tokens=B, wanted=n_seg, segments=n_seg, table_width=W, kinds=1 if self.decode else 3)
        self.work_caps = [None if p is None else attention_plan.plan_limits(B, p.tile_tokens, pk.target_ctas, p.ctas_per_item, n_seg)
                          for p in pk.plans]
        host, self.layout, self.sizes = pk.pack([], self.caps, self.work_caps)
        self.pinned = torch.from_numpy(host.copy()).pin_memory()
        self.native = NativeDecodePacker(pk, self.caps, self.work_caps, self.layout, self.pinned.numpy()) if self.decode else None
        self.dev = self.pinned.to(runner.device)
        self.nbytes = host.nbytes
        self.state = pk.to_state(self.dev, self.layout, self.sizes, full=True)
        self.tokens = torch.zeros(1 + n_seg, dtype=torch.int32, device=runner.device)
        # the status word and the chosen tokens come back by a copy that is part of the captured step
        self.tokens_host = torch.zeros(1 + n_seg, dtype=torch.int32).pin_memory()
        self.staging = None     # host buffer of a step packed ahead of time (prepack)
        # The decode form's pinned buffer is read by the replay's first node.  A caller that replays this
        # step again without having waited for the replay before it (the engine waits: it needs the
        # tokens) must not overwrite the buffer under a replay that has not started yet: an event marks
        # each replay's end and is waited for (on the host) before the buffer is written again.
        # The general form is copied in by a copy of its own before the replay, from two pinned buffers
        # in turn, each guarded by an event behind its copy: the next step can be packed while this one
        # runs (a 2048-token step takes 0.3 ms to pack and 3.4 ms to run).
        self._replayed = torch.cuda.Event()
        self._pending = False
        self._pinned = [self.pinned] if self.decode else [self.pinned, torch.from_numpy(host.copy()).pin_memory()]
        self._copied = [torch.cuda.Event() for _ in self._pinned]
        self._copy_pending = [False for _ in self._pinned]
        self._turn = 0
        # Warm up on a side stream (library handles, workspaces), then capture.
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side), torch.no_grad():
            for _ in range(2):
                self._body()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        before = ops.LAUNCHES
        # The step is one captured graph, or, where mixers are not ``graph_safe``, graphs with those
        # mixers between them: ("graph", CUDAGraph) and ("eager", fn, buffer) in the order they run.
        self.pieces = []
        self._ctx = None
        piecewise = not all(getattr(b.mixer, "graph_safe", False) for b in runner.model.blocks)
        # The collector must not run inside the capture: freeing an older engine's graphs
        # there (they die in reference cycles, at a time of the collector's choosing) is a
        # call the capture forbids, and the capture would be invalidated.
        gc.collect()
        collecting = gc.isenabled()
        gc.disable()
        try:
            with torch.no_grad():
                self._begin_piece()
                self._body(self._outside if piecewise else None)
                self._end_piece()
        finally:
            if collecting:
                gc.enable()
        self.graph = self.pieces[0][1] if len(self.pieces) == 1 else None     # (the whole step, when it is one graph)
        self.launches = ops.LAUNCHES - before

    def _begin_piece(self):
        # one memory pool for all of this runner's captured steps: they never run at the same time, so
        # the activations of one may lie where another's did (a 2048-token step holds some 150 MB)
        g = torch.cuda.CUDAGraph()
        self._ctx = torch.cuda.graph(g, pool=self.runner.graph_pool)
        self._ctx.__enter__()
        self.pieces.append(("graph", g))

    def _end_piece(self):
        self._ctx.__exit__(None, None, None)
        self._ctx = None

    def _outside(self, fn, like):
        """A mixer that cannot be captured: the capture ends before it and begins again behind it; the
        mixer reads what the graph before it left (fixed addresses) and its result is copied into a
        fixed buffer that the graph behind it reads."""
        self._end_piece()
        buf = torch.empty_like(like)
        buf.copy_(fn())
        self.pieces.append(("eager", fn, buf))
        self._begin_piece()
        return buf

    def replay(self):
        if self.graph is not None:
            self.graph.replay()
            return
        with torch.no_grad():
            for piece in self.pieces:
                if piece[0] == "graph":
                    piece[1].replay()
                else:
                    piece[2].copy_(piece[1]())

    def _body(self, outside=None):
        r = self.runner
        if self.decode:
            self.dev.copy_(self.pinned, non_blocking=True)  # the step's packed buffer: the graph's first node
        self.logits = r.model.forward(self.state, r.caches, outside)
        ops.sample(self.logits, self.state.temperature, self.state.uniform, self.tokens[1:])
        self.tokens[:1].copy_(r.rt.status)
        self.tokens_host.copy_(self.tokens, non_blocking=True)

    def _segments_of(self, entries, ahead=0):
        """(first token, tokens, tokens in the cache before, state slot) of every request of the step: what
        mixers that loop over the step on the host read (the captured pieces read the packed buffer)."""
        cache, segs, t0 = self.runner.cache, [], 0
        for e in entries:
            rc = cache.get(e.request_id)
            segs.append((t0, len(e.tokens), rc.tokens + ahead, rc.state_slot))
            t0 += len(e.tokens)
        return segs

    # -- a decode step packed ahead of time (while the step before it runs) ---------------------------
    def prepack(self, entries, temperature) -> None:
        """Fill a host buffer of the step's layout for requests that each stand one token further than
        their committed count; token ids and the sampling's uniform numbers come at launch."""
        if self.staging is None:
            self.pinned_np = self.pinned.numpy()
            self.staging = np.zeros_like(self.pinned_np)
        self.native.pack(entries, temperature, np.zeros(len(entries), dtype=np.float32) if temperature is not None else None,
                         ahead=1, out=self.staging)
        self._staged_segments = self._segments_of(entries, ahead=1) if self.graph is None else None

    def launch_prepacked(self, tokens, uniform):
        """Put the token ids (and uniform numbers) into the buffer ``prepack`` filled, and replay."""
        r = self.runner
        n = len(tokens)
        o = self.layout["tokens"][0]
        self.staging[o:o + n] = tokens
        if uniform is not None:
            o = self.layout["uniform"][0]
            self.staging[o:o + n] = np.asarray(uniform, dtype=np.float32).view(np.int32)
        self._before_write()
        np.copyto(self.pinned_np, self.staging)
        if self.graph is None:
            self.state.host_segments = self._staged_segments
        self._replay()
        r.bytes_h2d = self.nbytes
        r.last_launches = self.launches
        r.tokens_host = self.tokens_host[:1 + n]
        return self.logits[:n], self.tokens[:1 + n]

    def _before_write(self):
        if self._pending:
            self._replayed.synchronize()
            self._pending = False

    def _replay(self):
        self.replay()
        self._replayed.record()
        self._pending = True

    def run(self, entries, temperature, uniform):
        r = self.runner
        if self.graph is None:
            self.state.host_segments = self._segments_of(entries)
        if self.decode:
            self._before_write()
            if self.native is not None:
                self.native.pack(entries, temperature, uniform)     # straight into the pinned buffer
            else:
                host, _, _ = r.packer.pack(entries, self.caps, self.work_caps, temperature, uniform)
                self.pinned.numpy()[:] = host
            self._replay()
        else:
            host, _, _ = r.packer.pack(entries, self.caps, self.work_caps, temperature, uniform)
            i = self._turn
            self._turn = (i + 1) % len(self._pinned)
            if self._copy_pending[i]:
                self._copied[i].synchronize()               # the copy that last read this buffer (long done, as a rule)
            self._pinned[i].numpy()[:] = host
            self.dev.copy_(self._pinned[i], non_blocking=True)
            self._copied[i].record()
            self._copy_pending[i] = True
            self.replay()
        r.bytes_h2d = self.nbytes
        r.last_launches = self.launches
        n = sum(len(e.want) for e in entries)
        r.tokens_host = self.tokens_host[:1 + n]
        return self.logits[:n], self.tokens[:1 + n]


class ModelRunner:
    def __init__(self, model_dir: str, dtype="bfloat16", page_size: int = 16, num_pages: Optional[int] = None,
                 cache_bytes: Optional[int] = None, max_requests: int = 64, device: str = "cuda:0",
                 prefix_cache: bool = True, use_graphs: bool = True, max_graph_batch: int = 256):
        if not torch.cuda.is_available():
            raise KernelError("no CUDA device: this engine has no CPU path")
        ops.lib()  # build or load the kernels now; fails loudly if that cannot be done
        self.device = torch.device(device)
        torch.cuda.set_device(self.device)
        self.dtype = parse_dtype(dtype)
        # float32 means float32: no TF32 or other reduced-precision matrix mode
        torch.backends.cuda.matmul.allow_tf32 = False
        torch.backends.cudnn.allow_tf32 = False
        torch.set_float32_matmul_precision("highest")
        self.arch, self.config = load_config(model_dir)
        self.spec = self.arch.describe(self.config)
        self.rt = Runtime(self.device, self.dtype)
        with torch.no_grad():
            self.model = DecoderModel(self.spec, self.rt)
            tensors = load_weights(model_dir, self.model.tensor_specs(), self.dtype, self.device)
            self.model.bind(tensors)
            del tensors
        needs = self.model.cache_needs()
        probe = CacheManager(needs, page_size, 1, 1, self.dtype, self.device, allocate_device=False)
        if num_pages is None:
            if cache_bytes is None:
                raise ConfigError("give the cache a size: num_pages or cache_bytes")
            # pages = budget / bytes per page, at least one (crates/pagedllm/src/batch.rs:53-57)
            num_pages = max(1, cache_bytes // max(1, page_size * probe.bytes_per_token()))
        self.cache = CacheManager(needs, page_size, num_pages, max_requests, self.dtype, self.device,
                                  prefix_cache=prefix_cache)
        self.caches = self.cache.layer_caches()
        # How each group's attention is cut into work items is what its mixers wish (those of one group alike);
        # a group whose mixers wish for nothing gets tables and slots only.
        plans = []
        for g in self.cache.groups:
            wishes = {self.model.blocks[self.model.schedule[i].layer].mixer.plan_wish(page_size) for i in g.entries}
            if len(wishes) != 1:
                raise ConfigError(f"the mixers that share a cache group wish for different attention plans: {sorted(map(str, wishes))}")
            w = wishes.pop()
            plans.append(None if w is None else GroupPlanConfig(w.tile_tokens, w.ctas_per_item, g.window, w.heads, w.head_dim))
        # CTAs an attention launch should have before splits stop: one full wave at two CTAs an SM
        self.packer = StepPacker(self.cache, plans, 2 * ops.sm_count(), self.spec.vocab_size, self.spec.max_positions,
                                 self.device)
        self.vocab_size = self.spec.vocab_size
        # A captured step replays fixed launches.  A mixer that loops over the step on the host (it says
        # so by graph_safe = False) is left out of the capture and launched between the captured pieces,
        # where its block can be run in halves around it; else it keeps the engine on plain launches.
        self.use_graphs = use_graphs and self.model.capturable()
        self.max_graph_batch = max_graph_batch
        self._graphs = {}
        self.graph_pool = torch.cuda.graph_pool_handle()
        # the engine's token budget a step: steps of prompt portions that fill more than half of it are
        # captured once and replayed (None: such steps are launched kernel by kernel)
        self.graph_step_tokens: Optional[int] = None
        self.bytes_h2d = 0        # bytes the last step copied to the device
        self.tokens_host: Optional[torch.Tensor] = None   # pinned copy of the last step's (status, tokens), valid
                                                          # once the stream is synchronized; None: not made
        self.last_launches = 0    # kernels of this library the last step launched

    # -- the step ----------------------------------------------------------------------
    def step(self, entries: Sequence[StepEntry], check: bool = True, trace: Optional[dict] = None) -> torch.Tensor:
        """Run one batch.  Returns float32 logits [wanted, vocab] on the device, in
        the order of the entries and of their ``want`` lists.  Pages for the new
        tokens must have been reserved; nothing is committed.  With ``trace`` (a
        dict) the parts store copies of what they leave at module boundaries
        there, under the checkpoint's names (``Runtime.trace``)."""
        self.rt.trace = trace
        try:
            logits, _ = self.step_and_sample(entries, None, None, check=check)
        finally:
            self.rt.trace = None
        return logits

    def step_and_sample(self, entries: Sequence[StepEntry], temperature, uniform, check: bool = False):
        """The step, followed (when ``temperature`` and ``uniform`` are given, one per
        wanted row) by the sampling kernel.  Returns (logits, tokens): tokens is an
        int32 device tensor [1 + wanted] whose first entry is the kernels' status
        word, so one copy brings both back.  A step of single decoded tokens runs
        as a replayed CUDA graph when graphs are on."""
        if not entries:
            return torch.zeros((0, self.vocab_size), dtype=torch.float32, device=self.device), None
        self.bytes_h2d = 0
        self.tokens_host = None
        if self.use_graphs and temperature is not None:
            if all(len(e.tokens) == 1 and list(e.want) == [0] for e in entries):
                g = self._decode_graph(entries)
            else:
                g = self._portion_graph(entries)
            if g is not None:
                return g.run(entries, temperature, uniform)
        host, layout, sizes = self.packer.pack(entries, temperature=temperature, uniform=uniform)
        pinned = torch.from_numpy(host).pin_memory()
        dev = pinned.to(self.device, non_blocking=True)
        self.bytes_h2d = host.nbytes
        state = self.packer.to_state(dev, layout, sizes)
        tokens = None
        before = ops.LAUNCHES
        with torch.no_grad():
            logits = self.model.forward(state, self.caches)
            if temperature is not None and state.n_wanted:
                tokens = torch.empty(1 + state.n_wanted, dtype=torch.int32, device=self.device)
                ops.sample(logits, state.temperature, state.uniform, tokens[1:])
                tokens[:1].copy_(self.rt.status)
        self.last_launches = ops.LAUNCHES - before
        if check:
            self.check_status()
        return logits, tokens

    def prepack_decode(self, entries: Sequence[StepEntry], temperature):
        """Get the next decode step ready on the host while the current one runs: the captured step for
        these requests, its buffer filled for positions one further than committed (pages reserved by the
        caller).  Returns the step to ``launch_prepacked`` once the token ids are known, or None when such
        steps are not captured."""
        if not self.use_graphs or temperature is None:
            return None
        g = self._decode_graph(entries)
        if g is None or g.native is None:
            return None
        g.prepack(entries, temperature)
        return g

    # -- decode steps as CUDA graphs ------------------------------------------------------
    def _decode_graph(self, entries):
        n = len(entries)
        if n > self.max_graph_batch:
            return None
        B = 1
        while B < n:
            B *= 2
        width = max((len(self.cache.get(e.request_id).tables[gi].blocks) for e in entries
                     for gi in range(len(self.cache.groups))), default=1)
        W = 64
        while W < width:
            W *= 2
        key = (B, W)
        g = self._graphs.get(key)
        if g is None:
            g = _DecodeGraph(self, B, W)
            self._graphs[key] = g
        return g

    def _portion_graph(self, entries):
        """The captured step for portions of prompts (beside decoded tokens), when the engine
        runs under a token budget: one capture per (budget, requests, table width), replayed for
        every step that fills more than half of it.  Smaller steps are launched one by one, so
        that no step computes mostly padding."""
        cap = self.graph_step_tokens
        total = sum(len(e.tokens) for e in entries)
        if not cap or total > cap or 2 * total <= cap or len(entries) > self.max_graph_batch:
            return None
        S = 1
        while S < len(entries):
            S *= 2
        if sum(len(e.want) for e in entries) > S:
            return None     # (generation wants one place a request at most; a step that wants more is launched plainly)
        width = max((len(self.cache.get(e.request_id).tables[gi].blocks) for e in entries
                     for gi in range(len(self.cache.groups))), default=1)
        W = 64
        while W < width:
            W *= 2
        key = (cap, W, S)
        g = self._graphs.get(key)
        if g is None:
            g = _DecodeGraph(self, cap, W, segments=S)
            self._graphs[key] = g
        return g

    def capture_ahead(self, max_batch: int, table_width: int = 64) -> int:
        """Capture, before the first request needs them, the steps the engine replays: decode steps of 1, 2, 4, ...
        up to ``max_batch`` requests and, under a token budget, the budget's steps of as many requests, for block
        tables of up to ``table_width`` pages (wider ones are captured when a request first grows that long).
        A capture takes some 40 ms; without this the first requests pay for them.  Returns how many were made."""
        if not self.use_graphs:
            return 0
        made, B = 0, 1
        while True:
            b = min(B, self.max_graph_batch)
            if (b, table_width) not in self._graphs:
                self._graphs[(b, table_width)] = _DecodeGraph(self, b, table_width)
                made += 1
            cap = self.graph_step_tokens
            if cap and b <= cap and (cap, table_width, b) not in self._graphs:
                self._graphs[(cap, table_width, b)] = _DecodeGraph(self, cap, table_width, segments=b)
                made += 1
            if B >= max_batch or b >= self.max_graph_batch:
                return made
            B *= 2

    def check_status(self) -> None:
        code = int(self.rt.status.item())
        if code:
            self.rt.status.zero_()
            what = [name for bit, name in ((1, "a token id outside the vocabulary"), (2, "a cache slot outside the pool"),
                                          (4, "a position outside the rotary table"), (8, "a page id outside the pool"),
                                          (16, "a wait for a copy that ran out (attention)"),
                                          (32, "a key range that does not start on a tile boundary"),
                                          (64, "a wait that ran out in the tcgen05 product"),
                                          (128, "a wait that ran out in the tcgen05 attention"))
                    if code & bit]
            raise KernelError("a kernel met " + (", ".join(what) or f"status {code}"))

    # -- sizes -------------------------------------------------------------------------------
    def weight_bytes(self) -> int:
        seen, total = set(), 0
        for p in self.model.parts():
            for v in vars(p).values():
                if isinstance(v, torch.Tensor) and v.data_ptr() not in seen:
                    seen.add(v.data_ptr())
                    total += v.numel() * v.element_size()
        return total
