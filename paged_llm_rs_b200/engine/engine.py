"""The engine loop: plan a step, run it, choose tokens, commit
(crates/pagedllm-server/src/engine.rs:180-303 in the reference, without the
server around it).  Token ids go in and token ids come out.

    engine = Engine("model_dir", dtype="bfloat16")
    outputs = engine.generate([[1, 2, 3], [4, 5]], max_tokens=16)

Options carry the names and defaults of the reference's command line
(crates/pagedllm-server/src/main.rs:20-71): block_size 16, cache_mib 3584,
max_batch 16, chunk 128 (None = "off": prompts run whole), prefix_cache on.
"""

from __future__ import annotations

from collections import OrderedDict
from typing import Dict, Iterable, List, Optional, Sequence as Seq

import numpy as np
import torch

from ..errors import ConfigError, EngineError
from ..kernels import ops
from ..sampling.sampler import SamplingParams, sample_host
from .runner import ModelRunner
from .scheduler import Finish, Outcome, Plan, Scheduler, Sequence
from .step import StepEntry


class Engine:
    def __init__(self, model: str, dtype="bfloat16", block_size: int = 16, cache_mib: int = 3584,
                 blocks: Optional[int] = None, max_batch: int = 16, chunk: Optional[int] = 128,
                 prefix_cache: bool = True, device: str = "cuda:0", max_requests: Optional[int] = None,
                 max_prefill_seqs: int = 1, lookahead: bool = True, reference_draw_order: bool = False, runner=None):
        """``reference_draw_order``: temperature requests without top-k / top-p are drawn on the host
        in the reference's order (falling probability) instead of on the device (token ids upward):
        the same distribution, and for a given seed the reference's tokens.
        ``runner``: something that steps like a ``ModelRunner`` (cache, spec, vocab_size,
        step_and_sample, prepack_decode, check_status), to drive the loop without a model."""
        if chunk is not None and chunk < 1:
            raise ConfigError("chunk 0 would carry nothing")
        self.runner = runner if runner is not None else ModelRunner(
            model, dtype=dtype, page_size=block_size, num_pages=blocks,
            cache_bytes=None if blocks is not None else cache_mib << 20,
            max_requests=max_requests or max(256, 2 * max_batch), device=device, prefix_cache=prefix_cache)
        self.runner.graph_step_tokens = chunk if (chunk is not None and chunk <= 8192) else None
        self.scheduler = Scheduler(self.runner.cache, max_batch=max_batch, chunk=chunk,
                                   max_positions=self.runner.spec.max_positions, max_prefill_seqs=max_prefill_seqs)
        self.reference_draw_order = bool(reference_draw_order)
        self._next_id = 0
        self._seqs: Dict[int, Sequence] = {}
        # how the last FINISH_MEMORY requests ended (older ones are forgotten: an engine lives long)
        self._finish: "OrderedDict[int, Finish]" = OrderedDict()
        self.last_error: Optional[EngineError] = None   # what failed the last failed step
        self.bytes_d2h = 0  # bytes the last step copied back to the host
        # While a decode step runs on the GPU the host gets the next one ready (pages, positions, tables,
        # attention work: everything but the token ids), so that between two steps the GPU waits only for
        # the tokens to be read, checked for an ending, written into the buffer, and the replay.
        self.lookahead = bool(lookahead)
        self._inflight = None   # (plan, what _launch returned) of a step that runs and is not yet committed

    # -- requests ------------------------------------------------------------------------
    def submit(self, prompt: Seq[int], max_tokens: int = 512, temperature: float = 0.0,
               top_k: Optional[int] = None, top_p: Optional[float] = None, seed: int = 0,
               stop_tokens: Iterable[int] = ()) -> int:
        if temperature <= 0.0:
            top_k = top_p = None  # an explicit greedy request drops the nucleus settings (routes.rs:106-126)
        params = SamplingParams(float(temperature), top_k, top_p, self.reference_draw_order)
        V = self.runner.vocab_size
        if any((not 0 <= int(t) < V) for t in prompt):
            raise ConfigError(f"a prompt token lies outside the vocabulary of {V}")
        rid = self._next_id
        self._next_id += 1
        seq = Sequence(rid, prompt, params, max_tokens, stop_tokens, seed)
        self._seqs[rid] = seq
        self.scheduler.submit(seq)
        return rid

    FINISH_MEMORY = 4096

    def cancel(self, rid: int) -> None:
        """End a request now; its pages go back at once.  A step that is already running may still
        write the request's keys and values into those pages: it does so in stream order before any
        step that is planned after this call, so a new owner of a page (which names the page only
        after its own step is committed) never reads them.  When nothing is left to run, the step in
        flight is waited for here and its status checked, so that no step outlives its requests."""
        self.scheduler.cancel(rid)
        if self._inflight is not None and not self.scheduler.has_work():
            plan, ctx = self._inflight
            self._inflight = None
            try:
                self._collect(plan, ctx)               # its tokens belong to nobody any more
            except EngineError as e:
                self.last_error = e

    # -- one step ------------------------------------------------------------------------
    def step(self) -> Optional[Outcome]:
        """Plan, run, sample and commit one step.  None when there is nothing to do.  On return the
        step after it may already be running (a decode step that follows a decode step with the same
        requests): its tokens come with the next call.

        A step that fails (a kernel refuses its arguments, or the status word says that a kernel
        met an index out of range or a wait that ran out) ends every request that was in it with
        ``Finish.ERROR``, since none of them can tell what was written before it stopped
        (crates/pagedllm-server/src/engine.rs:338-348); their pages and state slots go back, the
        other requests go on, and ``last_error`` holds the cause."""
        if self._inflight is None:
            plan = self.scheduler.plan()
            if plan.kind == "idle":
                return None
            if plan.kind in ("refused", "outgrown"):
                return self._note(self.scheduler.commit(plan, []))
            try:
                self._inflight = (plan, self._launch(plan))
            except EngineError as e:
                return self._fail(plan, e)
        plan, ctx = self._inflight
        self._inflight = None                          # (whatever goes wrong below, this step is not collected twice)
        try:
            ahead = self._prepare_next(plan, ctx)      # host work beside the GPU
            tokens = self._collect(plan, ctx)          # waits for the step
        except EngineError as e:
            return self._fail(plan, e)
        if ahead is not None:
            seqs, graph = ahead
            if not self.scheduler.waiting and not any(self.scheduler.ends_with(s, t) for s, t in zip(seqs, tokens)):
                try:
                    self._inflight = self._launch_prepared(seqs, graph, tokens)
                except EngineError as e:
                    out = self._note(self.scheduler.commit(plan, tokens))
                    failed = self._fail(Plan("decode", [s.id for s in seqs], [(s.id, 1) for s in seqs]), e)
                    out.finished += failed.finished
                    return out
        return self._note(self.scheduler.commit(plan, tokens))

    def _fail(self, plan: Plan, error: EngineError) -> Outcome:
        self.last_error = error
        return self._note(self.scheduler.fail([rid for rid, _ in plan.advanced]))

    def _note(self, out: Outcome) -> Outcome:
        for rid, why in out.finished:
            self._finish[rid] = why
            self._finish.move_to_end(rid)
        while len(self._finish) > self.FINISH_MEMORY:
            self._finish.popitem(last=False)
        return out

    def _sampling_rows(self, seqs):
        """Temperatures for the sampling kernel, a uniform number for every row that draws (greedy rows
        leave their generator alone, sampler.rs:119-121), and the rows drawn on the host instead."""
        n = len(seqs)
        temp = np.zeros(n, dtype=np.float32)
        uni = np.zeros(n, dtype=np.float32)
        host_rows = []
        for i, s in enumerate(seqs):
            p = s.sampling
            if not p.on_device:
                host_rows.append(i)
            elif not p.is_greedy:
                temp[i] = p.temperature
                uni[i] = s.rng.next_f32()
        return temp, uni, host_rows

    def _launch(self, plan: Plan):
        """One packed copy to the device, the model, the sampling kernel; nothing is waited for."""
        seqs = [self._seqs[rid] for rid in plan.ids]
        temp, uni, host_rows = self._sampling_rows(seqs)
        logits, tokens_dev = self.runner.step_and_sample(plan.entries, temp, uni)
        return seqs, logits, tokens_dev, self.runner.tokens_host, host_rows

    def _collect(self, plan: Plan, ctx) -> List[int]:
        """The step's status word and tokens, one copy back.  Rows of requests with top-k or top-p are
        copied back as logits and drawn on the host."""
        seqs, logits, tokens_dev, back, host_rows = ctx
        if tokens_dev is None:
            self.bytes_d2h = 0
            return []
        if back is not None:     # a captured step copies them to pinned memory itself
            torch.cuda.current_stream().synchronize()
        else:
            back = tokens_dev.cpu()
        self.bytes_d2h = back.numel() * 4
        if int(back[0]):
            self.runner.check_status()
        tokens = back[1:].tolist()
        if host_rows:
            rows = logits[torch.tensor(host_rows, device=self.runner.device)].cpu().numpy()
            self.bytes_d2h += rows.nbytes
            for r, i in zip(rows, host_rows):
                tokens[i] = sample_host(r, seqs[i].sampling, seqs[i].rng)
        return tokens

    def _prepare_next(self, plan: Plan, ctx):
        """While ``plan`` runs: if the step after it will be the same requests decoding again, reserve
        their pages and pack that step (all but the token ids).  Returns (requests, captured step) or None."""
        if not self.lookahead or plan.kind != "decode" or ctx[4] or ctx[2] is None:
            return None
        seqs = self.scheduler.continuation(plan)
        if seqs is None or any(not s.sampling.on_device for s in seqs):
            return None
        temp = np.asarray([0.0 if s.sampling.is_greedy else s.sampling.temperature for s in seqs], dtype=np.float32)
        graph = self.runner.prepack_decode([StepEntry(s.id, [0], [0]) for s in seqs], temp)
        return None if graph is None else (seqs, graph)

    def _launch_prepared(self, seqs, graph, tokens: List[int]):
        """The step ``_prepare_next`` packed, now that the tokens it starts from are known."""
        uni = None       # (all rows greedy: nothing to draw, the buffer holds zeros)
        if any(not s.sampling.is_greedy for s in seqs):
            _, uni, _ = self._sampling_rows(seqs)
        logits, tokens_dev = graph.launch_prepacked(tokens, uni)
        self.scheduler.count_decode_step(len(seqs))
        plan = Plan("decode", [s.id for s in seqs], [(s.id, 1) for s in seqs],
                    [StepEntry(s.id, [t], [0]) for s, t in zip(seqs, tokens)])
        return plan, (seqs, logits, tokens_dev, self.runner.tokens_host, [])

    def warm_up(self) -> int:
        """Capture the steps this engine replays (decode steps up to ``max_batch`` requests, the token budget's
        steps) now instead of when the first requests need them.  Returns how many captures were made."""
        ahead = getattr(self.runner, "capture_ahead", None)
        return ahead(self.scheduler.max_batch) if ahead is not None else 0

    # -- whole generations -----------------------------------------------------------------
    def run_until_done(self) -> None:
        while self.scheduler.has_work():
            if self.step() is None:
                if self.scheduler.has_work():
                    raise RuntimeError("the scheduler is idle with requests left: the cache is too small to run any")
                break

    def generate(self, prompts: Seq[Seq[int]], max_tokens: int = 512, temperature: float = 0.0,
                 top_k: Optional[int] = None, top_p: Optional[float] = None, seed: int = 0,
                 stop_tokens: Iterable[int] = ()) -> List[List[int]]:
        """Generate for every prompt; returns the produced token ids per prompt
        (stop tokens are not part of the output)."""
        stop = tuple(stop_tokens)
        ids = [self.submit(p, max_tokens, temperature, top_k, top_p, seed, stop) for p in prompts]
        self.run_until_done()
        outs = [list(self._seqs[i].output) for i in ids]
        for i in ids:
            self._seqs.pop(i, None)
        return outs

    def finish_reason(self, rid: int) -> Optional[Finish]:
        return self._finish.get(rid)

    def metrics(self) -> dict:
        m = self.scheduler.metrics
        d = dict(vars(m))
        d["prefix_hit_rate"] = m.prefix_hit_rate()
        d["mean_batch"] = m.mean_batch()
        d["pages"] = self.runner.cache.num_pages
        d["pages_free"] = self.runner.cache.available()
        for gi, g in enumerate(self.runner.cache.groups):
            a = g.allocator
            d[f"group{gi}"] = dict(hits=a.hits, misses=a.misses, evictions=a.evictions, handed_out=a.handed_out)
        return d
