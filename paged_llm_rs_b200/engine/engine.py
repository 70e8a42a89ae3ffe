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

from typing import Dict, Iterable, List, Optional, Sequence as Seq

import numpy as np
import torch

from ..errors import ConfigError
from ..kernels import ops
from ..sampling.sampler import SamplingParams, sample_host
from .runner import ModelRunner
from .scheduler import Finish, Outcome, Plan, Scheduler, Sequence


class Engine:
    def __init__(self, model: str, dtype="bfloat16", block_size: int = 16, cache_mib: int = 3584,
                 blocks: Optional[int] = None, max_batch: int = 16, chunk: Optional[int] = 128,
                 prefix_cache: bool = True, device: str = "cuda:0", max_requests: Optional[int] = None,
                 max_prefill_seqs: int = 1):
        if chunk is not None and chunk < 1:
            raise ConfigError("chunk 0 would carry nothing")
        self.runner = ModelRunner(model, dtype=dtype, page_size=block_size, num_pages=blocks,
                                  cache_bytes=None if blocks is not None else cache_mib << 20,
                                  max_requests=max_requests or max(256, 2 * max_batch), device=device,
                                  prefix_cache=prefix_cache)
        self.runner.graph_step_tokens = chunk if (chunk is not None and chunk <= 8192) else None
        self.scheduler = Scheduler(self.runner.cache, max_batch=max_batch, chunk=chunk,
                                   max_positions=self.runner.spec.max_positions, max_prefill_seqs=max_prefill_seqs)
        self._next_id = 0
        self._seqs: Dict[int, Sequence] = {}
        self._finish: Dict[int, Finish] = {}
        self.bytes_d2h = 0  # bytes the last step copied back to the host

    # -- requests ------------------------------------------------------------------------
    def submit(self, prompt: Seq[int], max_tokens: int = 512, temperature: float = 0.0,
               top_k: Optional[int] = None, top_p: Optional[float] = None, seed: int = 0,
               stop_tokens: Iterable[int] = ()) -> int:
        if temperature <= 0.0:
            top_k = top_p = None  # an explicit greedy request drops the nucleus settings (routes.rs:106-126)
        params = SamplingParams(float(temperature), top_k, top_p)
        V = self.runner.vocab_size
        if any((not 0 <= int(t) < V) for t in prompt):
            raise ConfigError(f"a prompt token lies outside the vocabulary of {V}")
        rid = self._next_id
        self._next_id += 1
        seq = Sequence(rid, prompt, params, max_tokens, stop_tokens, seed)
        self._seqs[rid] = seq
        self.scheduler.submit(seq)
        return rid

    def cancel(self, rid: int) -> None:
        self.scheduler.cancel(rid)

    # -- one step ------------------------------------------------------------------------
    def step(self) -> Optional[Outcome]:
        """Plan, run, sample and commit one step.  None when there is nothing to do."""
        plan = self.scheduler.plan()
        if plan.kind == "idle":
            return None
        if plan.kind in ("refused", "outgrown"):
            out = self.scheduler.commit(plan, [])
        else:
            tokens = self._run(plan)
            out = self.scheduler.commit(plan, tokens)
        for rid, why in out.finished:
            self._finish[rid] = why
        return out

    def _run(self, plan: Plan) -> List[int]:
        """The step and the choice of tokens: one packed copy to the device, the
        model, the sampling kernel, one copy of status word and tokens back.  Rows
        of requests with top-k or top-p are copied back as logits and drawn on the host."""
        seqs = [self._seqs[rid] for rid in plan.ids]
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
                uni[i] = s.rng.next_f32()   # greedy rows leave their generator alone (sampler.rs:119-121)
        logits, tokens_dev = self.runner.step_and_sample(plan.entries, temp, uni)
        if tokens_dev is None:
            self.bytes_d2h = 0
            return []
        back = self.runner.tokens_host
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
