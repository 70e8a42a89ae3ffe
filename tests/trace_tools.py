"""Helpers for the replay tests: run bin/trace_run on a list of steps and collect
what it wrote; the plain implementation's logits for a request."""

import json
import os
import subprocess
import sys
import tempfile

import numpy as np
import torch

import plain_qwen3 as P

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TRACE_RUN = os.path.join(ROOT, "bin", "trace_run")


def replay(model_dir, dtype, steps, max_tokens, vocab, page_size=None, prefix_cache=False, graphs=False,
           step_tokens=None):
    """Run the steps through bin/trace_run in one process.  Returns {step: [wanted, vocab]};
    with ``prefix_cache`` the key "prefix" holds what trace_run wrote about shared pages."""
    out = tempfile.mkdtemp(prefix="trace_out_")
    text = "".join(json.dumps(s) + "\n" for s in steps)
    cmd = [sys.executable, TRACE_RUN, "--model", model_dir, "--dtype", dtype, "--out", out, "--max-tokens", str(max_tokens)]
    if page_size is not None:
        cmd += ["--page-size", str(page_size)]
    if prefix_cache:
        cmd += ["--prefix-cache", "on"]
    if graphs:
        cmd += ["--graphs", "on"] + (["--step-tokens", str(step_tokens)] if step_tokens else [])
    r = subprocess.run(cmd, input=text, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, f"trace_run failed:\n{r.stdout[-2000:]}\n{r.stderr[-4000:]}"
    done = [l for l in r.stdout.splitlines() if l.startswith("done ")]
    assert [int(l.split()[1]) for l in done] == [s["step"] for s in steps]
    res = {}
    for f in os.listdir(out):
        if f.endswith(".f32"):
            res[int(f[:-4])] = np.fromfile(os.path.join(out, f), dtype="<f4").reshape(-1, vocab)
    if prefix_cache:
        with open(os.path.join(out, "prefix.json")) as f:
            res["prefix"] = json.load(f)
    return res


def plain_logits(model_dir, tokens):
    """float64 logits [len(tokens), vocab] of the plain implementation on the stored weights."""
    cfg, w = P.load_model(model_dir, torch.float64)
    return P.forward(cfg, w, list(tokens)).numpy()


class TraceBuilder:
    """Collects steps and remembers which rows of which step belong to which
    position of which request."""

    def __init__(self):
        self.steps = []
        self.where = []  # (step, row, request, position)
        self.fed = {}    # request -> tokens fed so far

    def step(self, entries, end=()):
        """entries: (request id, tokens, want) with want = places among these tokens."""
        k = len(self.steps)
        row = 0
        es = []
        entries = [e for e in entries if len(e[1])]
        live = set(self.fed) | {e[0] for e in entries}
        assert len(live) <= 4, f"step {k}: {len(live)} requests live"
        for rid, toks, want in entries:
            base = self.fed.get(rid, 0)
            for w in want:
                self.where.append((k, row, rid, base + w))
                row += 1
            self.fed[rid] = base + len(toks)
            es.append(dict(id=rid, tokens=[int(t) for t in toks], want=[int(w) for w in want]))
        for rid in end:
            self.fed.pop(rid, None)
        self.steps.append(dict(step=k, entries=es, end=list(end)))
        return k

    def collect(self, results):
        """{request: {position: logits}} from trace_run's files."""
        out = {}
        for k, row, rid, pos in self.where:
            out.setdefault(rid, {})[pos] = results[k][row]
        return out

    def retire(self, rid, new_name):
        """Let a later request use the id ``rid`` again: what was collected under it so far is
        kept under ``new_name``."""
        self.where = [(k, row, new_name if r == rid else r, pos) for k, row, r, pos in self.where]
