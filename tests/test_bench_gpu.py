"""The measuring program's side paths run: its comparison with the reference's own attention kernel
(compiled from the reference's source where a copy lies under baseline/_ref) launches both kernels on
the same keys, values and queries and must find the same numbers; a short run of the bench prints a
line with the keys the record needs."""

import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run_bench(*args):
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True, cwd=ROOT, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    lines = [l for l in p.stdout.splitlines() if l.startswith("{")]
    assert lines, p.stdout[-500:]
    return json.loads(lines[-1])


def test_the_reference_kernel_comparison_runs_and_agrees():
    out = run_bench("--only", "reference-kernel")
    if "unavailable" in out:
        pytest.skip(out["unavailable"])
    assert out["max_abs_diff"] < 0.01
    for key in ("h16_b8_ctx4096", "h32_b64_ctx4096"):
        assert out[key + "_ref_us"] > 0 and 0 < out[key + "_ours_us"] < out[key + "_ref_us"]


def test_a_short_bench_run_prints_the_record():
    out = run_bench("--steps", "3", "--warmup", "3", "--layers", "2", "--no-shapes")
    for key in ("metric", "value", "ms_per_step", "e2e", "gpu_launches", "clocks", "prefill", "roofline", "config",
                "points", "generate"):
        assert key in out, key
    assert out["config"]["layers"] == 2 and out["config"]["layers_of_shape"] == 28
    assert out["gpu_launches"] > 0 and out["e2e"]["h2d_bytes_per_step"] > 0 and out["e2e"]["d2h_bytes_per_step"] > 0
    assert 0 < out["roofline"]["frac"] < 1.2 and 0 < out["prefill"]["frac"] < 1.2
    assert out["points"]["decode_b1"] > 0 and out["points"]["decode_b64"] > out["points"]["decode_b1"]
    assert "error" not in out["generate"] and out["generate"]["generated_tokens_s"] > 0


def test_the_long_prompt_mode_times_every_portion():
    out = run_bench("--only", "long-prompt", "--context", "6144", "--layers", "2")
    assert out["tokens"] == 6144 and out["whole_prompt_ms"] > 0
    first, last = out["portion_at_0"], out["portion_at_4096"]
    assert 0 < first["bf16_frac"] < 1.2 and 0 < last["bf16_frac"] < 1.2
    assert last["attention_share_of_flops"] > first["attention_share_of_flops"]
