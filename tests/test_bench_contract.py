"""bench.py's contract: what it prints for more than one GPU and for the reference arm (no
GPU needed), and, marked gpu, one short run whose line carries every key the contract names."""
import json
import subprocess
import sys

import pytest

from conftest import ROOT

BENCH = str(ROOT / "bench.py")


def run(*args):
    return subprocess.run([sys.executable, BENCH, *map(str, args)], capture_output=True, text=True, timeout=900)


def test_more_than_one_gpu_is_one_line_and_exit_code_2():
    r = run("--gpus", 2, "--steps", 1, "--warmup", 1)
    assert r.returncode == 2
    assert len(r.stdout.strip().splitlines()) == 1 and "single-GPU" in r.stdout


def test_the_reference_arm_says_why_it_is_unavailable():
    r = run("--impl", "reference", "--gpus", 1, "--steps", 1, "--warmup", 1)
    assert r.returncode == 0
    rec = json.loads(r.stdout.strip().splitlines()[-1])
    assert rec["impl"] == "reference" and isinstance(rec["unavailable"], str) and rec["unavailable"]


def test_prompts_must_fit_the_context():
    r = run("--context", 1024, "--prompt-len", "900:1000", "--steps", 128)
    assert r.returncode == 2 and "fit the context" in r.stderr


@pytest.mark.gpu
def test_a_short_run_prints_the_whole_contract():
    r = run("--layers", 1, "--steps", 4, "--warmup", 3, "--batch", 2, "--no-points")
    assert r.returncode == 0, r.stderr[-2000:]
    rec = json.loads(r.stdout.strip().splitlines()[-1])
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better",
                "scaling", "vs_baseline", "dtype", "data", "config", "clocks", "e2e", "gpu_launches",
                "prefill", "roofline", "points"):
        assert key in rec, key
    assert rec["n_gpus"] == 1 and rec["steps"] == 4 and rec["warmup"] == 3 and rec["value"] > 0
    cfg = rec["config"]
    assert len(cfg) <= 20 and all(not isinstance(v, (dict, list)) for v in cfg.values())
    assert cfg["layers"] == 1 and cfg["layers_of_shape"] == 36 and cfg["global_batch"] == 2
    assert set(rec["prefill"]) == {"value", "tokens", "ms", "frac"} and rec["prefill"]["tokens"] == 2048
    assert set(rec["roofline"]) == {"bound", "achieved", "peak", "unit", "frac"} and rec["roofline"]["bound"] == "hbm"
    assert abs(rec["roofline"]["frac"] - rec["roofline"]["achieved"] / rec["roofline"]["peak"]) < 1e-3
    assert {"value", "unit", "h2d_bytes_per_step", "d2h_bytes_per_step"} <= set(rec["e2e"])
    assert rec["e2e"]["h2d_bytes_per_step"] > 0 and rec["e2e"]["d2h_bytes_per_step"] > 0
    assert rec["gpu_launches"] > 0
    assert {"sm_mhz", "sm_max_mhz", "reasons"} <= set(rec["clocks"])
