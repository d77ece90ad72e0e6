"""The parts of bench.py's contract that need no GPU: more than one GPU is refused with one line and
exit code 2; the reference arm always prints exactly one JSON line and exits 0 -- either the
measurement with the keys of this package's own line, or the reason why it could not run."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

LINE_KEYS = {"metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
             "vs_baseline", "dtype", "data", "config", "e2e", "gpu_launches", "prefill", "roofline", "points", "clocks",
             "impl", "spread"}


def run(*args):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True, timeout=900)


def one_json_line(p):
    assert p.returncode == 0, p.stderr[-2000:]
    lines = [l for l in p.stdout.splitlines() if l.strip()]
    assert len(lines) == 1, p.stdout
    return json.loads(lines[0])


def test_more_than_one_gpu_is_refused_with_one_line():
    for impl in ("ours", "reference"):
        p = run("--gpus", "2", "--steps", "2", "--warmup", "1", "--impl", impl)
        assert p.returncode == 2
        lines = [l for l in p.stdout.splitlines() if l.strip()]
        assert len(lines) == 1 and "one GPU" in lines[0]


def test_reference_arm_without_a_gpu_prints_its_reason():
    import torch
    if torch.cuda.is_available():
        pytest.skip("covered by the gpu test below")
    d = one_json_line(run("--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "1"))
    assert d["impl"] == "reference" and d["unavailable"]


@pytest.mark.gpu
def test_reference_arm_measures_the_reference_with_the_same_keys():
    if not os.path.isdir(os.path.join(ROOT, "baseline", "_ref", "inference_engine")):
        pytest.skip("the reference is not installed under baseline/_ref")
    d = one_json_line(run("--impl", "reference", "--steps", "4", "--warmup", "3", "--layers", "2", "--points", "",
                          "--prefill-tokens", "256"))
    assert d["impl"] == "reference"
    if "unavailable" in d:          # the reason must be the real exception, not a fixed sentence
        assert ":" in d["unavailable"]
        pytest.skip(d["unavailable"])
    assert LINE_KEYS <= set(d), sorted(LINE_KEYS - set(d))
    assert d["config"]["same_config"] is True and d["config"]["layers"] == 2
    assert d["value"] > 0 and d["e2e"]["value"] > 0 and d["e2e"]["value"] <= d["value"] * 1.05
    assert d["e2e"]["h2d_bytes_per_step"] > 0 and d["e2e"]["d2h_bytes_per_step"] > 0


@pytest.mark.gpu
def test_own_arm_prints_every_key_of_the_contract():
    d = one_json_line(run("--steps", "4", "--warmup", "3", "--layers", "2", "--points", "1", "--prefill-tokens", "256"))
    assert LINE_KEYS <= set(d), sorted(LINE_KEYS - set(d))
    assert d["impl"] == "ours" and d["gpu_launches"] > 0 and d["spread"]["repeats"] >= 3
    assert d["config"]["layers"] == 2 and d["config"]["layers_full"] == 22
    assert len(d["config"]) <= 20 and not any(isinstance(v, (dict, list)) for v in d["config"].values())
