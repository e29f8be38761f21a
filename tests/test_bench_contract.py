"""The parts of bench.py's contract that need no GPU: more than one GPU is refused with one line and exit code 2,
and the reference arm always prints one JSON line and exits 0 (here, without a CUDA device, its `unavailable` form)."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run(*args):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True, timeout=300)


def test_more_than_one_gpu_is_refused_in_one_line():
    r = run("--gpus", "2", "--steps", "2", "--warmup", "1")
    assert r.returncode == 2
    lines = [l for l in r.stdout.splitlines() if l.strip()]
    assert len(lines) == 1 and "one GPU" in lines[0]


def test_reference_arm_prints_one_json_line():
    import torch
    if torch.cuda.is_available():
        import pytest
        pytest.skip("with a GPU the arm runs gpt-fast itself, which takes minutes; bench.py --impl reference is run by hand")
    r = run("--impl", "reference", "--steps", "2", "--warmup", "1")
    assert r.returncode == 0, r.stderr[-500:]
    lines = [l for l in r.stdout.splitlines() if l.strip()]
    assert len(lines) == 1
    out = json.loads(lines[0])
    assert out["impl"] == "reference" and "unavailable" in out


def test_reference_arm_imports_nothing_of_this_library():
    src = open(os.path.join(ROOT, "baseline", "reference_arm.py")).read()
    assert "gpt_fast_b200" not in src.replace("Nothing of gpt_fast_b200 is imported here", "")


def test_design_option_pairs_a_llama_of_equal_size():
    """`--design lasezen` sets the design beside a Llama decoder of the same width, depth and vocabulary and nearly the
    same number of weights (counted from the two weight plans)."""
    import math
    sys.path.insert(0, ROOT)
    import bench
    import gpt_fast_b200 as gf
    from gpt_fast_b200.config.registry import architecture_for

    def weights(cfg):
        arch = architecture_for(cfg)
        return sum(math.prod(s.shape) for s in arch.weight_plan(arch.parse(cfg)).sources().values())
    for name in ("lasezen-1b", "lasezen-7b"):
        cfg = gf.config_from_name(name)
        twin = bench.llama_twin(cfg)
        assert twin["hidden_size"] == cfg["width"] and twin["num_hidden_layers"] == len(cfg["layers"]) and twin["vocab_size"] == cfg["vocab"]
        assert abs(weights(twin) - weights(cfg)) < 0.05 * weights(cfg)
    r = run("--design", "nothing-of-the-kind")
    assert r.returncode == 2 and "no size table" in r.stdout
