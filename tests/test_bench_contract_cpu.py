"""bench.py's command-line contract where it can be checked without a GPU: the reference arm prints
one JSON line with the agreed keys, and the product arm refuses to run without a CUDA device."""
import json
import os
import subprocess
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(*args, env=None):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True,
                          timeout=900, cwd=ROOT, env=env)


def test_reference_arm_prints_one_json_line_with_the_contract_keys():
    # a one-process-per-GPU launcher hands its children OMP_NUM_THREADS=1; the arm must still use the host's cores
    r = _run("--impl", "reference", "--steps", "1", "--warmup", "0", env={**os.environ, "OMP_NUM_THREADS": "1"})
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [l for l in r.stdout.splitlines() if l.strip().startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["metric"] == "moe_layer_tokens_per_s" and d["unit"] == "tokens/s"
    for key in ("value", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling", "vs_baseline", "dtype",
                "data", "config", "cpu_baseline", "e2e"):
        assert key in d, key
    assert d["value"] > 0 and d["config"]["workload"].startswith("moe_ffn_layer")
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["cores"] == len(os.sched_getaffinity(0))
    assert d["e2e"]["h2d_bytes_per_step"] == 0 and d["e2e"]["d2h_bytes_per_step"] == 0


def test_product_arm_has_no_cpu_path():
    if torch.cuda.is_available():
        return  # on a GPU box the product arm is exercised by the driver
    r = _run("--steps", "1", "--warmup", "0")
    assert r.returncode != 0
    assert "CUDA" in (r.stderr + r.stdout)


def test_reference_arm_does_not_load_the_product_library():
    """The CPU arm is the baseline: it must run without the package (and so without libb200moe.so) ever
    being imported; the input generators are loaded by path."""
    code = ("import sys, bench; c = bench.cpu_sample_inputs(128); "
            "assert not any(m == 'ascend_kernel_b200' or m.startswith('ascend_kernel_b200.') for m in sys.modules); "
            "maps = open('/proc/self/maps').read(); assert 'libb200moe' not in maps; print('clean')")
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert r.returncode == 0 and "clean" in r.stdout, r.stderr[-2000:]


def test_hashed_inputs_are_reproducible_and_uniform():
    """The layer's weights are a hash of (seed, element index): the same call gives the same bits, a slice
    of experts equals the same experts of a larger slice, and the bytes are spread over all 256 values."""
    from ascend_kernel_b200 import inputs

    a = inputs.hashed_bytes((64, 1024), 77, "cpu", torch.int8)
    assert torch.equal(a, inputs.hashed_bytes((64, 1024), 77, "cpu", torch.int8))
    assert not torch.equal(a, inputs.hashed_bytes((64, 1024), 78, "cpu", torch.int8))
    h = torch.bincount(a.view(torch.uint8).reshape(-1).long(), minlength=256)
    assert int(h.min()) > 150 and int(h.max()) < 380          # 65 536 draws over 256 bins: 256 +- 16
    one = inputs.config4("cpu", n_tokens=2, hidden=64, n_experts=4, inter=32, top_k=2, seed=4, expert_lo=2, expert_hi=3)
    two = inputs.config4("cpu", n_tokens=2, hidden=64, n_experts=4, inter=32, top_k=2, seed=4, expert_lo=1, expert_hi=4)
    for k in ("w13", "s13", "o13", "w2", "s2", "o2"):
        assert torch.equal(one[k][0], two[k][1]), k
    u = inputs.hashed_uniform((4096,), -4.0, 4.0, 5, "cpu").float()
    assert -4.0 <= float(u.min()) and float(u.max()) <= 4.0 and abs(float(u.mean())) < 0.2
