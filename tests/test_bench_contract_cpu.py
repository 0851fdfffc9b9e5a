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
