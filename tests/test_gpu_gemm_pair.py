"""The CTA-pair (tcgen05 cta_group::2) variant of the grouped GEMM, selected per process with
B200MOE_GEMM_KERNEL=pair: same parity bar as the default kernel."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

SCRIPT = r"""
import sys, torch
sys.path.insert(0, %r)
from tests.test_gpu_gemm import _int8_case, run_gemm
from tests.util import assert_close_to_golden, bf16, load
from oracle import oracle as O
for counts, K, N, off in [([127, 129, 0, 1, 300], 192, 512, True), ([600], 128, 256, True), ([5] * 70, 64, 256, False)]:
    x, w, scale, offset, cnt = _int8_case(counts, K, N, 13, off)
    gold = O.golden_f32(x, w, scale, offset, cnt, "int8", O.GROUP_LIST_COUNTS)
    out, st = run_gemm(x, w, scale, offset, cnt, "int8", gl_type=1)
    assert st == (0, 0), st
    assert_close_to_golden(out, gold)
d = load("gemm_fp8.npz")
w, s = torch.from_numpy(d["weight"]), torch.from_numpy(d["scale"])
x, gl = bf16(d["x_bits"]), torch.from_numpy(d["group_list"])
out, st = run_gemm(x, w, s, None, gl, "fp8")
assert st == (0, 0)
assert_close_to_golden(out, O.golden_f32(x, w, s, None, gl, "fp8"))
d = load("gemm_fp4.npz")
w = torch.from_numpy(d["uni_weight_ascend"])
s, x, gl = bf16(d["uni_scale_bits"]), bf16(d["uni_x_bits"]), torch.from_numpy(d["uni_group_list"])
out, st = run_gemm(x, w, s, None, gl, "fp4")
assert st == (0, 0)
assert_close_to_golden(out, O.golden_f32(x, w, s, None, gl, "fp4"))
print("pair kernel ok")
""" % ROOT


def test_pair_kernel_parity():
    env = dict(os.environ, B200MOE_GEMM_KERNEL="pair")
    r = subprocess.run([sys.executable, "-c", SCRIPT], capture_output=True, text=True, env=env, timeout=600, cwd=ROOT)
    assert r.returncode == 0 and "pair kernel ok" in r.stdout, r.stdout[-2000:] + r.stderr[-3000:]
