"""The four Python tests the reference ships, run unmodified (apart from the device string)
against the CPU oracle.  This is what pins the oracle to the reference's executable spec.
Skipped where the reference checkout is absent (e.g. on the GPU box)."""
import os
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
# the reference checkout: $ASCEND_KERNEL_REFERENCE, else a directory `reference` beside this repository
REF = os.environ.get("ASCEND_KERNEL_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")

SCRIPTS = [
    "grouped_gemm/test/python/test_group_gemm_fp8.py",
    "grouped_gemm/test/python/test_group_gemm_fp4.py",
    "grouped_soft_gemv/test/python/test_group_soft_gemv_fp8.py",
    "grouped_soft_gemv/test/python/test_group_soft_gemv_fp4.py",
]


@pytest.mark.skipif(not os.path.isdir(REF), reason="reference checkout not present")
@pytest.mark.parametrize("script", SCRIPTS)
def test_reference_script_passes_against_oracle(script):
    r = subprocess.run([sys.executable, os.path.join(HERE, "ref_shim_runner.py"), os.path.join(REF, script)],
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
