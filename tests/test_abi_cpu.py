"""CPU-only checks of the boundary: the shared library loads, exports every symbol the header
declares, and rejects bad arguments with status codes before touching the GPU."""
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _lib():
    from ascend_kernel_b200 import _abi

    return _abi


def test_library_exports_every_declared_symbol():
    abi = _lib()
    header = open(os.path.join(ROOT, "include", "b200moe.h")).read()
    declared = set(re.findall(r"\b(b200moe_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    for name in sorted(declared):
        assert hasattr(abi.lib, name), f"{name} declared in include/b200moe.h but not exported"
    assert declared == set(abi.EXPORTS)
    assert abi.version().split(".")[0] == "1"


P = 4096  # an aligned, non-null fake pointer: argument validation never dereferences it


@pytest.mark.parametrize("fn", ["b200moe_grouped_gemm", "b200moe_grouped_gemv"])
def test_argument_validation_returns_status_codes(fn):
    abi = _lib()
    f = getattr(abi.lib, fn)
    ok = dict(M=8, K=256, N=512, G=4, ct=2, glt=0, lay=0)

    def call(**kw):
        a = dict(ok, **kw)
        ptrs = a.get("ptrs", [P] * 6)
        return f(*ptrs, a["M"], a["K"], a["N"], a["G"], a["ct"], a["glt"], a["lay"], a.get("ws", P), a.get("wsb", 1 << 20),
                 None)

    assert call(ct=9) == 1                      # compute type
    assert call(ptrs=[None, P, P, P, P, P]) == 2
    assert call(K=100) == 3 and call(N=100) == 3 and call(G=0) == 3 and call(M=-1) == 3
    assert call(ct=0, K=192) == 3               # fp8 needs K % 128 == 0
    assert call(ptrs=[P + 2, P, P, P, P, P]) == 4
    assert call(ws=None) == 5 and call(wsb=8) == 5
    assert call(glt=5) == 6 and call(lay=7) == 6
    assert call(M=0) == 0                       # nothing to do, nothing launched
    # fp8 takes what the reference takes (N % 128 == 0); the other modes need whole 256-column tiles
    assert call(ct=0, N=384, M=0) == 0 and call(ct=0, N=448, M=0) == 3
    assert call(ct=2, N=384, M=0) == 3 and call(ct=1, N=384, M=0) == 3
    if fn == "b200moe_grouped_gemm":
        assert call(ct=4, M=0) == 0             # bf16: the matmul phase alone
        assert call(ct=4, ptrs=[P, P, None, None, P, P], M=8, ws=None) == 5   # no scale needed; reaches the workspace check
    else:
        assert call(ct=4) == 1                  # the GEMV has no bf16 mode


def test_dequant_validation():
    abi = _lib()
    assert abi.lib.b200moe_fp4_dequant(P, None, P, 48, 0, None) == 3
    assert abi.lib.b200moe_fp4_dequant(P, None, P, 64, 1, None) == 2   # scale kind 1 without scale
    assert abi.lib.b200moe_fp4_dequant(P, None, P, 64, 5, None) == 6
    assert abi.lib.b200moe_fp4_dequant(None, None, None, 0, 0, None) == 0
    assert abi.lib.b200moe_fp4_layout(P, P, 1, 100, 256, 1, None) == 3
    assert abi.lib.b200moe_fp8_dequant(P, P, P, 1, 192, 256, None) == 3          # K % 128
    assert abi.lib.b200moe_fp8_dequant(P, P, P, 1, 128, 384, None) != 3          # N % 128 is enough
    assert abi.lib.b200moe_fp8_dequant(P, None, P, 1, 128, 128, None) == 2
    assert abi.lib.b200moe_fp4_dequant_bf16_scale(P, P, P, 1, 64, 128, 0, None) == 3
    assert abi.lib.b200moe_fp4_dequant_bf16_scale(P, P, P, 1, 64, 256, 3, None) == 6
    assert abi.lib.b200moe_fp4_scale_fold(P, P, P, 2, 64, 8, 3, None) == 3       # one or two global scales
    assert abi.lib.b200moe_fp4_scale_fold(P, P, P, 0, 64, 8, 1, None) == 0
    assert abi.lib.b200moe_pack_weight_int8(P, P, 1, 100, 256, 0, None) == 3
    assert abi.lib.b200moe_grouped_gemm_int8_packed(P, P, P, None, P, P, 8, 64, 128, 1, 0, 0, P, 1 << 20, None) == 3
    assert abi.lib.b200moe_grouped_gemm_int8_packed(P, P, P, None, P, P, 0, 64, 256, 1, 0, 0, P, 1 << 20, None) == 0


def test_python_mirror_rejects_cpu_tensors_and_bad_compute_type():
    import torch

    import ascend_kernel_b200 as ak

    x = torch.zeros(4, 256, dtype=torch.bfloat16)
    w = torch.zeros(2, 256, 256, dtype=torch.int8)
    s = torch.zeros(2, 256, dtype=torch.bfloat16)
    gl = torch.tensor([2, 4])
    out = torch.zeros(4, 256, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="Host tiling failed"):
        ak.grouped_gemm(x, w, s, s, gl, "fp16", out)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        ak.grouped_gemm(x, w, s, s, gl, "int8", out)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        ak.grouped_soft_gemv(x, w, s, gl, "int8", out)


def test_workspace_sizes():
    abi = _lib()
    assert abi.lib.b200moe_grouped_gemm_workspace_bytes(1000, 256, 512, 4, 2, 0) == 256 + 4096
    assert abi.lib.b200moe_grouped_gemm_workspace_bytes(1000, 256, 512, 4, 0, 0) == 256
    # pre-shuffled fp4 weights are read in place: no canonical copy in the workspace
    assert abi.lib.b200moe_grouped_gemm_workspace_bytes(8, 256, 512, 4, 1, 1) == 256
    assert abi.lib.b200moe_grouped_gemv_workspace_bytes(8, 256, 512, 4, 2, 0) == 256
    # fp4 GEMV: the rows' f16 exponents (padded to 256 bytes) and x as scaled f16
    assert abi.lib.b200moe_grouped_gemv_workspace_bytes(8, 256, 512, 4, 1, 1) == 256 + 256 + 8 * 256 * 2


def test_install_check_lists_the_reference_operators():
    """The drop-in module exposes the reference's operator names (and the additions); the check fails
    loudly for a name the module lacks."""
    from ascend_kernel_b200 import check_installed_ops as chk

    chk.check(verbose=False)
    assert chk.REFERENCE_OPS == ["grouped_soft_gemv", "grouped_gemm"]
    chk.ADDED_OPS.append("no_such_operator")
    try:
        with pytest.raises(RuntimeError, match="no_such_operator"):
            chk.check(verbose=False)
    finally:
        chk.ADDED_OPS.pop()
