"""The reference's weight formats as standalone operators (FP8 128x128-block and FP4 per-16-k dequant,
the two-level FP4 scale fold), the bf16 grouped GEMM (the reference's matmul phase alone) and the
shapes the reference accepts for fp8 (N a multiple of 128, not of 256), through the C ABI."""
import pytest
import torch

from oracle import oracle as O
from tests.test_gpu_gemm import SENTINEL, run_gemm
from tests.util import assert_close_to_golden, bf16, load, same_bits

pytestmark = pytest.mark.gpu


def test_fp8_dequant_bit_exact_against_reference_golden():
    import ascend_kernel_b200 as ak

    d = load("gemm_fp8.npz")
    w, s = torch.from_numpy(d["weight"]), torch.from_numpy(d["scale"])
    out = torch.empty(w.shape, dtype=torch.bfloat16, device="cuda")
    ak.fp8_dequant(w.cuda(), s.cuda(), out)
    torch.cuda.synchronize()
    assert same_bits(out, bf16(d["wd_bits"]))          # the reference's anti_quant_fp8 on the same bytes
    # every code (0x7F / 0xFF decode to +-480) against a few scales, and a matrix with N % 256 == 128
    gen = torch.Generator().manual_seed(3)
    w = torch.randint(0, 256, (3, 256, 384), generator=gen, dtype=torch.uint8)
    w[0, 0, :256] = torch.arange(256, dtype=torch.uint8)
    s = torch.randn(3, 2, 3, generator=gen)
    out = torch.empty(w.shape, dtype=torch.bfloat16, device="cuda")
    ak.fp8_dequant(w.cuda(), s.cuda(), out)
    torch.cuda.synchronize()
    assert same_bits(out, O.dequant_fp8(w, s, round_bf16=True).to(torch.bfloat16))


@pytest.mark.parametrize("prefix", ["ref_", "uni_"])
@pytest.mark.parametrize("layout", ["ascend", "canonical"])
def test_fp4_dequant_bf16_scale_bit_exact_against_reference_golden(prefix, layout):
    import ascend_kernel_b200 as ak

    d = load("gemm_fp4.npz")
    w = torch.from_numpy(d[prefix + ("weight_ascend" if layout == "ascend" else "weight_canonical")])
    s = bf16(d[prefix + "scale_bits"])
    out = torch.empty(w.shape[0], w.shape[1], 2 * w.shape[2], dtype=torch.bfloat16, device="cuda")
    ak.fp4_dequant_bf16_scale(w.cuda(), s.cuda(), out, weight_layout=layout)
    torch.cuda.synchronize()
    # the fixture holds expert 0 (all experts share their weights); -0 * scale keeps its sign in both
    assert same_bits(out[0], bf16(d[prefix + "wd0_bits"]))
    wc = O.ascend_unshuffle(w) if layout == "ascend" else w
    assert same_bits(out, O.dequant_fp4(wc, s, round_bf16=True).to(torch.bfloat16))


def test_fp4_scale_fold_bit_exact_against_reference_helper():
    import ascend_kernel_b200 as ak

    d = load("scale_fold.npz")
    for tag in ("one", "two"):
        got = ak.fp4_scale_fold(bf16(d[tag + "_block_bits"]).cuda(), torch.from_numpy(d[tag + "_global"]).cuda())
        torch.cuda.synchronize()
        assert same_bits(got, bf16(d[tag + "_folded_bits"])), tag


@pytest.mark.parametrize("counts,K,N", [([1], 64, 256), ([127, 129, 0, 1, 300], 192, 512), ([40, 260], 448, 256)])
def test_bf16_grouped_gemm_matches_oracle(counts, K, N):
    """computeType "bf16": weights already bf16, no scale -- and the two-phase form of the reference
    (dequantise to a bf16 buffer, then multiply) equals its fused fp8 operator bit for bit."""
    import ascend_kernel_b200 as ak

    gen = torch.Generator().manual_seed(5)
    G = len(counts)
    cnt = torch.tensor(counts, dtype=torch.int64)
    M = int(cnt.sum()) + 3
    x = torch.randn(M, K, generator=gen).to(torch.bfloat16)
    w = (torch.randn(G, K, N, generator=gen) * 0.05).to(torch.bfloat16)
    out = torch.full((M, N), SENTINEL, dtype=torch.bfloat16, device="cuda")
    ws = ak.grouped_gemm(x.cuda(), w.cuda(), None, None, cnt.cuda(), "bf16", out, group_list_type=1, return_workspace=True)
    torch.cuda.synchronize()
    assert ak.read_status(ws) == (0, 0)
    gold = O.golden_f32(x, w, None, None, cnt, "bf16", O.GROUP_LIST_COUNTS)
    assert_close_to_golden(out, gold)
    assert (out[M - 3:].float() == SENTINEL).all()
    if K % 128 == 0 and N % 128 == 0:
        w8 = torch.randint(0, 256, (G, K, N), generator=gen, dtype=torch.uint8)
        s8 = torch.randn(G, K // 128, N // 128, generator=gen)
        fused, _ = run_gemm(x, w8, s8, None, cnt, "fp8", gl_type=1)
        wd = torch.empty(G, K, N, dtype=torch.bfloat16, device="cuda")
        ak.fp8_dequant(w8.cuda(), s8.cuda(), wd)
        two_phase = torch.full((M, N), SENTINEL, dtype=torch.bfloat16, device="cuda")
        ak.grouped_gemm(x.cuda(), wd, None, None, cnt.cuda(), "bf16", two_phase, group_list_type=1)
        torch.cuda.synchronize()
        assert same_bits(fused, two_phase)


@pytest.mark.parametrize("N", [128, 384, 1664])
def test_fp8_accepts_n_multiple_of_128_like_the_reference(N):
    """grouped_matmul_antiquant.h:587-591 and grouped_soft_gemv_tiling.cpp:105-128 need K % 128 == 0 and
    N % 128 == 0 only."""
    import ascend_kernel_b200 as ak

    gen = torch.Generator().manual_seed(N)
    G, K = 3, 256
    cnt = torch.tensor([140, 0, 37], dtype=torch.int64)
    cs = torch.cumsum(cnt, 0)
    M = int(cnt.sum()) + 2
    x = torch.randn(M, K, generator=gen).to(torch.bfloat16)
    w = torch.randint(0, 256, (G, K, N), generator=gen, dtype=torch.uint8)
    s = torch.randn(G, K // 128, N // 128, generator=gen)
    out, st = run_gemm(x, w, s, None, cs, "fp8")
    assert st == (0, 0)
    assert_close_to_golden(out, O.golden_f32(x, w, s, None, cs, "fp8"))
    assert (out[M - 2:].float() == SENTINEL).all()
    # decode-sized rows through the GEMV
    cnt_v = torch.tensor([1, 4, 2], dtype=torch.int64)
    cs_v = torch.cumsum(cnt_v, 0)
    xv = x[:7].contiguous()
    out_v = torch.full((7, N), SENTINEL, dtype=torch.bfloat16, device="cuda")
    ak.grouped_soft_gemv(xv.cuda(), w.cuda(), s.cuda(), cs_v.cuda(), "fp8", out_v)
    torch.cuda.synchronize()
    assert_close_to_golden(out_v, O.golden_f32(xv, w, s, None, cs_v, "fp8", gemv=True), ulps=2.0)
    # what the reference rejects stays rejected
    with pytest.raises(RuntimeError):
        bad = torch.full((M, N + 64), SENTINEL, dtype=torch.bfloat16, device="cuda")
        ak.grouped_gemm(x.cuda(), torch.zeros(G, K, N + 64, dtype=torch.uint8, device="cuda"),
                        torch.zeros(G, K // 128, (N + 64) // 128, device="cuda"), None, cs.cuda(), "fp8", bad)


def test_device_findings_reach_the_caller_without_a_workspace():
    """An invalid group_list is clamped on the device and must still be reported to a caller that never
    looks at a workspace: through last_status / check_status of the python mirror, through the MoE layer
    and through the drop-in module."""
    import ascend_kernel_b200 as ak
    from ascend_kernel_b200 import cinfer_ascendc

    gen = torch.Generator().manual_seed(1)
    x = torch.randn(30, 64, generator=gen).to(torch.bfloat16).cuda()
    w = torch.randint(-128, 128, (2, 64, 256), generator=gen, dtype=torch.int8).cuda()
    s = torch.ones(2, 256, dtype=torch.bfloat16, device="cuda")
    out = torch.zeros(30, 256, dtype=torch.bfloat16, device="cuda")
    ak.check_status()                                        # clean slate
    good = torch.tensor([10, 30], dtype=torch.int64, device="cuda")
    bad = torch.tensor([20, 5], dtype=torch.int64, device="cuda")   # not monotone
    ak.grouped_gemm(x, w, s, None, good, "int8", out)
    assert ak.last_status() == (0, 0)
    ak.grouped_gemm(x, w, s, None, bad, "int8", out)
    ak.grouped_gemm(x, w, s, None, good, "int8", out)        # a later good call does not hide the finding
    assert ak.last_status() == (1, 1)
    with pytest.raises(RuntimeError, match="group_list"):
        ak.check_status()
    assert ak.last_status() == (0, 0)                        # check_status cleared it
    cinfer_ascendc.check_status()
    cinfer_ascendc.grouped_gemm(x, w, s, torch.zeros(0, device="cuda"), bad, "int8", out)
    assert tuple(cinfer_ascendc.last_status()) == (1, 1)
    with pytest.raises(RuntimeError, match="group_list"):
        cinfer_ascendc.check_status()
