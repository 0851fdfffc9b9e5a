"""Antiquant grouped GEMM (tcgen05 kernel) through the C ABI against the CPU oracle and the
reference-derived fixtures."""
import pytest
import torch

from oracle import oracle as O
from tests.util import assert_close_to_golden, bf16, load, same_bits

pytestmark = pytest.mark.gpu
SENTINEL = -768.0  # exactly representable in bf16


def run_gemm(x, w, scale, offset, gl, ct, gl_type=0, layout="ascend"):
    import ascend_kernel_b200 as ak

    N = w.shape[2] * (2 if ct in ("fp4", "int4") else 1)
    out = torch.full((x.shape[0], N), SENTINEL, dtype=torch.bfloat16, device="cuda")
    ws = ak.grouped_gemm(x.cuda(), w.cuda(), scale.cuda(), None if offset is None else offset.cuda(), gl.cuda(), ct,
                         out, group_list_type=gl_type, weight_layout=layout, return_workspace=True)
    torch.cuda.synchronize()
    return out, ak.read_status(ws)


def test_config0_int8_parity():
    from ascend_kernel_b200 import inputs

    c = inputs.config0()
    gold = O.golden_f32(c["x"], c["weight"], c["scale"], c["offset"], c["counts"], "int8", O.GROUP_LIST_COUNTS)
    out, st = run_gemm(c["x"], c["weight"], c["scale"], c["offset"], c["counts"], "int8", gl_type=1)
    assert st == (0, 0)
    rl2, mx, frac = assert_close_to_golden(out, gold)
    print(f"config0: rel-L2 {rl2:.2e} max-abs {mx:.3f} differing {frac:.4f}")


def _int8_case(counts, K, N, seed, with_offset, extra_rows=0):
    gen = torch.Generator().manual_seed(seed)
    G = len(counts)
    counts = torch.tensor(counts, dtype=torch.int64)
    M = int(counts.sum()) + extra_rows
    x = torch.randn(M, K, generator=gen).to(torch.bfloat16)
    w = torch.randint(-128, 128, (G, K, N), generator=gen, dtype=torch.int8)
    scale = (torch.rand(G, N, generator=gen) * 0.009 + 0.001).to(torch.bfloat16)
    offset = (torch.rand(G, N, generator=gen) * 8 - 4).to(torch.bfloat16) if with_offset else None
    return x, w, scale, offset, counts


@pytest.mark.parametrize("counts,K,N,with_offset", [
    ([1], 64, 256, False),                       # smallest legal problem
    ([127, 129, 0, 1, 300], 192, 512, True),     # ragged m, empty expert, several m-tiles
    ([0, 0, 256, 0], 448, 256, True),            # one expert owns everything, K spans 7 stages
    ([2100], 128, 512, True),                    # > 16 m-tiles: more than one L2 super-tile
    ([5] * 70, 64, 256, False),                  # many tiny experts
])
def test_int8_matches_oracle(counts, K, N, with_offset):
    x, w, scale, offset, cnt = _int8_case(counts, K, N, 13, with_offset)
    gold = O.golden_f32(x, w, scale, offset, cnt, "int8", O.GROUP_LIST_COUNTS)
    out, st = run_gemm(x, w, scale, offset, cnt, "int8", gl_type=1)
    assert st == (0, 0)
    assert_close_to_golden(out, gold)
    out2, _ = run_gemm(x, w, scale, offset, torch.cumsum(cnt, 0), "int8", gl_type=0)
    assert same_bits(out, out2)


def test_largest_expert_count_and_all_empty_groups():
    """1024 experts (the limit of the in-kernel schedule, and the largest shared-memory footprint) with
    0..3 rows each; then a group list that gives every expert zero rows: nothing is written."""
    gen = torch.Generator().manual_seed(23)
    counts = torch.randint(0, 4, (1024,), generator=gen).tolist()
    x, w, scale, offset, cnt = _int8_case(counts, 64, 256, 29, True)
    gold = O.golden_f32(x, w, scale, offset, cnt, "int8", O.GROUP_LIST_COUNTS)
    out, st = run_gemm(x, w, scale, offset, cnt, "int8", gl_type=1)
    assert st == (0, 0)
    assert_close_to_golden(out, gold)
    out0, st0 = run_gemm(x, w, scale, offset, torch.zeros_like(cnt), "int8", gl_type=1)
    assert st0 == (0, 0)
    assert (out0.float() == SENTINEL).all()


def test_rows_past_last_boundary_untouched():
    x, w, scale, offset, cnt = _int8_case([100, 30], 128, 256, 17, True, extra_rows=50)
    out, st = run_gemm(x, w, scale, offset, torch.cumsum(cnt, 0), "int8")
    assert st == (0, 0)
    assert (out[130:].float() == SENTINEL).all()
    gold = O.golden_f32(x, w, scale, offset, torch.cumsum(cnt, 0), "int8")
    assert_close_to_golden(out, gold)


def test_int8_weights_are_exact_on_the_tensor_cores():
    # x = one-hot rows, scale 1, no offset: the output is the int8 weight row itself, exactly
    G, K, N = 2, 128, 256
    gen = torch.Generator().manual_seed(1)
    w = torch.randint(-128, 128, (G, K, N), generator=gen, dtype=torch.int8)
    x = torch.zeros(2 * K, K, dtype=torch.bfloat16)
    x[torch.arange(2 * K), torch.arange(2 * K) % K] = 1
    scale = torch.ones(G, N, dtype=torch.bfloat16)
    out, st = run_gemm(x, w, scale, None, torch.tensor([K, K]), "int8", gl_type=1)
    assert st == (0, 0)
    assert torch.equal(out.cpu().float(), w.reshape(2 * K, N).float())


def test_fp8_reference_fixture_bit_exact_weights():
    d = load("gemm_fp8.npz")
    w, s = torch.from_numpy(d["weight"]), torch.from_numpy(d["scale"])
    x, gl = bf16(d["x_bits"]), torch.from_numpy(d["group_list"])
    out, st = run_gemm(x, w, s, torch.zeros_like(s), gl, "fp8")
    assert st == (0, 0)
    # the reference's own bar: allclose(atol=0.02) (test_group_gemm_fp8.py:71) is for x = ones;
    # here x ~ N(0,1): compare against the golden with the stated tolerance
    gold = O.golden_f32(x, w, s, None, gl, "fp8")
    assert_close_to_golden(out, gold)
    # one-hot x reads the dequantised weights back: bit-exact against the reference's dequant
    K = w.shape[1]
    eye = torch.eye(K, dtype=torch.bfloat16)
    out2, _ = run_gemm(eye, w[:1].contiguous(), s[:1].contiguous(), None, torch.tensor([K]), "fp8")
    # (x = identity sums +0 terms onto every weight, so a -0 weight reads back as +0: compare values)
    assert torch.equal(out2.cpu().float(), bf16(d["wd_bits"])[0].float())


@pytest.mark.parametrize("prefix", ["ref_", "uni_"])
@pytest.mark.parametrize("layout", ["ascend", "canonical"])
def test_fp4_reference_fixture(prefix, layout):
    d = load("gemm_fp4.npz")
    w = torch.from_numpy(d[prefix + ("weight_ascend" if layout == "ascend" else "weight_canonical")])
    s, x, gl = bf16(d[prefix + "scale_bits"]), bf16(d[prefix + "x_bits"]), torch.from_numpy(d[prefix + "group_list"])
    out, st = run_gemm(x, w, s, torch.zeros_like(s), gl, "fp4", layout=layout)
    assert st == (0, 0)
    n_rows = int(gl[-1])  # rows past the last boundary are not written (the fixture holds zeros there)
    assert torch.allclose(out.cpu().float()[:n_rows], bf16(d[prefix + "y_bits"]).float()[:n_rows],
                          atol=0.15)  # test_group_gemm_fp4.py:225
    assert (out[n_rows:].float() == SENTINEL).all()
    gold = O.golden_f32(x, w, s, None, gl, "fp4", weight_layout=layout)
    assert_close_to_golden(out, gold)
    K = w.shape[1]
    eye = torch.eye(K, dtype=torch.bfloat16)
    out2, _ = run_gemm(eye, w[:1].contiguous(), s[:1].contiguous(), None, torch.tensor([K]), "fp4", layout=layout)
    assert torch.equal(out2.cpu().float(), bf16(d[prefix + "wd0_bits"]).float())


def test_bad_group_list_is_clamped_and_reported():
    x, w, scale, offset, cnt = _int8_case([10, 20], 64, 256, 9, False)
    out, st = run_gemm(x, w, scale, None, torch.tensor([20, 5]), "int8")
    assert st[0] == 1 and st[1] == 1


def _int4_case(counts, K, N, seed, with_offset):
    gen = torch.Generator().manual_seed(seed)
    G = len(counts)
    counts = torch.tensor(counts, dtype=torch.int64)
    M = int(counts.sum())
    x = torch.randn(M, K, generator=gen).to(torch.bfloat16)
    w = torch.randint(0, 256, (G, K, N // 2), generator=gen, dtype=torch.uint8).view(torch.int8)
    scale = (torch.rand(G, K // 128, N, generator=gen) * 0.045 + 0.005).to(torch.bfloat16)
    offset = (torch.rand(G, K // 128, N, generator=gen) * 4 - 2).to(torch.bfloat16) if with_offset else None
    return x, w, scale, offset, counts


@pytest.mark.parametrize("counts,K,N,with_offset", [
    ([16, 48, 32, 32], 256, 512, True),
    ([127, 129, 0, 1, 300], 384, 256, True),
    ([70, 3], 128, 512, False),
])
def test_int4_per_group_scales_match_oracle(counts, K, N, with_offset):
    x, w, scale, offset, cnt = _int4_case(counts, K, N, 23, with_offset)
    gold = O.golden_f32(x, w, scale, offset, cnt, "int4", O.GROUP_LIST_COUNTS)
    out, st = run_gemm(x, w, scale, offset, cnt, "int4", gl_type=1)
    assert st == (0, 0)
    assert_close_to_golden(out, gold)
