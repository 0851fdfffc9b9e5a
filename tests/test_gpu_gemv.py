"""Grouped soft GEMV through the C ABI against the CPU oracle and the reference-derived fixtures."""
import pytest
import torch

from oracle import oracle as O
from tests.util import assert_close_to_golden, bf16, load

pytestmark = pytest.mark.gpu
SENTINEL = -768.0  # exactly representable in bf16


def run_gemv(x, w, scale, gl, ct, offset=None, gl_type=0, layout="ascend"):
    import ascend_kernel_b200 as ak

    N = w.shape[2] * (2 if ct in ("fp4", "int4") else 1)
    out = torch.full((x.shape[0], N), SENTINEL, dtype=torch.bfloat16, device="cuda")
    ws = ak.grouped_soft_gemv(x.cuda(), w.cuda(), scale.cuda(), gl.cuda(), ct, out, group_list_type=gl_type,
                              weight_layout=layout, offset=None if offset is None else offset.cuda(),
                              return_workspace=True)
    torch.cuda.synchronize()
    return out, ak.read_status(ws)


def _int8_case(counts, K, N, seed, with_offset):
    gen = torch.Generator().manual_seed(seed)
    G = len(counts)
    counts = torch.tensor(counts, dtype=torch.int64)
    M = int(counts.sum())
    x = torch.randn(M, K, generator=gen).to(torch.bfloat16)
    w = torch.randint(-128, 128, (G, K, N), generator=gen, dtype=torch.int8)
    scale = (torch.rand(G, N, generator=gen) * 0.009 + 0.001).to(torch.bfloat16)
    offset = (torch.rand(G, N, generator=gen) * 8 - 4).to(torch.bfloat16) if with_offset else None
    return x, w, scale, offset, counts


@pytest.mark.parametrize("counts,K,N,with_offset", [
    ([1, 1, 1, 1], 256, 256, False),
    ([1, 0, 2, 4, 0, 3], 512, 512, True),
    ([0, 0, 5, 9, 1], 192, 768, True),       # more than 4 rows per expert, K not a multiple of 128
    ([2] * 40, 128, 256, False),             # more work items than resident CTAs per expert slab
    ([3, 2, 4, 7], 64, 256, True),           # one k block only; 2..4 rows take the tensor-core path
    ([2, 3, 4, 1, 8, 2], 7168, 512, True),   # benchmark K
])
def test_int8_matches_oracle(counts, K, N, with_offset):
    x, w, scale, offset, cnt = _int8_case(counts, K, N, 7, with_offset)
    gold = O.golden_f32(x, w, scale, offset, cnt, "int8", O.GROUP_LIST_COUNTS, gemv=True)
    out, st = run_gemv(x, w, scale, cnt, "int8", offset, gl_type=1)
    assert st == (0, 0)
    assert_close_to_golden(out, gold)
    # cumulative group_list gives the same result
    out2, _ = run_gemv(x, w, scale, torch.cumsum(cnt, 0), "int8", offset, gl_type=0)
    assert torch.equal(out.cpu().view(torch.int16), out2.cpu().view(torch.int16))


def test_rows_past_last_boundary_untouched():
    x, w, scale, offset, cnt = _int8_case([1, 2, 1], 128, 256, 9, True)
    x = torch.cat([x, torch.randn(3, 128).to(torch.bfloat16)])  # 3 rows owned by nobody
    out, st = run_gemv(x, w, scale, torch.cumsum(cnt, 0), "int8", offset)
    assert st == (0, 0)
    assert (out[4:].float() == SENTINEL).all() and (out[:4].float() != SENTINEL).any()


def test_fp8_reference_fixture():
    d = load("gemv_fp8.npz")
    w, s = torch.from_numpy(d["weight"]), torch.from_numpy(d["scale"])
    x, gl = bf16(d["x_bits"]), torch.from_numpy(d["group_list"])
    out, st = run_gemv(x, w, s, gl, "fp8")
    assert st == (0, 0)
    want = bf16(d["y_bits"]).float()
    # the reference's own bar for this op: allclose(rtol=0.02) (test_group_soft_gemv_fp8.py:80)
    assert torch.allclose(out.cpu().float(), want, rtol=0.02, atol=1e-2)
    gold = O.golden_f32(x, w, s, None, gl, "fp8", gemv=True)
    assert_close_to_golden(out, gold, ulps=2.0)


def test_fp8_all_codes_and_many_rows():
    gen = torch.Generator().manual_seed(3)
    G, K, N = 3, 256, 256
    w = torch.arange(256, dtype=torch.uint8).repeat(G * K * N // 256).reshape(G, K, N)
    w = w[:, torch.randperm(K, generator=gen)]
    s = torch.randn(G, K // 128, N // 128, generator=gen)
    cnt = torch.tensor([3, 0, 6], dtype=torch.int64)
    x = torch.randn(9, K, generator=gen).to(torch.bfloat16)
    gold = O.golden_f32(x, w, s, None, torch.cumsum(cnt, 0), "fp8", gemv=True)
    out, st = run_gemv(x, w, s, torch.cumsum(cnt, 0), "fp8")
    assert st == (0, 0)
    assert_close_to_golden(out, gold, ulps=2.0)


@pytest.mark.parametrize("prefix", ["ref_", "uni_"])
@pytest.mark.parametrize("layout", ["ascend", "canonical"])
def test_fp4_reference_fixture(prefix, layout):
    d = load("gemv_fp4.npz")
    w = torch.from_numpy(d[prefix + ("weight_ascend" if layout == "ascend" else "weight_canonical")])
    s, x, gl = bf16(d[prefix + "scale_bits"]), bf16(d[prefix + "x_bits"]), torch.from_numpy(d[prefix + "group_list"])
    out, st = run_gemv(x, w, s, gl, "fp4", layout=layout)
    assert st == (0, 0)
    # reference bar: allclose(atol=0.5) against the bf16-weight golden (test_group_soft_gemv_fp4.py:223)
    assert torch.allclose(out.cpu().float(), bf16(d[prefix + "y_bits"]).float(), atol=0.5)
    gold = O.golden_f32(x, w, s, None, gl, "fp4", weight_layout=layout, gemv=True)
    assert_close_to_golden(out, gold, ulps=2.0)


def _fp4_case(counts, K, N, seed):
    gen = torch.Generator().manual_seed(seed)
    G = len(counts)
    cnt = torch.tensor(counts, dtype=torch.int64)
    x = torch.randn(int(cnt.sum()), K, generator=gen).to(torch.bfloat16)
    w = torch.randint(0, 256, (G, K, N // 2), generator=gen, dtype=torch.uint8)      # every code, both signs of zero
    scale = (torch.rand(G, K // 16, N, generator=gen) * 0.09 + 0.01).to(torch.bfloat16)
    return x, w, scale, cnt


@pytest.mark.parametrize("layout", ["canonical", "ascend"])
@pytest.mark.parametrize("counts,K,N", [
    ([1, 1, 1, 1], 64, 256),                 # one step of one k group
    ([1, 0, 2, 4, 0, 3], 192, 512),          # three steps: the look-ahead of four runs out inside the loop
    ([0, 5, 9, 1, 3], 448, 768),             # more than four rows per expert
    ([2, 3, 4, 1], 7168, 512),               # benchmark K
])
def test_fp4_tensor_core_path_matches_oracle(counts, K, N, layout):
    """fp4 on random codes: x rows are held as f16 (each scaled by a power of two) and the products run on the
    tensor core; rows of very different magnitude, including ones far outside the f16 range, stay exact."""
    import ascend_kernel_b200 as ak

    x, w, scale, cnt = _fp4_case(counts, K, N, 41)
    row_mag = torch.tensor([2.0 ** e for e in (0, 60, -70, 17, -3, 100, -110, 5, 30, -45)])[torch.arange(x.shape[0]) % 10]
    x = (x.float() * row_mag[:, None]).to(torch.bfloat16)
    gold = O.golden_f32(x, w, scale, None, cnt, "fp4", O.GROUP_LIST_COUNTS, weight_layout="canonical", gemv=True)
    wd = ak.fp4_layout(w.cuda(), to_ascend=True).cpu() if layout == "ascend" else w
    out, st = run_gemv(x, wd, scale, cnt, "fp4", gl_type=1, layout=layout)
    assert st == (0, 0)
    # row by row, each brought back to unit magnitude (a power of two: exact), so that every row is held to the bar
    inv = (1.0 / row_mag)[:, None]
    assert_close_to_golden((out.cpu().float() * inv).to(torch.bfloat16), gold * inv, ulps=2.0)


@pytest.mark.parametrize("layout", ["canonical", "ascend"])
def test_fp4_rows_that_are_not_exact_in_f16_take_the_fp32_path(layout):
    """A row whose elements span more than the f16 format holds (here 2^-100 beside 1), an infinity and a NaN:
    those items fall back to the fp32 multiply-adds; the small elements still count where the weights of the
    large ones are zero."""
    import ascend_kernel_b200 as ak

    x, w, scale, cnt = _fp4_case([2, 4, 1], 256, 256, 43)
    x = x.clone()
    x[0, 5] = 2.0 ** -100                    # expert 0: not representable beside its neighbours
    x[1] = 0
    x[1, 7], x[1, 9] = 2.0 ** -60, 3.0       # row 1: the weight under the large element is zero below
    w[0, 9] = 0                              # (both nibbles of every column: code 0)
    x[2, 3] = float("inf")                   # expert 1: non-finite values are propagated, not scaled
    x[6, 1] = float("nan")
    gold = O.golden_f32(x, w, scale, None, cnt, "fp4", O.GROUP_LIST_COUNTS, weight_layout="canonical", gemv=True)
    wd = ak.fp4_layout(w.cuda(), to_ascend=True).cpu() if layout == "ascend" else w
    out, st = run_gemv(x, wd, scale, cnt, "fp4", gl_type=1, layout=layout)
    assert st == (0, 0)
    o = out.cpu().float()
    finite = torch.isfinite(gold)
    assert torch.equal(torch.isnan(o), torch.isnan(gold)) and torch.equal(torch.isinf(o), torch.isinf(gold))
    assert_close_to_golden(torch.where(finite, o, torch.zeros_like(o)).to(torch.bfloat16),
                           torch.where(finite, gold, torch.zeros_like(gold)), ulps=2.0)
    assert float(o[1].abs().max()) > 0 and float(o[1].abs().max()) < 1e-15   # row 1 is made of its small element only
    assert_close_to_golden((o[1:2] * 2.0 ** 60).to(torch.bfloat16), gold[1:2] * 2.0 ** 60, ulps=2.0)


def test_bad_group_list_is_clamped_and_reported():
    x, w, scale, offset, cnt = _int8_case([1, 2, 1], 128, 256, 9, False)
    bad = torch.tensor([1, 0, 99], dtype=torch.int64)  # not monotone, then beyond M
    out, st = run_gemv(x, w, scale, bad, "int8")
    assert st[0] == 1


@pytest.mark.parametrize("counts,K,N,with_offset", [([1, 0, 2, 4, 0, 3], 256, 512, True), ([1, 6], 384, 256, False)])
def test_int4_per_group_scales_match_oracle(counts, K, N, with_offset):
    gen = torch.Generator().manual_seed(29)
    G = len(counts)
    cnt = torch.tensor(counts, dtype=torch.int64)
    M = int(cnt.sum())
    x = torch.randn(M, K, generator=gen).to(torch.bfloat16)
    w = torch.randint(0, 256, (G, K, N // 2), generator=gen, dtype=torch.uint8).view(torch.int8)
    scale = (torch.rand(G, K // 128, N, generator=gen) * 0.045 + 0.005).to(torch.bfloat16)
    offset = (torch.rand(G, K // 128, N, generator=gen) * 4 - 2).to(torch.bfloat16) if with_offset else None
    gold = O.golden_f32(x, w, scale, offset, cnt, "int4", O.GROUP_LIST_COUNTS, gemv=True)
    out, st = run_gemv(x, w, scale, cnt, "int4", offset, gl_type=1)
    assert st == (0, 0)
    assert_close_to_golden(out, gold)
