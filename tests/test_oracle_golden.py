"""Pins the CPU oracle to the fixtures generated from the reference's own Python helpers
(tests/golden/make_golden.py).  CPU only."""
import numpy as np
import torch

from oracle import oracle as O
from tests.util import bf16, load, same_bits


def test_decode_tables_match_reference_bit_tricks():
    d = load("decode_tables.npz")
    assert same_bits(O.e4m3_table().to(torch.bfloat16), bf16(d["e4m3_bf16_bits"]))
    assert same_bits(O.e2m1_table().to(torch.bfloat16), bf16(d["e2m1_bf16_bits"]))


def test_decode_tables_known_answers():
    t4 = O.e2m1_table().tolist()
    assert t4[:8] == [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]
    assert t4[9:] == [-0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0]
    assert np.signbit(np.float32(t4[8])) and t4[8] == 0.0
    t8 = O.e4m3_table()
    assert t8[0x7F] == 480.0 and t8[0xFF] == -480.0  # no NaN handling in the reference decode
    assert t8[0x01] == 2.0 ** -9 and t8[0x08] == 2.0 ** -6 and t8[0x38] == 1.0
    ref = torch.arange(256, dtype=torch.uint8).view(torch.float8_e4m3fn).float()
    ok = ~torch.isnan(ref)
    assert torch.equal(t8[ok], ref[ok])


def test_fp4_layouts_match_reference_repack():
    d = load("fp4_layout.npz")
    canon = torch.from_numpy(d["canonical"])
    asc = torch.from_numpy(d["ascend"])
    assert torch.equal(O.ascend_shuffle(canon), asc)
    assert torch.equal(O.ascend_unshuffle(asc), canon)
    # canonical = codes along N, low nibble even n; source was packed along K, low nibble even k
    pk = torch.from_numpy(d["packed_along_k"])
    codes_nk = O.fp4_unpack(pk)  # [G, N, K]
    assert torch.equal(O.fp4_unpack(canon), codes_nk.transpose(1, 2))
    # closed form of the permutation
    G, K, C = canon.shape
    flat_c = canon.reshape(-1)
    flat_a = asc.reshape(-1)
    rng = np.random.default_rng(0)
    for _ in range(500):
        r = int(rng.integers(0, G * K))
        c = int(rng.integers(0, C))
        assert flat_a[O.ascend_offset(r, c, C)] == flat_c[r * C + c]


def test_gemm_fp8_matches_reference_golden():
    d = load("gemm_fp8.npz")
    w, s = torch.from_numpy(d["weight"]), torch.from_numpy(d["scale"])
    wd = O.dequant_fp8(w, s, round_bf16=True).to(torch.bfloat16)
    assert same_bits(wd, bf16(d["wd_bits"]))
    x, gl = bf16(d["x_bits"]), torch.from_numpy(d["group_list"])
    out = torch.zeros(x.shape[0], w.shape[2], dtype=torch.bfloat16)
    O.grouped_gemm(x, w, s, torch.zeros_like(s), gl, "fp8", out)
    assert same_bits(out, bf16(d["y_bits"]))


def test_gemv_fp8_keeps_fp32_weights():
    d = load("gemv_fp8.npz")
    w, s = torch.from_numpy(d["weight"]), torch.from_numpy(d["scale"])
    wd = O.dequant_fp8(w, s, round_bf16=False)
    assert torch.equal(wd, torch.from_numpy(d["wd_f32"]))
    x, gl = bf16(d["x_bits"]), torch.from_numpy(d["group_list"])
    out = torch.zeros(x.shape[0], w.shape[2], dtype=torch.bfloat16)
    O.grouped_soft_gemv(x, w, s, gl, "fp8", out)
    assert same_bits(out, bf16(d["y_bits"]))


def _fp4_case(d, p, gemv):
    w = torch.from_numpy(d[p + "weight_ascend"])
    assert torch.equal(O.ascend_unshuffle(w), torch.from_numpy(d[p + "weight_canonical"]))
    s = bf16(d[p + "scale_bits"])
    wd = O.dequant_fp4(O.ascend_unshuffle(w), s, round_bf16=True).to(torch.bfloat16)
    assert same_bits(wd[0], bf16(d[p + "wd0_bits"])) and same_bits(wd[3], wd[0])
    x, gl = bf16(d[p + "x_bits"]), torch.from_numpy(d[p + "group_list"])
    out = torch.zeros(x.shape[0], 2 * w.shape[2], dtype=torch.bfloat16)
    if gemv:
        O.grouped_soft_gemv(x, w, s, gl, "fp4", out)
        # the reference golden rounds weights to bf16, the GEMV kernel does not: tolerance of
        # test_group_soft_gemv_fp4.py:223
        assert torch.allclose(out.float(), bf16(d[p + "y_bits"]).float(), atol=0.5)
    else:
        O.grouped_gemm(x, w, s, torch.zeros_like(s), gl, "fp4", out)
        assert same_bits(out, bf16(d[p + "y_bits"]))


def test_gemm_fp4_matches_reference_golden():
    d = load("gemm_fp4.npz")
    _fp4_case(d, "ref_", False)
    _fp4_case(d, "uni_", False)


def test_gemv_fp4_within_reference_tolerance():
    d = load("gemv_fp4.npz")
    _fp4_case(d, "ref_", True)
    _fp4_case(d, "uni_", True)


def test_group_list_semantics():
    x = torch.arange(12, dtype=torch.float32).reshape(6, 2).to(torch.bfloat16)
    wd = torch.stack([torch.eye(2) * (g + 1) for g in range(3)])
    cum = O.grouped_matmul(x, wd, torch.tensor([2, 2, 5]))
    cnt = O.grouped_matmul(x, wd, torch.tensor([2, 0, 3]), O.GROUP_LIST_COUNTS)
    assert torch.equal(torch.nan_to_num(cum, 7.0), torch.nan_to_num(cnt, 7.0))
    assert torch.isnan(cum[5]).all() and torch.equal(cum[4], x[4].float() * 3)
    out = torch.full((6, 2), -1.0, dtype=torch.bfloat16)
    O._store(out, cum)
    assert (out[5] == -1).all()  # rows past the last boundary are left untouched


def test_e8m0_dequant_exact():
    gen = torch.Generator().manual_seed(2)
    codes = torch.randint(0, 256, (4, 64), generator=gen, dtype=torch.uint8)
    sc = torch.randint(119, 128, (4, 4), generator=gen, dtype=torch.uint8)
    out = O.fp4_dequant_e8m0(codes, sc)
    v = O.e2m1_table()[O.fp4_unpack(codes).long()].double()
    ex = v * torch.pow(2.0, sc.double() - 127).repeat_interleave(32, dim=-1)
    assert torch.equal(out.double(), ex)
    assert torch.equal(O.fp4_dequant_e8m0(codes, None).double(), v)


def test_scale_fold_matches_reference_helper():
    """The two-level FP4 scale fold against the output of the reference's own anti_quant_fp8_scale."""
    d = load("scale_fold.npz")
    for tag in ("one", "two"):
        got = O.fp4_scale_fold(bf16(d[tag + "_block_bits"]), torch.from_numpy(d[tag + "_global"]))
        assert same_bits(got, bf16(d[tag + "_folded_bits"])), tag
