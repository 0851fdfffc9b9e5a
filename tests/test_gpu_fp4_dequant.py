"""FP4(e2m1) -> BF16 dequantisation through the C ABI: bit-exact against the CPU oracle."""
import pytest
import torch

from oracle import oracle as O
from tests.util import same_bits

pytestmark = pytest.mark.gpu


def _run(codes, scale):
    import ascend_kernel_b200 as ak

    out = torch.full((*codes.shape[:-1], codes.shape[-1] * 2), 7.0, dtype=torch.bfloat16, device="cuda")
    ak.fp4_dequant(codes.cuda(), None if scale is None else scale.cuda(), out)
    torch.cuda.synchronize()
    return out.cpu()


def test_all_codes_all_bench_exponents():
    # every byte value (all code pairs) under each exponent of the benchmark range 119..127
    codes = torch.arange(256, dtype=torch.uint8).repeat_interleave(16).reshape(256, 16)  # one 32-block each
    for s in range(119, 128):
        scale = torch.full((256, 1), s, dtype=torch.uint8)
        assert same_bits(_run(codes, scale), O.fp4_dequant_e8m0(codes, scale)), s


def test_seeded_random_bit_exact_ragged_size():
    gen = torch.Generator().manual_seed(2)
    # 3 x 2080 elements: not a multiple of the per-block work of the kernel
    codes = torch.randint(0, 256, (3, 1040), generator=gen, dtype=torch.uint8)
    scale = torch.randint(119, 128, (3, 65), generator=gen, dtype=torch.uint8)
    assert same_bits(_run(codes, scale), O.fp4_dequant_e8m0(codes, scale))
    assert same_bits(_run(codes, None), O.fp4_dequant_e8m0(codes, None))


def test_extreme_exponents():
    codes = torch.arange(256, dtype=torch.uint8).repeat_interleave(16).reshape(256, 16)
    for s in (0, 1, 2, 60, 126, 128, 200, 253, 254):
        scale = torch.full((256, 1), s, dtype=torch.uint8)
        got, want = _run(codes, scale), O.fp4_dequant_e8m0(codes, scale)
        assert same_bits(got, want), s
    got = _run(codes, torch.full((256, 1), 255, dtype=torch.uint8))
    assert torch.isnan(got.float()).all()  # e8m0 255 is NaN


def test_empty_and_errors():
    import ascend_kernel_b200 as ak
    from ascend_kernel_b200 import _abi

    out = torch.empty(0, dtype=torch.bfloat16, device="cuda")
    ak.fp4_dequant(torch.empty(0, dtype=torch.uint8, device="cuda"), None, out)
    rc = _abi.lib.b200moe_fp4_dequant(16, None, 16, 48, 0, None)  # 48 is not a multiple of 32
    assert rc == 3


def test_large_property_linearity_in_exponent():
    # 64 Mi elements: doubling every exponent doubles every output exactly
    gen = torch.Generator(device="cuda").manual_seed(5)
    n = 1 << 26
    codes = torch.randint(0, 256, (n // 2,), generator=gen, device="cuda", dtype=torch.uint8)
    s0 = torch.randint(119, 127, (n // 32,), generator=gen, device="cuda", dtype=torch.uint8)
    import ascend_kernel_b200 as ak

    a = torch.empty(n, dtype=torch.bfloat16, device="cuda")
    b = torch.empty(n, dtype=torch.bfloat16, device="cuda")
    ak.fp4_dequant(codes, s0, a)
    ak.fp4_dequant(codes, s0 + 1, b)
    assert torch.equal(a.float() * 2, b.float())
    # spot check of a slice against the oracle
    sl = slice(123 * 32 // 2, 123 * 32 // 2 + 4096)
    want = O.fp4_dequant_e8m0(codes[sl].cpu(), s0[123:123 + 256].cpu())
    assert same_bits(a[123 * 32:123 * 32 + 8192].cpu(), want)


def test_fp4_layout_roundtrip_matches_oracle():
    import ascend_kernel_b200 as ak
    from tests.util import load

    d = load("fp4_layout.npz")
    canon = torch.from_numpy(d["canonical"]).cuda()
    asc = torch.from_numpy(d["ascend"]).cuda()
    assert torch.equal(ak.fp4_layout(canon, True), asc)
    assert torch.equal(ak.fp4_layout(asc, False), canon)
