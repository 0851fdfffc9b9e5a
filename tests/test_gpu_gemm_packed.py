"""Int8 grouped GEMM on tile-packed weights (dequantised weights as the MMA's A operand in tensor
memory) through the C ABI, against the CPU oracle and against the generic kernel."""
import pytest
import torch

from oracle import oracle as O
from tests.test_gpu_gemm import SENTINEL, _int8_case, run_gemm
from tests.util import assert_close_to_golden, same_bits

pytestmark = pytest.mark.gpu


def run_packed(x, w, scale, offset, gl, gl_type=1, gate_up=False):
    import ascend_kernel_b200 as ak
    from ascend_kernel_b200 import ops

    wp = ops.pack_weight_int8(w.cuda(), gate_up=gate_up)
    n_out = w.shape[2] // 2 if gate_up else w.shape[2]
    out = torch.full((x.shape[0], n_out), SENTINEL, dtype=torch.bfloat16, device="cuda")
    ws = ops.grouped_gemm_packed(x.cuda(), wp, scale.cuda(), None if offset is None else offset.cuda(), gl.cuda(), out,
                                 group_list_type=gl_type, gate_up_silu=gate_up, return_workspace=True)
    torch.cuda.synchronize()
    return out, ak.read_status(ws)


def test_packed_weights_are_exact_on_the_tensor_cores():
    # x = one-hot rows, scale 1, no offset: the output is the int8 weight row itself, exactly; checks
    # the packed byte order, the tensor-memory operand layout and the transposed epilogue at once
    G, K, N = 2, 128, 512
    gen = torch.Generator().manual_seed(1)
    w = torch.randint(-128, 128, (G, K, N), generator=gen, dtype=torch.int8)
    x = torch.zeros(2 * K, K, dtype=torch.bfloat16)
    x[torch.arange(2 * K), torch.arange(2 * K) % K] = 1
    scale = torch.ones(G, N, dtype=torch.bfloat16)
    out, st = run_packed(x, w, scale, None, torch.tensor([K, K]))
    assert st == (0, 0)
    assert torch.equal(out.cpu().float(), w.reshape(2 * K, N).float())


@pytest.mark.parametrize("counts,K,N,with_offset", [
    ([1], 64, 256, False),                         # smallest legal problem
    ([127, 129, 0, 1, 300, 160, 161], 192, 512, True),  # ragged rows, empty expert, 1-3 m-tiles per expert
    ([0, 0, 256, 0], 448, 256, True),              # one expert owns everything, K spans 7 stages
    ([2100], 128, 512, True),                      # 14 m-tiles: more than one L2 super-tile
    ([5] * 70, 64, 256, False),                    # many tiny experts
    ([137, 120, 144, 16, 17], 7168, 256, True),    # the layer's K: 112 stages per tile
])
def test_packed_matches_oracle_and_generic_kernel(counts, K, N, with_offset):
    x, w, scale, offset, cnt = _int8_case(counts, K, N, 13, with_offset, extra_rows=7)
    gold = O.golden_f32(x, w, scale, offset, cnt, "int8", O.GROUP_LIST_COUNTS)
    out, st = run_packed(x, w, scale, offset, cnt)
    assert st == (0, 0)
    assert_close_to_golden(out, gold)
    n_rows = int(cnt.sum())
    assert (out[n_rows:].float() == SENTINEL).all()      # rows of no expert are never written
    ref, _ = run_gemm(x, w, scale, offset, cnt, "int8", gl_type=1)
    # the same exact products summed in fp32, possibly in another order
    assert float((out.float() - ref.float()).abs().max()) <= 0.02 * float(ref.float().abs().max())
    out2, _ = run_packed(x, w, scale, offset, torch.cumsum(cnt, 0), gl_type=0)
    assert same_bits(out, out2)


@pytest.mark.parametrize("counts,K,I", [([33, 0, 150, 170], 256, 256), ([128, 140], 1024, 128)])
def test_packed_gate_up_silu_matches_unfused_operators(counts, K, I):
    import ascend_kernel_b200 as ak

    x, w, scale, offset, cnt = _int8_case(counts, K, 2 * I, 31, True)
    out, st = run_packed(x, w, scale, offset, cnt, gate_up=True)
    assert st == (0, 0)
    h, _ = run_gemm(x, w, scale, offset, cnt, "int8", gl_type=1)
    want = ak.silu_mul(h)
    torch.cuda.synchronize()
    o, g = out.float().cpu(), want.float().cpu()
    assert O.rel_l2(o, g) < 2e-3
    gold_h = O.golden_f32(x, w, scale, offset, cnt, "int8", O.GROUP_LIST_COUNTS).to(torch.bfloat16).float()
    gold = (torch.nn.functional.silu(gold_h[:, :I]) * gold_h[:, I:]).to(torch.bfloat16).float()
    assert O.rel_l2(o, gold) < 4e-3


def test_packed_bad_group_list_is_clamped_and_reported():
    x, w, scale, offset, cnt = _int8_case([10, 20], 64, 256, 9, False)
    out, st = run_packed(x, w, scale, None, torch.tensor([20, 5]), gl_type=0)
    assert st[0] == 1 and st[1] == 1


def test_packed_scatter_stores_rows_where_the_codes_say():
    """The scatter variant against the plain one: row r lands at row (code & 0xffffffff) of destination tensor
    (code >> 32); a code naming no destination or a row past the destination's end is skipped."""
    from ascend_kernel_b200 import ops

    x, w, scale, offset, cnt = _int8_case([137, 0, 20, 161], 256, 512, 3, True)
    M, N = x.shape[0], w.shape[2]
    want, st = run_packed(x, w, scale, offset, cnt)
    assert st == (0, 0)
    gen = torch.Generator().manual_seed(8)
    perm = torch.randperm(M, generator=gen)
    base = (torch.arange(M) % 2).to(torch.int64)              # two destination tensors, rows alternate
    code = (base << 32) | perm.to(torch.int64)
    code[5] = (7 << 32) | 0                                    # no such destination
    code[9] = (0 << 32) | (M + 10)                             # row past the end
    d0 = torch.full((M, N), SENTINEL, dtype=torch.bfloat16, device="cuda")
    d1 = torch.full((M, N), SENTINEL, dtype=torch.bfloat16, device="cuda")
    wp = ops.pack_weight_int8(w.cuda())
    ops.grouped_gemm_packed_scatter(x.cuda(), wp, scale.cuda(), offset.cuda(), cnt.cuda(), code.cuda(),
                                    [d0.data_ptr(), d1.data_ptr()], M, group_list_type=1)
    torch.cuda.synchronize()
    got = torch.stack([d0, d1])
    for r in range(M):
        if r in (5, 9):
            continue
        assert torch.equal(got[int(base[r]), int(perm[r])].view(torch.int16), want[r].view(torch.int16)), r
    written = torch.zeros(2, M, dtype=torch.bool)
    keep = torch.ones(M, dtype=torch.bool)
    keep[5] = keep[9] = False
    written[base[keep], perm[keep]] = True
    assert bool((got[~written.cuda()].float() == SENTINEL).all())   # nothing else was touched


@pytest.mark.parametrize("K,N", [(192, 256), (7168, 512)])
def test_row_sums_from_the_gather_give_the_same_bits(K, N):
    """gather_rows(with_sums=True) adds the rows up in the order of the GEMM's own row-sum pass: a packed GEMM that is
    handed those sums returns exactly what it returns when it computes them itself."""
    from ascend_kernel_b200 import ops

    counts = [5, 0, 137, 33, 160, 1]
    x, w, scale, offset, cnt = _int8_case(counts, K, N, 23, True)
    src = torch.randn(50, K, generator=torch.Generator().manual_seed(5)).to(torch.bfloat16).cuda()
    index = torch.randint(0, 50, (int(cnt.sum()),), generator=torch.Generator().manual_seed(6), dtype=torch.int32).cuda()
    rows, sums = ops.gather_rows(src, index, with_sums=True)
    assert torch.equal(rows, ops.gather_rows(src, index))
    assert torch.allclose(sums.cpu(), rows.cpu().float().sum(1), rtol=1e-4, atol=1e-2)
    wp = ops.pack_weight_int8(w.cuda())
    a = torch.full((rows.shape[0], N), SENTINEL, dtype=torch.bfloat16, device="cuda")
    b = torch.full_like(a, SENTINEL)
    ops.grouped_gemm_packed(rows, wp, scale.cuda(), offset.cuda(), cnt.cuda(), a, group_list_type=1)
    ops.grouped_gemm_packed(rows, wp, scale.cuda(), offset.cuda(), cnt.cuda(), b, group_list_type=1, x_rowsum=sums)
    torch.cuda.synchronize()
    assert torch.equal(a.view(torch.int16), b.view(torch.int16))
    gold = O.golden_f32(rows.cpu(), w, scale, offset, cnt, "int8", O.GROUP_LIST_COUNTS)
    assert_close_to_golden(b, gold)
