"""The benchmark configurations at full size.  The CPU oracle cannot produce whole outputs of
these sizes in seconds, so parity is checked through properties that do not depend on size --
exact linearity under scaling by two, invariance under a permutation of the rows of an expert,
agreement of the two independent kernels (GEMM and GEMV) on the same data, rows of no expert left
untouched -- and by the oracle on a sample of rows, experts and tokens."""
import pytest
import torch

from oracle import oracle as O
from tests.util import assert_close_to_golden

pytestmark = pytest.mark.gpu
SENTINEL = -768.0


def _sample_rows_against_oracle(c, y, counts, rows, ct="int8", gemv=False):
    """Oracle on single rows: the row's expert is found from the counts, its weights come to the CPU."""
    starts = torch.cumsum(counts, 0) - counts
    for r in rows:
        g = int(torch.searchsorted(torch.cumsum(counts, 0), torch.tensor(r), right=True))
        assert starts[g] <= r < starts[g] + counts[g]
        sl = slice(g, g + 1)
        gold = O.golden_f32(c["x"][r:r + 1].cpu(), c["weight"][sl].cpu(), c["scale"][sl].cpu(),
                            None if c["offset"] is None else c["offset"][sl].cpu(), torch.tensor([1]), ct,
                            O.GROUP_LIST_COUNTS, gemv=gemv)
        assert_close_to_golden(y[r:r + 1], gold)


def _stratified_rows(counts, n_experts=8):
    """Rows to check with the oracle, grouped by expert: experts spread over the load ranks (the largest,
    the smallest non-empty one and others in between), and inside each the rows at the tile boundaries of
    both grouped-GEMM kernels (127/128/129, 159/160/161, 255/256/257), the first two and the last two."""
    starts = torch.cumsum(counts, 0) - counts
    order = torch.argsort(counts, descending=True)
    nonempty = [int(e) for e in order if counts[e] > 0]
    picks = sorted({nonempty[int(round(i * (len(nonempty) - 1) / (n_experts - 1)))] for i in range(n_experts)})
    out = {}
    for e in picks:
        n = int(counts[e])
        local = sorted({r for r in (0, 1, 127, 128, 129, 159, 160, 161, 255, 256, 257, n - 2, n - 1) if 0 <= r < n})
        out[e] = [int(starts[e]) + r for r in local]
    return out


def _check_rows_by_expert(c, y, counts, ct, layout="ascend", gemv=False, ulps=1.0, n_experts=8):
    """The oracle on the stratified rows: one dequantisation per sampled expert, all of its rows at once,
    whole rows (so the first and the last column tile are covered).  Returns the number of rows checked."""
    n = 0
    for e, rows in _stratified_rows(counts, n_experts).items():
        sl = slice(e, e + 1)
        xr = c["x"][rows].cpu()
        gold = O.golden_f32(xr, c["weight"][sl].cpu(), c["scale"][sl].cpu(),
                            None if c.get("offset") is None else c["offset"][sl].cpu(), torch.tensor([len(rows)]), ct,
                            O.GROUP_LIST_COUNTS, weight_layout=layout, gemv=gemv)
        assert_close_to_golden(y[rows], gold, ulps=ulps)
        n += len(rows)
    return n


def test_prefill_gemm_config3_properties():
    import ascend_kernel_b200 as ak
    from ascend_kernel_b200 import inputs

    c = inputs.config3("cuda")
    counts = c["counts"].cpu()
    M, N = c["x"].shape[0], c["weight"].shape[2]
    # three extra rows owned by nobody
    x = torch.cat([c["x"], torch.randn(3, c["x"].shape[1], device="cuda").to(torch.bfloat16)])
    y = torch.full((M + 3, N), SENTINEL, dtype=torch.bfloat16, device="cuda")
    ws = ak.grouped_gemm(x, c["weight"], c["scale"], c["offset"], c["counts"], "int8", y, group_list_type=1,
                         return_workspace=True)
    torch.cuda.synchronize()
    assert ak.read_status(ws) == (0, 0)
    assert bool((y[M:] == SENTINEL).all())
    assert not bool((y[:M] == SENTINEL).all(dim=1).any())
    # the oracle on rows of the largest expert, the smallest non-empty one and a few others
    order = torch.argsort(counts, descending=True)
    starts = torch.cumsum(counts, 0) - counts
    nonempty = order[counts[order] > 0]
    picks = [int(starts[nonempty[0]]), int(starts[nonempty[0]] + counts[nonempty[0]] - 1), int(starts[nonempty[-1]]),
             int(starts[nonempty[len(nonempty) // 2]] + 1), 0, M - 1]
    _sample_rows_against_oracle(dict(c, x=x), y, counts, picks)
    assert _check_rows_by_expert(dict(c, x=x), y, counts, "int8", n_experts=12) >= 64
    # the packed entry point on the same problem (experts from 0 to 16 000 rows: up to 105 m-tiles of one
    # expert): the same exact products, summed per tile in the same k order
    from ascend_kernel_b200 import ops

    yp = torch.full((M + 3, N), SENTINEL, dtype=torch.bfloat16, device="cuda")
    wp = ops.pack_weight_int8(c["weight"])
    ws = ops.grouped_gemm_packed(x, wp, c["scale"], c["offset"], c["counts"], yp, group_list_type=1, return_workspace=True)
    torch.cuda.synchronize()
    assert ak.read_status(ws) == (0, 0)
    del wp
    assert bool((yp[M:] == SENTINEL).all())
    assert _check_rows_by_expert(dict(c, x=x), yp, counts, "int8", n_experts=12) >= 64
    assert float((yp[:M].float() - y[:M].float()).abs().max()) <= 0.02 * float(y[:M].float().abs().max())
    del yp
    # linearity: scaling x by two scales every output by two, exactly (no rounding is involved)
    y2 = torch.empty_like(y)
    ak.grouped_gemm((x.float() * 2).to(torch.bfloat16), c["weight"], c["scale"], c["offset"], c["counts"], "int8", y2,
                    group_list_type=1)
    torch.cuda.synchronize()
    assert torch.equal((y[:M].float() * 2).to(torch.bfloat16).view(torch.int16), y2[:M].view(torch.int16))
    # rows are independent: reversing the rows of every expert reverses its outputs, bit for bit
    idx = torch.cat([torch.arange(int(s) + int(n) - 1, int(s) - 1, -1) for s, n in zip(starts, counts) if n > 0]).cuda()
    y3 = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    ak.grouped_gemm(x[:M][idx].contiguous(), c["weight"], c["scale"], c["offset"], c["counts"], "int8", y3,
                    group_list_type=1)
    torch.cuda.synchronize()
    assert torch.equal(y3.view(torch.int16), y[:M][idx].view(torch.int16))


@pytest.mark.parametrize("name", ["int4", "fp8", "fp4", "fp4_stored_order"])
def test_prefill_gemm_config3_other_formats_sampled_rows(name):
    """The other weight formats at the prefill shape (65 536 rows, Zipf split over 256 experts, K = 7168,
    N = 4096): int4 with per-128-k scale / offset (variant B of the benchmark configuration), and the
    reference's own fp8 and fp4 formats, the latter in the canonical and in the stored order."""
    import ascend_kernel_b200 as ak
    from ascend_kernel_b200 import inputs

    kind = "fp4" if name.startswith("fp4") else name
    layout = "ascend" if name == "fp4_stored_order" else "canonical"
    c = inputs.config3_variants("cuda", kind)
    if name == "fp4_stored_order":
        c["weight"] = ak.fp4_layout(c["weight"], to_ascend=True)
    counts = c["counts"].cpu()
    M, N = c["x"].shape[0], 4096
    y = torch.full((M, N), SENTINEL, dtype=torch.bfloat16, device="cuda")
    gl = c["counts"] if kind == "int4" else torch.cumsum(c["counts"], 0)
    ws = ak.grouped_gemm(c["x"], c["weight"], c["scale"], c["offset"], gl, kind, y,
                         group_list_type=1 if kind == "int4" else 0, weight_layout=layout, return_workspace=True)
    torch.cuda.synchronize()
    assert ak.read_status(ws) == (0, 0)
    assert not bool((y == SENTINEL).all(dim=1).any())
    assert _check_rows_by_expert(c, y, counts, kind, layout=layout, n_experts=12) >= 64


def test_decode_gemv_config1_against_gemm_and_oracle():
    import ascend_kernel_b200 as ak
    from ascend_kernel_b200 import inputs

    c = inputs.config1("cuda")
    counts = c["counts"].cpu()
    M, N = c["x"].shape[0], c["weight"].shape[2]
    yv = torch.full((M, N), SENTINEL, dtype=torch.bfloat16, device="cuda")
    ws = ak.grouped_soft_gemv(c["x"], c["weight"], c["scale"], c["counts"], "int8", yv, group_list_type=1,
                              return_workspace=True)
    ym = torch.full((M, N), SENTINEL, dtype=torch.bfloat16, device="cuda")
    ak.grouped_gemm(c["x"], c["weight"], c["scale"], None, c["counts"], "int8", ym, group_list_type=1)
    torch.cuda.synchronize()
    assert ak.read_status(ws)[0] == 0
    # two independent kernels, same exact weights, fp32 accumulation in different orders
    a, b = yv.float(), ym.float()
    assert O.rel_l2(a, b) < 2e-3
    assert float(((a - b).abs() > torch.maximum(torch.full_like(b, 2e-2), 2.0 ** (torch.floor(torch.log2(b.abs().clamp_min(1e-30))) - 7))).float().mean()) == 0.0
    rows = [0, M // 3, M - 1]
    _sample_rows_against_oracle(c, yv, counts, rows, gemv=True)
    assert _check_rows_by_expert(c, yv, counts, "int8", gemv=True, n_experts=24) >= 24
    # linearity
    yv2 = torch.empty_like(yv)
    ak.grouped_soft_gemv((c["x"].float() * 2).to(torch.bfloat16), c["weight"], c["scale"], c["counts"], "int8", yv2,
                         group_list_type=1)
    torch.cuda.synchronize()
    assert torch.equal((yv.float() * 2).to(torch.bfloat16).view(torch.int16), yv2.view(torch.int16))


def test_decode_gemv_config1_pass2_and_reference_formats():
    """The decode routing (32 tokens x top-8 over 256 experts) on the down-projection shape (K = 2048,
    N = 7168, int8) and on the gate/up shape with the reference's fp8 and fp4 formats.  The fp8 / fp4 GEMV
    keeps dequantised weights in fp32 and sums in another order than the golden: two bf16 steps are
    allowed where one step exceeds the absolute bound."""
    import ascend_kernel_b200 as ak
    from ascend_kernel_b200 import inputs

    counts = inputs.routed_counts(32, 256, 8, torch.Generator().manual_seed(1))
    M = int(counts.sum())
    gen = torch.Generator(device="cuda").manual_seed(11)
    # pass 2: int8, K = 2048 -> N = 7168
    K2, N2 = 2048, 7168
    c = dict(x=torch.randn(M, K2, generator=gen, device="cuda").to(torch.bfloat16),
             weight=inputs.int8_weights(256, K2, N2, gen, "cuda"),
             scale=(torch.rand(256, N2, generator=gen, device="cuda") * 0.009 + 0.001).to(torch.bfloat16), offset=None)
    y = torch.full((M, N2), SENTINEL, dtype=torch.bfloat16, device="cuda")
    ak.grouped_soft_gemv(c["x"], c["weight"], c["scale"], counts.cuda(), "int8", y, group_list_type=1)
    torch.cuda.synchronize()
    assert _check_rows_by_expert(c, y, counts, "int8", gemv=True, n_experts=24) >= 24
    del c, y
    torch.cuda.empty_cache()
    K1, N1 = 7168, 4096
    x1 = torch.randn(M, K1, generator=gen, device="cuda").to(torch.bfloat16)
    for name in ("fp8", "fp4", "fp4_stored_order"):
        kind = "fp4" if name.startswith("fp4") else name
        layout = "ascend" if name == "fp4_stored_order" else "canonical"
        cols = N1 if kind == "fp8" else N1 // 2
        w = torch.empty(256, K1, cols, dtype=torch.uint8, device="cuda")
        for g in range(256):
            w[g] = torch.randint(0, 256, (K1, cols), generator=gen, device="cuda", dtype=torch.uint8)
        if kind == "fp8":
            sc = torch.randn(256, K1 // 128, N1 // 128, generator=gen, device="cuda")
        else:
            sc = (torch.rand(256, K1 // 16, N1, generator=gen, device="cuda") * 3 + 0.25).to(torch.bfloat16)
            w = w.view(torch.int8)
            if layout == "ascend":
                w = ak.fp4_layout(w, to_ascend=True)
        y = torch.full((M, N1), SENTINEL, dtype=torch.bfloat16, device="cuda")
        ak.grouped_soft_gemv(x1, w, sc, counts.cuda(), kind, y, group_list_type=1, weight_layout=layout)
        torch.cuda.synchronize()
        c = dict(x=x1, weight=w, scale=sc, offset=None)
        assert _check_rows_by_expert(c, y, counts, kind, layout=layout, gemv=True, ulps=2.0, n_experts=16) >= 16, name
        del w, sc, y, c
        torch.cuda.empty_cache()


def test_fp4_dequant_config2_bit_exact_against_table_lookup():
    import ascend_kernel_b200 as ak
    from ascend_kernel_b200 import inputs

    d = inputs.config2("cuda")
    codes, scale = d["codes"], d["scale"]
    n = codes.numel() * 2
    out = torch.empty(n, dtype=torch.bfloat16, device="cuda")
    ak.fp4_dequant(codes, scale, out)
    torch.cuda.synchronize()
    lut = O.e2m1_table().cuda()  # 16 float32 values
    flat_c, flat_s = codes.reshape(-1), scale.reshape(-1)
    step = 1 << 26  # bytes of codes per chunk: bounds the temporaries of the check
    for i in range(0, flat_c.numel(), step):
        cb = flat_c[i:i + step].long()
        vals = torch.stack([lut[cb & 15], lut[cb >> 4]], dim=1).reshape(-1)           # low nibble = even element
        sc = torch.exp2(flat_s[i // 16:(i + cb.numel()) // 16].float() - 127.0)        # one scale per 32 elements
        want = (vals.reshape(-1, 32) * sc[:, None]).reshape(-1).to(torch.bfloat16)
        got = out[2 * i:2 * (i + cb.numel())]
        assert torch.equal(got.view(torch.int16), want.view(torch.int16)), i


def test_moe_layer_config4_sampled_tokens_against_oracle():
    from ascend_kernel_b200 import inputs
    from ascend_kernel_b200.moe_layer import MoELayer

    cfg = dict(n_tokens=4096, hidden=7168, n_experts=256, inter=2048, top_k=8, seed=4)
    c = inputs.config4("cuda", **cfg)
    layer = MoELayer(c["w13"], c["s13"], c["o13"], c["w2"], c["s2"], c["o2"], 256, 8)
    out = layer.forward(c["x"].cuda(), c["logits"].cuda())
    torch.cuda.synchronize()
    # tokens whose 8th and 9th largest logits differ (bf16 logits tie now and then, and a tie at the
    # boundary may be broken either way)
    srt = torch.sort(c["logits"].float(), dim=1, descending=True)[0]
    tie_free = (srt[:, 7] != srt[:, 8]).nonzero().flatten().tolist()
    toks = sorted({tie_free[int(round(i * (len(tie_free) - 1) / 15))] for i in range(16)})
    w, idx = O.route_topk(c["logits"][toks], 8)
    for i, t in enumerate(toks):
        acc = torch.zeros(cfg["hidden"], dtype=torch.float64)
        for j in range(8):
            e = int(idx[i, j])
            sl = slice(e, e + 1)
            one = torch.tensor([1])
            h = O.golden_f32(c["x"][t:t + 1], c["w13"][sl].cpu(), c["s13"][sl].cpu(), c["o13"][sl].cpu(), one, "int8",
                             O.GROUP_LIST_COUNTS).to(torch.bfloat16).float()
            I = cfg["inter"]
            act = (torch.nn.functional.silu(h[:, :I]) * h[:, I:]).to(torch.bfloat16)
            y = O.golden_f32(act, c["w2"][sl].cpu(), c["s2"][sl].cpu(), c["o2"][sl].cpu(), one, "int8",
                             O.GROUP_LIST_COUNTS).to(torch.bfloat16).double()
            acc += float(w[i, j]) * y[0]
        got = out[t].cpu().double()
        assert O.rel_l2(got, acc) < 4e-3, (t, O.rel_l2(got, acc))
