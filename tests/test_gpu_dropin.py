"""The compiled `cinfer_ascendc` module called the way the reference's own tests call it
(keyword arguments in their order, output written in place, no return value), on the
reference-derived fixtures."""
import pytest
import torch

from oracle import oracle as O
from tests.util import assert_close_to_golden, bf16, load

pytestmark = pytest.mark.gpu


def _module():
    from ascend_kernel_b200 import cinfer_ascendc

    return cinfer_ascendc


def test_grouped_gemm_fp8_call_shape_of_reference_test():
    m = _module()
    d = load("gemm_fp8.npz")
    w1w3 = torch.from_numpy(d["weight"]).cuda()
    scale = torch.from_numpy(d["scale"]).cuda()
    x = bf16(d["x_bits"]).cuda()
    expert_tokens = torch.from_numpy(d["group_list"]).cuda()
    scale_off = torch.zeros_like(scale)
    output = torch.zeros([x.shape[0], w1w3.shape[2]], device="cuda", dtype=torch.bfloat16)
    ret = m.grouped_gemm(x, w1w3, output=output, antiquantOffsetOptional=scale_off, antiquantScaleOptional=scale,
                         groupListOptional=expert_tokens, computeType="fp8")
    torch.cuda.synchronize()
    assert ret is None
    assert torch.allclose(output.cpu().float(), bf16(d["y_bits"]).float(), atol=0.02, rtol=1e-2)
    gold = O.golden_f32(x.cpu(), w1w3.cpu(), scale.cpu(), None, expert_tokens.cpu(), "fp8")
    assert_close_to_golden(output, gold)


def test_grouped_gemm_fp4_ascend_layout():
    m = _module()
    d = load("gemm_fp4.npz")
    w = torch.from_numpy(d["ref_weight_ascend"]).cuda()
    new_scale = bf16(d["ref_scale_bits"]).cuda()
    x = bf16(d["ref_x_bits"]).cuda()
    gl = torch.from_numpy(d["ref_group_list"]).cuda()
    output = torch.zeros([x.shape[0], w.shape[-1] * 2], dtype=x.dtype, device=x.device)
    m.grouped_gemm(x, w, output=output, antiquantOffsetOptional=torch.zeros_like(new_scale),
                   antiquantScaleOptional=new_scale, groupListOptional=gl, computeType="fp4")
    torch.cuda.synchronize()
    assert torch.allclose(output.cpu().float(), bf16(d["ref_y_bits"]).float(), atol=0.15)


def test_grouped_soft_gemv_fp8_and_fp4():
    m = _module()
    d = load("gemv_fp8.npz")
    w, s = torch.from_numpy(d["weight"]).cuda(), torch.from_numpy(d["scale"]).cuda()
    x, gl = bf16(d["x_bits"]).cuda(), torch.from_numpy(d["group_list"]).cuda()
    output = torch.zeros([x.shape[0], w.shape[2]], device="cuda", dtype=torch.bfloat16)
    m.grouped_soft_gemv(x, w, output=output, scale=s, groupList=gl, computeType="fp8")
    torch.cuda.synchronize()
    assert torch.allclose(output.cpu().float(), bf16(d["y_bits"]).float(), rtol=0.02, atol=1e-2)
    d = load("gemv_fp4.npz")
    w, s = torch.from_numpy(d["ref_weight_ascend"]).cuda(), bf16(d["ref_scale_bits"]).cuda()
    x, gl = bf16(d["ref_x_bits"]).cuda(), torch.from_numpy(d["ref_group_list"]).cuda()
    output = torch.zeros([x.shape[0], w.shape[-1] * 2], dtype=x.dtype, device=x.device)
    m.grouped_soft_gemv(x, w, output=output, scale=s, groupList=gl, computeType="fp4")
    torch.cuda.synchronize()
    assert torch.allclose(output.cpu().float(), bf16(d["ref_y_bits"]).float(), atol=0.5)


def test_int8_counts_mode_and_errors():
    m = _module()
    from ascend_kernel_b200 import inputs

    c = {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in inputs.config0().items()}
    out = torch.zeros(c["x"].shape[0], c["weight"].shape[2], dtype=torch.bfloat16, device="cuda")
    m.grouped_gemm(c["x"], c["weight"], c["scale"], c["offset"], c["counts"], "int8", out, group_list_type=1)
    torch.cuda.synchronize()
    gold = O.golden_f32(c["x"].cpu(), c["weight"].cpu(), c["scale"].cpu(), c["offset"].cpu(), c["counts"].cpu(),
                        "int8", O.GROUP_LIST_COUNTS)
    assert_close_to_golden(out, gold)
    with pytest.raises(RuntimeError, match="Host tiling failed"):
        m.grouped_gemm(c["x"], c["weight"], c["scale"], c["offset"], c["counts"], "fp16", out)
    with pytest.raises(RuntimeError):
        m.grouped_gemm(c["x"].cpu(), c["weight"], c["scale"], c["offset"], c["counts"], "int8", out)


def test_fp4_dequant_entry():
    m = _module()
    gen = torch.Generator().manual_seed(2)
    codes = torch.randint(0, 256, (8, 64), generator=gen, dtype=torch.uint8)
    sc = torch.randint(119, 128, (8, 4), generator=gen, dtype=torch.uint8)
    out = torch.empty(8, 128, dtype=torch.bfloat16, device="cuda")
    m.fp4_dequant(codes.cuda(), sc.cuda(), out)
    torch.cuda.synchronize()
    assert torch.equal(out.cpu().view(torch.int16), O.fp4_dequant_e8m0(codes, sc).view(torch.int16))


def test_hashed_inputs_have_the_same_bits_on_the_gpu_and_on_the_cpu():
    """The benchmark's CPU arm and GPU arm materialise the layer's weights separately; both must see the
    same bits."""
    from ascend_kernel_b200 import inputs

    for seed in (1, 9_000_017):
        assert torch.equal(inputs.hashed_bytes((300, 517), seed, "cuda", torch.int8).cpu(),
                           inputs.hashed_bytes((300, 517), seed, "cpu", torch.int8))
        assert torch.equal(inputs.hashed_uniform((5000,), 0.001, 0.01, seed, "cuda").cpu().view(torch.int16),
                           inputs.hashed_uniform((5000,), 0.001, 0.01, seed, "cpu").view(torch.int16))
    a = inputs.config4("cuda", n_tokens=2, hidden=64, n_experts=4, inter=32, top_k=2, seed=4, expert_lo=1, expert_hi=3)
    b = inputs.config4("cpu", n_tokens=2, hidden=64, n_experts=4, inter=32, top_k=2, seed=4, expert_lo=1, expert_hi=3)
    for k in ("w13", "s13", "o13", "w2", "s2", "o2"):
        assert torch.equal(a[k].cpu().view(torch.uint8), b[k].view(torch.uint8)), k


def test_packed_int8_path_of_the_compiled_module():
    """pack_weight_int8 + grouped_gemm_packed of the compiled module give the bits of its grouped_gemm."""
    m = _module()
    gen = torch.Generator().manual_seed(2)
    x = torch.randn(300, 128, generator=gen).to(torch.bfloat16).cuda()
    w = torch.randint(-128, 128, (3, 128, 512), generator=gen, dtype=torch.int8).cuda()
    s = (torch.rand(3, 512, generator=gen) * 0.009 + 0.001).to(torch.bfloat16).cuda()
    o = (torch.rand(3, 512, generator=gen) * 8 - 4).to(torch.bfloat16).cuda()
    gl = torch.tensor([137, 137, 300], dtype=torch.int64).cuda()
    a = torch.zeros(300, 512, dtype=torch.bfloat16, device="cuda")
    b = torch.zeros_like(a)
    m.grouped_gemm(x, w, s, o, gl, "int8", a)
    m.grouped_gemm_packed(x, m.pack_weight_int8(w), s, o, gl, b)
    torch.cuda.synchronize()
    assert torch.equal(a.view(torch.int16), b.view(torch.int16))
    assert tuple(m.last_status()) == (0, 0)
