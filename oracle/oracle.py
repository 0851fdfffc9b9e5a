"""CPU oracle for the MoE expert-GEMM hot path (TEST INFRASTRUCTURE, not product code).

Only the test-suite, the smoke check and the CPU-baseline leg of the benchmark may import this
module.  The product path (the CUDA kernels behind the C ABI) never routes through it.

It restates, in torch-CPU / numpy, what the reference operators compute:

* ``grouped_gemm``        grouped_gemm/op_kernel/grouped_matmul_antiquant.h:225-289 (group walk),
                          :408-457,537-692 (dequant driver), grouped_matmul.h:409-463 (bf16 matmul)
* ``grouped_soft_gemv``   grouped_soft_gemv/op_kernel/grouped_soft_gemv.h:235-293,
                          gemv_impl.h:147-398
* decode of FP8 e4m3      grouped_gemm/op_kernel/antiquant_impl.h:87-129 and the test golden
                          grouped_gemm/test/python/test_group_gemm_fp8.py:7-32
* decode of FP4 e2m1      antiquant_impl.h:41-85 and test_group_gemm_fp4.py:97-102
* FP4 weight pre-shuffle  test_group_gemm_fp4.py:105-142 (repack_weight, repack_weight_step2)

The bf16 cube matmul of the reference is closed CANN library code (``matmul::Matmul`` from
``lib/matmul_intf.h``, CANN 8.3.rc1) and the reference tests compare against the closed
``torch_npu.npu_grouped_matmul`` (torch_npu 2.6.0.post1); both are restated here as a per-expert
float32 ``x @ w`` over the cumulative ``group_list``.  Accumulation order is therefore not pinned
by the reference; everything up to the dequantised weights is pinned bit-exactly by the golden
fixtures under ``tests/golden`` (generated from the reference's own Python helpers).

The ``int8`` / ``int4`` modes and the e8m0 block-scaled FP4 dequantisation have no reference code;
they restate the benchmark configuration's formulas ``(W + offset) * scale`` and
``e2m1(code) * 2**(s-127)`` -- parity for those modes is unpinned by the reference.
"""
from __future__ import annotations

import numpy as np
import torch

E2M1_MAGNITUDES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)

GROUP_LIST_CUMSUM = 0
GROUP_LIST_COUNTS = 1


# --------------------------------------------------------------------------------------------
# decode tables
# --------------------------------------------------------------------------------------------
def e2m1_table() -> torch.Tensor:
    """16-entry float32 table of the FP4 e2m1 codes (sign in bit 3, code 8 is -0).

    Follows test_group_gemm_fp4.py:97-102: ((c & 8) << 12 | (c & 7) << 6) read as bf16, times
    bf16(0x7E80) = 2**126.
    """
    c = torch.arange(16, dtype=torch.int16)
    bits = ((c & 0x8) << 12) | ((c & 0x7) << 6)
    k = torch.tensor([0x7E80], dtype=torch.uint16).view(torch.bfloat16)
    return (bits.view(torch.bfloat16) * k).float()


def e4m3_table() -> torch.Tensor:
    """256-entry float32 table of the FP8 e4m3 codes as the reference decodes them.

    Follows test_group_gemm_fp8.py:11-14 / antiquant_impl.h:87-129: ((b & 0x80) << 8 |
    (b & 0x7F) << 4) read as bf16, times bf16(0x7B80) = 2**120.  There is no NaN handling:
    0x7F -> +480, 0xFF -> -480; subnormals (exponent field 0) are exact.
    """
    b = torch.arange(256, dtype=torch.int16)
    bits = ((b & 0x80) << 8) | ((b & 0x7F) << 4)
    k = torch.tensor([0x7B80], dtype=torch.uint16).view(torch.bfloat16)
    return (bits.view(torch.bfloat16) * k).float()


def e8m0_to_float(s: torch.Tensor) -> torch.Tensor:
    """e8m0 exponent byte -> float32 2**(s-127); 255 is NaN (OCP MX definition)."""
    s = s.to(torch.uint8)
    return s.view(torch.float8_e8m0fnu).float()


# --------------------------------------------------------------------------------------------
# FP4 layouts
# --------------------------------------------------------------------------------------------
def fp4_unpack(packed: torch.Tensor) -> torch.Tensor:
    """[..., C] bytes -> [..., 2C] codes, low nibble = even element (test_group_gemm_fp4.py:105-117)."""
    p = packed.contiguous().view(torch.uint8)
    lo = p & 0xF
    hi = p >> 4
    return torch.stack([lo, hi], dim=-1).reshape(*p.shape[:-1], p.shape[-1] * 2)


def fp4_pack(codes: torch.Tensor) -> torch.Tensor:
    """Inverse of fp4_unpack; returns int8 (the container dtype of grouped_gemm.cpp:76-83)."""
    c = codes.to(torch.uint8)
    return ((c[..., 1::2] << 4) | (c[..., 0::2] & 0xF)).view(torch.int8)


def ascend_shuffle(w: torch.Tensor) -> torch.Tensor:
    """Canonical [G,K,N/2] packed FP4 bytes -> the stored ("ascend") order.

    Restates repack_weight_step2 (test_group_gemm_fp4.py:129-142): rows flattened over (G,K) in
    blocks of 64 = (4,2,8), byte columns in blocks of 128 = (8,4,4); axes permuted
    (0,2,1,5,4,6,3,7).  Needs K % 64 == 0 and N % 256 == 0.
    """
    G, K, C = w.shape
    assert K % 64 == 0 and C % 128 == 0, "fp4 ascend layout needs K%64==0 and N%256==0"
    t = w.reshape(G * K // 64, 4, 2, 8, C // 128, 8, 4, 4)
    return t.permute(0, 2, 1, 5, 4, 6, 3, 7).contiguous().reshape(G, K, C)


def ascend_unshuffle(w: torch.Tensor) -> torch.Tensor:
    """Inverse of ascend_shuffle."""
    G, K, C = w.shape
    assert K % 64 == 0 and C % 128 == 0
    t = w.reshape(G * K // 64, 2, 4, 8, C // 128, 4, 8, 4)
    # forward: out axes = in axes (0,2,1,5,4,6,3,7); invert that permutation
    return t.permute(0, 2, 1, 6, 4, 3, 5, 7).contiguous().reshape(G, K, C)


def ascend_offset(r: int, c: int, C: int) -> int:
    """Closed form of ascend_shuffle: flat offset of canonical (row r, byte column c)."""
    R, a, b, c8 = r // 64, (r // 16) % 4, (r // 8) % 2, r % 8
    j, p, q, s = c // 128, (c // 16) % 8, (c // 4) % 4, c % 4
    J = C // 128
    return ((((((2 * R + b) * 4 + a) * 8 + p) * J + j) * 4 + q) * 8 + c8) * 4 + s


# --------------------------------------------------------------------------------------------
# dequantisation of the expert weights
# --------------------------------------------------------------------------------------------
def dequant_fp8(weight: torch.Tensor, scale: torch.Tensor, round_bf16: bool) -> torch.Tensor:
    """uint8 e4m3 codes [G,K,N] x fp32 scale [G,K/128,N/128] -> float32 [G,K,N].

    round_bf16=True is the GEMM path (antiquant_impl.h:171-208 casts to bf16 with RNE,
    test_group_gemm_fp8.py:27); False is the GEMV path (gemv_impl.h:147-199 keeps fp32,
    test_group_soft_gemv_fp8.py:27).
    """
    G, K, N = weight.shape
    assert K % 128 == 0 and N % 128 == 0, "fp8 needs K%128==0 and N%128==0"
    v = e4m3_table()[weight.view(torch.uint8).long()]
    s = scale.float().reshape(G, K // 128, 1, N // 128, 1)
    wd = (v.reshape(G, K // 128, 128, N // 128, 128) * s).reshape(G, K, N)
    return wd.to(torch.bfloat16).float() if round_bf16 else wd


def dequant_fp4(weight_canonical: torch.Tensor, scale: torch.Tensor, round_bf16: bool) -> torch.Tensor:
    """int8 packed e2m1 [G,K,N/2] (canonical) x bf16 scale [G,K/16,N] -> float32 [G,K,N].

    antiquant_impl.h:146-169,210-251: fp32 multiply then RNE cast to bf16 (GEMM);
    gemv_impl.h:147-199: fp32 multiply only (GEMV).
    """
    G, K, C = weight_canonical.shape
    N = 2 * C
    assert K % 16 == 0 and tuple(scale.shape) == (G, K // 16, N)
    v = e2m1_table()[fp4_unpack(weight_canonical).long()]
    s = scale.float().repeat_interleave(16, dim=1)
    wd = v * s
    return wd.to(torch.bfloat16).float() if round_bf16 else wd


def dequant_int8(weight: torch.Tensor, scale: torch.Tensor, offset: torch.Tensor | None) -> torch.Tensor:
    """(W + offset) * scale in float64; W int8 [G,K,N], scale/offset [G,N] (no reference code)."""
    w = weight.double()
    if offset is not None:
        w = w + offset.double().unsqueeze(1)
    return w * scale.double().unsqueeze(1)


def int4_unpack(packed: torch.Tensor) -> torch.Tensor:
    """[..., N/2] bytes -> [..., N] signed two's-complement int4 values, low nibble first."""
    c = fp4_unpack(packed).to(torch.int16)
    return torch.where(c >= 8, c - 16, c)


def dequant_int4(weight: torch.Tensor, scale: torch.Tensor, offset: torch.Tensor | None) -> torch.Tensor:
    """(W + offset) * scale in float64; W int4 pairs [G,K,N/2], scale/offset [G,K/128,N]."""
    w = int4_unpack(weight).double()
    G, K, N = w.shape
    assert K % 128 == 0 and tuple(scale.shape) == (G, K // 128, N)
    if offset is not None:
        w = w + offset.double().repeat_interleave(128, dim=1)
    return w * scale.double().repeat_interleave(128, dim=1)


def fp4_dequant_e8m0(codes: torch.Tensor, scale_e8m0: torch.Tensor | None) -> torch.Tensor:
    """Standalone FP4 -> BF16: packed bytes [..., L/2], one e8m0 byte per 32 elements of the last
    dimension ([..., L/32]) or None for scale 1.  Exact (no rounding for in-range exponents)."""
    v = e2m1_table()[fp4_unpack(codes).long()]
    if scale_e8m0 is not None:
        v = v * e8m0_to_float(scale_e8m0).repeat_interleave(32, dim=-1)
    return v.to(torch.bfloat16)


# --------------------------------------------------------------------------------------------
# group_list handling and the grouped contraction
# --------------------------------------------------------------------------------------------
def row_ranges(group_list: torch.Tensor, group_list_type: int = GROUP_LIST_CUMSUM):
    """[(r0, r1)] per expert.  Type 0: cumulative sums (grouped_matmul_utils.h:304-320,
    grouped_soft_gemv.h:10-16); type 1: per-expert counts (benchmark configurations)."""
    gl = [int(v) for v in group_list.tolist()]
    out, prev = [], 0
    for v in gl:
        if group_list_type == GROUP_LIST_CUMSUM:
            if v < prev:
                raise ValueError("group_list is not non-decreasing")
            out.append((prev, v))
            prev = v
        else:
            if v < 0:
                raise ValueError("negative count in group_list")
            out.append((prev, prev + v))
            prev += v
    return out


def grouped_matmul(x: torch.Tensor, wd: torch.Tensor, group_list: torch.Tensor,
                   group_list_type: int = GROUP_LIST_CUMSUM, acc=torch.float32) -> torch.Tensor:
    """out[r0_g:r1_g] = x[r0_g:r1_g] @ wd[g] (restates torch_npu.npu_grouped_matmul with
    split_item=2, group_type=0, group_list_type=0 as used by test_group_gemm_fp8.py:52-59).
    Rows at or beyond the last boundary are returned as NaN so callers can leave them untouched."""
    M, N = x.shape[0], wd.shape[-1]
    out = torch.full((M, N), float("nan"), dtype=acc)
    xf = x.to(acc)
    for g, (r0, r1) in enumerate(row_ranges(group_list, group_list_type)):
        if r1 > M:
            raise ValueError("group_list exceeds the number of rows of x")
        if r1 > r0:
            out[r0:r1] = xf[r0:r1] @ wd[g].to(acc)
    return out


def _store(output: torch.Tensor, res: torch.Tensor):
    """In-place write of the computed rows; rows never assigned to an expert stay untouched
    (grouped_matmul_antiquant.h:246-263: empty groups and trailing rows do no work)."""
    written = ~torch.isnan(res[:, 0]) if res.shape[1] else torch.zeros(res.shape[0], dtype=torch.bool)
    output[written] = res[written].to(output.dtype)


def grouped_gemm(x, weight, antiquantScaleOptional, antiquantOffsetOptional, groupListOptional,
                 computeType, output, group_list_type=GROUP_LIST_CUMSUM, weight_layout="ascend"):
    """Same keyword names as pybind.cpp:17-19.  fp8/fp4: offset accepted and ignored
    (grouped_matmul_antiquant.h:379 stores the pointer, nothing reads it)."""
    if computeType == "fp8":
        wd = dequant_fp8(weight, antiquantScaleOptional, round_bf16=True)
    elif computeType == "fp4":
        wc = ascend_unshuffle(weight) if weight_layout == "ascend" else weight
        wd = dequant_fp4(wc, antiquantScaleOptional, round_bf16=True)
    elif computeType == "int8":
        wd = dequant_int8(weight, antiquantScaleOptional, antiquantOffsetOptional)
    elif computeType == "int4":
        wd = dequant_int4(weight, antiquantScaleOptional, antiquantOffsetOptional)
    elif computeType == "bf16":  # the matmul phase alone (grouped_matmul.h:409-463): B = bf16 weights as they are
        wd = weight.float()
    else:
        raise RuntimeError("Host tiling failed!")  # grouped_gemm.cpp:10-16,129-133
    acc = torch.float64 if computeType in ("int8", "int4") else torch.float32
    _store(output, grouped_matmul(x, wd, groupListOptional, group_list_type, acc))


def grouped_soft_gemv(x, weight, scale, groupList, computeType, output,
                      group_list_type=GROUP_LIST_CUMSUM, weight_layout="ascend", offset=None):
    """Same keyword names as pybind.cpp:14-16.  Weights stay float32 after the dequant
    (gemv_impl.h:147-199), x is widened to float32, one RNE to bf16 at the end."""
    if computeType == "fp8":
        wd = dequant_fp8(weight, scale, round_bf16=False)
    elif computeType == "fp4":
        wc = ascend_unshuffle(weight) if weight_layout == "ascend" else weight
        wd = dequant_fp4(wc, scale, round_bf16=False)
    elif computeType == "int8":
        wd = dequant_int8(weight, scale, offset)
    elif computeType == "int4":
        wd = dequant_int4(weight, scale, offset)
    else:
        raise RuntimeError("Host tiling failed!")
    acc = torch.float64 if computeType in ("int8", "int4") else torch.float32
    _store(output, grouped_matmul(x, wd, groupList, group_list_type, acc))


def golden_f32(x, weight, scale, offset, group_list, compute_type, group_list_type=GROUP_LIST_CUMSUM,
               weight_layout="ascend", gemv=False) -> torch.Tensor:
    """Un-rounded float32 result [M,N] (NaN on rows owned by no expert)."""
    if compute_type == "fp8":
        wd = dequant_fp8(weight, scale, round_bf16=not gemv)
    elif compute_type == "fp4":
        wc = ascend_unshuffle(weight) if weight_layout == "ascend" else weight
        wd = dequant_fp4(wc, scale, round_bf16=not gemv)
    elif compute_type == "int8":
        wd = dequant_int8(weight, scale, offset)
    elif compute_type == "int4":
        wd = dequant_int4(weight, scale, offset)
    elif compute_type == "bf16":
        wd = weight.float()
    else:
        raise RuntimeError("Host tiling failed!")
    acc = torch.float64 if compute_type in ("int8", "int4") else torch.float32
    return grouped_matmul(x, wd, group_list, group_list_type, acc).float()


def fp4_scale_fold(block_scale: torch.Tensor, global_scale: torch.Tensor) -> torch.Tensor:
    """Two-level FP4 scale fold: block_scale bf16 [G,N,K/16] times the fp32 global scale [G,1,1] (or
    [G,2,1]: first / second half of the N rows), rounded to bf16, transposed to [G,K/16,N].
    Restates anti_quant_fp8_scale and the transpose that follows it
    (grouped_gemm/test/python/test_group_gemm_fp4.py:86-94,185-186): the in-place multiply of a bf16
    tensor by an fp32 one computes in fp32 and rounds once."""
    G, N, KB = block_scale.shape
    g = global_scale.float().reshape(G, -1)
    if g.shape[1] == 1:
        per_row = g.expand(G, N)
    else:
        per_row = torch.cat([g[:, :1].expand(G, N // 2), g[:, 1:2].expand(G, N - N // 2)], dim=1)
    folded = (block_scale.float() * per_row.unsqueeze(-1)).to(torch.bfloat16)
    return folded.transpose(-2, -1).contiguous()


# --------------------------------------------------------------------------------------------
# error metrics shared by the tests and the benchmark
# --------------------------------------------------------------------------------------------
def rel_l2(a: torch.Tensor, b: torch.Tensor) -> float:
    a, b = a.double(), b.double()
    den = float(b.norm())
    return float((a - b).norm()) / (den if den > 0 else 1.0)


def max_abs(a: torch.Tensor, b: torch.Tensor) -> float:
    return float((a.double() - b.double()).abs().max()) if a.numel() else 0.0


# --------------------------------------------------------------------------------------------
# expert-parallel MoE FFN layer (single-process golden of the benchmark's layer configuration)
# --------------------------------------------------------------------------------------------
def route_topk(logits: torch.Tensor, top_k: int):
    """softmax over experts -> top-k -> weights renormalised to sum 1 (float32).  Equal probabilities
    (equal bf16 logits) go to the lower expert index: a stable descending sort, not torch.topk, whose
    choice among ties is unspecified."""
    p = torch.softmax(logits.float(), dim=-1)
    ws, order = torch.sort(p, dim=-1, descending=True, stable=True)
    w, idx = ws[..., :top_k].contiguous(), order[..., :top_k].contiguous()
    return w / w.sum(dim=-1, keepdim=True), idx


def moe_layer(x, logits, w13, s13, o13, w2, s2, o2, top_k: int) -> torch.Tensor:
    """Golden of: route -> per-expert int8 antiquant GEMM gate|up -> SiLU(gate)*up (bf16) ->
    int8 antiquant GEMM down (bf16) -> weighted sum over the token's experts (fp32 -> bf16).
    w13 int8 [E,H,2I] (gate columns first), w2 int8 [E,I,H], scales/offsets [E,N]."""
    T, H = x.shape
    E = w13.shape[0]
    I = w2.shape[1]
    wts, idx = route_topk(logits, top_k)
    out = torch.zeros(T, H, dtype=torch.float32)
    for e in range(E):
        tok, slot = (idx == e).nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        xe = x[tok].double()
        wd1 = (w13[e].double() + (o13[e].double() if o13 is not None else 0.0)) * s13[e].double()
        h = (xe @ wd1).float().to(torch.bfloat16).float()
        act = (torch.nn.functional.silu(h[:, :I]) * h[:, I:]).to(torch.bfloat16)
        wd2 = (w2[e].double() + (o2[e].double() if o2 is not None else 0.0)) * s2[e].double()
        y = (act.double() @ wd2).float().to(torch.bfloat16).float()
        out.index_add_(0, tok, y * wts[tok, slot].unsqueeze(1))
    return out.to(torch.bfloat16)


def to_numpy_bits(t: torch.Tensor) -> np.ndarray:
    """bf16 tensor -> uint16 bit pattern array (fixtures are stored as bits)."""
    return t.contiguous().view(torch.uint16).numpy().copy()


def moe_layer_fp4_stored(x, logits, c13, s13, c2, s2, top_k: int) -> torch.Tensor:
    """Golden of the layer on FP4-stored experts: codes [E,H,2I/2] / [E,I,H/2] with one e8m0 scale per 32
    elements of the last dimension, dequantised to bf16 (exact), then route -> x @ W13 (bf16) ->
    SiLU(gate)*up (bf16) -> @ W2 (bf16) -> weighted sum over the token's experts (fp32 -> bf16)."""
    T, H = x.shape
    E, I = c13.shape[0], c2.shape[1]
    wts, idx = route_topk(logits, top_k)
    out = torch.zeros(T, H, dtype=torch.float32)
    for e in range(E):
        tok, slot = (idx == e).nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        wd1 = fp4_dequant_e8m0(c13[e], s13[e]).double()
        h = (x[tok].double() @ wd1).float().to(torch.bfloat16).float()
        act = (torch.nn.functional.silu(h[:, :I]) * h[:, I:]).to(torch.bfloat16)
        wd2 = fp4_dequant_e8m0(c2[e], s2[e]).double()
        y = (act.double() @ wd2).float().to(torch.bfloat16).float()
        out.index_add_(0, tok, y * wts[tok, slot].unsqueeze(-1))
    return out.to(torch.bfloat16)
