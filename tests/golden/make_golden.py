"""Generate the golden fixtures of this directory from the reference's own Python test helpers.

Run once, where the reference checkout is present:

    python tests/golden/make_golden.py /path/to/reference

The reference test files cannot be imported as modules (they import the NPU backend and run on
import), so the helper *functions* are lifted out of their source with ``ast`` and executed with
the device string "npu" replaced by "cpu".  The closed ``torch_npu.npu_grouped_matmul`` the tests
use as golden matmul is restated as a per-expert float32 ``x @ w`` over the cumulative
group_list; everything before that call (decode tables, dequantised weights, weight repacking)
is the reference's own code and is stored bit-exactly.

Outputs (all small, ``np.savez_compressed``):
  decode_tables.npz    e4m3 (256 codes) and e2m1 (16 codes) tables as bf16 bit patterns
  fp4_layout.npz       random bytes through repack_weight / repack_weight_step2
  gemm_fp8.npz         seeded small case: inputs, dequantised weights (bf16 bits), expected y
  gemm_fp4.npz         the reference fp4 pipeline (quantise, pack, repack, scale fold) on a
                       seeded case plus a uniform-random-code case
  gemv_fp8.npz / gemv_fp4.npz   the GEMV goldens (fp32 weights kept for fp8)
  scale_fold.npz       the two-level FP4 scale fold (anti_quant_fp8_scale + transpose) on seeded
                       scales, with one and with two global scales per expert
                       (``--only scale_fold`` writes this file alone)
"""
import ast
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def lift(path, names):
    """Execute only the named top-level functions / assignments of a reference test file."""
    src = open(path).read().replace('"npu"', '"cpu"').replace("'npu'", "'cpu'")
    tree = ast.parse(src)
    keep = []
    for node in tree.body:
        if isinstance(node, ast.FunctionDef) and node.name in names:
            keep.append(node)
        elif isinstance(node, ast.Assign) and any(
            isinstance(t, ast.Name) and t.id in names for t in node.targets
        ):
            keep.append(node)
    ns = {"torch": torch}
    exec(compile(ast.Module(body=keep, type_ignores=[]), path, "exec"), ns)
    missing = [n for n in names if n not in ns]
    assert not missing, missing
    return ns


def bits(t):
    return t.contiguous().view(torch.uint16).numpy().copy()


def grouped_matmul_f32(x, wd, cumsum):
    """Restatement of torch_npu.npu_grouped_matmul(split_item=2, group_type=0,
    group_list_type=0): rows [cs[g-1], cs[g]) of x times wd[g], float32 accumulate."""
    out = torch.zeros(x.shape[0], wd.shape[-1], dtype=torch.float32)
    prev = 0
    for g, c in enumerate(cumsum.tolist()):
        if c > prev:
            out[prev:c] = x[prev:c].float() @ wd[g].float()
        prev = c
    return out


def scale_fold_fixture(g4):
    """anti_quant_fp8_scale (test_group_gemm_fp4.py:86-94) followed by the transpose of :186."""
    gen = torch.Generator().manual_seed(41)
    out = {}
    for tag, G, N, KB, S in (("one", 3, 64, 8, 1), ("two", 2, 96, 12, 2)):
        block = (torch.randn(G, N, KB, generator=gen) * 100).clamp(-448, 448).to(torch.bfloat16)
        glob = (torch.rand(G, S, 1, generator=gen) * 0.01 + 1e-4).to(torch.float32)
        folded = g4["anti_quant_fp8_scale"](block.clone(), glob)      # bf16 [G, N, K/16]
        new_scale = folded.transpose(-2, -1).contiguous()              # [G, K/16, N]
        out[f"{tag}_block_bits"] = bits(block)
        out[f"{tag}_global"] = glob.numpy()
        out[f"{tag}_folded_bits"] = bits(new_scale)
    np.savez_compressed(f"{HERE}/scale_fold.npz", **out)


def main(ref, only=None):
    if only == "scale_fold":
        g4 = lift(f"{ref}/grouped_gemm/test/python/test_group_gemm_fp4.py", ["anti_quant_fp8_scale"])
        scale_fold_fixture(g4)
        print("scale_fold.npz", os.path.getsize(f"{HERE}/scale_fold.npz"))
        return
    g8 = lift(f"{ref}/grouped_gemm/test/python/test_group_gemm_fp8.py", ["anti_quant_fp8"])
    v8 = lift(f"{ref}/grouped_soft_gemv/test/python/test_group_soft_gemv_fp8.py", ["anti_quant_fp8"])
    g4 = lift(
        f"{ref}/grouped_gemm/test/python/test_group_gemm_fp4.py",
        ["FP4_E2M1_LEVELS", "to_fp4_e2m1_in_uint8", "from_fp4_e2m1_in_uint8",
         "pack_every_two_fp4_e2m1_in_uint8_to_one_uint8", "unpack_every_uint8_to_two_fp4_e2m1_in_uint8",
         "init_weight_and_scales", "do_dequant_b", "unpack_weight", "anti_quant_fp8_scale",
         "fp4_dequant", "repack_weight", "repack_weight_step2"],
    )

    # ---- decode tables ------------------------------------------------------------------
    codes = torch.arange(256, dtype=torch.uint8).reshape(1, 2, 128).repeat(1, 64, 1)  # [1,128,128]
    ones = torch.ones(1, 1, 1, dtype=torch.float32)
    t8 = g8["anti_quant_fp8"](codes, ones)[0, :2].reshape(256)
    t4 = g4["fp4_dequant"](torch.arange(16, dtype=torch.uint8))
    np.savez_compressed(f"{HERE}/decode_tables.npz", e4m3_bf16_bits=bits(t8), e2m1_bf16_bits=bits(t4))

    # ---- fp4 layouts --------------------------------------------------------------------
    gen = torch.Generator().manual_seed(11)
    # repack_weight input is [G, N, K/2] bytes packed along K (low nibble = even k)
    G, K, N = 2, 128, 256
    packed_k = torch.randint(0, 256, (G, N, K // 2), generator=gen, dtype=torch.uint8)
    canon = g4["repack_weight"](packed_k)  # int8 [G, K, N/2]
    shuf = g4["repack_weight_step2"](canon)
    np.savez_compressed(f"{HERE}/fp4_layout.npz", packed_along_k=packed_k.numpy(),
                        canonical=canon.numpy(), ascend=shuf.numpy())

    # ---- GEMM fp8 (shape of test_group_gemm_fp8.py:37-50 scaled down in K and N) ---------
    gen = torch.Generator().manual_seed(21)
    G, M, K, N = 4, 48, 256, 256
    w = torch.randint(0, 256, (G, K, N), generator=gen, dtype=torch.uint8)
    scale = torch.randn(G, K // 128, N // 128, generator=gen, dtype=torch.float32)
    x = torch.randn(M, K, generator=gen, dtype=torch.float32).to(torch.bfloat16)
    cs = torch.tensor([12, 25, 44, 48], dtype=torch.int64)
    wd = g8["anti_quant_fp8"](w, scale)  # bf16
    y = grouped_matmul_f32(x, wd, cs).to(torch.bfloat16)
    np.savez_compressed(f"{HERE}/gemm_fp8.npz", weight=w.numpy(), scale=scale.numpy(), x_bits=bits(x),
                        group_list=cs.numpy(), wd_bits=bits(wd), y_bits=bits(y))

    # ---- GEMV fp8 (test_group_soft_gemv_fp8.py:39-65: fp32 weights, fp32 x) ---------------
    gen = torch.Generator().manual_seed(22)
    G, M, K, N = 4, 4, 128, 256
    w = torch.randint(0, 256, (G, K, N), generator=gen, dtype=torch.uint8)
    scale = torch.randn(G, K // 128, N // 128, generator=gen, dtype=torch.float32)
    x = torch.randn(M, K, generator=gen, dtype=torch.float32).to(torch.bfloat16)
    cs = torch.tensor([1, 2, 3, 4], dtype=torch.int64)
    wd32 = v8["anti_quant_fp8"](w, scale)  # float32, not rounded
    assert wd32.dtype == torch.float32
    y = grouped_matmul_f32(x, wd32, cs).to(torch.bfloat16)
    np.savez_compressed(f"{HERE}/gemv_fp8.npz", weight=w.numpy(), scale=scale.numpy(), x_bits=bits(x),
                        group_list=cs.numpy(), wd_f32=wd32.numpy(), y_bits=bits(y))

    # ---- GEMM / GEMV fp4: the reference pipeline of test_group_gemm_fp4.py:160-217 -------
    def fp4_case(seed, dim, rows, cs, uniform_codes):
        torch.manual_seed(seed)
        gen = torch.Generator().manual_seed(seed)
        block = 16
        G = 4
        if uniform_codes:
            b = torch.randint(0, 256, (dim, dim // 2), generator=gen, dtype=torch.uint8)
            b_s = (torch.rand(dim, dim // block, generator=gen) * 3 + 0.25).to(torch.bfloat16)
            b_s_2 = torch.tensor([[0.37]], dtype=torch.float32)
        else:
            b, b_s, b_s_2 = g4["init_weight_and_scales"](dim, block)
        x = torch.randn(rows, dim, generator=gen, dtype=torch.float32).to(torch.bfloat16)
        b = b.unsqueeze(0).repeat(G, 1, 1)
        b_s = b_s.unsqueeze(0).repeat(G, 1, 1)
        b_s_2 = b_s_2.unsqueeze(0).repeat(G, 1, 1)
        canon = g4["repack_weight"](b)
        w_ascend = g4["repack_weight_step2"](canon)
        scale = g4["anti_quant_fp8_scale"](b_s.clone(), b_s_2)  # bf16 [G, N, K/16]
        new_scale = scale.transpose(-2, -1).contiguous()  # [G, K/16, N]
        w2 = g4["fp4_dequant"](g4["unpack_weight"](b))  # bf16 [G, N, K]
        for i in range(scale.shape[-1]):
            w2[:, :, i * 16:(i + 1) * 16] *= scale[:, :, i].unsqueeze(-1)  # bf16 multiply
        wd = w2.transpose(-2, -1).contiguous()  # [G, K, N] bf16
        y = grouped_matmul_f32(x, wd, cs).to(torch.bfloat16)
        return dict(weight_ascend=w_ascend.numpy(), weight_canonical=canon.numpy(),
                    scale_bits=bits(new_scale), x_bits=bits(x), group_list=cs.numpy(),
                    wd0_bits=bits(wd[0]), y_bits=bits(y))  # all G experts share weights: wd[0] only

    a = fp4_case(31, 256, 256, torch.tensor([2, 3, 4, 256], dtype=torch.int64), False)
    b = fp4_case(32, 256, 64, torch.tensor([5, 5, 37, 60], dtype=torch.int64), True)
    np.savez_compressed(f"{HERE}/gemm_fp4.npz", **{f"ref_{k}": v for k, v in a.items()},
                        **{f"uni_{k}": v for k, v in b.items()})
    a = fp4_case(33, 256, 4, torch.tensor([1, 2, 3, 4], dtype=torch.int64), False)
    b = fp4_case(34, 256, 4, torch.tensor([1, 2, 3, 4], dtype=torch.int64), True)
    np.savez_compressed(f"{HERE}/gemv_fp4.npz", **{f"ref_{k}": v for k, v in a.items()},
                        **{f"uni_{k}": v for k, v in b.items()})
    scale_fold_fixture(g4)
    for f in sorted(os.listdir(HERE)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(f"{HERE}/{f}"))


if __name__ == "__main__":
    import argparse

    ap = argparse.ArgumentParser()
    ap.add_argument("reference", help="path of the reference checkout")
    ap.add_argument("--only", choices=["scale_fold"], default=None, help="write this fixture alone")
    ns_ = ap.parse_args()
    main(ns_.reference, only=ns_.only)
