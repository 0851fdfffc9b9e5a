"""B200-native (sm_100a) implementation of the MoE expert-GEMM hot path of QingCheng-AI/ascend-kernel:
antiquant grouped GEMM, grouped soft GEMV and FP4 -> BF16 dequantisation behind a C ABI
(``include/b200moe.h``), with the reference's python operator interface on top.

Importing the package loads ``libb200moe.so`` and fails loudly if it has not been built.
"""
from . import _abi
from .ops import (check_status, combine, fp4_dequant, fp4_dequant_bf16_scale, fp4_layout, fp4_scale_fold, fp8_dequant,
                  gather_rows, grouped_gemm, grouped_gemm_packed, grouped_soft_gemv, last_status, pack_weight_int8,
                  read_status, silu_mul)

__all__ = ["grouped_gemm", "grouped_soft_gemv", "fp4_dequant", "fp4_dequant_bf16_scale", "fp8_dequant", "fp4_scale_fold",
           "fp4_layout", "pack_weight_int8", "grouped_gemm_packed", "silu_mul", "gather_rows", "combine", "read_status",
           "last_status", "check_status", "abi_version"]


def abi_version() -> str:
    return _abi.version()
