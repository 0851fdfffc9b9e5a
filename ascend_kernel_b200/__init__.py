"""B200-native (sm_100a) implementation of the MoE expert-GEMM hot path of QingCheng-AI/ascend-kernel:
antiquant grouped GEMM, grouped soft GEMV and FP4 -> BF16 dequantisation behind a C ABI
(``include/b200moe.h``), with the reference's python operator interface on top.

Importing the package loads ``libb200moe.so`` and fails loudly if it has not been built.
"""
from . import _abi
from .ops import (combine, fp4_dequant, fp4_layout, gather_rows, grouped_gemm, grouped_soft_gemv, read_status,
                  silu_mul)

__all__ = ["grouped_gemm", "grouped_soft_gemv", "fp4_dequant", "fp4_layout", "silu_mul", "gather_rows", "combine",
           "read_status", "abi_version"]


def abi_version() -> str:
    return _abi.version()
