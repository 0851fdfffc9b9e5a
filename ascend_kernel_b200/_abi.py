"""ctypes binding of the C ABI declared in ``include/b200moe.h``.

The shared library is the product; there is no fallback.  If ``libb200moe.so`` is missing the
import fails with instructions to build it, and every call raises when the library reports an
error status.
"""
from __future__ import annotations

import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libb200moe.so")

# enums of include/b200moe.h
CT = {"fp8": 0, "fp4": 1, "int8": 2, "int4": 3, "bf16": 4}
GROUP_LIST_CUMSUM, GROUP_LIST_COUNTS = 0, 1
LAYOUT = {"canonical": 0, "ascend": 1}
FP4_SCALE_NONE, FP4_SCALE_E8M0_PER32 = 0, 1
STATUS_BYTES = 256

EXPORTS = [
    "b200moe_grouped_gemm", "b200moe_grouped_gemm_workspace_bytes", "b200moe_grouped_gemv",
    "b200moe_grouped_gemv_workspace_bytes", "b200moe_fp4_dequant", "b200moe_fp4_layout", "b200moe_silu_mul",
    "b200moe_ep_finish", "b200moe_gather_rows", "b200moe_gather_rows_sum", "b200moe_grouped_gemm_int8_packed_rowsum", "b200moe_combine", "b200moe_read_status", "b200moe_read_sticky_status", "b200moe_strerror", "b200moe_version",
    "b200moe_moe_route", "b200moe_moe_regroup_index", "b200moe_grouped_gemm_int8_noalloc", "b200moe_grouped_gemm_int8_noalloc_max_rows", "b200moe_noalloc_read_status",
    "b200moe_ep_post_counts", "b200moe_ep_dispatch", "b200moe_ep_wait", "b200moe_ep_post", "b200moe_ep_combine",
    "b200moe_fp4_dequant_bf16_scale", "b200moe_fp8_dequant", "b200moe_fp4_scale_fold",
    "b200moe_silu_mul_dyn", "b200moe_grouped_gemm_int8_silu", "b200moe_pack_weight_int8", "b200moe_grouped_gemm_int8_packed", "b200moe_grouped_gemm_int8_packed_scatter",
    "b200moe_set_gemm_reserved_sms", "b200moe_ipc_alloc", "b200moe_ipc_open", "b200moe_ipc_close", "b200moe_ipc_free",
]

EP_MAX_WORLD = 8
IPC_HANDLE_BYTES = 64
EP_SIG_COUNTS, EP_SIG_ROWS, EP_SIG_RESULTS = 0, 1, 2


class EpComm(ctypes.Structure):
    """``b200moe_ep_comm`` of include/b200moe.h."""
    _fields_ = [("world", ctypes.c_int32), ("rank", ctypes.c_int32), ("n_experts", ctypes.c_int32),
                ("dispatch_ctas", ctypes.c_int32), ("cap_rows", ctypes.c_int64), ("hidden", ctypes.c_int64),
                ("peer_recv_x", ctypes.c_void_p * EP_MAX_WORLD), ("peer_y", ctypes.c_void_p * EP_MAX_WORLD),
                ("peer_counts", ctypes.c_void_p * EP_MAX_WORLD), ("peer_signal", ctypes.c_void_p * EP_MAX_WORLD),
                ("status", ctypes.c_void_p), ("step_counter", ctypes.c_void_p),
                ("peer_ret", ctypes.c_void_p * EP_MAX_WORLD), ("peer_ret_code", ctypes.c_void_p * EP_MAX_WORLD),
                ("cap_send", ctypes.c_int64), ("peer_recv_sum", ctypes.c_void_p * EP_MAX_WORLD)]


class B200MoeError(RuntimeError):
    def __init__(self, code: int, what: str):
        super().__init__(f"{what}: {strerror(code)} (status {code})")
        self.code = code


def _load() -> ctypes.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python ascend_kernel_b200/build.py` "
            "(there is no CPU or PyTorch fallback for these operators)")
    lib = ctypes.CDLL(LIB_PATH)
    vp, i64, i32, sz = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_size_t
    gemm_args = [vp, vp, vp, vp, vp, vp, i64, i64, i64, i64, i32, i32, i32, vp, sz, vp]
    lib.b200moe_grouped_gemm.argtypes = gemm_args
    lib.b200moe_grouped_gemm.restype = i32
    lib.b200moe_grouped_gemv.argtypes = gemm_args
    lib.b200moe_grouped_gemv.restype = i32
    for f in (lib.b200moe_grouped_gemm_workspace_bytes, lib.b200moe_grouped_gemv_workspace_bytes):
        f.argtypes = [i64, i64, i64, i64, i32, i32]
        f.restype = sz
    lib.b200moe_grouped_gemm_int8_silu.argtypes = [vp, vp, vp, vp, vp, vp, i64, i64, i64, i64, i32, vp, sz, vp]
    lib.b200moe_grouped_gemm_int8_silu.restype = i32
    lib.b200moe_pack_weight_int8.argtypes = [vp, vp, i64, i64, i64, i32, vp]
    lib.b200moe_pack_weight_int8.restype = i32
    lib.b200moe_grouped_gemm_int8_packed.argtypes = [vp, vp, vp, vp, vp, vp, i64, i64, i64, i64, i32, i32, vp, sz, vp]
    lib.b200moe_grouped_gemm_int8_packed.restype = i32
    lib.b200moe_grouped_gemm_int8_packed_rowsum.argtypes = [vp, vp, vp, vp, vp, vp, vp, i64, i64, i64, i64, i32, i32, vp, sz, vp]
    lib.b200moe_grouped_gemm_int8_packed_rowsum.restype = i32
    lib.b200moe_grouped_gemm_int8_packed_scatter.argtypes = [vp, vp, vp, vp, vp, vp, ctypes.POINTER(vp), i64, i64, i64, i64, i64,
                                                             i64, i32, vp, sz, vp]
    lib.b200moe_grouped_gemm_int8_packed_scatter.restype = i32
    lib.b200moe_set_gemm_reserved_sms.argtypes = [i32]
    lib.b200moe_set_gemm_reserved_sms.restype = i32
    lib.b200moe_grouped_gemm_int8_noalloc.argtypes = [vp, vp, vp, vp, vp, vp, i64, i64, i64, i64, i32, vp]
    lib.b200moe_grouped_gemm_int8_noalloc.restype = i32
    lib.b200moe_grouped_gemm_int8_noalloc_max_rows.argtypes = []
    lib.b200moe_grouped_gemm_int8_noalloc_max_rows.restype = i64
    lib.b200moe_noalloc_read_status.argtypes = [ctypes.POINTER(ctypes.c_int32), vp]
    lib.b200moe_noalloc_read_status.restype = i32
    lib.b200moe_fp4_dequant.argtypes = [vp, vp, vp, i64, i32, vp]
    lib.b200moe_fp4_dequant.restype = i32
    lib.b200moe_fp4_dequant_bf16_scale.argtypes = [vp, vp, vp, i64, i64, i64, i32, vp]
    lib.b200moe_fp4_dequant_bf16_scale.restype = i32
    lib.b200moe_fp8_dequant.argtypes = [vp, vp, vp, i64, i64, i64, vp]
    lib.b200moe_fp8_dequant.restype = i32
    lib.b200moe_fp4_scale_fold.argtypes = [vp, vp, vp, i64, i64, i64, i64, vp]
    lib.b200moe_fp4_scale_fold.restype = i32
    lib.b200moe_fp4_layout.argtypes = [vp, vp, i64, i64, i64, i32, vp]
    lib.b200moe_fp4_layout.restype = i32
    lib.b200moe_silu_mul.argtypes = [vp, vp, i64, i64, vp]
    lib.b200moe_silu_mul.restype = i32
    lib.b200moe_gather_rows.argtypes = [vp, vp, vp, i64, i64, vp]
    lib.b200moe_gather_rows.restype = i32
    lib.b200moe_gather_rows_sum.argtypes = [vp, vp, vp, vp, i64, i64, vp]
    lib.b200moe_gather_rows_sum.restype = i32
    lib.b200moe_combine.argtypes = [vp, vp, vp, vp, i64, i64, i64, vp]
    lib.b200moe_combine.restype = i32
    lib.b200moe_moe_route.argtypes = [vp, i64, i64, i64, vp, vp, vp, vp, vp, vp, vp]
    lib.b200moe_moe_route.restype = i32
    lib.b200moe_moe_regroup_index.argtypes = [vp, i64, i64, vp, vp, vp, vp]
    lib.b200moe_moe_regroup_index.restype = i32
    u64, comm = ctypes.c_uint64, ctypes.POINTER(EpComm)
    lib.b200moe_ep_post_counts.argtypes = [comm, vp, u64, vp]
    lib.b200moe_ep_dispatch.argtypes = [comm, vp, vp, i64, u64, vp, vp, vp, vp, vp]
    lib.b200moe_ep_wait.argtypes = [comm, i32, u64, vp]
    lib.b200moe_ep_post.argtypes = [comm, i32, u64, vp]
    lib.b200moe_ep_combine.argtypes = [comm, vp, vp, vp, vp, i64, i64, u64, vp]
    lib.b200moe_ep_finish.argtypes = [comm, vp, vp, vp, vp, i64, i64, u64, vp]
    lib.b200moe_ep_finish.restype = i32
    lib.b200moe_silu_mul_dyn.argtypes = [vp, vp, vp, i64, vp]
    lib.b200moe_ipc_alloc.argtypes = [sz, ctypes.POINTER(vp), ctypes.c_char_p]
    lib.b200moe_ipc_open.argtypes = [ctypes.c_char_p, ctypes.POINTER(vp)]
    lib.b200moe_ipc_close.argtypes = [vp]
    lib.b200moe_ipc_free.argtypes = [vp]
    for f in (lib.b200moe_ep_post_counts, lib.b200moe_ep_dispatch, lib.b200moe_ep_wait, lib.b200moe_ep_post,
              lib.b200moe_ep_combine, lib.b200moe_silu_mul_dyn, lib.b200moe_ipc_alloc, lib.b200moe_ipc_open,
              lib.b200moe_ipc_close, lib.b200moe_ipc_free):
        f.restype = i32
    lib.b200moe_read_status.argtypes = [vp, ctypes.POINTER(ctypes.c_int32), vp]
    lib.b200moe_read_status.restype = i32
    lib.b200moe_read_sticky_status.argtypes = [vp, ctypes.POINTER(ctypes.c_int32), i32, vp]
    lib.b200moe_read_sticky_status.restype = i32
    lib.b200moe_strerror.argtypes = [i32]
    lib.b200moe_strerror.restype = ctypes.c_char_p
    lib.b200moe_version.argtypes = []
    lib.b200moe_version.restype = ctypes.c_char_p
    return lib


lib = _load()


def strerror(code: int) -> str:
    return lib.b200moe_strerror(int(code)).decode()


def version() -> str:
    return lib.b200moe_version().decode()


def check(code: int, what: str) -> None:
    if code != 0:
        raise B200MoeError(code, what)
