"""Install check in the manner of the reference's ``check_installed_ops.py:6-19``: after a build, the
``cinfer_ascendc`` module must expose every operator the build installs.  The reference reads the list
from ``.installed_ops.txt``, written by its ``setup.py``; here the list is fixed (nothing is optional):
the reference's two open operators, under their reference names, and this build's additions.  The
reference's ``grouped_query_attention`` and ``incre_flash_attention`` are not in it -- their sources
were never published (``ascend-closed/README.md``).

    python -m ascend_kernel_b200.check_installed_ops
"""
REFERENCE_OPS = ["grouped_soft_gemv", "grouped_gemm"]                     # pybind.cpp:14-19 of the reference
ADDED_OPS = ["fp4_dequant", "fp4_dequant_bf16_scale", "fp8_dequant", "fp4_scale_fold", "pack_weight_int8",
             "grouped_gemm_packed", "last_status", "check_status"]


def check(verbose: bool = True) -> None:
    from . import cinfer_ascendc

    for op in REFERENCE_OPS + ADDED_OPS:
        if not hasattr(cinfer_ascendc, op):
            raise RuntimeError(f"Check installed ops failed: cinfer_ascendc has no attribute {op!r}")
        if verbose:
            print(f"{op} installed.")
    if verbose:
        print("Check installed ops passed.")


if __name__ == "__main__":
    check()
