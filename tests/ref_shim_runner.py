"""Run one of the reference's own Python test scripts on CPU against a stand-in
``cinfer_ascendc`` module.  Usage: python tests/ref_shim_runner.py <script.py>

Shims (nothing else is altered): the device string "npu" becomes "cpu", ``torch.npu.synchronize``
is a no-op, ``torch_npu.npu_grouped_matmul`` is a per-expert float32 ``x @ w`` over the cumulative
group_list, and ``cinfer_ascendc`` is the CPU oracle.  Exit status is the script's own.
"""
import os
import sys
import types

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from oracle import oracle as O  # noqa: E402


def npu_grouped_matmul(xs, ws, group_list=None, split_item=2, group_type=0, group_list_type=0, **kw):
    assert split_item == 2 and group_type == 0 and group_list_type == 0
    x, w = xs[0], ws[0]
    out = O.grouped_matmul(x, w.float(), group_list.cpu())
    return [torch.nan_to_num(out, nan=0.0).to(x.dtype)]


def main(path):
    sys.modules["torch_npu"] = types.SimpleNamespace(npu_grouped_matmul=npu_grouped_matmul)
    sys.modules["cinfer_ascendc"] = types.SimpleNamespace(
        grouped_gemm=O.grouped_gemm, grouped_soft_gemv=O.grouped_soft_gemv)
    torch.npu = types.SimpleNamespace(synchronize=lambda: None)
    src = open(path).read().replace('"npu"', '"cpu"').replace("'npu'", "'cpu'")
    exec(compile(src, path, "exec"), {"__name__": "__main__"})


if __name__ == "__main__":
    main(sys.argv[1])
