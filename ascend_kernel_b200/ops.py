"""Python mirror of the reference's operator interface over the C ABI (torch is used only for
device memory and the current stream).

``grouped_gemm`` / ``grouped_soft_gemv`` keep the keyword names of the reference's pybind module
(pybind.cpp:14-19 of the reference); outputs are caller-allocated and written in place, launches
are asynchronous on torch's current stream.  Trailing keywords (defaulted, so existing calls are
unchanged) select per-expert counts instead of cumulative sums and the canonical FP4 layout.
"""
from __future__ import annotations

import torch

from . import _abi
from ._abi import CT, LAYOUT

_lib = _abi.lib

# number of this package's kernels launched so far (the benchmark reads and resets it)
LAUNCHES = 0


def _count(n):
    global LAUNCHES
    LAUNCHES += n


def _ptr(t):
    return None if t is None else t.data_ptr()


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _need_cuda(**tensors):
    for name, t in tensors.items():
        if t is None:
            continue
        if not isinstance(t, torch.Tensor) or not t.is_cuda:
            raise RuntimeError(f"{name} must be a CUDA tensor (there is no CPU path)")
        if not t.is_contiguous():
            raise RuntimeError(f"{name} must be contiguous")


def _compute_type(computeType: str) -> int:
    if computeType not in CT:
        # the reference reports an unknown computeType this way (grouped_gemm.cpp:10-16,129-133)
        print(f'Invalid compute type: {computeType}. Supported: "fp4", "fp8", "int8", "int4", "bf16"')
        raise RuntimeError("Host tiling failed!")
    return CT[computeType]


def _check_common(x, weight, group_list, output, ct):
    if x.dtype != torch.bfloat16 or output.dtype != torch.bfloat16:
        raise RuntimeError("x and output must be bfloat16")
    if group_list.dtype != torch.int64:
        raise RuntimeError("group_list must be int64")
    if x.dim() != 2 or weight.dim() != 3 or output.dim() != 2:
        raise RuntimeError("expected x [M,K], weight [G,K,N(/2)], output [M,N]")
    if ct == CT["bf16"]:
        if weight.dtype != torch.bfloat16:
            raise RuntimeError("weight must be bfloat16 for computeType bf16")
    elif weight.element_size() != 1:
        raise RuntimeError("weight must be a 1-byte container (uint8 / int8)")
    M, K = x.shape
    G, Kw, Nw = weight.shape
    N = Nw * 2 if ct in (CT["fp4"], CT["int4"]) else Nw
    if Kw != K or tuple(output.shape) != (M, N) or group_list.numel() != G:
        raise RuntimeError(f"shape mismatch: x {tuple(x.shape)}, weight {tuple(weight.shape)}, "
                           f"output {tuple(output.shape)}, group_list {group_list.numel()}")
    return M, K, N, G


def _check_scale(scale, ct, G, K, N, what):
    want = {CT["fp8"]: ((G, K // 128, N // 128), torch.float32), CT["fp4"]: ((G, K // 16, N), torch.bfloat16),
            CT["int8"]: ((G, N), torch.bfloat16), CT["int4"]: ((G, K // 128, N), torch.bfloat16)}[ct]
    if tuple(scale.shape) != want[0] or scale.dtype != want[1]:
        raise RuntimeError(f"{what} must be {want[1]} of shape {want[0]}, got {scale.dtype} {tuple(scale.shape)}")


# One persistent workspace per (device, stream): its first 256 bytes hold the kernels' status words, of
# which words 4 / 5 keep the first finding of any call since they were last cleared (an invalid group
# list that was clamped, a bounded wait that expired).  `last_status` / `check_status` read them at the
# caller's synchronisation points, so a failed call cannot pass unnoticed even though no operator
# synchronises.  Calls on one stream run one after the other, so they can share the buffer.
_WS = {}


def _workspace(need, device):
    device = torch.device(device)
    idx = device.index if device.index is not None else torch.cuda.current_device()
    key = (idx, torch.cuda.current_stream(idx).cuda_stream)
    ws = _WS.get(key)
    if ws is None or ws.numel() < need:
        new = torch.zeros(max(int(need), 1 << 20), dtype=torch.uint8, device=torch.device("cuda", idx))
        if ws is not None:
            new[16:24].copy_(ws[16:24])  # carry the sticky status words over
        _WS[key] = ws = new
    return ws


def last_status(device=None, clear: bool = False):
    """(code, detail) of the first device-side finding of any operator call on ``device`` (default: the
    current one) since the status was last cleared; (0, 0) if none.  code 1: a group_list was invalid and
    rows were clamped (detail = expert index); 2: a bounded wait inside a kernel expired and the output
    is incomplete.  Synchronises the streams the operators ran on."""
    import ctypes

    idx = torch.cuda.current_device() if device is None else torch.device(device).index
    found = (0, 0)
    for (d, stream), ws in list(_WS.items()):
        if d != idx:
            continue
        out = (ctypes.c_int32 * 2)()
        with torch.cuda.device(d):
            _abi.check(_lib.b200moe_read_sticky_status(_ptr(ws), out, int(bool(clear)), stream), "read_sticky_status")
        if found == (0, 0) and out[0] != 0:
            found = (int(out[0]), int(out[1]))
    return found


def check_status(device=None):
    """Raises if an operator call on ``device`` left a device-side finding (and clears it)."""
    code, detail = last_status(device, clear=True)
    if code != 0:
        what = {1: "a group_list was invalid (rows were clamped); first bad expert index",
                2: "a bounded wait inside a kernel expired (results are incomplete); barrier id"}.get(code, "status")
        raise RuntimeError(f"b200moe device status {code}: {what} {detail}")


def _run(fn, ws_fn, what, x, weight, scale, offset, group_list, output, ct, group_list_type, layout, M, K, N, G):
    need = ws_fn(M, K, N, G, ct, layout)
    ws = _workspace(need, x.device)
    with torch.cuda.device(x.device):
        rc = fn(_ptr(x), _ptr(weight), _ptr(scale), _ptr(offset), _ptr(group_list), _ptr(output), M, K, N, G, ct,
                group_list_type, layout, _ptr(ws), need, _stream())
    _abi.check(rc, what)
    return ws


def grouped_gemm(x, weight, antiquantScaleOptional, antiquantOffsetOptional, groupListOptional, computeType,
                 output, group_list_type: int = 0, weight_layout: str = "ascend", return_workspace: bool = False):
    """output[rows of expert g] = bf16(x[rows of expert g] @ dequant(weight[g])).  Returns None
    (or the workspace tensor holding the device status words when ``return_workspace``)."""
    ct = _compute_type(computeType)
    _need_cuda(x=x, weight=weight, scale=antiquantScaleOptional, offset=antiquantOffsetOptional,
               group_list=groupListOptional, output=output)
    M, K, N, G = _check_common(x, weight, groupListOptional, output, ct)
    if ct == CT["bf16"]:
        antiquantScaleOptional = None  # the matmul phase alone: no scale, no offset
    else:
        _check_scale(antiquantScaleOptional, ct, G, K, N, "antiquantScaleOptional")
    offset = antiquantOffsetOptional if ct in (CT["int8"], CT["int4"]) else None  # ignored for fp8/fp4
    if offset is not None:
        _check_scale(offset, ct, G, K, N, "antiquantOffsetOptional")
    ws = _run(_lib.b200moe_grouped_gemm, _lib.b200moe_grouped_gemm_workspace_bytes, "grouped_gemm", x, weight,
              antiquantScaleOptional, offset, groupListOptional, output, ct, group_list_type,
              LAYOUT[weight_layout], M, K, N, G)
    if M > 0:  # GEMM + row sums for the int8 offset term (pre-shuffled fp4 weights are read in place)
        _count(1 + (offset is not None and ct == CT["int8"]))
    return ws if return_workspace else None


def interleave_gate_up(t, block: int = 128):
    """[..., 2I] with the gate columns first and the up columns after them -> the order
    grouped_gemm_silu takes: blocks of `block` gate columns followed by the up columns of the same
    indices.  Applies to the weight [G, K, 2I] and to its per-channel scale / offset [G, 2I]."""
    two_i = t.shape[-1]
    inter = two_i // 2
    if two_i % (2 * block) != 0:
        raise RuntimeError("2I must be a multiple of 256")
    j = torch.arange(two_i, device=t.device)
    b, r = j // (2 * block), j % (2 * block)
    src = torch.where(r < block, b * block + r, inter + b * block + (r - block))
    return t.index_select(t.dim() - 1, src).contiguous()


def grouped_gemm_silu(x, weight, scale, offset, group_list, output, group_list_type: int = 0,
                      return_workspace: bool = False):
    """output [M, I] = bf16(silu(gate) * up) of the int8 gate/up projection; ``weight`` / ``scale`` /
    ``offset`` in the interleaved column order of :func:`interleave_gate_up`."""
    _need_cuda(x=x, weight=weight, scale=scale, offset=offset, group_list=group_list, output=output)
    if x.dtype != torch.bfloat16 or output.dtype != torch.bfloat16 or group_list.dtype != torch.int64:
        raise RuntimeError("x and output must be bfloat16, group_list int64")
    if weight.dim() != 3 or weight.element_size() != 1:
        raise RuntimeError("weight must be int8 [G, K, 2I]")
    G, K, N = weight.shape
    M = x.shape[0]
    if x.shape[1] != K or tuple(output.shape) != (M, N // 2) or group_list.numel() != G:
        raise RuntimeError(f"shape mismatch: x {tuple(x.shape)}, weight {tuple(weight.shape)}, output {tuple(output.shape)}")
    _check_scale(scale, CT["int8"], G, K, N, "scale")
    if offset is not None:
        _check_scale(offset, CT["int8"], G, K, N, "offset")
    need = _lib.b200moe_grouped_gemm_workspace_bytes(M, K, N, G, CT["int8"], LAYOUT["canonical"])
    ws = _workspace(need, x.device)
    with torch.cuda.device(x.device):
        rc = _lib.b200moe_grouped_gemm_int8_silu(_ptr(x), _ptr(weight), _ptr(scale), _ptr(offset), _ptr(group_list),
                                                 _ptr(output), M, K, N, G, group_list_type, _ptr(ws), need, _stream())
    _abi.check(rc, "grouped_gemm_silu")
    if M > 0:
        _count(1 + (offset is not None))
    return ws if return_workspace else None


def pack_weight_int8(weight, gate_up: bool = False):
    """int8 [G, K, N] -> the tile-packed order grouped_gemm_packed reads (same shape, opaque contents).
    ``gate_up``: N = 2I with the gate columns first; tiles then pair gate and up columns."""
    _need_cuda(weight=weight)
    if weight.dim() != 3 or weight.element_size() != 1:
        raise RuntimeError("weight must be int8 [G, K, N]")
    G, K, N = weight.shape
    out = torch.empty_like(weight)
    with torch.cuda.device(weight.device):
        rc = _lib.b200moe_pack_weight_int8(_ptr(weight), _ptr(out), G, K, N, int(bool(gate_up)), _stream())
    _abi.check(rc, "pack_weight_int8")
    _count(1)
    return out


def grouped_gemm_packed(x, packed, scale, offset, group_list, output, group_list_type: int = 0,
                        gate_up_silu: bool = False, return_workspace: bool = False, x_rowsum=None):
    """int8 grouped GEMM on weights from :func:`pack_weight_int8`; ``scale`` / ``offset`` bf16 [G, N] in
    the original column order.  ``gate_up_silu``: output [M, N/2] = bf16(silu(gate) * up).  ``x_rowsum``: fp32
    [M] sums of the rows of x when the caller has them (``gather_rows(..., with_sums=True)``): the launch then
    makes no pass of its own over x for the offset term."""
    _need_cuda(x=x, packed=packed, scale=scale, offset=offset, group_list=group_list, output=output, x_rowsum=x_rowsum)
    if x_rowsum is not None and (x_rowsum.dtype != torch.float32 or x_rowsum.numel() < x.shape[0]):
        raise RuntimeError("x_rowsum must be float32 with one element per row of x")
    if x.dtype != torch.bfloat16 or output.dtype != torch.bfloat16 or group_list.dtype != torch.int64:
        raise RuntimeError("x and output must be bfloat16, group_list int64")
    if packed.dim() != 3 or packed.element_size() != 1:
        raise RuntimeError("packed must be the [G, K, N] tensor pack_weight_int8 returned")
    G, K, N = packed.shape
    M = x.shape[0]
    n_out = N // 2 if gate_up_silu else N
    if x.shape[1] != K or tuple(output.shape) != (M, n_out) or group_list.numel() != G:
        raise RuntimeError(f"shape mismatch: x {tuple(x.shape)}, packed {tuple(packed.shape)}, output {tuple(output.shape)}")
    _check_scale(scale, CT["int8"], G, K, N, "scale")
    if offset is not None:
        _check_scale(offset, CT["int8"], G, K, N, "offset")
    need = _lib.b200moe_grouped_gemm_workspace_bytes(M, K, N, G, CT["int8"], LAYOUT["canonical"])
    ws = _workspace(need, x.device)
    with torch.cuda.device(x.device):
        if x_rowsum is not None and offset is not None:
            rc = _lib.b200moe_grouped_gemm_int8_packed_rowsum(_ptr(x), _ptr(packed), _ptr(scale), _ptr(offset),
                                                              _ptr(x_rowsum), _ptr(group_list), _ptr(output), M, K, N, G,
                                                              group_list_type, int(bool(gate_up_silu)), _ptr(ws), need,
                                                              _stream())
        else:
            rc = _lib.b200moe_grouped_gemm_int8_packed(_ptr(x), _ptr(packed), _ptr(scale), _ptr(offset), _ptr(group_list),
                                                       _ptr(output), M, K, N, G, group_list_type, int(bool(gate_up_silu)),
                                                       _ptr(ws), need, _stream())
    _abi.check(rc, "grouped_gemm_packed")
    if M > 0:
        _count(1 + (offset is not None and x_rowsum is None))
    return ws if return_workspace else None


def set_gemm_reserved_sms(n: int) -> int:
    """SMs the persistent packed-weight GEMM kernels leave free from now on (process-wide; 0 = none);
    returns the previous value.  For callers that run other kernels beside a grouped GEMM."""
    return int(_lib.b200moe_set_gemm_reserved_sms(int(n)))


def grouped_gemm_packed_scatter(x, packed, scale, offset, group_list, row_code, dst_ptrs, dst_rows: int,
                                group_list_type: int = 0):
    """grouped_gemm_packed whose result row r is stored at row ``row_code[r] & 0xffffffff`` of the bf16
    [dst_rows, N] tensor at device address ``dst_ptrs[row_code[r] >> 32]`` (addresses may be other GPUs'
    memory mapped into this process)."""
    import ctypes

    _need_cuda(x=x, packed=packed, scale=scale, offset=offset, group_list=group_list, row_code=row_code)
    if x.dtype != torch.bfloat16 or group_list.dtype != torch.int64 or row_code.dtype != torch.int64:
        raise RuntimeError("x must be bfloat16, group_list and row_code int64")
    G, K, N = packed.shape
    M = x.shape[0]
    if x.shape[1] != K or group_list.numel() != G or row_code.numel() < M or not 1 <= len(dst_ptrs) <= 8:
        raise RuntimeError("shape mismatch")
    _check_scale(scale, CT["int8"], G, K, N, "scale")
    if offset is not None:
        _check_scale(offset, CT["int8"], G, K, N, "offset")
    need = _lib.b200moe_grouped_gemm_workspace_bytes(M, K, N, G, CT["int8"], LAYOUT["canonical"])
    ws = _workspace(need, x.device)
    bases = (ctypes.c_void_p * len(dst_ptrs))(*dst_ptrs)
    with torch.cuda.device(x.device):
        rc = _lib.b200moe_grouped_gemm_int8_packed_scatter(_ptr(x), _ptr(packed), _ptr(scale), _ptr(offset), _ptr(group_list),
                                                           _ptr(row_code), bases, len(dst_ptrs), dst_rows, M, K, N, G,
                                                           group_list_type, _ptr(ws), need, _stream())
    _abi.check(rc, "grouped_gemm_packed_scatter")
    if M > 0:
        _count(1 + (offset is not None))


def grouped_soft_gemv(x, weight, scale, groupList, computeType, output, group_list_type: int = 0,
                      weight_layout: str = "ascend", offset=None, return_workspace: bool = False):
    ct = _compute_type(computeType)
    _need_cuda(x=x, weight=weight, scale=scale, offset=offset, group_list=groupList, output=output)
    M, K, N, G = _check_common(x, weight, groupList, output, ct)
    _check_scale(scale, ct, G, K, N, "scale")
    if offset is not None:
        if ct not in (CT["int8"], CT["int4"]):
            raise RuntimeError("offset is only defined for int8 / int4")
        _check_scale(offset, ct, G, K, N, "offset")
    ws = _run(_lib.b200moe_grouped_gemv, _lib.b200moe_grouped_gemv_workspace_bytes, "grouped_soft_gemv", x, weight,
              scale, offset, groupList, output, ct, group_list_type, LAYOUT[weight_layout], M, K, N, G)
    if M > 0:
        _count(1)
    return ws if return_workspace else None


def fp4_dequant(codes, scale, output):
    """codes: uint8/int8 [..., L/2]; scale: uint8 e8m0 [..., L/32] or None; output bf16 [..., L]."""
    _need_cuda(codes=codes, scale=scale, output=output)
    n = codes.numel() * 2
    if output.dtype != torch.bfloat16 or output.numel() != n:
        raise RuntimeError("output must be bfloat16 with twice as many elements as codes has bytes")
    if scale is not None and (scale.element_size() != 1 or scale.numel() * 32 != n):
        raise RuntimeError("scale must hold one e8m0 byte per 32 elements")
    with torch.cuda.device(codes.device):
        rc = _lib.b200moe_fp4_dequant(_ptr(codes), _ptr(scale), _ptr(output), n,
                                      _abi.FP4_SCALE_NONE if scale is None else _abi.FP4_SCALE_E8M0_PER32, _stream())
    _abi.check(rc, "fp4_dequant")
    _count(1)


def fp4_dequant_bf16_scale(codes, scale, output, weight_layout: str = "ascend"):
    """The reference's FP4 weight format on its own: codes int8/uint8 [G, K, N/2], scale bf16 [G, K/16, N]
    -> output bf16 [G, K, N] = rne_bf16(e2m1 * scale), the weights its GEMM kernel multiplies with."""
    _need_cuda(codes=codes, scale=scale, output=output)
    G, K, C = codes.shape
    N = 2 * C
    if codes.element_size() != 1 or scale.dtype != torch.bfloat16 or tuple(scale.shape) != (G, K // 16, N):
        raise RuntimeError("codes: bytes [G, K, N/2]; scale: bfloat16 [G, K/16, N]")
    if output.dtype != torch.bfloat16 or tuple(output.shape) != (G, K, N):
        raise RuntimeError("output must be bfloat16 [G, K, N]")
    with torch.cuda.device(codes.device):
        rc = _lib.b200moe_fp4_dequant_bf16_scale(_ptr(codes), _ptr(scale), _ptr(output), G, K, N, LAYOUT[weight_layout],
                                                 _stream())
    _abi.check(rc, "fp4_dequant_bf16_scale")
    _count(1)


def fp8_dequant(codes, scale, output):
    """The reference's FP8 weight format on its own: codes uint8 [G, K, N], scale float32 [G, K/128, N/128] ->
    output bf16 [G, K, N] = rne_bf16(e4m3 * scale) (0x7F / 0xFF decode to +-480, as in the reference)."""
    _need_cuda(codes=codes, scale=scale, output=output)
    G, K, N = codes.shape
    if codes.element_size() != 1 or scale.dtype != torch.float32 or tuple(scale.shape) != (G, K // 128, N // 128):
        raise RuntimeError("codes: uint8 [G, K, N]; scale: float32 [G, K/128, N/128]")
    if output.dtype != torch.bfloat16 or tuple(output.shape) != (G, K, N):
        raise RuntimeError("output must be bfloat16 [G, K, N]")
    with torch.cuda.device(codes.device):
        rc = _lib.b200moe_fp8_dequant(_ptr(codes), _ptr(scale), _ptr(output), G, K, N, _stream())
    _abi.check(rc, "fp8_dequant")
    _count(1)


def fp4_scale_fold(block_scale, global_scale):
    """block_scale bf16 [G, N, K/16] x global_scale float32 [G, 1, 1] or [G, 2, 1] (gate / up halves of the N
    rows) -> bf16 [G, K/16, N]: the scale tensor the fp4 operators take."""
    _need_cuda(block_scale=block_scale, global_scale=global_scale)
    G, N, KB = block_scale.shape
    n_global = global_scale.numel() // max(G, 1)
    if block_scale.dtype != torch.bfloat16 or global_scale.dtype != torch.float32 or n_global not in (1, 2):
        raise RuntimeError("block_scale: bfloat16 [G, N, K/16]; global_scale: float32 [G, 1 or 2, 1]")
    out = torch.empty(G, KB, N, dtype=torch.bfloat16, device=block_scale.device)
    with torch.cuda.device(block_scale.device):
        rc = _lib.b200moe_fp4_scale_fold(_ptr(block_scale), _ptr(global_scale), _ptr(out), G, N, KB, n_global, _stream())
    _abi.check(rc, "fp4_scale_fold")
    _count(1)
    return out


def fp4_layout(src, to_ascend: bool):
    """[G,K,N/2] packed FP4 weights between the canonical and the stored ("ascend") order."""
    _need_cuda(src=src)
    G, K, C = src.shape
    dst = torch.empty_like(src)
    with torch.cuda.device(src.device):
        rc = _lib.b200moe_fp4_layout(_ptr(src), _ptr(dst), G, K, 2 * C, int(bool(to_ascend)), _stream())
    _abi.check(rc, "fp4_layout")
    _count(1)
    return dst


def silu_mul(h, out=None):
    _need_cuda(h=h, out=out)
    rows, two_i = h.shape
    if out is None:
        out = torch.empty(rows, two_i // 2, dtype=torch.bfloat16, device=h.device)
    with torch.cuda.device(h.device):
        rc = _lib.b200moe_silu_mul(_ptr(h), _ptr(out), rows, two_i // 2, _stream())
    _abi.check(rc, "silu_mul")
    _count(1)
    return out


def gather_rows(src, index, out=None, with_sums: bool = False):
    """out[i, :] = src[index[i], :]; ``with_sums``: returns (out, fp32 [n] row sums of out) -- the sums the int8
    grouped GEMMs need for their offset term, bit for bit."""
    _need_cuda(src=src, index=index, out=out)
    if index.dtype != torch.int32:
        raise RuntimeError("index must be int32")
    if out is None:
        out = torch.empty(index.numel(), src.shape[1], dtype=src.dtype, device=src.device)
    with torch.cuda.device(src.device):
        if with_sums:
            if src.dtype != torch.bfloat16:
                raise RuntimeError("row sums are defined for bfloat16 rows")
            sums = torch.empty(index.numel(), dtype=torch.float32, device=src.device)
            rc = _lib.b200moe_gather_rows_sum(_ptr(src), _ptr(index), _ptr(out), _ptr(sums), index.numel(), src.shape[1],
                                              _stream())
        else:
            rc = _lib.b200moe_gather_rows(_ptr(src), _ptr(index), _ptr(out), index.numel(), src.shape[1], _stream())
    _abi.check(rc, "gather_rows")
    _count(1)
    return (out, sums) if with_sums else out


def combine(y, slot, weight, out=None):
    _need_cuda(y=y, slot=slot, weight=weight, out=out)
    if slot.dtype != torch.int32 or weight.dtype != torch.float32:
        raise RuntimeError("slot must be int32 and weight float32")
    T, top_k = slot.shape
    if out is None:
        out = torch.empty(T, y.shape[1], dtype=torch.bfloat16, device=y.device)
    with torch.cuda.device(y.device):
        rc = _lib.b200moe_combine(_ptr(y), _ptr(slot), _ptr(weight), _ptr(out), T, top_k, y.shape[1], _stream())
    _abi.check(rc, "combine")
    _count(1)
    return out


def moe_route_buffers(n_tokens: int, n_experts: int, top_k: int, device):
    """The six tensors ``moe_route`` fills (its five results and its scratch), for callers that reuse them."""
    return (torch.empty(n_tokens, top_k, dtype=torch.int32, device=device),
            torch.empty(n_tokens, top_k, dtype=torch.float32, device=device),
            torch.empty(n_experts, dtype=torch.int64, device=device),
            torch.empty(n_tokens * top_k, dtype=torch.int32, device=device),
            torch.empty(n_tokens, top_k, dtype=torch.int32, device=device),
            torch.empty(2 * n_experts, dtype=torch.int32, device=device))


def moe_route(logits, top_k: int, out=None):
    """logits bf16 [T, E] -> (idx int32 [T,k], weight fp32 [T,k], counts int64 [E], token_of int32 [T*k],
    slot int32 [T,k]).  ``out``: the tuple of ``moe_route_buffers`` to fill instead of new tensors."""
    _need_cuda(logits=logits)
    if logits.dtype != torch.bfloat16:
        raise RuntimeError("logits must be bfloat16")
    T, E = logits.shape
    dev = logits.device
    idx, w, counts, token_of, slot, scratch = out if out is not None else moe_route_buffers(T, E, top_k, dev)
    if idx.shape != (T, top_k) or counts.numel() != E or token_of.numel() != T * top_k:
        raise RuntimeError("moe_route: output buffers of another shape")
    with torch.cuda.device(dev):
        rc = _lib.b200moe_moe_route(_ptr(logits), T, E, top_k, _ptr(idx), _ptr(w), _ptr(counts), _ptr(token_of),
                                    _ptr(slot), _ptr(scratch), _stream())
    _abi.check(rc, "moe_route")
    _count(3)
    return idx, w, counts, token_of, slot


def silu_mul_dyn(h, n_rows, out=None):
    """silu_mul over the first ``n_rows[0]`` rows of h (``n_rows``: int64 device tensor)."""
    _need_cuda(h=h, n_rows=n_rows, out=out)
    if h.dtype != torch.bfloat16 or n_rows.dtype != torch.int64:
        raise RuntimeError("h must be bfloat16 and n_rows int64")
    R, two_i = h.shape
    if out is None:
        out = torch.empty(R, two_i // 2, dtype=torch.bfloat16, device=h.device)
    with torch.cuda.device(h.device):
        rc = _lib.b200moe_silu_mul_dyn(_ptr(h), _ptr(out), _ptr(n_rows), two_i // 2, _stream())
    _abi.check(rc, "silu_mul_dyn")
    _count(1)
    return out


def moe_regroup_index(recv_counts, n_recv: int):
    """recv_counts int64 [world, e_local] (rows per source rank and local expert, arrival order) ->
    (pos int32 [n_recv], inv int32 [n_recv], local_counts int64 [e_local])."""
    _need_cuda(recv_counts=recv_counts)
    if recv_counts.dtype != torch.int64:
        raise RuntimeError("recv_counts must be int64")
    world, e_local = recv_counts.shape
    dev = recv_counts.device
    pos = torch.empty(n_recv, dtype=torch.int32, device=dev)
    inv = torch.empty(n_recv, dtype=torch.int32, device=dev)
    local_counts = torch.empty(e_local, dtype=torch.int64, device=dev)
    with torch.cuda.device(dev):
        rc = _lib.b200moe_moe_regroup_index(_ptr(recv_counts), world, e_local, _ptr(pos), _ptr(inv),
                                            _ptr(local_counts), _stream())
    _abi.check(rc, "moe_regroup_index")
    _count(1)
    return pos, inv, local_counts


def combine_to_host(y, slot, weight, out_host):
    """combine() writing its result straight into pinned host memory (the device -> host transfer of
    the layer output rides on the kernel's stores instead of a separate copy)."""
    _need_cuda(y=y, slot=slot, weight=weight)
    if not (isinstance(out_host, torch.Tensor) and out_host.is_pinned() and out_host.is_contiguous()
            and out_host.dtype == torch.bfloat16):
        raise RuntimeError("out_host must be a contiguous pinned bfloat16 host tensor")
    T, top_k = slot.shape
    if tuple(out_host.shape) != (T, y.shape[1]):
        raise RuntimeError("out_host has the wrong shape")
    with torch.cuda.device(y.device):
        rc = _lib.b200moe_combine(_ptr(y), _ptr(slot), _ptr(weight), out_host.data_ptr(), T, top_k, y.shape[1],
                                  _stream())
    _abi.check(rc, "combine")
    _count(1)
    return out_host


def read_status(ws):
    import ctypes

    out = (ctypes.c_int32 * 2)()
    _abi.check(_lib.b200moe_read_status(_ptr(ws), out, _stream()), "read_status")
    return int(out[0]), int(out[1])
