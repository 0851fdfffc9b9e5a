"""The allocation-free int8 grouped GEMM entry point (`b200moe_grouped_gemm_int8_noalloc`).

It exists for hosts that are not allowed to allocate device memory themselves -- for example an
operator plug-in living inside a framework whose own allocator owns the whole GPU, or a serving
loop that may not allocate once it is running -- and therefore cannot give the regular entry point
the workspace it asks for.  The scratch lives inside the library instead and is shared by all calls,
so the checks here are: same bits as the regular entry point, on two calls in a row (the second
call finds the first call's leftovers in the scratch), and a clear refusal beyond the row limit.

This file is named so that pytest collects it last.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(counts, K, N, seed, with_offset):
    gen = torch.Generator().manual_seed(seed)
    G = len(counts)
    counts = torch.tensor(counts, dtype=torch.int64)
    M = int(counts.sum())
    x = torch.randn(M, K, generator=gen).to(torch.bfloat16)
    w = torch.randint(-128, 128, (G, K, N), generator=gen, dtype=torch.int8)
    scale = (torch.rand(G, N, generator=gen) * 0.009 + 0.001).to(torch.bfloat16)
    offset = (torch.rand(G, N, generator=gen) * 8 - 4).to(torch.bfloat16) if with_offset else None
    return [t.cuda() if t is not None else None for t in (x, w, scale, offset, counts)]


def _noalloc(x, w, scale, offset, counts):
    from ascend_kernel_b200 import _abi

    M, K = x.shape
    G, _, N = w.shape
    y = torch.full((M, N), -768.0, dtype=torch.bfloat16, device="cuda")
    rc = _abi.lib.b200moe_grouped_gemm_int8_noalloc(
        x.data_ptr(), w.data_ptr(), scale.data_ptr(), None if offset is None else offset.data_ptr(),
        counts.data_ptr(), y.data_ptr(), M, K, N, G, 1, torch.cuda.current_stream().cuda_stream)
    assert rc == 0, _abi.strerror(rc)
    st = (ctypes.c_int32 * 2)()
    assert _abi.lib.b200moe_noalloc_read_status(st, torch.cuda.current_stream().cuda_stream) == 0
    assert (st[0], st[1]) == (0, 0)
    return y


def _regular(x, w, scale, offset, counts):
    import ascend_kernel_b200 as ak

    y = torch.full((x.shape[0], w.shape[2]), -768.0, dtype=torch.bfloat16, device="cuda")
    ak.grouped_gemm(x, w, scale, offset, counts, "int8", y, group_list_type=1)
    torch.cuda.synchronize()
    return y


def test_two_calls_in_a_row_match_the_regular_entry_point():
    first = _case([127, 129, 0, 1, 300], 192, 512, 13, True)
    second = _case([40, 0, 260], 128, 256, 14, True)       # fewer rows: stale row sums stay behind it
    third = _case([5, 90], 64, 256, 15, False)             # no offset: the row sums are not rewritten
    for args in (first, second, third):
        got = _noalloc(*args)
        want = _regular(*args)
        assert torch.equal(got.view(torch.int16), want.view(torch.int16))


def test_a_warmed_up_call_takes_no_device_memory():
    """After one warm-up call on the device (which loads the kernel image and looks up the scratch array's
    address), further calls leave the free device memory and torch's allocation count exactly as they
    were: nothing is allocated, by the driver or by torch, on behalf of the call."""
    from ascend_kernel_b200 import _abi

    x, w, scale, offset, counts = _case([40, 0, 260], 128, 256, 21, True)
    M, K = x.shape
    G, _, N = w.shape
    y = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream

    def call():
        rc = _abi.lib.b200moe_grouped_gemm_int8_noalloc(x.data_ptr(), w.data_ptr(), scale.data_ptr(), offset.data_ptr(),
                                                        counts.data_ptr(), y.data_ptr(), M, K, N, G, 1, stream)
        assert rc == 0, _abi.strerror(rc)

    call()                       # warm-up: module load, symbol lookup
    torch.cuda.synchronize()
    free0 = torch.cuda.mem_get_info()[0]
    live0 = torch.cuda.memory_stats()["allocation.all.current"]
    reserved0 = torch.cuda.memory_reserved()
    for _ in range(2):
        call()
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free0
        assert torch.cuda.memory_stats()["allocation.all.current"] == live0
        assert torch.cuda.memory_reserved() == reserved0


def test_rejects_more_rows_than_the_scratch_holds():
    from ascend_kernel_b200 import _abi

    limit = _abi.lib.b200moe_grouped_gemm_int8_noalloc_max_rows()
    assert limit == 65536
    p = 4096  # aligned, never dereferenced: the size check comes first
    rc = _abi.lib.b200moe_grouped_gemm_int8_noalloc(p, p, p, None, p, p, limit + 1, 256, 256, 4, 0, None)
    assert rc == 9 and "allocation-free" in _abi.strerror(rc)
    assert _abi.lib.b200moe_grouped_gemm_int8_noalloc(p, p, p, None, p, p, limit, 100, 256, 4, 0, None) == 3
