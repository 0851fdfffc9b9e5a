"""Expert-parallel token exchange over NVLink peer memory (host side).

``PeerExchange`` owns this rank's exchange buffers (allocated by the C library so that the
other processes of the node can map them through CUDA IPC), maps every peer's buffers, and wraps
the exchange kernels of ``include/b200moe.h`` (``b200moe_ep_*``).  With ``n_buffers`` = 2 or 3 the row,
count and return buffers exist that many times and a step uses the set its ``parity`` names, so that the
exchange of one step can run while the expert GEMMs of the step before still read the other set
(moe_layer.OverlappedSteps); the signal words are shared, their step numbers only grow.  torch.distributed is used once,
at construction, to pass the 64-byte IPC handles around; a layer step itself makes no collective
call and never synchronises with the host.
"""
from __future__ import annotations

import ctypes

import torch

from . import _abi, ops

_lib = _abi.lib


class _DeviceBuffer:
    """A raw device allocation exposed to torch through ``__cuda_array_interface__``."""

    def __init__(self, ptr: int, shape, typestr: str):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (ptr, False), "version": 2}


def _as_tensor(ptr: int, shape, dtype, device):
    """Zero-copy torch view of ``ptr`` (bf16 goes through int16: the interface has no bf16 code)."""
    if dtype == torch.bfloat16:
        return torch.as_tensor(_DeviceBuffer(ptr, shape, "<i2"), device=device).view(torch.bfloat16)
    code = {torch.int32: "<i4", torch.int64: "<i8", torch.uint8: "|u1", torch.float32: "<f4"}[dtype]
    return torch.as_tensor(_DeviceBuffer(ptr, shape, code), device=device)


class PeerExchange:
    def __init__(self, group, n_experts: int, hidden: int, cap_rows: int, device, n_buffers: int = 1):
        """``group``: the expert-parallel process group (all ranks on one node) or None for a single
        rank.  ``cap_rows``: rows this rank's receive / result buffers hold; the worst case is
        (tokens of all ranks) x top_k.  ``n_buffers``: 1, or 2 / 3 for steps that overlap."""
        if n_buffers not in (1, 2, 3):
            raise ValueError("n_buffers must be 1, 2 or 3")
        self.n_buffers = n_buffers
        self.device = torch.device(device)
        self.n_experts, self.hidden, self.cap_rows = n_experts, hidden, cap_rows
        if group is not None:
            import torch.distributed as dist

            self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        else:
            self.world, self.rank = 1, 0
        if self.world > _abi.EP_MAX_WORLD:
            raise RuntimeError(f"at most {_abi.EP_MAX_WORLD} ranks")
        self.step = 0
        # rows this rank itself dispatches at most (its tokens x top_k): the size of its return buffer
        self.cap_send = max(1, cap_rows // self.world)
        # bytes of ONE set; the sets of a doubled buffer follow one another in the same allocation
        one = {"recv_x": cap_rows * hidden * 2, "y": cap_rows * hidden * 2,
               "counts": -(-self.world * n_experts * 4 // 256) * 256, "signal": 3 * _abi.EP_MAX_WORLD * 8,
               "ret": self.cap_send * hidden * 2, "ret_code": cap_rows * 8,
               "recv_sum": -(-cap_rows * 4 // 256) * 256}
        doubled = ("recv_x", "counts", "ret", "ret_code", "recv_sum") if n_buffers > 1 else ()
        sizes = {name: nbytes * (n_buffers if name in doubled else 1) for name, nbytes in one.items()}
        self._own, handles = {}, {}
        with torch.cuda.device(self.device):
            for name, nbytes in sizes.items():
                p = ctypes.c_void_p()
                h = ctypes.create_string_buffer(_abi.IPC_HANDLE_BYTES)
                _abi.check(_lib.b200moe_ipc_alloc(nbytes, ctypes.byref(p), h), f"ipc_alloc({name})")
                self._own[name], handles[name] = p.value, bytes(h.raw)
        # every rank's handles -> pointers valid in this process
        self._peer = {name: [None] * self.world for name in sizes}
        self._opened = []
        if self.world > 1:
            import torch.distributed as dist

            everyone = [None] * self.world
            dist.all_gather_object(everyone, handles, group=group)
            with torch.cuda.device(self.device):
                for r, hs in enumerate(everyone):
                    for name in sizes:
                        if r == self.rank:
                            self._peer[name][r] = self._own[name]
                            continue
                        p = ctypes.c_void_p()
                        _abi.check(_lib.b200moe_ipc_open(hs[name], ctypes.byref(p)), f"ipc_open({name}, rank {r})")
                        self._peer[name][r] = p.value
                        self._opened.append(p.value)
            dist.barrier(group=group)  # nobody starts a step before every mapping exists
        else:
            for name in sizes:
                self._peer[name][0] = self._own[name]
        self.status = torch.zeros(4, dtype=torch.int32, device=self.device)
        self._done = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._step_dev = torch.zeros(1, dtype=torch.int64, device=self.device)
        self.device_steps = False  # True: the step number lives on the device (constant kernel arguments)

        def at(name, r, p):  # rank r's set p of buffer `name`, as mapped in this process
            return self._peer[name][r] + (p * one[name] if name in doubled else 0)

        self._comms = []
        for p in range(n_buffers):
            c = _abi.EpComm()
            c.world, c.rank, c.n_experts, c.cap_rows, c.hidden = self.world, self.rank, n_experts, cap_rows, hidden
            for r in range(self.world):
                c.peer_recv_x[r], c.peer_y[r] = at("recv_x", r, p), at("y", r, p)
                c.peer_counts[r], c.peer_signal[r] = at("counts", r, p), at("signal", r, p)
                c.peer_ret[r], c.peer_ret_code[r] = at("ret", r, p), at("ret_code", r, p)
                c.peer_recv_sum[r] = at("recv_sum", r, p)
            c.cap_send = self.cap_send
            c.status = self.status.data_ptr()
            c.step_counter = self._step_dev.data_ptr()
            self._comms.append(c)
        self._comm = self._comms[0]
        # torch views of the local row buffers (inputs / outputs of the grouped GEMMs), one per set
        self.recv_x_sets = [_as_tensor(at("recv_x", self.rank, p), (cap_rows, hidden), torch.bfloat16, self.device)
                            for p in range(n_buffers)]
        self.y = _as_tensor(self._own["y"], (cap_rows, hidden), torch.bfloat16, self.device)
        # results pushed back by the owners' down projections: this rank's return buffer (one row per
        # dispatched (token, j) pair, in sorted order), and the return addresses of the rows it received
        self.ret_sets = [_as_tensor(at("ret", self.rank, p), (self.cap_send, hidden), torch.bfloat16, self.device)
                         for p in range(n_buffers)]
        self.ret_code_sets = [_as_tensor(at("ret_code", self.rank, p), (cap_rows,), torch.int64, self.device)
                              for p in range(n_buffers)]
        self.ret_ptrs_sets = [[at("ret", r, p) for r in range(self.world)] for p in range(n_buffers)]
        # fp32 sum of every received row, stored by the sender beside the row
        self.recv_sum_sets = [_as_tensor(at("recv_sum", self.rank, p), (cap_rows,), torch.float32, self.device)
                              for p in range(n_buffers)]
        self.recv_sum = self.recv_sum_sets[0]
        self.recv_x, self.ret, self.ret_code, self.ret_ptrs = (self.recv_x_sets[0], self.ret_sets[0],
                                                               self.ret_code_sets[0], self.ret_ptrs_sets[0])

    # ---- one step ---------------------------------------------------------------------------
    def _s(self):
        return torch.cuda.current_stream().cuda_stream

    def begin_step(self) -> int:
        self.step += 1
        return self.step

    def use_device_steps(self):
        """From now on the step number is kept on the device and the kernels get step 0, so a layer
        pass has the same arguments every time.  Call between steps, with the stream idle."""
        torch.cuda.current_stream().synchronize()
        self._step_dev.fill_(self.step)
        self.device_steps = True

    def use_host_steps(self):
        """Back to step numbers passed by the host (what overlapping steps need: two of them are in
        flight, each kernel is told which one it belongs to).  Call between steps, with the device idle."""
        if self.device_steps:
            torch.cuda.synchronize(self.device)
            self.step = int(self._step_dev.item())
            self.device_steps = False

    def _step_arg(self, step=None) -> int:
        if step is not None:
            if self.device_steps:
                raise RuntimeError("explicit step numbers need use_host_steps()")
            return step
        return 0 if self.device_steps else self.step

    # Every kernel wrapper takes the buffer set (``parity``) and, for steps in flight beside one
    # another, the step number the kernel belongs to (default: the step begun last).
    def post_counts(self, counts, parity: int = 0, step: int = None):
        with torch.cuda.device(self.device):
            _abi.check(_lib.b200moe_ep_post_counts(ctypes.byref(self._comms[parity]), counts.data_ptr(),
                                                   self._step_arg(step), self._s()), "ep_post_counts")
        ops._count(1)

    def dispatch(self, x, token_of, parity: int = 0, step: int = None, out=None, max_ctas: int = 0):
        """-> (remote_pos int32 [rows], local_counts int64 [E/world], n_recv int64 [1]); ``out``: these
        three, preallocated.  ``max_ctas`` > 0 bounds the kernel's grid (a dispatch that shares the GPU
        with a grouped GEMM)."""
        self._comms[parity].dispatch_ctas = max_ctas
        n_rows = token_of.numel()
        if out is None:
            out = (torch.empty(n_rows, dtype=torch.int32, device=self.device),
                   torch.empty(self.n_experts // self.world, dtype=torch.int64, device=self.device),
                   torch.empty(1, dtype=torch.int64, device=self.device))
        remote_pos, local_counts, n_recv = out
        with torch.cuda.device(self.device):
            _abi.check(_lib.b200moe_ep_dispatch(ctypes.byref(self._comms[parity]), x.data_ptr(), token_of.data_ptr(),
                                                n_rows, self._step_arg(step), remote_pos.data_ptr(),
                                                local_counts.data_ptr(), n_recv.data_ptr(), self._done.data_ptr(),
                                                self._s()), "ep_dispatch")
        ops._count(1)
        return remote_pos, local_counts, n_recv

    def wait(self, which: int, step: int = None):
        with torch.cuda.device(self.device):
            _abi.check(_lib.b200moe_ep_wait(ctypes.byref(self._comm), which, self._step_arg(step), self._s()), "ep_wait")
        ops._count(1)

    def post(self, which: int, step: int = None):
        with torch.cuda.device(self.device):
            _abi.check(_lib.b200moe_ep_post(ctypes.byref(self._comm), which, self._step_arg(step), self._s()), "ep_post")
        ops._count(1)

    def finish(self, slot, weight, out=None, parity: int = 0, step: int = None):
        """End of a step whose results were pushed: signals this rank's results, waits for every rank's, then sums
        each token's rows of this rank's return buffer (set ``parity``) -- one launch."""
        T, top_k = slot.shape
        if out is None:
            out = torch.empty(T, self.hidden, dtype=torch.bfloat16, device=self.device)
        with torch.cuda.device(self.device):
            _abi.check(_lib.b200moe_ep_finish(ctypes.byref(self._comms[parity]), self.ret_sets[parity].data_ptr(),
                                              slot.data_ptr(), weight.data_ptr(), out.data_ptr(), T, top_k,
                                              self._step_arg(step), self._s()), "ep_finish")
        ops._count(1)
        return out

    def combine(self, remote_pos, slot, weight, out=None):
        T, top_k = slot.shape
        if out is None:
            out = torch.empty(T, self.hidden, dtype=torch.bfloat16, device=self.device)
        with torch.cuda.device(self.device):
            _abi.check(_lib.b200moe_ep_combine(ctypes.byref(self._comm), remote_pos.data_ptr(), slot.data_ptr(),
                                               weight.data_ptr(), out.data_ptr(), T, top_k, self._step_arg(), self._s()),
                       "ep_combine")
        ops._count(1)
        return out

    def read_status(self):
        """(0, _) = fine; (1, expert) = a receive buffer overflowed; (2, where) = a wait expired."""
        s = self.status.cpu()
        return int(s[0]), int(s[1])

    def close(self):
        """Unmaps the peers' buffers and frees this rank's.  All ranks must have finished their last
        step (synchronise and barrier first)."""
        with torch.cuda.device(self.device):
            for p in self._opened:
                _lib.b200moe_ipc_close(p)
            self._opened = []
            self.recv_x = self.y = self.ret = self.ret_code = None
            self.recv_x_sets = self.ret_sets = self.ret_code_sets = self.recv_sum_sets = []
            self.recv_sum = None
            for name, p in list(self._own.items()):
                _lib.b200moe_ipc_free(p)
            self._own = {}
