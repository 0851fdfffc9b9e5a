"""Expert-parallel MoE FFN layer built from the hot-path operators.

One process per GPU; experts are sharded contiguously over the ranks (expert e lives on rank
e // (E / world)).  Per step:

  route (softmax -> top-k -> renormalise) and sort   b200moe_moe_route
  of the (token, k) pairs by expert
  gather rows into expert order                      b200moe_gather_rows
  all-to-all of per-expert counts, then of rows      NCCL (torch.distributed), world > 1 only
  regroup received rows expert-major                 b200moe_moe_regroup_index + b200moe_gather_rows, world > 1 only
  grouped GEMM gate|up  [H -> 2I], int8 antiquant,   b200moe_grouped_gemm_int8_packed  (tcgen05; weights
  SiLU(gate) * up in its epilogue                    repacked once at construction)
  grouped GEMM down     [I -> H], int8 antiquant     b200moe_grouped_gemm_int8_packed
  inverse regroup, all-to-all back                   world > 1 only
  weighted sum over each token's k results           b200moe_combine

With ``exchange="p2p"`` the two all-to-alls, the count exchange, the host read of the split sizes
and the regroup passes are replaced by this package's exchange kernels (ep_exchange.py): rows are
stored straight into the owner's receive buffer over NVLink, already expert-major, each with its
fp32 sum beside it; the down projection's epilogue stores every result row into the return buffer of
the rank the row came from, and the weighted sum is local.  A step then has no host synchronisation,
and ``OverlappedSteps`` runs the exchange of one step beside the GEMMs of the step before.
On one rank the row gather also adds up each row, so the gate/up GEMM makes no pass of its own over
its input for the offset term.

With the NCCL exchange, data from peers lands in this GPU's own memory (the NCCL receive buffer)
before a kernel reads it.  torch is used for device memory, streams and the process group; routing, permutation
and every row-sized operation are this package's CUDA kernels.
"""
from __future__ import annotations

import torch

from . import ops


class CudaRowOps:
    """The row-sized operations of the layer, on this package's CUDA kernels."""

    route = staticmethod(ops.moe_route)
    combine_to_host = staticmethod(ops.combine_to_host)
    regroup_index = staticmethod(ops.moe_regroup_index)
    gather_rows = staticmethod(ops.gather_rows)
    combine = staticmethod(ops.combine)
    silu_mul = staticmethod(ops.silu_mul)
    grouped_gemm = staticmethod(ops.grouped_gemm)


class MoELayer:
    def __init__(self, w13, s13, o13, w2, s2, o2, n_experts: int, top_k: int, group=None, row_ops=CudaRowOps,
                 exchange: str = "nccl", max_tokens: int = 0, fuse_silu: bool = None, gemm: str = None,
                 weight_format: str = "int8", exchange_buffers: int = 1):
        """w13 int8 [E_local, H, 2I] (gate columns first), w2 int8 [E_local, I, H]; per-channel bf16
        scales/offsets [E_local, N].  ``group``: a torch.distributed process group or None.
        ``row_ops`` exists so the dispatch / regroup / combine index logic can be exercised by CPU
        ranks in the test-suite with stand-in row operations; the product always uses CudaRowOps.
        ``exchange``: "nccl" (all-to-all collectives) or "p2p" (this package's peer-memory kernels;
        needs ``max_tokens`` = the largest number of tokens a rank passes to forward, which sizes the
        receive buffers for the worst case max_tokens x world x top_k rows).
        ``fuse_silu`` (default: on with the CUDA row operations): SiLU(gate) * up runs in the epilogue
        of the first grouped GEMM; the layer then keeps w13 / s13 / o13 in the interleaved column
        order that kernel takes (a one-time copy made here) instead of the tensors passed in.
        ``gemm``: "packed" (default with the CUDA row operations) repacks both weight tensors once
        into the tile order of ``ops.grouped_gemm_packed`` and keeps only those copies -- the expert
        GEMMs then dequantise straight into tensor memory and SiLU(gate) * up runs in the first
        one's epilogue; "generic" calls the drop-in operator on the [G, K, N] tensors.
        ``weight_format="fp4"``: the experts are STORED as FP4 e2m1 -- w13 uint8 [E_local, H, 2I/2] and w2
        uint8 [E_local, I, H/2], two codes per byte along the last dimension, with s13 / s2 one e8m0 byte
        per 32 elements of the last dimension ([E_local, H, 2I/32] / [E_local, I, H/32]); o13 / o2 must be
        None.  Every pass dequantises them to bf16 buffers owned by the layer (FP4 -> BF16 kernel) and
        runs the bf16 grouped GEMM on those: the two-phase structure of the reference's own kernel
        (dequantise to a bf16 workspace, then multiply: grouped_matmul_antiquant.h:632-654,
        grouped_matmul.h:409-463) with the benchmark's storage format.
        ``exchange_buffers=2`` (p2p exchange only) doubles the exchange buffers, which ``OverlappedSteps``
        needs to run one step's token exchange beside the expert GEMMs of the step before."""
        self.ops = row_ops
        self.w13, self.s13, self.o13, self.w2, self.s2, self.o2 = w13, s13, o13, w2, s2, o2
        self.n_experts, self.top_k = n_experts, top_k
        self.group = group
        if group is not None:
            import torch.distributed as dist

            self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        else:
            self.world, self.rank = 1, 0
        self.e_local = w13.shape[0]
        assert self.e_local * self.world == n_experts
        self.hidden, self.inter = w13.shape[1], w2.shape[1]
        self.device = w13.device
        if weight_format not in ("int8", "fp4"):
            raise ValueError("weight_format must be 'int8' or 'fp4'")
        self.weight_format = weight_format
        self.bf13 = self.bf2 = None
        if weight_format == "fp4":
            if o13 is not None or o2 is not None or row_ops is not CudaRowOps:
                raise ValueError("FP4-stored experts take no offsets and run on the CUDA row operations only")
            if w13.shape[2] != self.inter or w2.shape[2] * 2 != self.hidden:
                raise ValueError("expected w13 [E, H, 2I/2] and w2 [E, I, H/2] packed codes")
            fuse_silu, gemm = False, "generic"
            # the bf16 weights of one pass: overwritten by every pass, never read across passes
            self.bf13 = torch.empty(self.e_local, self.hidden, 2 * self.inter, dtype=torch.bfloat16, device=self.device)
            self.bf2 = torch.empty(self.e_local, self.inter, self.hidden, dtype=torch.bfloat16, device=self.device)
        self.fuse_silu = (row_ops is CudaRowOps) if fuse_silu is None else bool(fuse_silu)
        if gemm is None:
            gemm = "packed" if (row_ops is CudaRowOps and self.fuse_silu) else "generic"
        if gemm not in ("packed", "generic"):
            raise ValueError("gemm must be 'packed' or 'generic'")
        self.gemm = gemm
        if gemm == "packed":
            self.w13 = ops.pack_weight_int8(w13, gate_up=True)
            self.w2 = ops.pack_weight_int8(w2, gate_up=False)
        elif self.fuse_silu:
            self.w13 = ops.interleave_gate_up(w13)
            self.s13 = ops.interleave_gate_up(s13)
            self.o13 = None if o13 is None else ops.interleave_gate_up(o13)
        self.px = None
        if exchange == "p2p":
            from .ep_exchange import PeerExchange

            if max_tokens <= 0:
                raise ValueError('exchange="p2p" needs max_tokens')
            self.px = PeerExchange(group, n_experts, self.hidden, max_tokens * self.world * top_k, self.device,
                                   n_buffers=exchange_buffers)
        elif exchange != "nccl":
            raise ValueError("exchange must be 'nccl' or 'p2p'")
        self.gather_sums = True  # one rank: the row gather also produces the row sums of the gate/up GEMM
        self.timing = None  # [ev0..ev3] around GEMM1 / SiLU / GEMM2, filled by forward(record=True)
        self.phases = None  # [(name, event)] phase boundaries of the last forward(record=True)
        # called on the host when the rows of the step have been enqueued to reach their experts and the
        # expert GEMMs come next (HostPipeline starts the neighbouring steps' host copies there)
        self.mid_hook = None

    def read_status(self, clear: bool = True):
        """Device-side findings of the passes run so far, read at a synchronisation point of the caller's
        choosing (it waits for the layer's stream): raises if a grouped GEMM saw an invalid group list or
        a bounded wait expired, in an operator or in the token exchange; returns (0, 0) otherwise."""
        code, detail = ops.last_status(self.device, clear=clear)
        if code == 0 and self.px is not None:
            code, detail = self.px.read_status()
        if code != 0:
            raise RuntimeError(f"MoE layer: device status {code} (detail {detail}): "
                               + ("invalid group list, rows were clamped" if code == 1 else
                                  "a bounded wait expired, results are incomplete"))
        return code, detail

    def _mid(self):
        if self.mid_hook is not None:
            self.mid_hook()

    def _experts(self, rows, counts, record, y=None, n_rows=None, scatter=None, rows_sum=None):
        """rows [R, H] expert-major with per-local-expert counts -> [R, H] (into ``y`` when given).
        ``n_rows``: int64 device tensor with the number of rows in use when R is only a capacity.
        ``scatter`` = (row_code, destination pointers, destination rows): the down projection stores
        each result row where its code says (the return buffer of the rank the token came from) instead
        of into ``y``; packed GEMMs only.  ``rows_sum``: fp32 sums of the rows when the caller has them (the
        packed gate/up GEMM then skips its own pass over the rows)."""
        R = rows.shape[0]
        if y is None:
            y = torch.empty(R, self.hidden, dtype=torch.bfloat16, device=self.device)
        if R == 0:
            return y
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)] if record else None
        self.timing = None
        if ev:
            ev[0].record()
        if self.weight_format == "fp4":
            ops.fp4_dequant(self.w13, self.s13, self.bf13)
            h = torch.empty(R, 2 * self.inter, dtype=torch.bfloat16, device=self.device)
            ops.grouped_gemm(rows, self.bf13, None, None, counts, "bf16", h, group_list_type=1)
            if ev:
                ev[1].record()
            act = ops.silu_mul(h) if n_rows is None else ops.silu_mul_dyn(h, n_rows)
            if ev:
                ev[2].record()
            ops.fp4_dequant(self.w2, self.s2, self.bf2)
            ops.grouped_gemm(act, self.bf2, None, None, counts, "bf16", y, group_list_type=1)
            if ev:
                ev[3].record()
                self.timing = ev
            return y
        if self.gemm == "packed":
            act = torch.empty(R, self.inter, dtype=torch.bfloat16, device=self.device)
            ops.grouped_gemm_packed(rows, self.w13, self.s13, self.o13, counts, act, group_list_type=1,
                                    gate_up_silu=True, x_rowsum=rows_sum)
            if ev:
                ev[1].record()
                ev[2].record()
            if scatter is not None:
                ops.grouped_gemm_packed_scatter(act, self.w2, self.s2, self.o2, counts, scatter[0], scatter[1], scatter[2],
                                                group_list_type=1)
            else:
                ops.grouped_gemm_packed(act, self.w2, self.s2, self.o2, counts, y, group_list_type=1)
            if ev:
                ev[3].record()
                self.timing = ev
            return y
        if self.fuse_silu:
            act = torch.empty(R, self.inter, dtype=torch.bfloat16, device=self.device)
            ops.grouped_gemm_silu(rows, self.w13, self.s13, self.o13, counts, act, group_list_type=1)
            if ev:
                ev[1].record()
        else:
            h = torch.empty(R, 2 * self.inter, dtype=torch.bfloat16, device=self.device)
            self.ops.grouped_gemm(rows, self.w13, self.s13, self.o13, counts, "int8", h, group_list_type=1)
            if ev:
                ev[1].record()
            act = self.ops.silu_mul(h) if n_rows is None else ops.silu_mul_dyn(h, n_rows)
        if ev:
            ev[2].record()
        self.ops.grouped_gemm(act, self.w2, self.s2, self.o2, counts, "int8", y, group_list_type=1)
        if ev:
            ev[3].record()
            self.timing = ev
        return y

    # ---- one step --------------------------------------------------------------------------
    def forward(self, x, logits, record: bool = False, out_host=None):
        """x bf16 [T, H], logits bf16 [T, E] on this rank's device -> bf16 [T, H] (on the device, or
        written by the combine kernel into the pinned host tensor ``out_host`` when one is given)."""
        def finish(y, slot, wts):
            if out_host is not None:
                return self.ops.combine_to_host(y, slot, wts, out_host)
            return self.ops.combine(y, slot, wts)

        marks = [] if record else None

        def mark(name):
            if marks is not None:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record()
                marks.append((name, ev))

        mark("start")
        idx, wts, counts, token_of, slot = self.ops.route(logits, self.top_k)
        if self.px is not None:
            px = self.px
            if x.shape[0] * self.world * self.top_k > px.cap_rows:
                raise RuntimeError("more tokens than max_tokens")
            px.begin_step()
            px.post_counts(counts)
            mark("route")
            remote_pos, local_counts, n_recv = px.dispatch(x, token_of)
            px.wait(1)                                            # rows of every source rank have landed
            mark("dispatch")
            self._mid()
            if self.gemm == "packed":
                # the down projection hands every result row straight back to the rank its token came from
                # (stores over NVLink from the GEMM's epilogue); the weighted sum is then local
                self._experts(px.recv_x, local_counts, record, y=px.y, n_rows=n_recv,
                              scatter=(px.ret_code, px.ret_ptrs, px.cap_send), rows_sum=px.recv_sum)
                mark("experts")
                if out_host is None and x.shape[0] > 0:
                    # one launch: signal this rank's pushes, wait for every owner's, sum each token's rows
                    out = px.finish(slot, wts)
                else:
                    px.post(2)                                    # this rank's pushes are complete and visible
                    px.wait(2)                                    # every owner has pushed this rank's rows
                    out = finish(px.ret, slot, wts)
            else:
                self._experts(px.recv_x, local_counts, record, y=px.y, n_rows=n_recv)
                px.post(2)                                        # results of this rank are complete
                mark("experts")
                out = px.combine(remote_pos, slot, wts, out=out_host)  # a pinned host tensor is written directly
            mark("combine")
            self.phases = marks
            return out
        # one rank on the packed GEMMs: the gather also adds up each row (the gate/up GEMM's offset term needs
        # the sums and would otherwise read all rows once more)
        sums = None
        if (self.gather_sums and self.world == 1 and self.gemm == "packed" and self.o13 is not None
                and self.ops is CudaRowOps):
            send, sums = ops.gather_rows(x, token_of, with_sums=True)
        else:
            send = self.ops.gather_rows(x, token_of)             # [T*k, H] sorted by expert
        mark("route+gather")

        if self.world == 1:
            self._mid()
            y = self._experts(send, counts, record, rows_sum=sums)
            mark("experts")
            out = finish(y, slot, wts)
            mark("combine")
            self.phases = marks
            return out

        import torch.distributed as dist

        # per (destination rank, local expert) counts out, per (source rank, local expert) counts in
        send_counts = counts.reshape(self.world, self.e_local)
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts, group=self.group)
        # the variable all-to-all needs its split sizes on the host
        both = torch.stack([send_counts.sum(1), recv_counts.sum(1)]).cpu()
        in_split, out_split = both[0].tolist(), both[1].tolist()
        n_recv = int(sum(out_split))
        recv = torch.empty(n_recv, self.hidden, dtype=torch.bfloat16, device=self.device)
        dist.all_to_all_single(recv, send, out_split, in_split, group=self.group)
        mark("dispatch")

        # received order is (source rank, expert); the grouped GEMM wants expert-major
        pos, inv, local_counts = self.ops.regroup_index(recv_counts, n_recv)
        rows = self.ops.gather_rows(recv, inv)
        mark("regroup")
        self._mid()
        y = self._experts(rows, local_counts, record)
        mark("experts")
        back = self.ops.gather_rows(y, pos)                      # source-major again
        ret = torch.empty(send.shape[0], self.hidden, dtype=torch.bfloat16, device=self.device)
        dist.all_to_all_single(ret, back, in_split, out_split, group=self.group)
        mark("return")
        out = finish(ret, slot, wts)
        mark("combine")
        self.phases = marks
        return out

    def forward_host(self, x_host, logits_host, out_host=None):
        """End-to-end call with host buffers: pinned host -> device copies of this step's inputs,
        the layer, and the device -> host read of the result."""
        lg = logits_host.to(self.device, non_blocking=True)
        x = x_host.to(self.device, non_blocking=True)
        if out_host is None:
            out_host = torch.empty(x_host.shape, dtype=torch.bfloat16, pin_memory=True)
        self.forward(x, lg, out_host=out_host)
        torch.cuda.current_stream().synchronize()
        return out_host


class OverlappedSteps:
    """Steps of a p2p layer with the token exchange of step k+1 beside the expert GEMMs of step k.

    A step is split over two streams.  The exchange stream routes the step's tokens, posts the counts
    and stores the rows into their owners' receive buffers; the caller's stream waits for every rank's
    rows, runs the two grouped GEMMs (the second pushes each result row back to its source rank), waits
    for the pushes of the other ranks and sums each token's rows.  Steps alternate between the two
    buffer sets of the exchange, so step k+1's rows land in one set while step k's GEMMs read the
    other; step k+2's exchange waits for step k's weighted sum.  The persistent GEMM kernels leave
    ``reserve_sms`` multiprocessors free (``ops.set_gemm_reserved_sms``): their CTAs fill an SM, and the
    routing and row-store kernels of the next step need somewhere to run.  Nothing here synchronises
    with the host or calls a collective; every device-side wait is bounded as in the serial pass.

    ``submit`` takes inputs that are COMPLETE on the device when it is called (or by the ``ready`` event)
    and must stay untouched until the step's ``rows_sent`` event; results come back in submission order.
    All ranks must submit the same number of steps, and ``drain`` before the object is dropped or the layer's
    serial pass is used again.  The layer must have been built with
    ``exchange="p2p", exchange_buffers=2`` and the packed GEMMs."""

    def __init__(self, layer: "MoELayer", n_tokens: int, reserve_sms: int = 8, late_sum: bool = False,
                 defer_sum: bool = False):
        """``late_sum``: the end of a step -- the wait for the other ranks' pushes and the weighted sum -- also
        runs on the exchange stream, beside the NEXT step's gate/up GEMM, so the caller's stream goes from one
        step's down projection straight to the next step's gate/up GEMM and a slow peer's pushes are waited for
        off the critical path; both GEMMs then leave ``reserve_sms`` SMs free.  A step's result is then
        complete by the event of the handle ``submit`` returns (set by the next ``submit`` or by ``flush``),
        not in the order of the caller's stream.  Off by default: measured 2-4 % slower on 2 and 4 GPUs (the
        down projection gives up SMs as well and the sum runs on the few that are free).
        ``defer_sum`` (needs ``exchange_buffers=3``): the end of a step stays on the caller's stream but is
        enqueued after the NEXT step's GEMMs, so the wait for the slowest peer's pushes finds them long done
        -- the ranks stop meeting at a barrier every step; steps then rotate over three buffer sets (the
        exchange of step k+2 must not wait for the sum of step k, which now comes after step k+1's GEMMs).
        Results are complete by the handle's event, one ``submit`` (or ``flush``) later."""
        if layer.px is None or layer.px.n_buffers < 2 or layer.gemm != "packed":
            raise RuntimeError('OverlappedSteps needs exchange="p2p", exchange_buffers=2 or 3 and the packed GEMMs')
        if late_sum and defer_sum:
            raise ValueError("late_sum and defer_sum exclude one another")
        if defer_sum and layer.px.n_buffers < 3:
            raise RuntimeError("defer_sum needs exchange_buffers=3")
        self.layer, self.n_tokens, self.reserve_sms, self.late_sum = layer, n_tokens, reserve_sms, late_sum
        self.defer_sum, self.n_sets = defer_sum, (3 if defer_sum else 2)
        dev, px = layer.device, layer.px
        px.use_host_steps()
        self.s_x = torch.cuda.Stream(dev, priority=-1)
        # serial passes enqueued before this point on the caller's stream use the first buffer set
        self.s_x.wait_stream(torch.cuda.current_stream())
        n_rows = n_tokens * layer.top_k
        self.sets = []
        for _ in range(self.n_sets):
            self.sets.append(dict(
                route=ops.moe_route_buffers(n_tokens, layer.n_experts, layer.top_k, dev),
                disp=(torch.empty(n_rows, dtype=torch.int32, device=dev),
                      torch.empty(layer.e_local, dtype=torch.int64, device=dev),
                      torch.empty(1, dtype=torch.int64, device=dev)),
                act=torch.empty(px.cap_rows, layer.inter, dtype=torch.bfloat16, device=dev),
                done=None))
        self.n = 0
        self.rows_sent = None  # event: the rows of the step submitted last have left (its inputs are free)
        self.tail = None       # late_sum: what is left to enqueue of the step submitted last

    def _finish(self, tail):
        """Waits for every owner's pushes of the step, then sums each token's rows: on the exchange stream
        (late_sum) or on the caller's (defer_sum)."""
        layer, px = self.layer, self.layer.px
        stream = self.s_x if self.late_sum else torch.cuda.current_stream()
        with torch.cuda.stream(stream):
            stream.wait_event(tail["posted"])
            px.wait(2, step=tail["step"])
            handle = tail["handle"]
            if tail["out_free"] is not None:     # whoever last read the caller's output buffer
                stream.wait_event(tail["out_free"])
            if handle.out is None:               # (allocated on that stream: wait for the event before use elsewhere)
                handle.out = torch.empty(self.n_tokens, layer.hidden, dtype=torch.bfloat16, device=layer.device)
            layer.ops.combine(px.ret_sets[tail["parity"]], tail["slot"], tail["wts"], handle.out)
            handle.event = torch.cuda.Event()
            handle.event.record(stream)
            if self.defer_sum:
                self.sets[tail["parity"]]["done"] = handle.event

    def flush(self):
        """late_sum / defer_sum: enqueues the end of the step submitted last without waiting for a next step."""
        if self.tail is not None:
            tail, self.tail = self.tail, None
            self._finish(tail)

    def submit(self, x, logits, ready=None, out=None, out_free=None, record: bool = False):
        """One step.  Returns a handle: ``handle.out`` is the bf16 [T, H] result (``out`` if given; it is written
        once the event ``out_free`` has completed), complete once ``handle.event`` has -- which, without
        ``late_sum``, is in the order of the caller's stream.  ``record=True`` leaves CUDA events around the
        two GEMMs in ``layer.timing``."""
        layer, px = self.layer, self.layer.px
        if x.shape[0] != self.n_tokens:
            raise RuntimeError("OverlappedSteps was built for another token count")
        p = self.n % self.n_sets
        self.n += 1
        st = self.sets[p]
        step = px.begin_step()
        main = torch.cuda.current_stream()
        with torch.cuda.stream(self.s_x):
            if ready is not None:
                self.s_x.wait_event(ready)
            if st["done"] is not None:       # the step before last: its weighted sum has read this set
                self.s_x.wait_event(st["done"])
            idx, wts, counts, token_of, slot = layer.ops.route(logits, layer.top_k, out=st["route"])
            px.post_counts(counts, parity=p, step=step)
            # two 1024-thread CTAs per reserved SM: the dispatch never takes an SM the GEMMs could use
            _, local_counts, n_recv = px.dispatch(x, token_of, parity=p, step=step, out=st["disp"],
                                                  max_ctas=2 * self.reserve_sms)
            sent = torch.cuda.Event()
            sent.record(self.s_x)
        self.rows_sent = sent
        # late_sum: the previous step's end follows this step's exchange on the exchange stream (its own set of
        # buffers is the other one; the step before that, which used this set, ended before this exchange began)
        if self.late_sum:
            self.flush()
        main.wait_event(sent)
        px.wait(1, step=step)                # rows of every source rank have landed
        # The gate/up GEMM makes room: the next step's exchange is released when the previous step's weighted
        # sum ends, so it runs beside this kernel.  Without late_sum the down projection takes every SM (a
        # late exchange kernel would wait for that GEMM's first CTA to leave: time, not correctness).
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)] if record else None
        if ev:
            ev[0].record()
        prev = ops.set_gemm_reserved_sms(self.reserve_sms)
        try:
            ops.grouped_gemm_packed(px.recv_x_sets[p], layer.w13, layer.s13, layer.o13, local_counts, st["act"],
                                    group_list_type=1, gate_up_silu=True, x_rowsum=px.recv_sum_sets[p])
            if ev:
                ev[1].record()
                ev[2].record()
            if not self.late_sum:
                ops.set_gemm_reserved_sms(prev)  # (defer_sum too: nothing runs beside the down projection)
            ops.grouped_gemm_packed_scatter(st["act"], layer.w2, layer.s2, layer.o2, local_counts,
                                            px.ret_code_sets[p], px.ret_ptrs_sets[p], px.cap_send, group_list_type=1)
        finally:
            ops.set_gemm_reserved_sms(prev)
        if ev:
            ev[3].record()
        layer.timing = ev
        handle = StepResult(out)
        if self.late_sum or self.defer_sum:
            px.post(2, step=step)            # this rank's pushes are complete and visible
            posted = torch.cuda.Event()
            posted.record(main)
            if self.defer_sum:
                self.flush()                 # the previous step's end, behind this step's GEMMs on this stream
            self.tail = dict(step=step, parity=p, slot=slot, wts=wts, posted=posted, handle=handle, out_free=out_free)
            if self.late_sum:
                st["done"] = None            # the exchange stream itself orders the sets' reuse
            return handle
        if out_free is not None:
            main.wait_event(out_free)
        # one launch: signal this rank's pushes, wait for every owner's, sum each token's rows
        handle.out = px.finish(slot, wts, out=out, parity=p, step=step)
        st["done"] = torch.cuda.Event()
        st["done"].record(main)
        handle.event = st["done"]
        return handle

    def drain(self):
        """Waits (on the host) for everything submitted."""
        self.flush()
        self.s_x.synchronize()
        torch.cuda.current_stream().synchronize()


class StepResult:
    """Result of a submitted overlapped step: ``out`` once ``event`` (a CUDA event) has completed."""

    def __init__(self, out=None):
        self.out, self.event = out, None


class GraphedLayer:
    """One layer pass recorded as CUDA graphs and replayed: a step then costs the host two graph
    launches instead of a dozen kernel launches and as many allocations.  The pass is recorded in two
    parts that share a memory pool -- up to the point where the rows are with their experts, and from
    the expert GEMMs on -- so that a caller can put an event between them.  Needs a pass without host
    synchronisation: one rank, or ``exchange="p2p"`` (whose step number moves to the device so that
    the recorded kernel arguments stay valid).  With several ranks every rank must construct its
    GraphedLayer and call it the same number of times."""

    def __init__(self, layer: MoELayer, n_tokens: int):
        if layer.world > 1 and layer.px is None:
            raise RuntimeError("the NCCL exchange reads split sizes on the host and cannot be recorded")
        self.layer = layer
        dev = layer.device
        self.x = torch.zeros(n_tokens, layer.hidden, dtype=torch.bfloat16, device=dev)
        self.logits = torch.zeros(n_tokens, layer.n_experts, dtype=torch.bfloat16, device=dev)
        if layer.px is not None:
            layer.px.use_device_steps()
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):  # warm-up outside the recording (lazy initialisation, allocator pools)
                layer.forward(self.x, self.logits)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        before = ops.LAUNCHES
        self.head, self.tail = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
        pool = torch.cuda.graph_pool_handle()
        saved_hook = layer.mid_hook
        split = {"done": False}

        def cut():  # end of the first recording, start of the second, same stream and pool
            self.head.capture_end()
            self.tail.capture_begin(pool=pool)
            split["done"] = True

        layer.mid_hook = cut
        try:
            with torch.cuda.stream(side):
                self.head.capture_begin(pool=pool)
                try:
                    self.out = layer.forward(self.x, self.logits)
                finally:
                    (self.tail if split["done"] else self.head).capture_end()
        finally:
            layer.mid_hook = saved_hook
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        if not split["done"]:
            raise RuntimeError("the layer pass never reached its expert GEMMs while being recorded")
        self.launches = ops.LAUNCHES - before
        ops.LAUNCHES = before

    def __call__(self, x=None, logits=None, mid_event=None):
        """Runs one pass on the current stream; ``x`` / ``logits`` (device or pinned host tensors) are
        copied into the recorded inputs first.  ``mid_event`` is recorded between the two parts.
        Returns the recorded output tensor, which the next call overwrites."""
        if x is not None:
            self.x.copy_(x, non_blocking=True)
        if logits is not None:
            self.logits.copy_(logits, non_blocking=True)
        self.head.replay()
        if mid_event is not None:
            mid_event.record()
        self.tail.replay()
        ops._count(self.launches)
        return self.out


class PendingResult:
    """Handle of a submitted step.  ``synchronize`` returns when the step's result is in its host
    buffer (it enqueues the copy first if the pipeline was still holding it back)."""

    def __init__(self, pipe, step):
        self.pipe, self.step = pipe, step
        self.event = None  # set when the device -> host copy has been enqueued

    def synchronize(self):
        if self.event is None:
            self.pipe.flush()
        self.event.synchronize()


class HostPipeline:
    """Host-buffer calls with ``depth`` steps in flight.

    ``submit`` enqueues one step: the copy of its pinned-host inputs on a copy-in stream, the layer
    on the caller's current stream, the copy of its result to pinned host memory on a copy-out
    stream.  Step i+1's input copy and step i-1's output copy overlap step i's kernels (PCIe is
    full duplex, the copy engines are independent of the SMs); every step still moves all of its
    inputs and its whole result.  Both copies are held back until step i's rows are with their
    experts: host copies that run beside the routing and exchange kernels slow those down (measured:
    +0.25 ms per step on 2 GPUs), beside the expert GEMMs they cost nothing.  The copy of the last
    submitted step's result is therefore enqueued by the next ``submit``, by ``flush`` or by
    ``drain``.  ``submit`` returns a PendingResult; ``drain`` waits for everything submitted."""

    def __init__(self, layer: MoELayer, depth: int = 2, graphed: GraphedLayer = None,
                 overlapped: "OverlappedSteps" = None):
        """``graphed``: a GraphedLayer of ``layer`` for the token count the pipeline will be fed;
        the kernels of a step are then two graph launches.  ``overlapped``: an OverlappedSteps of
        ``layer`` instead: a step's token exchange then runs beside the GEMMs of the step before, its
        input copy is released as soon as the rows of the step that last used the slot have left, and
        its result is copied out as soon as it exists (the exchange is off the critical path there, so
        nothing is held back)."""
        if depth < 2:
            raise ValueError("depth must be at least 2")
        if graphed is not None and overlapped is not None:
            raise ValueError("graphed and overlapped exclude one another")
        self.layer, self.depth, self.graphed, self.overlapped = layer, depth, graphed, overlapped
        self.s_in, self.s_out = torch.cuda.Stream(layer.device), torch.cuda.Stream(layer.device)
        self.slots = [dict(x=None, lg=None, out=None, in_done=None, comp_done=None, out_done=None)
                      for _ in range(depth)]
        self.n = 0
        self.last_mid = None  # event between the two parts of the step submitted last
        self.pending = None   # (slot, out_host, PendingResult) of the step whose result copy is held back

    def _copy_out(self, after):
        """Enqueues the held-back result copy once ``after`` (an event) has completed."""
        if self.pending is None:
            return
        sl, out_host, handle = self.pending
        self.pending = None
        with torch.cuda.stream(self.s_out):
            if after is not None:
                self.s_out.wait_event(after)
            self.s_out.wait_event(sl["comp_done"])
            out_host.copy_(sl["out"], non_blocking=True)
            sl["out_done"] = torch.cuda.Event()
            sl["out_done"].record(self.s_out)
        handle.event = sl["out_done"]

    def _copy_out_overlapped(self):
        """Overlapped steps: enqueues the result copy of the pending step behind the step's own event."""
        if self.pending is None:
            return
        sl, out_host, handle, res = self.pending
        self.pending = None
        with torch.cuda.stream(self.s_out):
            self.s_out.wait_event(res.event)
            out_host.copy_(sl["out"], non_blocking=True)
            sl["out_done"] = torch.cuda.Event()
            sl["out_done"].record(self.s_out)
        handle.event = sl["out_done"]

    def flush(self):
        """Enqueues the result copy of the step submitted last without waiting for a next step."""
        if self.overlapped is not None:
            self.overlapped.flush()
            self._copy_out_overlapped()
            return
        self._copy_out(None)

    def submit(self, x_host, logits_host, out_host):
        sl = self.slots[self.n % self.depth]
        step = self.n
        self.n += 1
        main = torch.cuda.current_stream()
        if sl["x"] is None or sl["x"].shape != x_host.shape:
            sl["x"] = torch.empty(x_host.shape, dtype=x_host.dtype, device=self.layer.device)
            sl["lg"] = torch.empty(logits_host.shape, dtype=logits_host.dtype, device=self.layer.device)
        if self.overlapped is not None:
            with torch.cuda.stream(self.s_in):
                if sl.get("rows_sent") is not None:      # the exchange that last read these input buffers
                    self.s_in.wait_event(sl["rows_sent"])
                sl["lg"].copy_(logits_host, non_blocking=True)
                sl["x"].copy_(x_host, non_blocking=True)
                sl["in_done"] = torch.cuda.Event()
                sl["in_done"].record(self.s_in)
            if sl["out"] is None or sl["out"].shape != x_host.shape:
                sl["out"] = torch.empty(x_host.shape, dtype=torch.bfloat16, device=self.layer.device)
            # (with the late sum this call also enqueues the end of the step submitted before: its event exists now)
            res = self.overlapped.submit(sl["x"], sl["lg"], ready=sl["in_done"], out=sl["out"], out_free=sl["out_done"])
            sl["rows_sent"] = self.overlapped.rows_sent
            self._copy_out_overlapped()
            handle = PendingResult(self, step)
            self.pending = (sl, out_host, handle, res)
            if res.event is not None:
                self._copy_out_overlapped()
            return handle
        with torch.cuda.stream(self.s_in):
            # the previous step's rows are with their experts; that step follows, on the same stream,
            # the one that last read these input buffers
            if self.last_mid is not None:
                self.s_in.wait_event(self.last_mid)
            if sl["comp_done"] is not None:
                self.s_in.wait_event(sl["comp_done"])
            sl["lg"].copy_(logits_host, non_blocking=True)
            sl["x"].copy_(x_host, non_blocking=True)
            sl["in_done"] = torch.cuda.Event()
            sl["in_done"].record(self.s_in)
        main.wait_event(sl["in_done"])
        if sl["out_done"] is not None:               # the copy that last read this slot's result
            main.wait_event(sl["out_done"])
        mid = torch.cuda.Event()
        if self.graphed is not None:
            res = self.graphed(sl["x"], sl["lg"], mid_event=mid)
            if sl["out"] is None or sl["out"].shape != res.shape:
                sl["out"] = torch.empty_like(res)
            sl["out"].copy_(res, non_blocking=True)  # the recorded output is overwritten by the next step
        else:
            saved = self.layer.mid_hook
            self.layer.mid_hook = lambda: mid.record(main)
            try:
                sl["out"] = self.layer.forward(sl["x"], sl["lg"])
            finally:
                self.layer.mid_hook = saved
        sl["comp_done"] = torch.cuda.Event()
        sl["comp_done"].record(main)
        self.last_mid = mid
        self._copy_out(mid)                          # the previous step's result, beside this step's GEMMs
        handle = PendingResult(self, step)
        self.pending = (sl, out_host, handle)
        return handle

    def drain(self):
        self.flush()
        main = torch.cuda.current_stream()
        for sl in self.slots:
            if sl["out_done"] is not None:
                main.wait_event(sl["out_done"])
        main.synchronize()
