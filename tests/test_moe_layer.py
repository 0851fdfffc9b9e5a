"""Expert-parallel MoE layer: index logic on CPU ranks (gloo, world size 2) with stand-in row
operations, and the CUDA path on one GPU, both against the single-process oracle."""
import os
import socket
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from oracle import oracle as O  # noqa: E402


class TorchRowOps:
    """CPU stand-ins with the semantics of the CUDA row kernels (tests only)."""

    @staticmethod
    def route(logits, top_k):
        w, idx = O.route_topk(logits, top_k)
        T = logits.shape[0]
        flat = idx.reshape(-1)
        order = torch.argsort(flat, stable=True)
        token_of = (order // top_k).to(torch.int32)
        slot = torch.empty_like(order)
        slot[order] = torch.arange(order.numel())
        counts = torch.bincount(flat, minlength=logits.shape[1])
        return idx.to(torch.int32), w.contiguous(), counts, token_of, slot.reshape(T, top_k).to(torch.int32)

    @staticmethod
    def regroup_index(recv_counts, n_recv):
        world, e_local = recv_counts.shape
        blk = recv_counts.reshape(-1)
        src_start = torch.cumsum(blk, 0) - blk
        em = recv_counts.t().contiguous().reshape(-1)
        em_start = (torch.cumsum(em, 0) - em).reshape(e_local, world).t().reshape(-1)
        pos = torch.repeat_interleave(em_start - src_start, blk, output_size=n_recv) + torch.arange(n_recv)
        inv = torch.empty_like(pos)
        inv[pos] = torch.arange(n_recv)
        return pos.to(torch.int32), inv.to(torch.int32), recv_counts.sum(0)

    @staticmethod
    def gather_rows(src, index, out=None):
        return src[index.long()].contiguous()

    @staticmethod
    def combine(y, slot, weight, out=None):
        acc = (y[slot.long()].float() * weight.unsqueeze(-1)).sum(1)
        return acc.to(torch.bfloat16)

    @staticmethod
    def silu_mul(h, out=None):
        I = h.shape[1] // 2
        return (torch.nn.functional.silu(h[:, :I].float()) * h[:, I:].float()).to(torch.bfloat16)

    @staticmethod
    def grouped_gemm(x, w, s, o, gl, ct, out, group_list_type=0, **kw):
        O.grouped_gemm(x, w, s, o, gl, ct, out, group_list_type=group_list_type)


def small_case(seed=4, T=48, H=128, E=8, I=64, k=2):
    gen = torch.Generator().manual_seed(seed)
    x = torch.randn(T, H, generator=gen).to(torch.bfloat16)
    logits = torch.randn(T, E, generator=gen).to(torch.bfloat16)
    w13 = torch.randint(-128, 128, (E, H, 2 * I), generator=gen, dtype=torch.int8)
    w2 = torch.randint(-128, 128, (E, I, H), generator=gen, dtype=torch.int8)
    s13 = (torch.rand(E, 2 * I, generator=gen) * 0.009 + 0.001).to(torch.bfloat16)
    o13 = (torch.rand(E, 2 * I, generator=gen) * 8 - 4).to(torch.bfloat16)
    s2 = (torch.rand(E, H, generator=gen) * 0.009 + 0.001).to(torch.bfloat16)
    o2 = (torch.rand(E, H, generator=gen) * 8 - 4).to(torch.bfloat16)
    return dict(x=x, logits=logits, w13=w13, s13=s13, o13=o13, w2=w2, s2=s2, o2=o2, top_k=k, E=E)


def close(out, gold):
    # fp32 sums in a different order, silu via expf on the GPU: a few bf16 steps at most
    o, g = out.float(), gold.float()
    assert O.rel_l2(o, g) < 4e-3, O.rel_l2(o, g)
    assert float((o - g).abs().max()) <= 0.05 * float(g.abs().max())


def test_single_process_index_logic_matches_oracle():
    from ascend_kernel_b200.moe_layer import MoELayer

    c = small_case()
    layer = MoELayer(c["w13"], c["s13"], c["o13"], c["w2"], c["s2"], c["o2"], c["E"], c["top_k"], None, TorchRowOps)
    out = layer.forward(c["x"], c["logits"])
    gold = O.moe_layer(c["x"], c["logits"], c["w13"], c["s13"], c["o13"], c["w2"], c["s2"], c["o2"], c["top_k"])
    close(out, gold)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _step_inputs(c, step):
    """Inputs of step `step`: the case's tokens, rows reversed on odd steps."""
    if step % 2 == 0:
        return c["x"], c["logits"]
    return torch.flip(c["x"], [0]).contiguous(), torch.flip(c["logits"], [0]).contiguous()


def _rank_main(rank, world, port, q, cuda=False, case_kw=None, exchange="nccl", steps=1):
    import torch.distributed as dist

    from ascend_kernel_b200.moe_layer import CudaRowOps, MoELayer

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    if cuda:
        os.environ["NCCL_NVLS_ENABLE"] = "0"
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    else:
        dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        c = small_case(**(case_kw or {}))
        dev = torch.device("cuda", rank) if cuda else torch.device("cpu")
        el, tl = c["E"] // world, c["x"].shape[0] // world
        sl = slice(rank * el, (rank + 1) * el)
        w = [c[k][sl].contiguous().to(dev) for k in ("w13", "s13", "o13", "w2", "s2", "o2")]
        overlap, defer = exchange in ("p2p+overlap", "p2p+defer"), exchange == "p2p+defer"
        if overlap:
            exchange = "p2p"
        layer = MoELayer(*w, c["E"], c["top_k"], dist.group.WORLD, CudaRowOps if cuda else TorchRowOps,
                         exchange=exchange, max_tokens=tl, exchange_buffers=(3 if defer else 2) if overlap else 1)
        outs = []
        if overlap:
            # every step enqueued before the host looks at anything: the exchange of a step runs beside the
            # GEMMs of the one before
            from ascend_kernel_b200.moe_layer import OverlappedSteps

            ins = [tuple(t[rank * tl:(rank + 1) * tl].to(dev) for t in _step_inputs(c, step)) for step in range(steps)]
            torch.cuda.synchronize()
            # (the six-step test runs the late sum)
            ov = OverlappedSteps(layer, tl, reserve_sms=8, late_sum=(steps % 2 == 0 and not defer), defer_sum=defer)
            res = [ov.submit(x, lg) for x, lg in ins]
            ov.drain()
            res = [h.out for h in res]
            outs = [r.cpu().view(torch.int16).numpy() for r in res]
            # and the serial pass still works on the same layer afterwards
            x, lg = ins[0]
            assert torch.equal(layer.forward(x, lg).cpu().view(torch.int16), res[0].cpu().view(torch.int16))
        for step in range(0 if overlap else steps):
            x, lg = _step_inputs(c, step)
            out = layer.forward(x[rank * tl:(rank + 1) * tl].to(dev), lg[rank * tl:(rank + 1) * tl].to(dev))
            outs.append(out.cpu().view(torch.int16).numpy())
        if cuda:
            torch.cuda.synchronize()
        status = layer.px.read_status() if layer.px is not None else (0, 0)
        dist.barrier()  # peers may still be reading this rank's result buffer until they are done too
        if layer.px is not None:
            layer.px.close()
        q.put((rank, (outs if steps > 1 else outs[0], status) if exchange == "p2p" else outs[0]))  # ("p2p+overlap" -> "p2p" above)
    finally:
        dist.destroy_process_group()


def test_two_cpu_ranks_dispatch_and_combine_match_oracle():
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = dict(q.get(timeout=240) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    c = small_case()
    gold = O.moe_layer(c["x"], c["logits"], c["w13"], c["s13"], c["o13"], c["w2"], c["s2"], c["o2"], c["top_k"])
    out = torch.cat([torch.from_numpy(got[r]).view(torch.bfloat16) for r in range(2)])
    close(out, gold)
    # and identical to the single-process run of the same stand-in operations
    from ascend_kernel_b200.moe_layer import MoELayer

    one = MoELayer(c["w13"], c["s13"], c["o13"], c["w2"], c["s2"], c["o2"], c["E"], c["top_k"], None,
                   TorchRowOps).forward(c["x"], c["logits"])
    assert torch.equal(out.view(torch.int16), one.view(torch.int16))


@pytest.mark.gpu
def test_cuda_layer_matches_oracle():
    from ascend_kernel_b200.moe_layer import MoELayer

    c = small_case(T=200, H=256, E=8, I=256, k=2)
    d = {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in c.items()}
    layer = MoELayer(d["w13"], d["s13"], d["o13"], d["w2"], d["s2"], d["o2"], c["E"], c["top_k"])
    out = layer.forward(d["x"], d["logits"])
    torch.cuda.synchronize()
    gold = O.moe_layer(c["x"], c["logits"], c["w13"], c["s13"], c["o13"], c["w2"], c["s2"], c["o2"], c["top_k"])
    close(out.cpu(), gold)
    host = layer.forward_host(c["x"].pin_memory(), c["logits"].pin_memory())
    assert torch.equal(host.view(torch.int16), out.cpu().view(torch.int16))


@pytest.mark.gpu
def test_host_pipeline_matches_single_calls():
    """Five different batches through the two-steps-in-flight host pipeline give the bits of the
    one-at-a-time host call (buffer reuse across slots must not mix steps up)."""
    from ascend_kernel_b200.moe_layer import HostPipeline, MoELayer

    c = small_case(T=200, H=256, E=8, I=256, k=2)
    d = {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in c.items()}
    layer = MoELayer(d["w13"], d["s13"], d["o13"], d["w2"], d["s2"], d["o2"], c["E"], c["top_k"])
    g = torch.Generator().manual_seed(11)
    xs = [torch.randn(c["x"].shape, generator=g).to(torch.bfloat16).pin_memory() for _ in range(5)]
    lgs = [c["logits"][torch.randperm(c["logits"].shape[0], generator=g)].contiguous().pin_memory() for _ in range(5)]
    want = [layer.forward_host(x, lg).clone() for x, lg in zip(xs, lgs)]
    pipe = HostPipeline(layer, depth=2)
    outs = [torch.empty(c["x"].shape, dtype=torch.bfloat16).pin_memory() for _ in range(5)]
    handles = [pipe.submit(x, lg, o) for x, lg, o in zip(xs, lgs, outs)]
    # a result is in its host buffer once its handle has been waited for: the first because the next
    # submit enqueued its copy, the last because the wait itself does
    handles[0].synchronize()
    assert torch.equal(outs[0].view(torch.int16), want[0].view(torch.int16))
    assert handles[-1].event is None
    handles[-1].synchronize()
    assert torch.equal(outs[-1].view(torch.int16), want[-1].view(torch.int16))
    pipe.drain()
    for o, w in zip(outs, want):
        assert torch.equal(o.view(torch.int16), w.view(torch.int16))
    with pytest.raises(ValueError):
        HostPipeline(layer, depth=1)


@pytest.mark.gpu
def test_graphed_layer_replays_match_eager_calls():
    """The recorded pass (direct path and peer-memory exchange) replayed on new inputs gives the bits
    of the eager call, also through the host pipeline."""
    from ascend_kernel_b200.moe_layer import GraphedLayer, HostPipeline, MoELayer

    c = small_case(T=200, H=256, E=8, I=256, k=2)
    d = {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in c.items()}
    w = [d[k] for k in ("w13", "s13", "o13", "w2", "s2", "o2")]
    eager = MoELayer(*w, c["E"], c["top_k"])
    for exchange in ("nccl", "p2p"):  # one rank: "nccl" is the direct path
        layer = MoELayer(*w, c["E"], c["top_k"], exchange=exchange, max_tokens=200)
        g = GraphedLayer(layer, 200)
        for step in range(3):
            x, lg = _step_inputs(c, step)
            want = eager.forward(x.cuda(), lg.cuda())
            got = g(x.cuda(), lg.cuda())
            torch.cuda.synchronize()
            assert torch.equal(got.view(torch.int16), want.view(torch.int16)), (exchange, step)
        pipe = HostPipeline(layer, depth=2, graphed=g)
        outs = [torch.empty(200, 256, dtype=torch.bfloat16).pin_memory() for _ in range(4)]
        for step in range(4):
            x, lg = _step_inputs(c, step)
            pipe.submit(x.pin_memory(), lg.pin_memory(), outs[step])
        pipe.drain()
        for step in range(4):
            x, lg = _step_inputs(c, step)
            want = eager.forward(x.cuda(), lg.cuda()).cpu()
            assert torch.equal(outs[step].view(torch.int16), want.view(torch.int16)), (exchange, step)
        if layer.px is not None:
            assert layer.px.read_status()[0] == 0
            layer.px.close()


@pytest.mark.gpu
def test_fused_silu_gemm_equals_gemm_then_silu_bit_for_bit():
    """b200moe_grouped_gemm_int8_silu on interleaved weights = b200moe_grouped_gemm + b200moe_silu_mul
    on the plain ones, on ragged groups (empty expert, one row, more than one tile, rows of nobody)."""
    import ascend_kernel_b200 as ak
    from ascend_kernel_b200 import ops

    gen = torch.Generator().manual_seed(5)
    G, K, I = 5, 192, 384
    counts = torch.tensor([3, 0, 300, 1, 129], dtype=torch.int64)
    M = int(counts.sum()) + 2
    x = torch.randn(M, K, generator=gen).to(torch.bfloat16).cuda()
    w = torch.randint(-128, 128, (G, K, 2 * I), generator=gen, dtype=torch.int8).cuda()
    s = (torch.rand(G, 2 * I, generator=gen) * 0.009 + 0.001).to(torch.bfloat16).cuda()
    o = (torch.rand(G, 2 * I, generator=gen) * 8 - 4).to(torch.bfloat16).cuda()
    for off in (o, None):
        h = torch.zeros(M, 2 * I, dtype=torch.bfloat16, device="cuda")
        ak.grouped_gemm(x, w, s, off, counts.cuda(), "int8", h, group_list_type=1)
        want = ak.silu_mul(h)
        got = torch.full((M, I), -768.0, dtype=torch.bfloat16, device="cuda")
        ws = ops.grouped_gemm_silu(x, ops.interleave_gate_up(w), ops.interleave_gate_up(s),
                                   None if off is None else ops.interleave_gate_up(off), counts.cuda(), got,
                                   group_list_type=1, return_workspace=True)
        torch.cuda.synchronize()
        assert ak.read_status(ws) == (0, 0)
        assert torch.equal(got[:M - 2].view(torch.int16), want[:M - 2].view(torch.int16))
        assert bool((got[M - 2:] == -768.0).all())


@pytest.mark.gpu
def test_layer_with_and_without_fused_silu_agree_bit_for_bit():
    from ascend_kernel_b200.moe_layer import MoELayer

    c = small_case(T=200, H=256, E=8, I=256, k=2)
    d = {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in c.items()}
    w = [d[k] for k in ("w13", "s13", "o13", "w2", "s2", "o2")]
    a = MoELayer(*w, c["E"], c["top_k"], fuse_silu=True, gemm="generic").forward(d["x"], d["logits"])
    b = MoELayer(*w, c["E"], c["top_k"], fuse_silu=False, gemm="generic").forward(d["x"], d["logits"])
    torch.cuda.synchronize()
    assert torch.equal(a.view(torch.int16), b.view(torch.int16))


@pytest.mark.gpu
def test_layer_on_packed_weights_agrees_with_the_drop_in_operator_path():
    """The layer's default (weights repacked once, dequantised into tensor memory) against the same
    layer on the [G, K, N] tensors through the drop-in grouped GEMM, and both against the oracle."""
    from ascend_kernel_b200.moe_layer import MoELayer

    c = small_case(T=400, H=256, E=8, I=256, k=4)
    d = {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in c.items()}
    w = [d[k] for k in ("w13", "s13", "o13", "w2", "s2", "o2")]
    packed = MoELayer(*w, c["E"], c["top_k"])
    assert packed.gemm == "packed"
    a = packed.forward(d["x"], d["logits"])
    b = MoELayer(*w, c["E"], c["top_k"], gemm="generic").forward(d["x"], d["logits"])
    torch.cuda.synchronize()
    gold = O.moe_layer(c["x"], c["logits"], c["w13"], c["s13"], c["o13"], c["w2"], c["s2"], c["o2"], c["top_k"])
    close(a.cpu(), gold)
    close(b.cpu(), gold)
    assert O.rel_l2(a.float().cpu(), b.float().cpu()) < 2e-3


@pytest.mark.gpu
def test_layer_on_fp4_stored_experts_matches_oracle():
    """Experts stored as FP4 e2m1 with e8m0 block scales, dequantised to bf16 in every pass and multiplied by
    the bf16 grouped GEMM, against the CPU golden of the same two phases."""
    from ascend_kernel_b200.moe_layer import MoELayer

    gen = torch.Generator().manual_seed(9)
    T, H, E, I, k = 300, 256, 8, 256, 2
    x = torch.randn(T, H, generator=gen).to(torch.bfloat16)
    logits = torch.randn(T, E, generator=gen).to(torch.bfloat16)
    c13 = torch.randint(0, 256, (E, H, I), generator=gen, dtype=torch.uint8)
    s13 = torch.randint(119, 128, (E, H, 2 * I // 32), generator=gen, dtype=torch.uint8)
    c2 = torch.randint(0, 256, (E, I, H // 2), generator=gen, dtype=torch.uint8)
    s2 = torch.randint(119, 128, (E, I, H // 32), generator=gen, dtype=torch.uint8)
    layer = MoELayer(c13.cuda(), s13.cuda(), None, c2.cuda(), s2.cuda(), None, E, k, weight_format="fp4")
    out = layer.forward(x.cuda(), logits.cuda())
    torch.cuda.synchronize()
    layer.read_status()
    # the layer's bf16 weight buffers hold the exact dequantised values
    assert torch.equal(layer.bf13.cpu().view(torch.int16), O.fp4_dequant_e8m0(c13, s13).view(torch.int16))
    gold = O.moe_layer_fp4_stored(x, logits, c13, s13, c2, s2, k)
    close(out.cpu(), gold)
    with pytest.raises(ValueError):
        MoELayer(c13.cuda(), s13.cuda(), s13.cuda(), c2.cuda(), s2.cuda(), None, E, k, weight_format="fp4")


@pytest.mark.gpu
def test_layer_reports_device_findings():
    """MoELayer.read_status raises when a kernel of an earlier pass left a finding (here: a grouped GEMM
    called directly with a group list that is not monotone) and is quiet otherwise."""
    import ascend_kernel_b200 as ak
    from ascend_kernel_b200.moe_layer import MoELayer

    c = small_case(T=64, H=256, E=8, I=256, k=2)
    d = {k_: (v.cuda() if torch.is_tensor(v) else v) for k_, v in c.items()}
    layer = MoELayer(d["w13"], d["s13"], d["o13"], d["w2"], d["s2"], d["o2"], c["E"], c["top_k"])
    ak.check_status()
    layer.forward(d["x"], d["logits"])
    assert layer.read_status() == (0, 0)
    out = torch.zeros(64, 512, dtype=torch.bfloat16, device="cuda")
    bad = torch.tensor([40, 3, 3, 3, 3, 3, 3, 3], dtype=torch.int64, device="cuda")  # cumulative list going down
    ak.grouped_gemm(d["x"], d["w13"], d["s13"], d["o13"], bad, "int8", out)
    layer.forward(d["x"], d["logits"])
    with pytest.raises(RuntimeError, match="group list"):
        layer.read_status()
    assert layer.read_status() == (0, 0)


@pytest.mark.gpu
def test_aux_kernels_match_torch():
    import ascend_kernel_b200 as ak

    gen = torch.Generator().manual_seed(0)
    h = torch.randn(37, 512, generator=gen).to(torch.bfloat16)
    got = ak.silu_mul(h.cuda()).cpu().float()
    want = TorchRowOps.silu_mul(h).float()
    assert torch.allclose(got, want, rtol=2e-2, atol=1e-3)
    src = torch.randn(50, 256, generator=gen).to(torch.bfloat16)
    idx = torch.randint(0, 50, (77,), generator=gen, dtype=torch.int32)
    assert torch.equal(ak.gather_rows(src.cuda(), idx.cuda()).cpu().view(torch.int16), src[idx.long()].view(torch.int16))
    slot = torch.randint(0, 50, (20, 4), generator=gen, dtype=torch.int32)
    w = torch.rand(20, 4, generator=gen)
    got = ak.combine(src.cuda(), slot.cuda(), w.cuda()).cpu().float()
    want = (src[slot.long()].float() * w.unsqueeze(-1)).sum(1)
    assert torch.allclose(got, want, rtol=1e-2, atol=1e-2)


@pytest.mark.gpu
def test_two_gpu_ranks_match_oracle():
    """Expert-parallel layer over NCCL on two GPUs (skipped on a single-GPU box)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    kw = dict(T=200, H=256, E=8, I=256, k=2)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, q, True, kw)) for r in range(2)]
    for p in procs:
        p.start()
    got = dict(q.get(timeout=300) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    c = small_case(**kw)
    gold = O.moe_layer(c["x"], c["logits"], c["w13"], c["s13"], c["o13"], c["w2"], c["s2"], c["o2"], c["top_k"])
    out = torch.cat([torch.from_numpy(got[r]).view(torch.bfloat16) for r in range(2)])
    close(out, gold)


@pytest.mark.gpu
def test_peer_memory_exchange_single_rank_matches_direct_path():
    """exchange="p2p" with one rank (the rank is its own peer): every exchange kernel runs, and
    three steps in a row give the bits of the direct path."""
    from ascend_kernel_b200.moe_layer import MoELayer

    c = small_case(T=200, H=256, E=8, I=256, k=2)
    d = {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in c.items()}
    w = [d[k] for k in ("w13", "s13", "o13", "w2", "s2", "o2")]
    direct = MoELayer(*w, c["E"], c["top_k"])
    p2p = MoELayer(*w, c["E"], c["top_k"], exchange="p2p", max_tokens=256)
    for step in range(3):
        x, lg = _step_inputs(c, step)
        n = 200 - 40 * step  # fewer tokens each step: stale rows of earlier steps must not leak in
        a = direct.forward(x[:n].cuda(), lg[:n].cuda())
        b = p2p.forward(x[:n].cuda(), lg[:n].cuda())
        torch.cuda.synchronize()
        assert torch.equal(a.view(torch.int16), b.view(torch.int16)), step
    assert p2p.px.read_status()[0] == 0
    host = torch.empty(120, 256, dtype=torch.bfloat16).pin_memory()
    p2p.forward(c["x"][:120].cuda(), c["logits"][:120].cuda(), out_host=host)
    torch.cuda.synchronize()
    want = direct.forward(c["x"][:120].cuda(), c["logits"][:120].cuda())
    assert torch.equal(host.view(torch.int16), want.cpu().view(torch.int16))
    p2p.px.close()


@pytest.mark.gpu
def test_peer_memory_wait_expires_with_status_instead_of_hanging():
    """A wait for a signal nobody posts gives up after its time limit, records status 2 and leaves
    the context usable: the next complete step is still right."""
    import time

    from ascend_kernel_b200 import _abi
    from ascend_kernel_b200.moe_layer import MoELayer

    c = small_case(T=64, H=256, E=8, I=256, k=2)
    d = {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in c.items()}
    w = [d[k] for k in ("w13", "s13", "o13", "w2", "s2", "o2")]
    p2p = MoELayer(*w, c["E"], c["top_k"], exchange="p2p", max_tokens=64)
    p2p.px.begin_step()
    t0 = time.time()
    p2p.px.wait(_abi.EP_SIG_ROWS)  # no dispatch ran in this step: the rows signal never comes
    torch.cuda.synchronize()
    assert 1.0 < time.time() - t0 < 10.0
    assert p2p.px.read_status()[0] == 2
    p2p.px.status.zero_()
    # a dispatch whose counts never arrive (a step was opened, nobody posted counts) stores no row anywhere,
    # and a combine whose results are never signalled reads none: the buffers keep what they held
    from ascend_kernel_b200 import ops

    p2p.px.recv_x.fill_(-3.0)
    p2p.px.y.fill_(-5.0)
    p2p.px.begin_step()
    _, wts, _, token_of, slot = ops.moe_route(d["logits"], c["top_k"])
    remote_pos, _, _ = p2p.px.dispatch(d["x"], token_of)
    late = p2p.px.combine(remote_pos, slot, wts)
    torch.cuda.synchronize()
    assert p2p.px.read_status()[0] == 2
    assert bool((remote_pos == -1).all())
    assert bool((p2p.px.recv_x == -3.0).all()) and bool((p2p.px.y == -5.0).all())
    assert bool((late == 0).all())
    p2p.px.status.zero_()
    out = p2p.forward(d["x"], d["logits"])
    want = MoELayer(*w, c["E"], c["top_k"]).forward(d["x"], d["logits"])
    torch.cuda.synchronize()
    assert torch.equal(out.view(torch.int16), want.view(torch.int16))
    assert p2p.px.read_status()[0] == 0
    p2p.px.close()


@pytest.mark.gpu
def test_two_gpu_ranks_peer_memory_exchange_matches_oracle():
    """The peer-memory exchange on two GPUs, three steps with changing inputs (skipped on a
    single-GPU box: kernels that wait for each other never share one GPU)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    kw = dict(T=200, H=256, E=8, I=256, k=2)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, q, True, kw, "p2p", 3)) for r in range(2)]
    for p in procs:
        p.start()
    got = dict(q.get(timeout=300) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    c = small_case(**kw)
    for r in range(2):
        assert got[r][1][0] == 0, got[r][1]
    for step in range(3):
        x, lg = _step_inputs(c, step)
        gold = O.moe_layer(x, lg, c["w13"], c["s13"], c["o13"], c["w2"], c["s2"], c["o2"], c["top_k"])
        out = torch.cat([torch.from_numpy(got[r][0][step]).view(torch.bfloat16) for r in range(2)])
        close(out, gold)


@pytest.mark.gpu
def test_overlapped_steps_single_rank_match_direct_path():
    """Steps whose exchange runs on a second stream beside the GEMMs of the step before (one rank, which is
    its own peer): seven steps enqueued without a host synchronisation give the bits of the direct path,
    with the GEMMs leaving SMs free and with none reserved; the layer's serial pass and a recorded pass
    still work afterwards."""
    from ascend_kernel_b200 import ops
    from ascend_kernel_b200.moe_layer import GraphedLayer, MoELayer, OverlappedSteps

    c = small_case(T=200, H=256, E=8, I=256, k=2)
    d = {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in c.items()}
    w = [d[k] for k in ("w13", "s13", "o13", "w2", "s2", "o2")]
    direct = MoELayer(*w, c["E"], c["top_k"])
    p2p = MoELayer(*w, c["E"], c["top_k"], exchange="p2p", max_tokens=200, exchange_buffers=2)
    ins = []
    for step in range(7):
        x, lg = _step_inputs(c, step)
        ins.append((torch.roll(x, step, 0).cuda(), torch.roll(lg, 3 * step, 0).cuda()))
    want = [direct.forward(x, lg) for x, lg in ins]
    torch.cuda.synchronize()
    for reserve, late in ((8, True), (0, False), (4, False), (8, True)):
        ov = OverlappedSteps(p2p, 200, reserve_sms=reserve, late_sum=late)
        got = [ov.submit(x, lg) for x, lg in ins]
        assert all(h.event is not None for h in got[:-1]) and (got[-1].event is None) == late
        ov.drain()
        assert ops.set_gemm_reserved_sms(0) == 0          # restored after every step
        for step, (a, b) in enumerate(zip(want, got)):
            assert torch.equal(a.view(torch.int16), b.out.view(torch.int16)), (reserve, late, step)
    assert p2p.px.read_status()[0] == 0
    # the sum of a step deferred behind the next step's GEMMs: three buffer sets
    p3 = MoELayer(*w, c["E"], c["top_k"], exchange="p2p", max_tokens=200, exchange_buffers=3)
    ov = OverlappedSteps(p3, 200, defer_sum=True)
    got = [ov.submit(x, lg) for x, lg in ins]
    assert got[-1].event is None and all(h.event is not None for h in got[:-1])
    ov.drain()
    for step, (a, b) in enumerate(zip(want, got)):
        assert torch.equal(a.view(torch.int16), b.out.view(torch.int16)), ("defer", step)
    assert p3.px.read_status()[0] == 0
    p3.px.close()
    # host buffers in, host buffers out, three steps in flight over overlapped steps (both kinds of step end)
    from ascend_kernel_b200.moe_layer import HostPipeline

    for late in (True, False):
        pipe = HostPipeline(p2p, depth=3, overlapped=OverlappedSteps(p2p, 200, late_sum=late))
        host_in = [(x.cpu().pin_memory(), lg.cpu().pin_memory()) for x, lg in ins]
        host_out = [torch.empty(200, 256, dtype=torch.bfloat16).pin_memory() for _ in ins]
        handles = [pipe.submit(x, lg, o) for (x, lg), o in zip(host_in, host_out)]
        handles[2].synchronize()
        assert torch.equal(want[2].cpu().view(torch.int16), host_out[2].view(torch.int16))
        pipe.drain()
        for step, (a, b) in enumerate(zip(want, host_out)):
            assert torch.equal(a.cpu().view(torch.int16), b.view(torch.int16)), (late, step)
    b = p2p.forward(*ins[1])
    assert torch.equal(want[1].view(torch.int16), b.view(torch.int16))
    g = GraphedLayer(p2p, 200)
    out = g(*ins[2]).clone()
    torch.cuda.synchronize()
    assert torch.equal(want[2].view(torch.int16), out.view(torch.int16))
    with pytest.raises(RuntimeError):                     # recorded passes keep the step number on the device
        p2p.px.post(2, step=5)
    ov = OverlappedSteps(p2p, 200)                        # ... and overlapped steps take it back
    got = ov.submit(*ins[3])
    ov.drain()
    assert torch.equal(want[3].view(torch.int16), got.out.view(torch.int16))
    assert p2p.px.read_status()[0] == 0
    p2p.px.close()


@pytest.mark.gpu
def test_two_gpu_ranks_overlapped_steps_match_oracle():
    """Overlapped steps on two GPUs: six steps with changing inputs, all enqueued up front."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    _two_gpu_overlapped(dict(T=200, H=256, E=8, I=256, k=2), "p2p+overlap", 6)


@pytest.mark.gpu
def test_two_gpu_ranks_overlapped_steps_with_deferred_sum_match_oracle():
    """The same with a step's weighted sum enqueued behind the next step's GEMMs (three buffer sets): seven
    steps, so every set is used at least twice."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    _two_gpu_overlapped(dict(T=200, H=256, E=8, I=256, k=2), "p2p+defer", 7)


def _two_gpu_overlapped(kw, exchange, steps):
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, q, True, kw, exchange, steps)) for r in range(2)]
    for p in procs:
        p.start()
    got = dict(q.get(timeout=300) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    c = small_case(**kw)
    for r in range(2):
        assert got[r][1][0] == 0, got[r][1]
    for step in range(steps):
        x, lg = _step_inputs(c, step)
        gold = O.moe_layer(x, lg, c["w13"], c["s13"], c["o13"], c["w2"], c["s2"], c["o2"], c["top_k"])
        out = torch.cat([torch.from_numpy(got[r][0][step]).view(torch.bfloat16) for r in range(2)])
        close(out, gold)


@pytest.mark.gpu
def test_route_and_regroup_kernels_match_torch():
    import ascend_kernel_b200 as ak
    from ascend_kernel_b200 import ops

    gen = torch.Generator().manual_seed(3)
    T, E, k = 333, 256, 8
    # distinct, bf16-exact logits per token (no ties, so the selected set is unambiguous)
    logits = torch.stack([torch.randperm(E, generator=gen) for _ in range(T)]).float().div(16).sub(8).to(torch.bfloat16)
    idx, w, counts, token_of, slot = ops.moe_route(logits.cuda(), k)
    torch.cuda.synchronize()
    rw, ridx = O.route_topk(logits, k)
    # same expert sets and weights
    got_sorted, order = torch.sort(idx.cpu().long(), dim=1)
    want_sorted, worder = torch.sort(ridx, dim=1)
    tie_free = (got_sorted == want_sorted).all(1)
    assert tie_free.all()
    assert torch.allclose(torch.gather(w.cpu(), 1, order)[tie_free], torch.gather(rw, 1, worder)[tie_free], rtol=1e-4, atol=1e-6)
    assert torch.allclose(w.cpu().sum(1), torch.ones(T), atol=1e-5)
    assert torch.equal(counts.cpu(), torch.bincount(idx.cpu().long().reshape(-1), minlength=E))
    # slot / token_of are a consistent permutation, grouped by expert
    pos = slot.cpu().long().reshape(-1)
    assert torch.equal(torch.sort(pos)[0], torch.arange(T * k))
    assert torch.equal(token_of.cpu().long()[pos], torch.arange(T * k) // k)
    expert_of_pos = torch.empty(T * k, dtype=torch.long)
    expert_of_pos[pos] = idx.cpu().long().reshape(-1)
    assert (expert_of_pos[1:] >= expert_of_pos[:-1]).all()
    # regroup index
    rc = torch.randint(0, 7, (4, 16), generator=gen)
    n = int(rc.sum())
    p, inv, lc = ops.moe_regroup_index(rc.cuda(), n)
    tp, tinv, tlc = TorchRowOps.regroup_index(rc, n)
    assert torch.equal(p.cpu(), tp) and torch.equal(inv.cpu(), tinv) and torch.equal(lc.cpu(), tlc)
