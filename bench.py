#!/usr/bin/env python
"""Benchmark of the MoE expert-GEMM hot path on B200.

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...        # the CPU golden path on the host cores

One step = one pass of the expert-parallel MoE FFN layer (benchmark configuration 4: 4096 tokens,
hidden 7168, 256 experts, intermediate 2048, top-8, int8 antiquant weights with per-channel
scale/offset) over a batch of seeded synthetic tokens.  The global batch is fixed (strong
scaling): each of the N ranks holds 4096/N tokens and 256/N experts.

Rank 0 prints ONE JSON line.  `value` is whole-job tokens/s with inputs resident in HBM; `e2e` is
the same metric through the public host-buffer call (`HostPipeline.submit`: pinned host -> device
copies of every step's inputs and the device -> host read of every step's result inside the timed
region, two steps in flight -- three on several GPUs -- so that the copies of neighbouring steps overlap
the expert GEMMs; `single_step_latency_ms` is the unpipelined `MoELayer.forward_host`).  On several GPUs
(peer-memory exchange) the steps are `OverlappedSteps`: a step's routing and token dispatch run on a second
stream beside the previous step's gate/up GEMM; `phases_ms_rank0` then comes from serial passes made before
the timed region, `--no-overlap` times the serial pass itself.  `roofline` covers the
dominant kernel of the step (the tcgen05 grouped GEMM, both launches); `kernels` (N=1 only) holds
the three hot-path kernels at their own benchmark configurations (prefill grouped GEMM, decode
grouped GEMV, FP4 dequant) with their roofline fractions of the measured peaks; `cpu_baseline` is
the CPU oracle (torch-CPU float32 golden path) timed on this box's host cores on a bounded sample.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

CFG = dict(n_tokens=4096, hidden=7168, n_experts=256, inter=2048, top_k=8, seed=4)
# dram bytes / algorithmic bytes of the layer's grouped GEMMs, from a profiler capture of a small case
DRAM_OVER_ALGORITHMIC = 1.00
CPU_SAMPLE_EVERY = 32  # the CPU legs time every 32nd expert by load rank (8 of 256) with all its routed rows
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def inputs_module():
    """ascend_kernel_b200/inputs.py loaded by path: it needs only torch, and importing it through the
    package would load the CUDA library, which the CPU arm must not map."""
    import importlib.util

    spec = importlib.util.spec_from_file_location("_b200moe_inputs", os.path.join(ROOT, "ascend_kernel_b200", "inputs.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            d = json.load(open(p))
            return {k: float(d[k]) for k in FALLBACK_PEAKS}, "measured"
        except Exception:
            pass
    return dict(FALLBACK_PEAKS), "fallback"


# ------------------------------------------------------------------------------------------------
# clocks during the timed region
# ------------------------------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc = index, None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None
        return self

    def __exit__(self, *exc):
        self.result = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return
        time.sleep(0.25)  # let at least a few samples through even for a short timed region
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except Exception:
            self.proc.kill()
            return
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [v.strip() for v in line.split(",")]
            if len(f) < 6:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for n, v in zip(names, f[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if sm:
            self.result = {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                           "samples": len(sm)}


# ------------------------------------------------------------------------------------------------
# CPU golden path (oracle) on a bounded sample -- the cpu_baseline leg and the reference arm
# ------------------------------------------------------------------------------------------------
def cpu_sample_inputs(every: int):
    """Routing of the full configuration; weights only for every `every`-th expert by load rank."""
    import torch

    from oracle import oracle as O

    inputs = inputs_module()
    c = inputs.config4("cpu", expert_lo=0, expert_hi=0, **CFG)
    wts, idx = O.route_topk(c["logits"], CFG["top_k"])
    counts = torch.bincount(idx.reshape(-1), minlength=CFG["n_experts"])
    by_load = torch.argsort(counts, descending=True)
    chosen = by_load[every // 2::every].tolist()
    weights = {e: inputs.config4("cpu", n_tokens=1, hidden=CFG["hidden"], n_experts=CFG["n_experts"],
                                 inter=CFG["inter"], top_k=CFG["top_k"], seed=CFG["seed"], expert_lo=e,
                                 expert_hi=e + 1) for e in chosen}
    return c, idx, counts, chosen, weights


def cpu_moe_sample(every: int, prepared=None):
    """Times the CPU golden path over the sampled experts' routed rows (weight generation is
    outside the timed region).  Returns (tokens_per_s, seconds, rows, description)."""
    import torch

    c, idx, counts, chosen, weights = prepared if prepared is not None else cpu_sample_inputs(every)
    rows_total, t_total = 0, 0.0
    I = CFG["inter"]
    for e in chosen:
        tok = (idx == e).nonzero(as_tuple=True)[0]
        if tok.numel() == 0:
            continue
        w = weights[e]
        xr = c["x"][tok]
        t0 = time.perf_counter()
        wd1 = (w["w13"][0].float() + w["o13"][0].float()) * w["s13"][0].float()
        h = (xr.float() @ wd1).to(torch.bfloat16).float()
        act = (torch.nn.functional.silu(h[:, :I]) * h[:, I:]).to(torch.bfloat16).float()
        wd2 = (w["w2"][0].float() + w["o2"][0].float()) * w["s2"][0].float()
        _ = (act @ wd2).to(torch.bfloat16)
        t_total += time.perf_counter() - t0
        rows_total += int(tok.numel())
    tok_s = (rows_total / CFG["top_k"]) / t_total if t_total > 0 else 0.0
    desc = (f"{len(chosen)} of {CFG['n_experts']} experts (every {every}th by load rank) with all their routed rows "
            f"({rows_total} of {CFG['n_tokens'] * CFG['top_k']} rows), float32 torch-CPU dequant + matmul; "
            f"tokens/s = rows/top_k/time")
    return tok_s, t_total, rows_total, desc


def use_all_host_cores():
    """Give torch's CPU kernels every core this process may run on, and return the count.  A launcher
    that starts one process per GPU sets OMP_NUM_THREADS=1 for its children, which would leave the
    CPU arm with a single thread."""
    import torch

    try:
        cores = len(os.sched_getaffinity(0))
    except AttributeError:
        cores = os.cpu_count() or 1
    torch.set_num_threads(max(1, cores))
    return torch.get_num_threads()


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch

    threads = use_all_host_cores()
    every = CPU_SAMPLE_EVERY
    prepared = cpu_sample_inputs(every)
    for _ in range(args.warmup):
        cpu_moe_sample(every, prepared)
    vals, secs = [], 0.0
    for _ in range(args.steps):
        v, t, rows, desc = cpu_moe_sample(every, prepared)
        vals.append(v)
        secs += t
    value = statistics.mean(vals) if vals else 0.0
    line = {
        "impl": "reference", "metric": "moe_layer_tokens_per_s", "value": value, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * secs / max(1, args.steps), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args.gpus),
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": desc},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "note": "the reference's device code targets Ascend NPUs and cannot run here; this arm times the CPU "
                "restatement of its golden path (oracle port) on the host cores",
    }
    print(json.dumps(line), flush=True)


def workload_config(n_gpus):
    return {"workload": "moe_ffn_layer_int8_antiquant (benchmark configuration 4)", **CFG,
            "experts_per_gpu": CFG["n_experts"] // n_gpus, "tokens_per_gpu": CFG["n_tokens"] // n_gpus,
            "parallelism": f"ep{n_gpus}",
            "l2": "no flush: per-GPU working set (expert weights) is far larger than the 126 MB L2"}


# ------------------------------------------------------------------------------------------------
# per-kernel lines (N = 1)
# ------------------------------------------------------------------------------------------------
LAST_BACK_TO_BACK_MS = None


def time_launches(fn, n_warm, n_iter, n_sustained=50):
    """CUDA-event time of one call of fn (its own kernels only): the median of the first n_iter calls after
    an idle second (the clocks a kernel timed alone sees), which is returned, and the median of
    n_sustained further calls issued back to back (the clocks inside a long run, usually under the power
    cap), left in LAST_BACK_TO_BACK_MS."""
    global LAST_BACK_TO_BACK_MS
    import torch

    torch.cuda.synchronize()
    time.sleep(1.0)
    for _ in range(n_warm):
        fn()
    torch.cuda.synchronize()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n_iter + n_sustained)]
    for a, b in evs:
        a.record()
        fn()
        b.record()
    torch.cuda.synchronize()
    times = [a.elapsed_time(b) for a, b in evs]
    LAST_BACK_TO_BACK_MS = statistics.median(times[n_iter:]) if n_sustained else None
    return statistics.median(times[:n_iter])


def kernel_lines(peaks, quick=False, which=("gemm", "gemv", "dequant")):
    import torch

    import ascend_kernel_b200 as ak
    from ascend_kernel_b200 import inputs

    dev = "cuda"
    out = {}
    # ---- prefill grouped GEMM (configuration 3, variant A) ----
    # quick cases stay larger than L2 and below 2 GB of weights; the GEMV one has 64 experts so that
    # its work items (active experts x 16 slabs) fill the 296 resident CTAs more than twice
    n_quick = 64 if tuple(which) == ("gemv",) else 32
    c = inputs.config3(dev) if not quick else inputs.config3(dev, n_rows=8192, n_experts=n_quick)
    M, K = c["x"].shape
    G, _, N = c["weight"].shape
    y = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
    if "gemm" in which:
      ms = time_launches(lambda: ak.grouped_gemm(c["x"], c["weight"], c["scale"], c["offset"], c["counts"], "int8", y,
                                               group_list_type=1), 3, 10)
      flops = 2.0 * M * K * N
      out["grouped_gemm_prefill_int8"] = {
        "ms": ms, "ms_back_to_back": LAST_BACK_TO_BACK_MS, "tflops": flops / ms / 1e9, "frac_of_measured_sustained": flops / ms / 1e9 / peaks["bf16_tflops_sustained"],
        "frac_of_measured_burst": flops / ms / 1e9 / peaks["bf16_tflops"], "frac_of_spec_2250": flops / ms / 1e9 / 2250.0,
        "shape": {"M": M, "K": K, "N": N, "G": G, "active_experts": int((c["counts"] > 0).sum())}}
    if "gemm" in which:
      # the same problem through the packed entry point (weights repacked once, outside the timed region)
      from ascend_kernel_b200 import ops as _ops

      wp = _ops.pack_weight_int8(c["weight"])
      ms = time_launches(lambda: _ops.grouped_gemm_packed(c["x"], wp, c["scale"], c["offset"], c["counts"], y,
                                                          group_list_type=1), 3, 10)
      out["grouped_gemm_prefill_int8_packed"] = {
        "ms": ms, "ms_back_to_back": LAST_BACK_TO_BACK_MS, "tflops": flops / ms / 1e9,
        "frac_of_measured_sustained": flops / ms / 1e9 / peaks["bf16_tflops_sustained"],
        "frac_of_measured_burst": flops / ms / 1e9 / peaks["bf16_tflops"], "frac_of_spec_2250": flops / ms / 1e9 / 2250.0}
      del wp
      torch.cuda.empty_cache()
    # ---- decode grouped GEMV (configuration 1): reuse the weight tensor ----
    # decode routing: 32 tokens x top-8 over 256 experts (quick: the same 1 row per expert on average)
    counts = inputs.routed_counts(max(1, G // 8), G, 8, torch.Generator().manual_seed(1)).to(dev)
    Mv = int(counts.sum())
    xv = c["x"][:Mv].contiguous()
    yv = torch.empty(Mv, N, dtype=torch.bfloat16, device=dev)
    n_act = int((counts > 0).sum())
    if "gemv" in which:
      ms = time_launches(lambda: ak.grouped_soft_gemv(xv, c["weight"], c["scale"], counts, "int8", yv,
                                                    group_list_type=1), 3, 10)
      by = n_act * K * N + 2.0 * Mv * K + 2.0 * Mv * N + n_act * N * 2
      out["grouped_gemv_decode_int8_pass1"] = {"ms": ms, "ms_back_to_back": LAST_BACK_TO_BACK_MS, "gbs": by / ms / 1e6, "frac_of_measured": by / ms / 1e6 / peaks["hbm_gbs"],
                                             "frac_of_spec_8000": by / ms / 1e6 / 8000.0,
                                             "shape": {"M": Mv, "K": K, "N": N, "G": G, "active_experts": n_act}}
    del c, y, xv, yv
    torch.cuda.empty_cache()
    # ---- the other weight formats at the prefill shape (int4 = configuration 3 variant B; fp8 / fp4 = the
    # reference's own formats, cumulative group_list; fp4 in the canonical order and in the reference's
    # stored order, which the kernel reads in place) ----
    if "gemm" in which:
        for name in ("int4", "fp8", "fp4", "fp4_stored_order"):
            kind = "fp4" if name.startswith("fp4") else name
            layout = "ascend" if name == "fp4_stored_order" else "canonical"
            c = (inputs.config3_variants(dev, kind) if not quick
                 else inputs.config3_variants(dev, kind, n_rows=8192, n_experts=32))
            M, K = c["x"].shape
            y = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
            gl = c["counts"] if kind == "int4" else torch.cumsum(c["counts"], 0)
            off = c["offset"] if kind == "int4" else torch.zeros(1, device=dev)
            fn = (lambda: ak.grouped_gemm(c["x"], c["weight"], c["scale"], off, gl, kind, y,
                                          group_list_type=1 if kind == "int4" else 0, weight_layout=layout))
            ms = time_launches(fn, 2, 5, 50)
            flops = 2.0 * M * K * N
            out[f"grouped_gemm_prefill_{name}"] = {"ms": ms, "ms_back_to_back": LAST_BACK_TO_BACK_MS, "tflops": flops / ms / 1e9,
                                                   "frac_of_measured_burst": flops / ms / 1e9 / peaks["bf16_tflops"],
                                                   "frac_of_measured_sustained": flops / ms / 1e9 / peaks["bf16_tflops_sustained"]}
            del c, y
            torch.cuda.empty_cache()
    if not quick and "gemv" in which:
        gen = torch.Generator(device=dev).manual_seed(11)
        K2, N2 = 2048, 7168
        w2 = inputs.int8_weights(G, K2, N2, gen, dev)
        s2 = (torch.rand(G, N2, generator=gen, device=dev) * 0.009 + 0.001).to(torch.bfloat16)
        x2 = torch.randn(Mv, K2, generator=gen, device=dev).to(torch.bfloat16)
        y2 = torch.empty(Mv, N2, dtype=torch.bfloat16, device=dev)
        ms = time_launches(lambda: ak.grouped_soft_gemv(x2, w2, s2, counts, "int8", y2, group_list_type=1), 3, 10)
        by = n_act * K2 * N2 + 2.0 * Mv * K2 + 2.0 * Mv * N2 + n_act * N2 * 2
        out["grouped_gemv_decode_int8_pass2"] = {"ms": ms, "ms_back_to_back": LAST_BACK_TO_BACK_MS, "gbs": by / ms / 1e6, "frac_of_measured": by / ms / 1e6 / peaks["hbm_gbs"],
                                                 "frac_of_spec_8000": by / ms / 1e6 / 8000.0,
                                                 "shape": {"M": Mv, "K": K2, "N": N2, "G": G, "active_experts": n_act}}
        del w2, s2, x2, y2
        torch.cuda.empty_cache()
    if "gemv" in which:
        gen = torch.Generator(device=dev).manual_seed(12)
        # the reference's own weight formats at the pass-1 shape (same routing): fp8 with fp32 block
        # scales, fp4 (canonical layout) with bf16 scales per 16 k rows
        K1, N1 = 7168, 4096
        x1 = torch.randn(Mv, K1, generator=gen, device=dev).to(torch.bfloat16)
        y1 = torch.empty(Mv, N1, dtype=torch.bfloat16, device=dev)
        for name in ("fp8", "fp4", "fp4_stored_order"):
            kind = "fp4" if name.startswith("fp4") else name
            cols = N1 if kind == "fp8" else N1 // 2
            w1 = torch.empty(G, K1, cols, dtype=torch.uint8, device=dev)
            for g in range(G):
                w1[g] = torch.randint(0, 256, (K1, cols), generator=gen, device=dev, dtype=torch.uint8)
            if kind == "fp8":
                s1 = torch.randn(G, K1 // 128, N1 // 128, generator=gen, device=dev)
                sbytes = n_act * (K1 // 128) * (N1 // 128) * 4
            else:
                s1 = (torch.rand(G, K1 // 16, N1, generator=gen, device=dev) * 3 + 0.25).to(torch.bfloat16)
                w1 = w1.view(torch.int8)
                sbytes = n_act * (K1 // 16) * N1 * 2
            layout = "ascend" if name == "fp4_stored_order" else "canonical"
            ms = time_launches(lambda: ak.grouped_soft_gemv(x1, w1, s1, counts, kind, y1, group_list_type=1,
                                                            weight_layout=layout), 3, 10)
            by = n_act * K1 * cols + sbytes + 2.0 * Mv * K1 + 2.0 * Mv * N1
            out[f"grouped_gemv_decode_{name}"] = {"ms": ms, "ms_back_to_back": LAST_BACK_TO_BACK_MS, "gbs": by / ms / 1e6,
                                                  "frac_of_measured": by / ms / 1e6 / peaks["hbm_gbs"],
                                                  "shape": {"M": Mv, "K": K1, "N": N1, "G": G, "active_experts": n_act}}
            del w1, s1
            torch.cuda.empty_cache()
        del x1, y1
    if "dequant" not in which:
        return out
    # ---- FP4 dequant (configuration 2) ----
    d = inputs.config2(dev) if not quick else inputs.config2(dev, shape=(32, 2048, 7168))
    n = d["codes"].numel() * 2
    o = torch.empty(n, dtype=torch.bfloat16, device=dev)
    ms = time_launches(lambda: ak.fp4_dequant(d["codes"], d["scale"], o), 3, 10)
    by = n * (0.5 + 1.0 / 32 + 2.0)
    out["fp4_dequant_e8m0"] = {"ms": ms, "ms_back_to_back": LAST_BACK_TO_BACK_MS, "gbs": by / ms / 1e6, "frac_of_measured": by / ms / 1e6 / peaks["hbm_gbs"],
                               "frac_of_spec_8000": by / ms / 1e6 / 8000.0, "elements": n}
    del d, o
    torch.cuda.empty_cache()
    return out


# ------------------------------------------------------------------------------------------------
# correctness of the measured configuration, outside every timed region
# ------------------------------------------------------------------------------------------------
def parity_check(out_dev, x_host, lg_host, dev, n_check=8, tol=4e-3):
    """The CPU golden path on `n_check` of this rank's tokens against the layer's output `out_dev`
    (the rows of this rank's tokens, on the device).  A token needs the weights of its top-k experts,
    wherever they live: each is materialised on the device from its hash (the same bits every rank
    holds), copied to the host and put through the float32 CPU formulas.  Returns (worst rel-L2, count)."""
    import torch

    from ascend_kernel_b200 import inputs
    from oracle import oracle as O

    lg = lg_host.float()
    k = CFG["top_k"]
    srt = torch.sort(lg, dim=1, descending=True)[0]
    tie_free = (srt[:, k - 1] != srt[:, k]).nonzero().flatten().tolist()  # a tie at the boundary may go either way
    toks = sorted({tie_free[int(round(i * (len(tie_free) - 1) / max(1, n_check - 1)))] for i in range(n_check)})
    w, idx = O.route_topk(lg_host[toks], k)
    I = CFG["inter"]
    cache, worst = {}, 0.0
    for i, t in enumerate(toks):
        acc = torch.zeros(CFG["hidden"], dtype=torch.float64)
        for j in range(k):
            e = int(idx[i, j])
            if e not in cache:
                if len(cache) >= 12:
                    cache.clear()
                c = inputs.config4(dev, n_tokens=1, hidden=CFG["hidden"], n_experts=CFG["n_experts"], inter=I, top_k=k,
                                   seed=CFG["seed"], expert_lo=e, expert_hi=e + 1)
                cache[e] = {n: c[n][0].cpu() for n in ("w13", "s13", "o13", "w2", "s2", "o2")}
            p = cache[e]
            wd1 = (p["w13"].float() + p["o13"].float()) * p["s13"].float()
            h = (x_host[t:t + 1].float() @ wd1).to(torch.bfloat16).float()
            act = (torch.nn.functional.silu(h[:, :I]) * h[:, I:]).to(torch.bfloat16).float()
            wd2 = (p["w2"].float() + p["o2"].float()) * p["s2"].float()
            y = (act @ wd2).to(torch.bfloat16).double()
            acc += float(w[i, j]) * y[0]
        worst = max(worst, O.rel_l2(out_dev[t].cpu().double(), acc))
    return worst, len(toks)


def fp4_stored_line(peaks, steps=5, warmup=2):
    """Configuration 4 with its experts STORED as FP4 e2m1 (+ e8m0 scale per 32) and dequantised to bf16
    in every pass (the reference kernel's own two phases: dequantise to a bf16 buffer, then the bf16
    grouped matmul).  One GPU, device-resident inputs."""
    import torch

    from ascend_kernel_b200 import inputs
    from ascend_kernel_b200.moe_layer import MoELayer

    dev = torch.device("cuda", torch.cuda.current_device())
    c = inputs.config4_fp4(dev, **CFG)
    layer = MoELayer(c["c13"], c["s13"], None, c["c2"], c["s2"], None, CFG["n_experts"], CFG["top_k"], weight_format="fp4")
    x, lg = c["x"].to(dev), c["logits"].to(dev)
    for _ in range(warmup):
        layer.forward(x, lg)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        layer.forward(x, lg)
    e1.record()
    torch.cuda.synchronize()
    layer.read_status()
    ms = e0.elapsed_time(e1) / steps
    E, H, I = CFG["n_experts"], CFG["hidden"], CFG["inter"]
    elems = E * (H * 2 * I + I * H)
    rows = CFG["n_tokens"] * CFG["top_k"]
    # packed codes + scales in, bf16 weights out, bf16 weights in again, activations
    by = elems * (0.5 + 1.0 / 32 + 2.0 + 2.0) + rows * 2.0 * (H + 2 * I + 2 * I + I + I + H)
    return {"ms_per_step": ms, "tokens_per_s": CFG["n_tokens"] / (ms / 1e3), "steps": steps,
            "roofline": {"bound": "hbm", "achieved": by / ms / 1e6, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": by / ms / 1e6 / peaks["hbm_gbs"], "algorithmic_bytes": by},
            "what": "FP4 e2m1 experts (e8m0 scale per 32) -> bf16 buffers per pass (fp4_dequant_kernel) -> bf16 grouped GEMM"}


def layer_gemm_case(quick: bool):
    """The two expert GEMMs of the layer alone, on rows distributed like the layer's (128 +- 11 per expert):
    a case for profiler captures (--quick: 32 experts, about 1.4 GB of weights)."""
    import torch

    from ascend_kernel_b200 import ops

    dev = "cuda"
    G = 32 if quick else 256
    gen = torch.Generator(device=dev).manual_seed(0)
    cnt = torch.clamp((torch.randn(G, generator=gen, device=dev) * 11.3 + 128).round(), 1, 400).to(torch.int64)
    M = int(cnt.sum())
    H, I = CFG["hidden"], CFG["inter"]
    out = {"rows": M, "experts": G}
    for name, K, N, gate_up in (("gate_up_silu", H, 2 * I, True), ("down", I, H, False)):
        x = torch.randn(M, K, generator=gen, device=dev).to(torch.bfloat16)
        w = torch.randint(-128, 128, (G, K, N), generator=gen, device=dev, dtype=torch.int8)
        sc = (torch.rand(G, N, generator=gen, device=dev) * 0.009 + 0.001).to(torch.bfloat16)
        of = (torch.rand(G, N, generator=gen, device=dev) * 8 - 4).to(torch.bfloat16)
        wp = ops.pack_weight_int8(w, gate_up=gate_up)
        del w
        y = torch.empty(M, N // 2 if gate_up else N, dtype=torch.bfloat16, device=dev)
        ms = time_launches(lambda: ops.grouped_gemm_packed(x, wp, sc, of, cnt, y, group_list_type=1, gate_up_silu=gate_up),
                           3, 10, 0)
        out[name] = {"ms": ms, "tflops": 2.0 * M * K * N / ms / 1e9,
                     "algorithmic_bytes": G * K * N + 2.0 * M * K + 2.0 * M * (N // 2 if gate_up else N) + 4.0 * G * N}
        del x, wp, y
        torch.cuda.empty_cache()
    return out


# ------------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------------
def bind_to_gpu_numa_node(torch, index: int):
    """Restricts this process to the CPUs of the NUMA node the GPU hangs off (read from sysfs), so that the
    pinned host buffers it allocates next are local to that GPU's PCIe root.  One process per GPU only; returns
    the node, or None when the topology cannot be read (nothing is changed then).  CPU affinity of this process
    is the only thing touched."""
    try:
        p = torch.cuda.get_device_properties(index)
        bdf = "%04x:%02x:%02x.0" % (p.pci_domain_id, p.pci_bus_id, p.pci_device_id)
        node = int(open(f"/sys/bus/pci/devices/{bdf}/numa_node").read())
        if node < 0:
            return None
        cpus = set()
        for part in open(f"/sys/devices/system/node/node{node}/cpulist").read().strip().split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        cpus &= os.sched_getaffinity(0)
        if not cpus:
            return None
        os.sched_setaffinity(0, cpus)
        return node
    except Exception:  # no sysfs, no such attribute, not permitted: run unbound
        return None


def run_ours(args):
    import torch

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the operators have no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    # several ranks share the host: each keeps its pinned buffers on its own GPU's NUMA node
    numa_node = bind_to_gpu_numa_node(torch, local_rank) if world > 1 else None
    group = None
    if world > 1:
        import torch.distributed as dist

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
        group = dist.group.WORLD

    import ascend_kernel_b200 as ak  # noqa: F401  (fails loudly if the CUDA library is missing)
    from ascend_kernel_b200 import inputs, ops
    from ascend_kernel_b200.moe_layer import MoELayer

    peaks, peak_kind = load_peaks()
    E, T = CFG["n_experts"], CFG["n_tokens"]
    assert E % world == 0 and T % world == 0
    e_local, t_local = E // world, T // world
    c = inputs.config4(dev, expert_lo=rank * e_local, expert_hi=(rank + 1) * e_local, **CFG)
    exchange = args.exchange if (world > 1 or args.single_rank_exchange) else "direct"
    # several ranks on the peer-memory exchange: a step's token exchange runs beside the GEMMs of the step before
    overlap = exchange == "p2p" and not args.no_overlap
    layer = MoELayer(c["w13"], c["s13"], c["o13"], c["w2"], c["s2"], c["o2"], E, CFG["top_k"], group,
                     exchange="p2p" if exchange == "p2p" else "nccl", max_tokens=t_local,
                     exchange_buffers=(3 if args.defer_sum else 2) if overlap else 1)
    layer.gather_sums = not args.no_gather_sums
    x_host = c["x"][rank * t_local:(rank + 1) * t_local].contiguous().pin_memory()
    lg_host = c["logits"][rank * t_local:(rank + 1) * t_local].contiguous().pin_memory()
    x, lg = x_host.to(dev), lg_host.to(dev)

    def barrier():
        if world > 1:
            import torch.distributed as dist

            dist.barrier(group=group)
        torch.cuda.synchronize()

    def max_over_ranks(v: float) -> float:
        if world == 1:
            return v
        import torch.distributed as dist

        t = torch.tensor([v], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
        return float(t.item())

    # ---- correctness of exactly this configuration (all ranks, the exchange in use), before anything is
    # warmed up or timed: the host works for several seconds here and the GPU idles
    out_dev = layer.forward(x, lg)
    barrier()
    worst, n_checked = parity_check(out_dev, x_host, lg_host, dev)
    worst = max_over_ranks(worst)
    parity = {"tokens": n_checked * world, "rel_l2_max": worst, "tol": 4e-3, "ok": bool(worst <= 4e-3),
              "against": "CPU golden path (float32) on sampled tokens of every rank, experts fetched wherever they live"}
    del out_dev
    barrier()

    # ---- device-resident timing ----
    from ascend_kernel_b200.moe_layer import GraphedLayer, HostPipeline, OverlappedSteps

    gemm_ms, gemm_events, phase_events = 0.0, [], []
    ov = None
    if overlap:
        # the phases of a step, from serial passes outside the timed region (overlapped steps have no
        # phase boundaries on one stream)
        for i in range(6):
            layer.forward(x, lg, record=i > 1)
            if i > 1 and layer.phases is not None:
                phase_events.append(layer.phases)
        barrier()
        ov = OverlappedSteps(layer, t_local, reserve_sms=args.reserve_sms, late_sum=args.late_sum, defer_sum=args.defer_sum)

    def one_step(record=False):
        if ov is not None:
            return ov.submit(x, lg, record=record)
        layer.forward(x, lg, record=record)
        return None

    def settle(last):  # overlapped steps: the caller's stream waits for the end of the last one
        if last is not None:
            ov.flush()
            torch.cuda.current_stream().wait_event(last.event)

    last = None
    for _ in range(args.warmup):
        last = one_step()
    settle(last)
    barrier()
    ops.LAUNCHES = 0
    with ClockSampler(local_rank) as clk:
        barrier()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.profiler.start()  # lets `ncu --profile-from-start off` list only the timed steps
        ev0.record()
        t_host = time.perf_counter()
        for _ in range(args.steps):
            last = one_step(record=True)
            if layer.timing is not None:
                gemm_events.append(layer.timing)
            if ov is None and layer.phases is not None:
                phase_events.append(layer.phases)
        settle(last)
        ev1.record()
        host_ms_per_step = (time.perf_counter() - t_host) * 1e3 / args.steps  # the host's launch work per step
        barrier()
        torch.cuda.profiler.stop()
    launches = ops.LAUNCHES / max(1, args.steps)
    total_ms = max_over_ranks(ev0.elapsed_time(ev1))
    for ev in gemm_events:
        gemm_ms += ev[0].elapsed_time(ev[1]) + ev[2].elapsed_time(ev[3])
    ms_per_step = total_ms / args.steps
    value = T / (ms_per_step / 1e3)
    phases = {}
    for marks in phase_events:
        for (n0, e0), (n1, e1) in zip(marks[:-1], marks[1:]):
            phases[n1] = phases.get(n1, 0.0) + e0.elapsed_time(e1) / len(phase_events)

    # ---- end to end through the host-buffer call ----
    out_host = torch.empty(t_local, CFG["hidden"], dtype=torch.bfloat16).pin_memory()
    for _ in range(min(3, args.warmup)):
        layer.forward_host(x_host, lg_host, out_host)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        layer.forward_host(x_host, lg_host, out_host)
    e1.record()
    barrier()
    latency_ms = max_over_ranks(e0.elapsed_time(e1)) / args.steps
    # the same calls with steps in flight (copy-in / kernels / copy-out on three streams); the kernels of a
    # step are overlapped steps where those ran above, else one CUDA-graph launch where the step has no host
    # synchronisation
    graphed = GraphedLayer(layer, t_local) if (exchange != "nccl" and ov is None) else None
    depth = 3 if ov is not None else 2
    pipe = HostPipeline(layer, depth=depth, graphed=graphed, overlapped=ov)
    outs = [out_host] + [torch.empty_like(out_host).pin_memory() for _ in range(depth - 1)]
    for i in range(max(depth, min(3, args.warmup))):
        pipe.submit(x_host, lg_host, outs[i % depth])
    pipe.drain()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    t_host = time.perf_counter()
    for i in range(args.steps):
        pipe.submit(x_host, lg_host, outs[i % depth])
    host_ms_per_submit = (time.perf_counter() - t_host) * 1e3 / args.steps  # the host's own work per step
    pipe.drain()
    e1.record()
    barrier()
    e2e_ms = max_over_ranks(e0.elapsed_time(e1)) / args.steps
    exchange_status = list(layer.px.read_status()) if layer.px is not None else None
    h2d = (x_host.numel() * 2 + lg_host.numel() * 2) * world
    d2h = out_host.numel() * 2 * world

    # ---- roofline of the dominant kernel (both grouped-GEMM launches of a step, this rank) ----
    rows_local = T * CFG["top_k"] / world  # expectation; exact rows differ per rank by routing
    flops_step = 2.0 * rows_local * (CFG["hidden"] * 2 * CFG["inter"] + CFG["inter"] * CFG["hidden"])
    gemm_ms_step = gemm_ms / max(1, len(gemm_events))
    H_, I_ = CFG["hidden"], CFG["inter"]
    algo_bytes = (E / world) * (H_ * 2 * I_ + I_ * H_) + rows_local * 2.0 * (H_ + 2 * I_ + I_ + H_)
    traffic = DRAM_OVER_ALGORITHMIC * algo_bytes
    achieved = flops_step / gemm_ms_step / 1e9 if gemm_ms_step > 0 else 0.0
    sm_mhz = clk.result.get("sm_mhz")
    roofline = {"bound": "tensor", "kernel": "grouped_gemm_packed_kernel (2 launches per step, rank 0)",
                "achieved": achieved, "peak": peaks["bf16_tflops_sustained"], "unit": "TFLOP/s",
                "frac": achieved / peaks["bf16_tflops_sustained"], "peak_kind": f"{peak_kind} (sustained cuBLAS bf16)",
                "frac_burst": achieved / peaks["bf16_tflops"], "peak_burst": peaks["bf16_tflops"],
                "frac_of_spec_2250": achieved / 2250.0,
                "traffic": traffic, "traffic_unit": "bytes per step (both launches)",
                "traffic_source": f"algorithmic bytes (weights once + x + y) x {DRAM_OVER_ALGORITHMIC}: dram bytes / "
                                  "algorithmic bytes of one profiler capture of `--workload layer_gemm --quick` (32 "
                                  "experts, rows distributed like the layer's); the full-size launch is too large to capture",
                "ms_per_step_in_kernel": gemm_ms_step,
                "gemm_mcycles_per_step": (gemm_ms_step * sm_mhz / 1e3) if sm_mhz else None}

    line = {
        "metric": "moe_layer_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16 x int8 -> fp32 accumulate", "data": "synthetic",
        "config": workload_config(world), "exchange": exchange, "exchange_status": exchange_status,
        # what a step spends outside its two grouped GEMMs (routing, exchange, waits, weighted sum, launch gaps): with
        # overlapped steps the exchange of phases_ms_rank0 is no longer part of it
        "outside_gemm_ms_per_step_rank0": ms_per_step - gemm_ms_step,
        "exchange_overlapped": ({"reserved_sms": args.reserve_sms, "late_sum": args.late_sum, "defer_sum": args.defer_sum, "phases_from": "serial passes before the timed region"}
                                if ov is not None else False),
        "e2e": {"value": T / (e2e_ms / 1e3), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": e2e_ms, "steps_in_flight": depth, "cuda_graph": graphed is not None,
                "exchange_overlapped": ov is not None, "host_ms_per_submit_rank0": host_ms_per_submit,
                "host_numa_node_rank0": numa_node,
                "single_step_latency_ms": latency_ms},
        "host_launch_ms_per_step_rank0": host_ms_per_step,
        "gpu_launches": launches * args.steps, "gpu_launches_per_step": launches,
        "roofline": roofline, "clocks": clk.result, "phases_ms_rank0": {k: round(v, 4) for k, v in phases.items()},
        "parity_check": parity,
    }
    if world == 1 and rank == 0:
        del layer, c
        torch.cuda.empty_cache()
        if not args.no_kernels:
            line["moe_layer_fp4_stored"] = fp4_stored_line(peaks)
            torch.cuda.empty_cache()
            kernels = kernel_lines(peaks, quick=args.quick)
            kernels["peaks"] = {**peaks, "kind": peak_kind}
            # their own line, ahead of the headline line: a reader of the output's tail loses nothing
            print(json.dumps({"kernels": kernels}), flush=True)
            line["kernels"] = {k: {f: v[f] for f in ("ms", "ms_back_to_back", "tflops", "gbs", "frac_of_measured",
                                                      "frac_of_measured_sustained", "frac_of_measured_burst") if f in v}
                               for k, v in kernels.items() if k != "peaks"}
        if not args.no_cpu:
            # the bounded sample of the reference arm (8 of the 256 experts), passes repeated until about ten
            # seconds are timed
            use_all_host_cores()
            prepared = cpu_sample_inputs(CPU_SAMPLE_EVERY)
            cpu_moe_sample(CPU_SAMPLE_EVERY, prepared)  # warm-up (thread pool, allocator)
            rows_sum, secs, passes = 0, 0.0, 0
            while secs < 10.0 and passes < 40:
                _, t, rows, desc = cpu_moe_sample(CPU_SAMPLE_EVERY, prepared)
                rows_sum, secs, passes = rows_sum + rows, secs + t, passes + 1
            tok_s = rows_sum / CFG["top_k"] / secs
            line["cpu_baseline"] = {"value": tok_s, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": "port",
                                    "sample": f"{passes} passes over " + desc, "seconds": secs}
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist

        torch.cuda.synchronize()
        dist.barrier(group=group)  # peers may read this rank's exchange buffers until they are done too
        dist.destroy_process_group()
    if not parity["ok"]:
        raise SystemExit(f"parity check failed: rel-L2 {parity['rel_l2_max']:.3e} > {parity['tol']}")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="moe", choices=["moe", "gemm", "gemv", "dequant", "layer_gemm"],
                    help="moe: the benchmark line; others: one kernel alone (for profiling)")
    ap.add_argument("--exchange", default="p2p", choices=["p2p", "nccl"],
                    help="token exchange between ranks (N > 1): this package's peer-memory kernels or NCCL all-to-all")
    ap.add_argument("--single-rank-exchange", action="store_true",
                    help="one GPU: run the peer-memory exchange kernels all the same (the rank is its own peer), "
                         "which puts the routing and row gather of a step beside the GEMMs of the step before")
    ap.add_argument("--no-gather-sums", action="store_true",
                    help="one GPU: the gate/up GEMM adds up the rows of x itself instead of taking the sums from the gather")
    ap.add_argument("--no-overlap", action="store_true",
                    help="several ranks, p2p: run a step's token exchange serially before its GEMMs")
    ap.add_argument("--defer-sum", action="store_true",
                    help="overlapped steps: a step's wait for the peers' pushes and its weighted sum follow the NEXT "
                         "step's GEMMs on the same stream (three buffer sets): no barrier between the ranks every step")
    ap.add_argument("--late-sum", action="store_true",
                    help="overlapped steps: wait for the peers' pushes and sum beside the next step's GEMMs (measured slower)")
    ap.add_argument("--reserve-sms", type=int, default=8,
                    help="SMs the grouped GEMMs leave to the next step's exchange kernels when steps overlap")
    ap.add_argument("--no-kernels", action="store_true", help="skip the per-kernel lines (N=1)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline sample")
    ap.add_argument("--quick", action="store_true", help="small shapes for the per-kernel lines (profiling)")
    args = ap.parse_args()
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args)
    elif args.workload != "moe":
        # one hot-path kernel alone at its own benchmark configuration (--quick: a small case of
        # the same kernel, sized for profiler captures)
        import torch

        torch.cuda.set_device(0)
        peaks, kind = load_peaks()
        line = {"workload": args.workload, "quick": args.quick, "peaks": {**peaks, "kind": kind},
                "kernels": (layer_gemm_case(args.quick) if args.workload == "layer_gemm"
                            else kernel_lines(peaks, quick=args.quick, which=(args.workload,)))}
        print(json.dumps(line), flush=True)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
