"""Seeded synthetic inputs with the shapes, sizes and value distributions of the benchmark
configurations (DeepSeek-V3 is only a shape donor; no dataset is involved).

Small cases are drawn on the CPU (so the CPU oracle and the GPU path see identical bits on any
machine) and moved to ``device``; full-size tensors are drawn directly on ``device``, except the MoE
layer's weights, which are a hash of the element index and so have the same bits wherever they are
materialised.  This module imports nothing but torch: the benchmark's CPU arm loads it by path, without
importing the package (and with it the CUDA library).
"""
from __future__ import annotations

import torch


def _gen(seed, device):
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return g


def _uniform(shape, lo, hi, gen, device, dtype=torch.bfloat16):
    return (torch.rand(shape, generator=gen, device=device) * (hi - lo) + lo).to(dtype)


# ---- counter-based values: the same bits on the CPU and on a GPU ------------------------------------
# torch's CPU and CUDA generators are different algorithms, so tensors drawn on the device cannot be
# reproduced on the host.  Where both sides must see the same bits (the benchmark's CPU arm and GPU arm)
# values are a hash of (seed, element index) instead: splitmix64's finaliser in int64 tensor arithmetic,
# which wraps the same way on both devices.
def _mix64(idx, seed: int):
    m34, m37, m33 = (1 << 34) - 1, (1 << 37) - 1, (1 << 33) - 1
    g = (seed * 0x9E3779B97F4A7C15 + 0x632BE59BD9B4E019) & 0x7FFFFFFFFFFFFFFF
    z = idx + g
    z = (z ^ ((z >> 30) & m34)) * -4658895280553007687    # 0xBF58476D1CE4E5B9 as int64
    z = (z ^ ((z >> 27) & m37)) * -7723592293110705685    # 0x94D049BB133111EB as int64
    return z ^ ((z >> 31) & m33)


def hashed_bytes(shape, seed: int, device, dtype=torch.uint8):
    """Bytes uniform over 0..255 (int8: -128..127), identical on every device, in chunks that bound the
    int64 temporaries."""
    n = 1
    for d in shape:
        n *= int(d)
    out = torch.empty(n, dtype=torch.uint8, device=device)
    step = 1 << 24
    for i in range(0, n, step):
        idx = torch.arange(i, min(n, i + step), dtype=torch.int64, device=device)
        out[i:i + idx.numel()] = (_mix64(idx, seed) & 0xFF).to(torch.uint8)
    out = out.reshape(shape)
    return out.view(torch.int8) if dtype == torch.int8 else out


def hashed_uniform(shape, lo: float, hi: float, seed: int, device, dtype=torch.bfloat16):
    """lo + (hi - lo) * u with u a 24-bit fraction of the hash, in float32 (one multiply, one add, each
    rounded on its own: the same on every device), then cast."""
    n = 1
    for d in shape:
        n *= int(d)
    idx = torch.arange(n, dtype=torch.int64, device=device)
    u = ((_mix64(idx, seed) >> 8) & 0xFFFFFF).to(torch.float32) * (1.0 / (1 << 24))
    return (u * (hi - lo) + lo).to(dtype).reshape(shape)


def int8_weights(G, K, N, gen, device):
    """int8 uniform on [-128, 127], drawn expert by expert to bound the temporary int64 buffer."""
    w = torch.empty(G, K, N, dtype=torch.int8, device=device)
    for g in range(G):
        w[g] = torch.randint(-128, 128, (K, N), generator=gen, device=device, dtype=torch.int8)
    return w


def zipf_counts(n_experts: int, total_rows: int, alpha: float, seed: int, n_zero: int = 4):
    """Per-expert row counts: popularity rank**-alpha over a seeded permutation of the experts,
    the ``n_zero`` least popular forced to 0, largest-remainder rounding so the sum is exact."""
    g = torch.Generator().manual_seed(seed)
    perm = torch.randperm(n_experts, generator=g)
    p = torch.arange(1, n_experts + 1, dtype=torch.float64) ** (-alpha)
    if n_zero:
        p[-n_zero:] = 0
    p = p / p.sum()
    raw = p * total_rows
    base = raw.floor().to(torch.int64)
    rem = int(total_rows - base.sum())
    if rem > 0:
        order = torch.argsort(raw - base, descending=True)
        base[order[:rem]] += 1
    counts = torch.empty(n_experts, dtype=torch.int64)
    counts[perm] = base
    assert int(counts.sum()) == total_rows
    return counts


def config0(device="cpu"):
    """Small antiquant grouped GEMM: 4 experts, counts [16,48,32,32], K=256, N=512, int8 weights,
    per-channel bf16 scale U(0.001,0.01) and offset U(-4,4)."""
    gen = _gen(0, "cpu")
    G, K, N = 4, 256, 512
    counts = torch.tensor([16, 48, 32, 32], dtype=torch.int64)
    M = int(counts.sum())
    x = torch.randn(M, K, generator=gen).to(torch.bfloat16)
    w = torch.randint(-128, 128, (G, K, N), generator=gen, dtype=torch.int8)
    scale = _uniform((G, N), 0.001, 0.01, gen, "cpu")
    offset = _uniform((G, N), -4.0, 4.0, gen, "cpu")
    t = dict(x=x, weight=w, scale=scale, offset=offset, counts=counts)
    return {k: v.to(device) for k, v in t.items()}


def routed_counts(n_tokens: int, n_experts: int, top_k: int, gen) -> torch.Tensor:
    """Per-expert counts when every token picks top_k distinct experts uniformly."""
    ids = torch.stack([torch.randperm(n_experts, generator=gen)[:top_k] for _ in range(n_tokens)])
    return torch.bincount(ids.reshape(-1), minlength=n_experts).to(torch.int64)


def config1(device, K=7168, N=4096, n_experts=256, n_tokens=32, top_k=8, seed=1):
    """Decode-shaped grouped GEMV: 32 tokens x top-8 over 256 experts -> 256 rows sorted by expert."""
    counts = routed_counts(n_tokens, n_experts, top_k, _gen(seed, "cpu"))
    gen = _gen(seed, device)
    M = int(counts.sum())
    x = torch.randn(M, K, generator=gen, device=device).to(torch.bfloat16)
    w = int8_weights(n_experts, K, N, gen, device)
    scale = _uniform((n_experts, N), 0.001, 0.01, gen, device)
    return dict(x=x, weight=w, scale=scale, offset=None, counts=counts.to(device))


def config2(device, shape=(256, 2048, 7168), seed=2):
    """FP4 dequant: packed bytes uniform over 0..255 (codes uniform over the 16 values), e8m0
    scale bytes uniform in 119..127, one per 32 elements of the last dimension."""
    gen = _gen(seed, device)
    lead, last = shape[:-1], shape[-1]
    codes = torch.empty(*lead, last // 2, dtype=torch.uint8, device=device)
    flat = codes.view(-1)
    step = 1 << 28
    for i in range(0, flat.numel(), step):
        n = min(step, flat.numel() - i)
        flat[i:i + n] = torch.randint(0, 256, (n,), generator=gen, device=device, dtype=torch.uint8)
    scale = torch.randint(119, 128, (*lead, last // 32), generator=gen, device=device, dtype=torch.uint8)
    return dict(codes=codes, scale=scale)


def config3(device, n_rows=65536, n_experts=256, K=7168, N=4096, seed=3, alpha=1.2):
    """Prefill-shaped antiquant grouped GEMM, variant A (int8, per-channel scale and offset)."""
    counts = zipf_counts(n_experts, n_rows, alpha, seed)
    gen = _gen(seed, device)
    x = torch.randn(n_rows, K, generator=gen, device=device).to(torch.bfloat16)
    w = int8_weights(n_experts, K, N, gen, device)
    scale = _uniform((n_experts, N), 0.001, 0.01, gen, device)
    offset = _uniform((n_experts, N), -4.0, 4.0, gen, device)
    return dict(x=x, weight=w, scale=scale, offset=offset, counts=counts.to(device))


def config3_variants(device, kind, n_rows=65536, n_experts=256, K=7168, N=4096, seed=3, alpha=1.2):
    """Same shape and row split as config3 with another weight format:
    "int4": two's-complement pairs [G,K,N/2], bf16 scale U(0.005,0.05) / offset U(-2,2) [G,K/128,N];
    "fp8":  e4m3 codes [G,K,N] (uniform bytes), fp32 scale ~N(0,1) [G,K/128,N/128] (reference format);
    "fp4":  e2m1 pairs [G,K,N/2] canonical order, bf16 scale U(0.25,3.25) [G,K/16,N] (reference format)."""
    counts = zipf_counts(n_experts, n_rows, alpha, seed)
    gen = _gen(seed, device)
    x = torch.randn(n_rows, K, generator=gen, device=device).to(torch.bfloat16)
    cols = N if kind == "fp8" else N // 2
    w = torch.empty(n_experts, K, cols, dtype=torch.uint8, device=device)
    for g in range(n_experts):
        w[g] = torch.randint(0, 256, (K, cols), generator=gen, device=device, dtype=torch.uint8)
    offset = None
    if kind == "int4":
        scale = _uniform((n_experts, K // 128, N), 0.005, 0.05, gen, device)
        offset = _uniform((n_experts, K // 128, N), -2.0, 2.0, gen, device)
        w = w.view(torch.int8)
    elif kind == "fp8":
        scale = torch.randn(n_experts, K // 128, N // 128, generator=gen, device=device, dtype=torch.float32)
    else:
        scale = _uniform((n_experts, K // 16, N), 0.25, 3.25, gen, device)
        w = w.view(torch.int8)
    return dict(x=x, weight=w, scale=scale, offset=offset, counts=counts.to(device))


def config4(device, n_tokens=4096, hidden=7168, n_experts=256, inter=2048, top_k=8, seed=4,
            expert_lo=0, expert_hi=None):
    """MoE FFN layer inputs.  Tokens and router logits are global (CPU generator); the weights of expert
    e are a hash of (seed, e, element index), so a rank can materialise only its own slice
    [expert_lo, expert_hi) and the CPU golden path can materialise single experts with the same bits."""
    expert_hi = n_experts if expert_hi is None else expert_hi
    gen = _gen(seed, "cpu")
    x = torch.randn(n_tokens, hidden, generator=gen).to(torch.bfloat16)
    logits = torch.randn(n_tokens, n_experts, generator=gen).to(torch.bfloat16)
    n_local = expert_hi - expert_lo
    w13 = torch.empty(n_local, hidden, 2 * inter, dtype=torch.int8, device=device)
    w2 = torch.empty(n_local, inter, hidden, dtype=torch.int8, device=device)
    s13 = torch.empty(n_local, 2 * inter, dtype=torch.bfloat16, device=device)
    o13 = torch.empty_like(s13)
    s2 = torch.empty(n_local, hidden, dtype=torch.bfloat16, device=device)
    o2 = torch.empty_like(s2)
    for e in range(expert_lo, expert_hi):
        i, se = e - expert_lo, (seed * 100003 + e) * 8
        w13[i] = hashed_bytes((hidden, 2 * inter), se, device, torch.int8)
        w2[i] = hashed_bytes((inter, hidden), se + 1, device, torch.int8)
        s13[i] = hashed_uniform((2 * inter,), 0.001, 0.01, se + 2, device)
        o13[i] = hashed_uniform((2 * inter,), -4.0, 4.0, se + 3, device)
        s2[i] = hashed_uniform((hidden,), 0.001, 0.01, se + 4, device)
        o2[i] = hashed_uniform((hidden,), -4.0, 4.0, se + 5, device)
    return dict(x=x, logits=logits, w13=w13, s13=s13, o13=o13, w2=w2, s2=s2, o2=o2, top_k=top_k)


def config4_tokens(n_tokens=4096, hidden=7168, n_experts=256, seed=4):
    """Only the tokens and router logits of config4 (bf16, CPU)."""
    gen = _gen(seed, "cpu")
    x = torch.randn(n_tokens, hidden, generator=gen).to(torch.bfloat16)
    logits = torch.randn(n_tokens, n_experts, generator=gen).to(torch.bfloat16)
    return x, logits


def config4_fp4(device, n_tokens=4096, hidden=7168, n_experts=256, inter=2048, top_k=8, seed=4,
                expert_lo=0, expert_hi=None):
    """The MoE layer with its expert weights STORED as FP4 e2m1 the way the dequantisation benchmark
    stores them: packed two per byte along the last dimension (low nibble = even element), one e8m0
    scale byte (uniform in 119..127, i.e. 2**-8 .. 2**0) per 32 elements of the last dimension.
    Tokens and router logits are those of config4; weights are drawn per expert."""
    expert_hi = n_experts if expert_hi is None else expert_hi
    gen = _gen(seed, "cpu")
    x = torch.randn(n_tokens, hidden, generator=gen).to(torch.bfloat16)
    logits = torch.randn(n_tokens, n_experts, generator=gen).to(torch.bfloat16)
    n_local = expert_hi - expert_lo
    c13 = torch.empty(n_local, hidden, inter, dtype=torch.uint8, device=device)           # [E, H, 2I/2]
    s13 = torch.empty(n_local, hidden, 2 * inter // 32, dtype=torch.uint8, device=device)
    c2 = torch.empty(n_local, inter, hidden // 2, dtype=torch.uint8, device=device)       # [E, I, H/2]
    s2 = torch.empty(n_local, inter, hidden // 32, dtype=torch.uint8, device=device)
    for e in range(expert_lo, expert_hi):
        i, se = e - expert_lo, (seed * 100003 + 50000 + e) * 8
        c13[i] = hashed_bytes(c13.shape[1:], se, device)
        s13[i] = 119 + hashed_bytes(s13.shape[1:], se + 1, device) % 9
        c2[i] = hashed_bytes(c2.shape[1:], se + 2, device)
        s2[i] = 119 + hashed_bytes(s2.shape[1:], se + 3, device) % 9
    return dict(x=x, logits=logits, c13=c13, s13=s13, c2=c2, s2=s2, top_k=top_k)
