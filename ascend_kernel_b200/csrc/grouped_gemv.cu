// Grouped GEMV for decode-sized expert batches (HBM-bandwidth kernel).
//
// Work item = (non-empty expert, slab of 256 output columns); persistent CTAs (two per SM) draw
// items from a ticket counter, experts with the most rows first, the slabs of an expert next to one another.  The expert's x rows (up to 4 per pass) are copied to shared memory
// once per item.  Every warp streams its share of the k rows straight from global memory with
// 128-bit coalesced loads, eight row pairs (8 x 512 B per warp) in flight before the first is
// consumed, decodes the packed weights in registers (byte / nibble unpack, no shared-memory
// staging of weights) and accumulates in fp32 with packed two-wide FMAs.  The 16 half-warp
// partial sums per column are combined with one shuffle and one pass through shared memory;
// scale and offset are applied in the fp32 epilogue and the result is rounded to bf16 once.
// Experts with more than 4 rows are processed 4 rows at a time (the weight slab is then re-read
// from L2).  int8 items with 2..4 rows, fp8 items and fp4 items use the tensor core for the multiply-adds
// (gv_compute_mma, gv_compute_fp4_mma); fp4 falls back to fp32 FMAs for x rows that are not exact in f16.
#include <cuda_fp16.h>

#include <cstdlib>

#include "common.cuh"

namespace b200moe {

constexpr int kGvSlabN = 256;
constexpr int kGvWarps = 8;
constexpr int kGvThreads = kGvWarps * 32;
constexpr int kGvUnroll = 8;                            // row pairs in flight per lane
constexpr int kGvWarpRows = 2 * kGvUnroll;              // k rows a warp consumes per step
constexpr int kGvIterRows = kGvWarps * kGvWarpRows;     // k rows a CTA consumes per step
constexpr int kGvRows = 4;                              // x rows per pass
constexpr int kGvXPad = 16;                             // bf16 elements between staged x rows (bank spread)
constexpr int kGvMmaParts = 4;                          // k groups of the tensor-core path
constexpr int kGvL2Steps = 4;                           // steps a warp requests into L2 ahead of its register loads

struct GemvArgs {
    const __nv_bfloat16* x;
    const uint8_t* weight;
    const void* scale;
    const __nv_bfloat16* offset;
    const int64_t* group_list;
    __nv_bfloat16* y;
    int M, K, N, G, gl_type;
    int* status;
    int fp4_stored;  // fp4 weights in the reference's pre-shuffled order, read in place
    const __half* x16;  // fp4: x as scaled f16 and the rows' exponents (gv_fp4_prepare_x_kernel), or null: fp32 path only
    const int* xexp;
};

typedef unsigned long long f32x2;  // two packed fp32 (sm_100 two-wide FP32 instructions)

__device__ __forceinline__ f32x2 pack2(float lo, float hi) {
    f32x2 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(f32x2 v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) {
    f32x2 r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
__device__ __forceinline__ f32x2 add2(f32x2 a, f32x2 b) {
    f32x2 r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b) {
    f32x2 r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}

__device__ __forceinline__ uint4 ldg_stream(const uint8_t* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
__device__ __forceinline__ uint2 ldg_stream8(const uint8_t* p) {
    uint2 v;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}

template <int MODE>
struct GvTraits {
    static constexpr bool kNibbles = (MODE == B200MOE_CT_FP4 || MODE == B200MOE_CT_INT4);
    static constexpr int kLaneBytes = kNibbles ? 8 : 16;  // 16 columns per lane
};

// Decode the lane's 16 columns of one weight row into eight fp32 pairs.
template <int MODE, bool kScaleFp4 = true>
__device__ __forceinline__ void gv_decode(const uint4& q, f32x2 (&w)[8], const f32x2 (&sc)[8], const f32x2 (&tc)[8]) {
    if constexpr (MODE == B200MOE_CT_INT8) {
        const uint32_t w4[4] = {q.x, q.y, q.z, q.w};
        const f32x2 kneg = pack2(-8388736.0f, -8388736.0f);  // -(2^23 + 128)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t u = w4[i] ^ 0x80808080u;  // biased byte: value + 128
            // 0x4B0000uu is the fp32 2^23 + uu
            const float f0 = __uint_as_float(prmt(u, 0x4B000000u, 0x7440u)), f1 = __uint_as_float(prmt(u, 0x4B000000u, 0x7441u));
            const float f2 = __uint_as_float(prmt(u, 0x4B000000u, 0x7442u)), f3 = __uint_as_float(prmt(u, 0x4B000000u, 0x7443u));
            w[2 * i] = add2(pack2(f0, f1), kneg);
            w[2 * i + 1] = add2(pack2(f2, f3), kneg);
        }
    } else if constexpr (MODE == B200MOE_CT_FP8) {
        const uint32_t w4[4] = {q.x, q.y, q.z, q.w};
        const f32x2 k120 = pack2(1.329227995784916e36f, 1.329227995784916e36f);  // 2^120
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float f[4];
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                // e4m3 bits moved under the fp32 exponent: value * 2^-120 (subnormals included)
                const uint32_t p = prmt(w4[i], 0u, 0x0444u | (b << 12));  // byte b -> bits 31..24
                f[b] = __uint_as_float(((p >> 4) & 0x07F00000u) | (p & 0x80000000u));
            }
            w[2 * i] = mul2(pack2(f[0], f[1]), k120);
            w[2 * i + 1] = mul2(pack2(f[2], f[3]), k120);
        }
    } else if constexpr (MODE == B200MOE_CT_INT4) {
        // (w + o) * s = w * s + o * s in fp32: sc holds s, tc holds o * s of the row's 128-k group
        const uint32_t w2[2] = {q.x ^ 0x88888888u, q.y ^ 0x88888888u};  // nibble + 8
        const f32x2 kneg = pack2(-8388616.0f, -8388616.0f);             // -(2^23 + 8)
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t word = w2[i >> 2];
            const int sh = 8 * (i & 3);
            const float f0 = __uint_as_float(((word >> sh) & 0xFu) | 0x4B000000u);
            const float f1 = __uint_as_float(((word >> (sh + 4)) & 0xFu) | 0x4B000000u);
            w[i] = fma2(add2(pack2(f0, f1), kneg), sc[i], tc[i]);
        }
    } else {  // FP4: q.x, q.y hold 16 codes; per-column scale of the current 16-row group
        const uint32_t w2[2] = {q.x, q.y};
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            uint32_t o[4];
            e2m1x8_to_bf16(w2[i], o);
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if constexpr (kScaleFp4)
                    w[4 * i + j] = mul2(pack2(__uint_as_float(o[j] << 16), __uint_as_float(o[j] & 0xFFFF0000u)), sc[4 * i + j]);
                else
                    w[4 * i + j] = pack2(__uint_as_float(o[j] << 16), __uint_as_float(o[j] & 0xFFFF0000u));
        }
    }
}

template <int MODE, int MB>
__device__ __forceinline__ void gv_compute(const GemvArgs& a, const __nv_bfloat16* xs, const float* xsum, float* red,
                                           int g, int r0, int rows_valid, int n0) {
    using T = GvTraits<MODE>;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int half = lane >> 4, l16 = lane & 15;
    const size_t row_bytes = T::kNibbles ? (size_t)a.N / 2 : (size_t)a.N;
    const uint8_t* wbase = a.weight + (size_t)g * a.K * row_bytes + (T::kNibbles ? n0 / 2 : n0) + l16 * T::kLaneBytes;
    const int col0 = n0 + l16 * 16;

    f32x2 acc[MB][8];
#pragma unroll
    for (int m = 0; m < MB; ++m)
#pragma unroll
        for (int c = 0; c < 8; ++c) acc[m][c] = 0ull;

    f32x2 sc[8], tc[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) sc[c] = tc[c] = 0ull;

    // int8 / fp8: the warp's rows of the steps kGvL2Steps ahead are requested into L2, one line per lane (16 rows
    // x the slab's 256-byte row segment): the register loads then wait for L2 instead of DRAM.  (The nibble
    // formats' versions of this function have no registers to spare for it.)
    const uint8_t* pf_base = a.weight + (size_t)g * a.K * row_bytes + n0 + 128 * (lane & 1);
    auto prefetch_step = [&](int k) {
        if constexpr (!T::kNibbles) {
            if (k + (lane >> 1) < a.K) asm volatile("prefetch.global.L2 [%0];" ::"l"(pf_base + (size_t)(k + (lane >> 1)) * row_bytes));
        }
    };
#pragma unroll
    for (int i = 0; i < kGvL2Steps; ++i) prefetch_step(warp * kGvWarpRows + i * kGvIterRows);
    for (int k0 = warp * kGvWarpRows; k0 < a.K; k0 += kGvIterRows) {
        prefetch_step(k0 + kGvL2Steps * kGvIterRows);
        // ---- issue all loads of this step first ----
        uint4 q[kGvUnroll];
        const uint8_t* p = wbase + (size_t)(k0 + half) * row_bytes;
#pragma unroll
        for (int u = 0; u < kGvUnroll; ++u) {
            if constexpr (T::kNibbles) {
                const uint2 v = ldg_stream8(p + (size_t)(2 * u) * row_bytes);
                q[u] = make_uint4(v.x, v.y, 0u, 0u);
            } else {
                q[u] = ldg_stream(p + (size_t)(2 * u) * row_bytes);
            }
        }
        // ---- x values of the 16 rows: lane uses rows k0 + 2u + half ----
        uint32_t xw[MB][kGvUnroll];
#pragma unroll
        for (int m = 0; m < MB; ++m) {
            const uint4* xp = reinterpret_cast<const uint4*>(xs + (size_t)m * (a.K + kGvXPad) + k0);
            const uint4 x0 = xp[0], x1 = xp[1];
            xw[m][0] = x0.x; xw[m][1] = x0.y; xw[m][2] = x0.z; xw[m][3] = x0.w;
            xw[m][4] = x1.x; xw[m][5] = x1.y; xw[m][6] = x1.z; xw[m][7] = x1.w;
        }
        float sf = 1.f;
        if constexpr (MODE == B200MOE_CT_FP8) {
            sf = __ldg(static_cast<const float*>(a.scale) + ((size_t)g * (a.K >> 7) + (k0 >> 7)) * (a.N >> 7) + (col0 >> 7));
        } else if constexpr (MODE == B200MOE_CT_FP4) {
            // one scale row per 16 k rows: exactly the rows of this step
            const uint4* sp = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(a.scale) +
                                                             ((size_t)g * (a.K >> 4) + (k0 >> 4)) * a.N + col0);
            const uint4 s0 = __ldg(sp), s1 = __ldg(sp + 1);
            const uint32_t sw[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
            for (int c = 0; c < 8; ++c) sc[c] = pack2(__uint_as_float(sw[c] << 16), __uint_as_float(sw[c] & 0xFFFF0000u));
        } else if constexpr (MODE == B200MOE_CT_INT4) {
            // one scale / offset row per 128 k rows; the 16 rows of this step lie inside one group
            const size_t so = ((size_t)g * (a.K >> 7) + (k0 >> 7)) * a.N + col0;
            const uint4* sp = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(a.scale) + so);
            const uint4 s0 = __ldg(sp), s1 = __ldg(sp + 1);
            uint4 o0 = make_uint4(0u, 0u, 0u, 0u), o1 = o0;
            if (a.offset != nullptr) {
                const uint4* op = reinterpret_cast<const uint4*>(a.offset + so);
                o0 = __ldg(op);
                o1 = __ldg(op + 1);
            }
            const uint32_t sw[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
            const uint32_t ow[8] = {o0.x, o0.y, o0.z, o0.w, o1.x, o1.y, o1.z, o1.w};
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                sc[c] = pack2(__uint_as_float(sw[c] << 16), __uint_as_float(sw[c] & 0xFFFF0000u));
                tc[c] = mul2(pack2(__uint_as_float(ow[c] << 16), __uint_as_float(ow[c] & 0xFFFF0000u)), sc[c]);
            }
        }
        // fp4 with one or two rows: the step's rows are one scale group, so the scale multiplies the fp32
        // sum of the step's products (x * e2m1 is exact in fp32) instead of every weight
        constexpr bool kGroupScale = (MODE == B200MOE_CT_FP4) && MB <= 2;
        f32x2 part[kGroupScale ? MB : 1][8];
        if constexpr (kGroupScale) {
#pragma unroll
            for (int m = 0; m < MB; ++m)
#pragma unroll
                for (int c = 0; c < 8; ++c) part[m][c] = 0ull;
        }
#pragma unroll
        for (int u = 0; u < kGvUnroll; ++u) {
            f32x2 w[8];
            gv_decode<MODE, !kGroupScale>(q[u], w, sc, tc);
#pragma unroll
            for (int m = 0; m < MB; ++m) {
                float xv = __uint_as_float(half ? (xw[m][u] & 0xFFFF0000u) : (xw[m][u] << 16));
                if constexpr (MODE == B200MOE_CT_FP8) xv *= sf;
                const f32x2 xx = pack2(xv, xv);
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    if constexpr (kGroupScale) part[m][c] = fma2(xx, w[c], part[m][c]);
                    else acc[m][c] = fma2(xx, w[c], acc[m][c]);
                }
            }
        }
        if constexpr (kGroupScale) {
#pragma unroll
            for (int m = 0; m < MB; ++m)
#pragma unroll
                for (int c = 0; c < 8; ++c) acc[m][c] = fma2(part[m][c], sc[c], acc[m][c]);
        }
    }

    // ---- combine the 16 partial sums per column -------------------------------------------------
#pragma unroll
    for (int m = 0; m < MB; ++m) {
        float v[16];
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            unpack2(acc[m][c], v[2 * c], v[2 * c + 1]);
            v[2 * c] += __shfl_xor_sync(0xffffffffu, v[2 * c], 16);
            v[2 * c + 1] += __shfl_xor_sync(0xffffffffu, v[2 * c + 1], 16);
        }
        if (half == 0) {
            float4* dst = reinterpret_cast<float4*>(red + ((warp * kGvRows + m) * kGvSlabN) + l16 * 16);
#pragma unroll
            for (int c = 0; c < 4; ++c) dst[c] = make_float4(v[4 * c], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]);
        }
    }
    __syncthreads();
    {
        const int t = threadIdx.x;  // column inside the slab
        const int n = n0 + t;
        float s_n = 1.f, so_n = 0.f;
        if constexpr (MODE == B200MOE_CT_INT8) {
            s_n = __bfloat162float(static_cast<const __nv_bfloat16*>(a.scale)[(size_t)g * a.N + n]);
            if (a.offset != nullptr) so_n = s_n * __bfloat162float(a.offset[(size_t)g * a.N + n]);
        }
#pragma unroll
        for (int m = 0; m < MB; ++m) {
            if (m < rows_valid) {
                float v = 0.f;
#pragma unroll
                for (int w = 0; w < kGvWarps; ++w) v += red[(w * kGvRows + m) * kGvSlabN + t];
                if constexpr (MODE == B200MOE_CT_INT8) v = fmaf(so_n, xsum[m], s_n * v);
                a.y[(size_t)(r0 + m) * a.N + n] = __float2bfloat16_rn(v);
            }
        }
    }
    __syncthreads();
}

// ---- 2..4 rows per expert, int8: the multiply-adds go to the tensor core ---------------------
// With more than one row the scalar path spends most of its issue slots on FMAs.  Here a warp
// multiplies a 16 (k) x 128 (columns) block of weights with up to four x rows per step using eight
// mma.sync m16n8k16 instructions, the weights as the 16 x 16 operand:
//   lane (g, t) = (lane / 4, lane % 4) loads rows k0 + 4t .. 4t+3, columns 16g .. 16g+15 (each load
//   instruction reads four full 128-byte lines) and feeds instruction j with columns 16g + 2j, +1:
//   operand row g <-> column 16g + 2j, row g + 8 <-> column 16g + 2j + 1, and the instruction's
//   k index {2t, 2t+1, 2t+8, 2t+9} <-> weight rows 4t .. 4t+3 (a summation index: any assignment
//   works as long as the x operand uses the same one).  One byte permute per two rows and two
//   columns puts (row, row + 1) pairs of a column side by side, then the exact int8 -> bf16
//   conversion of common.cuh applies; x pairs come from shared memory with one 8-byte load per step.
// The instruction count per weight byte no longer depends on the number of rows.
// Two e4m3 codes in the high bytes of the two 16-bit lanes (low bytes ignored) -> bf16x2, exact:
// exponent and mantissa bits go under the bf16 exponent, times 2^120 (subnormals included).
__device__ __forceinline__ uint32_t e4m3x2_hi_to_bf16(uint32_t t) {
    return mul_bf16x2(((t >> 4) & 0x07F007F0u) | (t & 0x80008000u), 0x7B807B80u);
}

__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                          uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// fp8 (e4m3) follows the same scheme: the bytes of rows (k, k+1) of a column are permuted into the
// high bytes of the two 16-bit lanes and decoded by bit placement (exact in bf16); the fp32 scale of
// the 128 x 128 block, uniform for a warp over a 128-row stretch, multiplies the stretch's partial sums.
template <int MODE>
__device__ __forceinline__ void gv_compute_mma(const GemvArgs& a, const __nv_bfloat16* xs, const float* xsum, float* red,
                                               int g_expert, int r0, int rows_valid, int n0) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int hc = warp & 1, kg = warp >> 1;  // column half of the slab, k group
    const size_t row_bytes = (size_t)a.N;
    const uint8_t* wbase = a.weight + (size_t)g_expert * a.K * row_bytes + n0 + 128 * hc + 16 * g + (size_t)(4 * t) * row_bytes;
    // x pairs of token g at the lane's four k rows (tokens beyond the valid rows contribute zeros)
    const __nv_bfloat16* xrow = xs + (size_t)(g < rows_valid ? g : 0) * (a.K + kGvXPad) + 4 * t;
    const bool x_on = g < rows_valid;

    float c[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j) c[j][0] = c[j][1] = c[j][2] = c[j][3] = 0.f;
    constexpr bool kBlockScale = (MODE == B200MOE_CT_FP8);
    float ct[kBlockScale ? 8 : 1][4];  // fp8: totals; `c` then holds the current 128-row stretch
    if constexpr (kBlockScale) {
#pragma unroll
        for (int j = 0; j < 8; ++j) ct[j][0] = ct[j][1] = ct[j][2] = ct[j][3] = 0.f;
    }

    constexpr int kStepRows = 16 * kGvMmaParts;  // k rows the CTA consumes per step
    // (fp8 accepts N % 256 == 128: in the last slab the warps of the second column half have no columns)
    const int k_end = (n0 + 128 * hc < a.N) ? a.K : 0;
    // two steps (2 x 16 rows of the warp's 128-byte row segment) per iteration: one line per lane into L2,
    // kGvL2Steps / 2 iterations ahead
    const uint8_t* pf_base = a.weight + (size_t)g_expert * a.K * row_bytes + n0 + 128 * hc;
    auto prefetch_iter = [&](int k) {
        const int kk = k + (lane >> 4) * kStepRows + (lane & 15);
        if (kk < k_end) asm volatile("prefetch.global.L2 [%0];" ::"l"(pf_base + (size_t)kk * row_bytes));
    };
#pragma unroll
    for (int i = 0; i < kGvL2Steps / 2; ++i) prefetch_iter(kg * 16 + i * 2 * kStepRows);
    for (int k0 = kg * 16; k0 < k_end; k0 += 2 * kStepRows) {
        prefetch_iter(k0 + (kGvL2Steps / 2) * 2 * kStepRows);
        const bool second = k0 + kStepRows < a.K;
        float sf = 1.f;
        if constexpr (kBlockScale)  // k0 and k0 + 64 lie in the same 128-row block (K % 128 == 0)
            sf = __ldg(static_cast<const float*>(a.scale) + ((size_t)g_expert * (a.K >> 7) + (k0 >> 7)) * (a.N >> 7) +
                       ((n0 + 128 * hc) >> 7));
        uint4 q[2][4];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            if (h == 1 && !second) break;
            const uint8_t* p = wbase + (size_t)(k0 + h * kStepRows) * row_bytes;
#pragma unroll
            for (int i = 0; i < 4; ++i) q[h][i] = ldg_stream(p + (size_t)i * row_bytes);
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            if (h == 1 && !second) break;
            uint2 xb = make_uint2(0u, 0u);
            if (x_on) xb = *reinterpret_cast<const uint2*>(xrow + k0 + h * kStepRows);
            const uint32_t r0w[4] = {q[h][0].x, q[h][0].y, q[h][0].z, q[h][0].w};
            const uint32_t r1w[4] = {q[h][1].x, q[h][1].y, q[h][1].z, q[h][1].w};
            const uint32_t r2w[4] = {q[h][2].x, q[h][2].y, q[h][2].z, q[h][2].w};
            const uint32_t r3w[4] = {q[h][3].x, q[h][3].y, q[h][3].z, q[h][3].w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
#pragma unroll
                for (int o = 0; o < 2; ++o) {  // byte pairs (0,1) and (2,3) of word i: instruction j = 2i + o
                    uint32_t a0, a1, a2, a3;
                    if constexpr (MODE == B200MOE_CT_INT8) {
                        const uint32_t sel = o == 0 ? 0x5410u : 0x7632u;
                        s8x4_to_bf16_even_odd(prmt(r0w[i], r1w[i], sel), a0, a1);  // (row 4t, 4t+1) at the two columns
                        s8x4_to_bf16_even_odd(prmt(r2w[i], r3w[i], sel), a2, a3);  // (row 4t+2, 4t+3)
                    } else {
                        // byte b of both rows into the high bytes of the two lanes (the low bytes are masked off)
                        const uint32_t s0 = o == 0 ? 0x4000u : 0x6020u, s1 = o == 0 ? 0x5010u : 0x7030u;
                        a0 = e4m3x2_hi_to_bf16(prmt(r0w[i], r1w[i], s0));
                        a1 = e4m3x2_hi_to_bf16(prmt(r0w[i], r1w[i], s1));
                        a2 = e4m3x2_hi_to_bf16(prmt(r2w[i], r3w[i], s0));
                        a3 = e4m3x2_hi_to_bf16(prmt(r2w[i], r3w[i], s1));
                    }
                    mma_16816(c[2 * i + o], a0, a1, a2, a3, xb.x, xb.y);
                }
            }
        }
        if constexpr (kBlockScale) {
#pragma unroll
            for (int j = 0; j < 8; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    ct[j][e] = fmaf(sf, c[j][e], ct[j][e]);
                    c[j][e] = 0.f;
                }
        }
    }
    if constexpr (kBlockScale) {
#pragma unroll
        for (int j = 0; j < 8; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) c[j][e] = ct[j][e];
    }

    // ---- partial sums of the four k groups -> shared memory -> per-column epilogue ----------------
    if (t < 2) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int col = 128 * hc + 16 * g + 2 * j;
#pragma unroll
            for (int e = 0; e < 2; ++e) {  // tokens 2t, 2t + 1
                const int tok = 2 * t + e;
                float* dst = red + (size_t)(kg * kGvRows + tok) * kGvSlabN + col;
                *reinterpret_cast<float2*>(dst) = make_float2(c[j][e], c[j][2 + e]);
            }
        }
    }
    __syncthreads();
    {
        const int tc = threadIdx.x;  // column inside the slab
        const int n = n0 + tc;
        float s_n = 1.f, so_n = 0.f;
        if constexpr (MODE == B200MOE_CT_INT8) {
            s_n = __bfloat162float(static_cast<const __nv_bfloat16*>(a.scale)[(size_t)g_expert * a.N + n]);
            if (a.offset != nullptr) so_n = s_n * __bfloat162float(a.offset[(size_t)g_expert * a.N + n]);
        }
#pragma unroll
        for (int m = 0; m < kGvRows; ++m) {
            if (m < rows_valid && n < a.N) {
                float v = 0.f;
#pragma unroll
                for (int w = 0; w < kGvMmaParts; ++w) v += red[(w * kGvRows + m) * kGvSlabN + tc];
                if constexpr (MODE == B200MOE_CT_INT8) v = fmaf(so_n, xsum[m], s_n * v);
                a.y[(size_t)(r0 + m) * a.N + n] = __float2bfloat16_rn(v);
            }
        }
    }
    __syncthreads();
}

// ---- fp4 weights in the reference's stored (pre-shuffled) order, read in place -----------------
// Canonical row 16a + 8b + c8 of 64-row block R, byte column 128j + 16p + 4q + s lives at
//   ((((((2R + b) * 4 + a) * 8 + p) * J + j) * 4 + q) * 8 + c8) * 4 + s,        J = N / 256,
// so 16 consecutive bytes are four consecutive rows of eight columns.  A lane therefore owns eight
// columns of the 256-column slab (lane = 16-byte chunk of the output row) and, per step, the 16 rows
// of one scale group: four 16-byte loads, one scale vector.  fp32 throughout; the scale of a group
// multiplies the fp32 sum of its 16 products (x * e2m1 is exact in fp32) instead of every weight.
// No conversion pass over the weights.
template <int MB>
__device__ __forceinline__ void gv_compute_fp4_stored(const GemvArgs& a, const __nv_bfloat16* xs, float* red, int g,
                                                      int r0, int rows_valid, int n0) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int J = a.N >> 8, j = n0 >> 8, p = lane >> 2, q = lane & 3;
    const uint8_t* wbase = a.weight + (size_t)g * a.K * ((size_t)a.N >> 1) + (size_t)j * 128 + q * 32;
    const size_t p_stride = (size_t)J * 128;  // bytes between consecutive (b, a, p) rows of the stored array
    const int col0 = n0 + lane * 8;

    f32x2 acc[MB][4];
#pragma unroll
    for (int m = 0; m < MB; ++m)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[m][c] = 0ull;

    for (int k0 = warp * 16; k0 < a.K; k0 += kGvWarps * 16) {
        const int R = k0 >> 6, aa = (k0 >> 4) & 3;
        uint4 wq[4];  // [2b + h]: rows k0 + 8b + 4h .. + 3
#pragma unroll
        for (int b = 0; b < 2; ++b) {
            const uint8_t* ptr = wbase + ((size_t)((2 * R + b) * 4 + aa) * 8 + p) * p_stride;
            wq[2 * b] = ldg_stream(ptr);
            wq[2 * b + 1] = ldg_stream(ptr + 16);
        }
        const uint4 s4 = __ldg(reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(a.scale) +
                                                              ((size_t)g * (a.K >> 4) + (k0 >> 4)) * a.N + col0));
        const uint32_t sw[4] = {s4.x, s4.y, s4.z, s4.w};
        f32x2 sc[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) sc[c] = pack2(__uint_as_float(sw[c] << 16), __uint_as_float(sw[c] & 0xFFFF0000u));
        uint32_t xw[MB][8];  // x of the 16 rows, two per word
#pragma unroll
        for (int m = 0; m < MB; ++m) {
            const uint4* xp = reinterpret_cast<const uint4*>(xs + (size_t)m * (a.K + kGvXPad) + k0);
            const uint4 x0 = xp[0], x1 = xp[1];
            xw[m][0] = x0.x; xw[m][1] = x0.y; xw[m][2] = x0.z; xw[m][3] = x0.w;
            xw[m][4] = x1.x; xw[m][5] = x1.y; xw[m][6] = x1.z; xw[m][7] = x1.w;
        }
        // the 16 rows of the step share one scale per column: sum x * e2m1 first (fp32), scale once
        f32x2 part[MB][4];
#pragma unroll
        for (int m = 0; m < MB; ++m)
#pragma unroll
            for (int c = 0; c < 4; ++c) part[m][c] = 0ull;
#pragma unroll
        for (int piece = 0; piece < 4; ++piece) {
            const uint32_t w4[4] = {wq[piece].x, wq[piece].y, wq[piece].z, wq[piece].w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int row = 4 * piece + i;  // 8b + 4h + i within the step
                uint32_t v[4];
                e2m1x8_to_bf16(w4[i], v);
                f32x2 wv[4];
#pragma unroll
                for (int c = 0; c < 4; ++c) wv[c] = pack2(__uint_as_float(v[c] << 16), __uint_as_float(v[c] & 0xFFFF0000u));
#pragma unroll
                for (int m = 0; m < MB; ++m) {
                    const uint32_t xx = xw[m][row >> 1];
                    const float xv = __uint_as_float((row & 1) ? (xx & 0xFFFF0000u) : (xx << 16));
                    const f32x2 x2 = pack2(xv, xv);
#pragma unroll
                    for (int c = 0; c < 4; ++c) part[m][c] = fma2(x2, wv[c], part[m][c]);
                }
            }
        }
#pragma unroll
        for (int m = 0; m < MB; ++m)
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[m][c] = fma2(part[m][c], sc[c], acc[m][c]);
    }
    // partial sums of the eight warps -> shared memory -> one thread per column
#pragma unroll
    for (int m = 0; m < MB; ++m) {
        float v[8];
#pragma unroll
        for (int c = 0; c < 4; ++c) unpack2(acc[m][c], v[2 * c], v[2 * c + 1]);
        float4* dst = reinterpret_cast<float4*>(red + ((warp * kGvRows + m) * kGvSlabN) + lane * 8);
        dst[0] = make_float4(v[0], v[1], v[2], v[3]);
        dst[1] = make_float4(v[4], v[5], v[6], v[7]);
    }
    __syncthreads();
    {
        const int t = threadIdx.x;
#pragma unroll
        for (int m = 0; m < MB; ++m) {
            if (m < rows_valid) {
                float v = 0.f;
#pragma unroll
                for (int w = 0; w < kGvWarps; ++w) v += red[(w * kGvRows + m) * kGvSlabN + t];
                a.y[(size_t)(r0 + m) * a.N + n0 + t] = __float2bfloat16_rn(v);
            }
        }
    }
    __syncthreads();
}


// ---- fp4, 1..4 rows per expert: decode by the e2m1 -> f16 conversion instruction, multiply-adds on the tensor core --
// The scalar fp4 paths spend their issue slots on the decode and the FMAs (about 6 instructions per weight with
// four rows; the HBM rate leaves room for fewer than 3).  Here the x rows are held in shared memory as f16 --
// each row scaled by a power of two so that its largest element lies in [2^14, 2^15); the staging code only
// takes this path when every element is then exactly representable, so x' * e2m1 products stay exact -- and a
// warp multiplies a 16 (k) x 128 (columns) block of weights with the x rows using eight mma.sync m16n8k16
// (f16 operands, fp32 accumulation), the weights as the 16 x 16 operand.  The 16 rows of a step are one scale
// group: the instruction starts from zero and its fp32 sums are multiplied by the group's bf16 scale per column
// into the running totals (the scale never touches a weight; gemv_impl.h:147-199 keeps the weights in fp32
// the same way).  The row's power of two is undone in the epilogue.
//   lane (g, t) = (lane / 4, lane % 4) owns k rows {2t, 2t+1, 2t+8, 2t+9} of the step -- the instruction's own k
//   indices -- and 16 columns: rows (2t, 2t+1) of eight columns are two 32-bit words; one shift and two logic
//   operations put the two rows' codes of a column into one byte, which the conversion instruction turns into
//   the f16 pair (row 2t, row 2t+1) the operand register wants.
//   canonical layout: columns 16g .. 16g+15 of the warp's 128 (four 8-byte loads cover four rows x 64 bytes);
//   stored order: the 8-column groups (p, q) = (4 hc + g / 4 + 2 i, g % 4), i = 0, 1, whose rows (2t, 2t+1) of
//   an 8-row block are 8 consecutive bytes (each load instruction covers two full 128-byte lines).
__device__ __forceinline__ void cvt_e2m1x8_f16(uint32_t w, uint32_t (&o)[4]) {
    // byte i of w = two codes -> f16x2 (low nibble in the low half)
    asm("{ .reg .b8 b0, b1, b2, b3; mov.b32 {b0, b1, b2, b3}, %4; cvt.rn.f16x2.e2m1x2 %0, b0; "
        "cvt.rn.f16x2.e2m1x2 %1, b1; cvt.rn.f16x2.e2m1x2 %2, b2; cvt.rn.f16x2.e2m1x2 %3, b3; }"
        : "=r"(o[0]), "=r"(o[1]), "=r"(o[2]), "=r"(o[3])
        : "r"(w));
}

__device__ __forceinline__ void mma_16816_f16_zero(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                   uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%10, %10, %10, %10};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}

constexpr int kGvFp4Ahead = 4;  // steps whose loads are in flight per warp (6: slower, measured)

constexpr int kGvFp4L2Ahead = 1;  // batches of kGvFp4Ahead steps requested into L2 before their loads are issued

template <bool kStored>
__device__ __forceinline__ void gv_compute_fp4_mma(const GemvArgs& a, const __half* xs, const int* xexp, float* red,
                                                   int g_expert, int r0, int rows_valid, int n0) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int hc = warp & 1, kg = warp >> 1;  // column half of the slab, k group
    const size_t row_bytes = (size_t)a.N >> 1;
    const uint8_t* wexp = a.weight + (size_t)g_expert * a.K * row_bytes;
    // first of the lane's 16 columns inside the slab (stored order: of its first group; the second is 64 further)
    const int c_first = kStored ? 128 * hc + 32 * (g >> 2) + 8 * (g & 3) : 128 * hc + 16 * g;
    const uint8_t* wbase;
    size_t p_stride = 0;
    if constexpr (kStored) {
        const int J = a.N >> 8, j = n0 >> 8;
        p_stride = (size_t)J * 128;
        wbase = wexp + (size_t)j * 128 + (g & 3) * 32 + 8 * t;
    } else {
        wbase = wexp + (size_t)(n0 >> 1) + 64 * hc + 8 * g + (size_t)(2 * t) * row_bytes;
    }
    const __half* xrow = xs + (size_t)(g < rows_valid ? g : 0) * (a.K + kGvXPad) + 2 * t;
    const bool x_on = g < rows_valid;
    const __nv_bfloat16* sbase = static_cast<const __nv_bfloat16*>(a.scale) + (size_t)g_expert * (a.K >> 4) * a.N + n0 + c_first;

    float acc[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;

    constexpr int kStepRows = 16 * kGvMmaParts;  // k rows the CTA consumes per step
    // q[0], q[1]: rows (2t, 2t+1) and (2t+8, 2t+9) of the lane's columns 0..7; q[2], q[3]: of its columns 8..15
    auto load = [&](int k, uint2 (&q)[4]) {
        if constexpr (kStored) {
            const int R = k >> 6, aa = (k >> 4) & 3;
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int b = 0; b < 2; ++b)
                    q[2 * i + b] = ldg_stream8(wbase + ((size_t)((2 * R + b) * 4 + aa) * 8 + 4 * hc + (g >> 2) + 2 * i) * p_stride);
        } else {
            const uint8_t* p = wbase + (size_t)k * row_bytes;
            // rows 2t, 2t+1, 2t+8, 2t+9: 16 columns = 8 bytes each
            const uint2 r0w = ldg_stream8(p), r1w = ldg_stream8(p + row_bytes);
            const uint2 r8w = ldg_stream8(p + 8 * row_bytes), r9w = ldg_stream8(p + 9 * row_bytes);
            q[0] = make_uint2(r0w.x, r1w.x);
            q[1] = make_uint2(r8w.x, r9w.x);
            q[2] = make_uint2(r0w.y, r1w.y);
            q[3] = make_uint2(r8w.y, r9w.y);
        }
    };
    // Four steps of the warp's weights and scales into L2, one line per lane: the weights of a step are 8 lines
    // (stored order: 2 row blocks x 4 line rows; canonical: 16 rows x 64 bytes, half a line each), its scales 2
    // lines.  The register loads, issued up to kGvFp4L2Ahead batches later, then wait for L2, not for DRAM.
    auto prefetch_group = [&](int k0) {
        const int h = lane >> 3, k = k0 + h * kStepRows;
        if (k >= a.K) return;
        const uint8_t* w;
        if constexpr (kStored) {
            const int R = k >> 6, aa = (k >> 4) & 3, i = (lane >> 2) & 1, b = (lane >> 1) & 1, gq = lane & 1;
            w = wexp + (size_t)(n0 >> 8) * 128 + ((size_t)((2 * R + b) * 4 + aa) * 8 + 4 * hc + gq + 2 * i) * p_stride;
        } else {
            w = wexp + (size_t)(n0 >> 1) + 64 * hc + (size_t)(k + 2 * (lane & 7)) * row_bytes;  // rows 2l and (same line pair) 2l+1
        }
        asm volatile("prefetch.global.L2 [%0];" ::"l"(w));
        if constexpr (!kStored) asm volatile("prefetch.global.L2 [%0];" ::"l"(w + row_bytes));
        if ((lane & 7) < 2) {
            const __nv_bfloat16* sp = static_cast<const __nv_bfloat16*>(a.scale) + ((size_t)g_expert * (a.K >> 4) + (k >> 4)) * a.N +
                                      n0 + 128 * hc + 64 * (lane & 7);
            asm volatile("prefetch.global.L2 [%0];" ::"l"(sp));
        }
    };
    auto compute = [&](int k, const uint2 (&q)[4]) {
        uint32_t b0 = 0u, b1 = 0u;
        if (x_on) {
            b0 = *reinterpret_cast<const uint32_t*>(xrow + k);
            b1 = *reinterpret_cast<const uint32_t*>(xrow + k + 8);
        }
        // the group's scales of the lane's 16 columns
        const __nv_bfloat16* sp = sbase + (size_t)(k >> 4) * a.N;
        const uint4 s0 = __ldg(reinterpret_cast<const uint4*>(sp));
        const uint4 s1 = __ldg(reinterpret_cast<const uint4*>(sp + (kStored ? 64 : 8)));
        const uint32_t sw[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
        for (int i = 0; i < 2; ++i) {  // columns 8i .. 8i+7 of the lane's 16
            const uint2 lo = q[2 * i], hi = q[2 * i + 1];
            // byte b: the codes of rows (r, r + 1) at column 2b (e_*) / 2b + 1 (o_*)
            const uint32_t e_lo = (lo.x & 0x0F0F0F0Fu) | ((lo.y << 4) & 0xF0F0F0F0u);
            const uint32_t o_lo = ((lo.x >> 4) & 0x0F0F0F0Fu) | (lo.y & 0xF0F0F0F0u);
            const uint32_t e_hi = (hi.x & 0x0F0F0F0Fu) | ((hi.y << 4) & 0xF0F0F0F0u);
            const uint32_t o_hi = ((hi.x >> 4) & 0x0F0F0F0Fu) | (hi.y & 0xF0F0F0F0u);
            uint32_t a0[4], a1[4], a2[4], a3[4];
            cvt_e2m1x8_f16(e_lo, a0);
            cvt_e2m1x8_f16(o_lo, a1);
            cvt_e2m1x8_f16(e_hi, a2);
            cvt_e2m1x8_f16(o_hi, a3);
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                float d[4];
                mma_16816_f16_zero(d, a0[b], a1[b], a2[b], a3[b], b0, b1);
                const float sc_e = __uint_as_float(sw[4 * i + b] << 16), sc_o = __uint_as_float(sw[4 * i + b] & 0xFFFF0000u);
                float* c = acc[4 * i + b];
                c[0] = fmaf(d[0], sc_e, c[0]);
                c[1] = fmaf(d[1], sc_e, c[1]);
                c[2] = fmaf(d[2], sc_o, c[2]);
                c[3] = fmaf(d[3], sc_o, c[3]);
            }
        }
    };
    constexpr int kBatchRows = kGvFp4Ahead * kStepRows;
    int k0 = kg * 16;
    int k_pf = k0;  // first step not yet requested into L2 (requests go out four steps at a time)
    for (; k0 + (kGvFp4Ahead - 1) * kStepRows < a.K; k0 += kBatchRows) {
        uint2 q[kGvFp4Ahead][4];
        for (; k_pf < k0 + kGvFp4L2Ahead * kBatchRows; k_pf += 4 * kStepRows) prefetch_group(k_pf);
#pragma unroll
        for (int h = 0; h < kGvFp4Ahead; ++h) load(k0 + h * kStepRows, q[h]);
#pragma unroll
        for (int h = 0; h < kGvFp4Ahead; ++h) compute(k0 + h * kStepRows, q[h]);
    }
    for (; k0 < a.K; k0 += kStepRows) {
        uint2 q1[4];
        load(k0, q1);
        compute(k0, q1);
    }

    // ---- partial sums of the four k groups -> shared memory -> per-column epilogue ----------------
    if (t < 2) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int col = c_first + (kStored ? 64 * (j >> 2) : 8 * (j >> 2)) + 2 * (j & 3);
#pragma unroll
            for (int e = 0; e < 2; ++e) {  // tokens 2t, 2t + 1
                float* dst = red + (size_t)(kg * kGvRows + 2 * t + e) * kGvSlabN + col;
                *reinterpret_cast<float2*>(dst) = make_float2(acc[j][e], acc[j][2 + e]);
            }
        }
    }
    __syncthreads();
    {
        const int tc = threadIdx.x;  // column inside the slab
#pragma unroll
        for (int m = 0; m < kGvRows; ++m) {
            if (m < rows_valid) {
                float v = 0.f;
#pragma unroll
                for (int w = 0; w < kGvMmaParts; ++w) v += red[(w * kGvRows + m) * kGvSlabN + tc];
                a.y[(size_t)(r0 + m) * a.N + n0 + tc] = __float2bfloat16_rn(scalbnf(v, xexp[m]));
            }
        }
    }
    __syncthreads();
}

// fp4 prepass, one CTA per x row: the row as f16, times 2^-e with e chosen so that its largest element lies in
// [2^14, 2^15), into x16; e into xexp -- or kGvNotF16 when some element is not exactly representable then (more
// than about 2^-32 below the row's largest, a bf16 subnormal, an infinity or a NaN): such rows take the fp32 path.
constexpr int kGvNotF16 = -(1 << 30);

__global__ void __launch_bounds__(256) gv_fp4_prepare_x_kernel(const __nv_bfloat16* __restrict__ x, __half* __restrict__ x16,
                                                               int* __restrict__ xexp, int K) {
    __shared__ int s_max, s_bad;
    const size_t row = blockIdx.x;
    const uint32_t* src = reinterpret_cast<const uint32_t*>(x + row * K);
    uint32_t* dst = reinterpret_cast<uint32_t*>(x16 + row * K);
    if (threadIdx.x == 0) { s_max = 0; s_bad = 0; }
    __syncthreads();
    uint32_t mx = 0u;
    for (int i = threadIdx.x; i < K / 2; i += blockDim.x) {
        const uint32_t w = __ldg(src + i);
        mx = max(mx, max(w & 0x7FFFu, (w >> 16) & 0x7FFFu));  // bf16 magnitudes order like integers
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if ((threadIdx.x & 31) == 0) atomicMax(&s_max, (int)mx);
    __syncthreads();
    const int e_max = s_max >> 7;                    // biased exponent of the largest magnitude
    const int sh = e_max == 0 ? 0 : e_max - 127 - 14;
    int bad = e_max == 255;
    for (int i = threadIdx.x; i < K / 2; i += blockDim.x) {
        const uint32_t w = __ldg(src + i);
        uint32_t out = 0u;
#pragma unroll
        for (int hlf = 0; hlf < 2; ++hlf) {
            const uint32_t b = hlf ? (w >> 16) : (w & 0xFFFFu);
            const uint32_t mag = b & 0x7FFFu, sign = b & 0x8000u;
            uint32_t h = sign;
            if (mag != 0u) {
                const int e = (int)(mag >> 7);
                const int E = e - sh - 112;                       // biased f16 exponent of the scaled value
                const uint32_t sig = (0x80u | (mag & 0x7Fu)) << 3;  // 11-bit significand, leading one at bit 10
                if (e == 0 || E > 30) bad = 1;
                else if (E >= 1) h = sign | ((uint32_t)E << 10) | (sig & 0x3FFu);
                else {
                    const int s = 1 - E;                          // f16 subnormal: exact only if no set bit is shifted out
                    if (s > 10 || (sig & ((1u << s) - 1u)) != 0u) bad = 1;
                    else h = sign | (sig >> s);
                }
            }
            out |= h << (16 * hlf);
        }
        dst[i] = out;
    }
    if (bad) atomicOr(&s_bad, 1);
    __syncthreads();
    if (threadIdx.x == 0) xexp[row] = s_bad ? kGvNotF16 : sh;
}

// fp4 is launched as two kernels over the same work items: PATH 1 takes the passes whose x rows are all exact as
// scaled f16 (tensor-core path), PATH 2 the others (fp32 multiply-adds; normally none, and the kernel leaves after
// walking the item list); PATH 0: every other mode, and fp4 without the prepass.  Separate kernels keep the
// registers of one path from weighing on the other.
template <int MODE, int PATH = 0>
__global__ void __launch_bounds__(kGvThreads, 2) grouped_gemv_kernel(const GemvArgs a) {
    extern __shared__ __align__(16) uint8_t smem_raw[];
    int* row_start = reinterpret_cast<int*>(smem_raw);
    int* active = row_start + (a.G + 1);
    int* n_active_p = active + a.G;
    uintptr_t p = (reinterpret_cast<uintptr_t>(n_active_p + 1) + 15) & ~uintptr_t(15);
    float* xsum = reinterpret_cast<float*>(p);                                   // [4]
    float* red = xsum + 4;                                                        // [8][4][256]
    __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(red + kGvWarps * kGvRows * kGvSlabN);  // [4][K]

    load_row_starts(a.group_list, a.G, a.M, a.gl_type, row_start, a.status);
    if (threadIdx.x == 0) {
        // non-empty experts, those with the most rows first (counting sort on min(rows, 5)): with
        // the ticket counter below the long items start early and the short ones fill the tail
        int n = 0;
        for (int b = 5; b >= 1; --b)
            for (int g = 0; g < a.G; ++g) {
                const int rows = row_start[g + 1] - row_start[g];
                if ((rows >= 5 ? 5 : rows) == b) active[n++] = g;
            }
        *n_active_p = n;
    }
    __syncthreads();

    const int n_slabs = (a.N + kGvSlabN - 1) / kGvSlabN;
    const int n_act = *n_active_p;
    const int n_items = n_act * n_slabs;
    const int kvec = a.K / 8;  // 16-byte vectors per x row
    int* ticket = a.status + (PATH == 2 ? 3 : 2);  // zeroed by the host before the launch
    __shared__ int s_item;
    __shared__ int xexp[kGvRows];
    for (;;) {
        __syncthreads();
        if (threadIdx.x == 0) s_item = atomicAdd(ticket, 1);
        __syncthreads();
        const int item = s_item;
        if (item >= n_items) break;
        // expert-major order: the CTAs that run at the same time hold neighbouring slabs of the same experts and
        // walk the same k rows together, so whole rows of the weight matrix are fetched close in time (DRAM
        // pages stay open: measured +1..6 % over slab-major order); the experts with the most rows still come first
        const int g = active[item / n_slabs];
        const int n0 = (item % n_slabs) * kGvSlabN;
        const int r0 = row_start[g], r1 = row_start[g + 1];
        for (int r = r0; r < r1; r += kGvRows) {
            const int rows = min(kGvRows, r1 - r);
            // fp4: the tensor-core path when every row of the pass is exact as scaled f16 (prepared by the prepass)
            bool fp4_mma = false;
            if constexpr (PATH != 0) {
                fp4_mma = true;
                for (int m = 0; m < rows; ++m) fp4_mma = fp4_mma && a.xexp[r + m] != kGvNotF16;
                if (fp4_mma != (PATH == 1)) continue;  // the other kernel's pass
                if (fp4_mma && threadIdx.x < rows) xexp[threadIdx.x] = a.xexp[r + threadIdx.x];
            }
            // ---- stage the x rows (and their sums, for the offset term) ----
            if (threadIdx.x < 4) xsum[threadIdx.x] = 0.f;
            __syncthreads();
            for (int m = 0; m < rows; ++m) {
                const uint4* src = fp4_mma ? reinterpret_cast<const uint4*>(a.x16 + (size_t)(r + m) * a.K)
                                           : reinterpret_cast<const uint4*>(a.x + (size_t)(r + m) * a.K);
                uint4* dst = reinterpret_cast<uint4*>(xs + (size_t)m * (a.K + kGvXPad));
                float s = 0.f;
                for (int i = threadIdx.x; i < kvec; i += kGvThreads) {
                    const uint4 v = __ldg(src + i);
                    dst[i] = v;
                    if (MODE == B200MOE_CT_INT8 && a.offset != nullptr) {
                        const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                        for (int j = 0; j < 4; ++j) s += __uint_as_float(w4[j] << 16) + __uint_as_float(w4[j] & 0xFFFF0000u);
                    }
                }
                if (MODE == B200MOE_CT_INT8 && a.offset != nullptr) {
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
                    if ((threadIdx.x & 31) == 0) atomicAdd(&xsum[m], s);
                }
            }
            __syncthreads();
            // fp8: the tensor-core path also wins with one row (its decode is two-wide); int8 with one
            // row is faster on the scalar path; fp4 takes the tensor-core path whenever x is exact in f16
            if constexpr (PATH == 1) {
                if (a.fp4_stored) gv_compute_fp4_mma<true>(a, reinterpret_cast<const __half*>(xs), xexp, red, g, r, rows, n0);
                else gv_compute_fp4_mma<false>(a, reinterpret_cast<const __half*>(xs), xexp, red, g, r, rows, n0);
            } else if (MODE == B200MOE_CT_FP4 && a.fp4_stored) {
                if (rows == 1) gv_compute_fp4_stored<1>(a, xs, red, g, r, rows, n0);
                else if (rows == 2) gv_compute_fp4_stored<2>(a, xs, red, g, r, rows, n0);
                else gv_compute_fp4_stored<4>(a, xs, red, g, r, rows, n0);
            } else if constexpr (MODE == B200MOE_CT_FP8) gv_compute_mma<MODE>(a, xs, xsum, red, g, r, rows, n0);
            else if (rows == 1) gv_compute<MODE, 1>(a, xs, xsum, red, g, r, rows, n0);
            else if constexpr (MODE == B200MOE_CT_INT8) gv_compute_mma<MODE>(a, xs, xsum, red, g, r, rows, n0);
            else if (rows == 2) gv_compute<MODE, 2>(a, xs, xsum, red, g, r, rows, n0);
            else gv_compute<MODE, 4>(a, xs, xsum, red, g, r, rows, n0);
        }
    }
}

static size_t gv_smem_bytes(int G, int K) {
    size_t b = sizeof(int) * (size_t)(2 * G + 2) + 16;
    b += sizeof(float) * (4 + kGvWarps * kGvRows * kGvSlabN);
    b += (size_t)kGvRows * (K + kGvXPad) * 2;
    return b;
}

template <int MODE, int PATH = 0>
static int gv_launch(const GemvArgs& a, cudaStream_t stream) {
    const size_t smem = gv_smem_bytes(a.G, a.K);
    if (smem > 227 * 1024) return B200MOE_ERR_SHAPE;
    B200MOE_CUDA_TRY(cudaFuncSetAttribute(grouped_gemv_kernel<MODE, PATH>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          (int)smem));
    const int per_sm = smem <= 110 * 1024 ? 2 : 1;
    grouped_gemv_kernel<MODE, PATH><<<per_sm * sm_count(), kGvThreads, smem, stream>>>(a);
    B200MOE_CUDA_TRY(cudaGetLastError());
    return B200MOE_OK;
}

}  // namespace b200moe

using namespace b200moe;

static size_t gv_fp4_exp_bytes(int64_t M) { return ((size_t)M * sizeof(int) + 255) / 256 * 256; }

extern "C" size_t b200moe_grouped_gemv_workspace_bytes(int64_t M, int64_t K, int64_t N, int64_t G, int compute_type,
                                                       int weight_layout) {
    (void)N; (void)G; (void)weight_layout;
    // status words and the work-item ticket; fp4 adds the rows' exponents and x as scaled f16
    size_t b = B200MOE_STATUS_BYTES;
    if (compute_type == B200MOE_CT_FP4 && M > 0 && K > 0) b += gv_fp4_exp_bytes(M) + (size_t)M * (size_t)K * 2;
    return b;
}

extern "C" int b200moe_grouped_gemv(const void* x, const void* weight, const void* scale, const void* offset,
                                    const int64_t* group_list, void* y, int64_t M, int64_t K, int64_t N, int64_t G,
                                    int compute_type, int group_list_type, int weight_layout, void* workspace,
                                    size_t workspace_bytes, void* stream) {
    if (compute_type < B200MOE_CT_FP8 || compute_type > B200MOE_CT_INT4) return B200MOE_ERR_COMPUTE_TYPE;
    if (group_list_type != B200MOE_GROUP_LIST_CUMSUM && group_list_type != B200MOE_GROUP_LIST_COUNTS)
        return B200MOE_ERR_ARGUMENT;
    if (weight_layout != B200MOE_LAYOUT_CANONICAL && weight_layout != B200MOE_LAYOUT_ASCEND)
        return B200MOE_ERR_ARGUMENT;
    if (M < 0 || K <= 0 || N <= 0 || G <= 0 || G > kMaxExperts || M > 0x7FFFFFF0LL || K > 0x7FFFFFF0LL ||
        N > 0x7FFFFFF0LL || G * K > 0x7FFFFFF0LL)
        return B200MOE_ERR_SHAPE;
    // fp8: what the reference takes (K and N multiples of its 128 x 128 scale block, i.e. a last slab of
    // 128 columns); the other modes work on whole 256-column slabs
    if (compute_type == B200MOE_CT_FP8 ? ((K % 128) != 0 || (N % 128) != 0) : ((K % 64) != 0 || (N % kGvSlabN) != 0))
        return B200MOE_ERR_SHAPE;
    if (compute_type == B200MOE_CT_INT4 && (K % 128) != 0) return B200MOE_ERR_SHAPE;
    if (M == 0) return B200MOE_OK;
    if (!x || !weight || !scale || !group_list || !y) return B200MOE_ERR_NULL_POINTER;
    if (!aligned16(x) || !aligned16(weight) || !aligned16(scale) || !aligned16(y) ||
        (offset && !aligned16(offset)))
        return B200MOE_ERR_ALIGNMENT;
    const size_t need = b200moe_grouped_gemv_workspace_bytes(M, K, N, G, compute_type, weight_layout);
    if (workspace == nullptr || workspace_bytes < need || !aligned16(workspace)) return B200MOE_ERR_WORKSPACE;

    cudaStream_t s = static_cast<cudaStream_t>(stream);
    B200MOE_CUDA_TRY(cudaMemsetAsync(workspace, 0, 16, s));
    GemvArgs a;
    a.x = static_cast<const __nv_bfloat16*>(x);
    a.weight = static_cast<const uint8_t*>(weight);
    a.scale = scale;
    a.offset = static_cast<const __nv_bfloat16*>(offset);
    a.group_list = group_list;
    a.y = static_cast<__nv_bfloat16*>(y);
    a.M = (int)M; a.K = (int)K; a.N = (int)N; a.G = (int)G;
    a.gl_type = group_list_type;
    a.status = static_cast<int*>(workspace);

    // fp4 in the stored (pre-shuffled) order is read in place
    a.fp4_stored = (compute_type == B200MOE_CT_FP4 && weight_layout == B200MOE_LAYOUT_ASCEND) ? 1 : 0;
    a.x16 = nullptr;
    a.xexp = nullptr;
    // (B200MOE_GEMV_FP4_SCALAR=1 keeps fp4 on the fp32 multiply-adds: comparison runs)
    static const bool fp4_scalar = [] { const char* e = getenv("B200MOE_GEMV_FP4_SCALAR"); return e && e[0] == '1'; }();
    if (compute_type == B200MOE_CT_FP4 && !fp4_scalar) {
        uint8_t* ws = static_cast<uint8_t*>(workspace) + B200MOE_STATUS_BYTES;
        a.xexp = reinterpret_cast<const int*>(ws);
        a.x16 = reinterpret_cast<const __half*>(ws + gv_fp4_exp_bytes(M));
        gv_fp4_prepare_x_kernel<<<(unsigned)M, 256, 0, s>>>(a.x, const_cast<__half*>(a.x16), const_cast<int*>(a.xexp), a.K);
        B200MOE_CUDA_TRY(cudaGetLastError());
    }
    switch (compute_type) {
        case B200MOE_CT_INT8: return gv_launch<B200MOE_CT_INT8>(a, s);
        case B200MOE_CT_FP8: return gv_launch<B200MOE_CT_FP8>(a, s);
        case B200MOE_CT_INT4: return gv_launch<B200MOE_CT_INT4>(a, s);
        default: {
            if (a.x16 == nullptr) return gv_launch<B200MOE_CT_FP4>(a, s);
            const int rc = gv_launch<B200MOE_CT_FP4, 1>(a, s);
            return rc != B200MOE_OK ? rc : gv_launch<B200MOE_CT_FP4, 2>(a, s);
        }
    }
}
