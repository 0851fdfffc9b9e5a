// Standalone dequantisation kernels (FP4 e2m1 with e8m0 block scales; the reference's two weight
// formats: FP4 with bf16 scales per 16 k and FP8 e4m3 with fp32 scales per 128 x 128 block), the FP4
// weight layout conversion and the two-level FP4 scale fold.
//
// Bandwidth kernel: 0.5 B of codes + 1/32 B of scale in, 2 B out per element.  Each thread owns
// one 32-bit word (8 codes) per step, so a warp reads 128 contiguous bytes and writes 512
// contiguous bytes per instruction; eight independent words per thread are in flight.
#include "common.cuh"

namespace b200moe {

constexpr int kDqThreads = 256;
constexpr int kDqUnroll = 8;

template <bool kScaled>
__global__ void __launch_bounds__(kDqThreads)
fp4_dequant_kernel(const uint32_t* __restrict__ codes, const uint8_t* __restrict__ scale,
                   uint4* __restrict__ out, long long n_words) {
    const long long base = (long long)blockIdx.x * (kDqThreads * kDqUnroll) + threadIdx.x;
    uint32_t w[kDqUnroll];
    uint32_t sc[kDqUnroll];
#pragma unroll
    for (int u = 0; u < kDqUnroll; ++u) {
        const long long i = base + (long long)u * kDqThreads;
        w[u] = 0;
        sc[u] = 127;
        if (i < n_words) {
            w[u] = __ldcs(codes + i);
            if (kScaled) sc[u] = __ldg(scale + (i >> 2));  // 32 elements = 4 words share a scale
        }
    }
#pragma unroll
    for (int u = 0; u < kDqUnroll; ++u) {
        const long long i = base + (long long)u * kDqThreads;
        if (i >= n_words) continue;
        uint32_t o[4];
        e2m1x8_to_bf16(w[u], o);
        if (kScaled) {
            // 2^(s-127) as bf16: exponent field s; s = 0 is the subnormal 2^-127, 255 is NaN
            uint32_t sb = sc[u] == 0 ? 0x0040u : (sc[u] == 255 ? 0x7FC0u : (sc[u] << 7));
            sb |= sb << 16;
#pragma unroll
            for (int j = 0; j < 4; ++j) o[j] = mul_bf16x2(o[j], sb);
        }
        __stcs(out + i, make_uint4(o[0], o[1], o[2], o[3]));
    }
}

// [G*K, C] bytes, C = N/2.  One thread moves 4 bytes (the innermost contiguous unit of the
// stored order).  Stored offset of canonical (row r, byte column c):
//   r = 64R + 16a + 8b + c8, c = 128j + 16p + 4q + s, J = C/128
//   off = ((((((2R+b)*4+a)*8+p)*J+j)*4+q)*8+c8)*4+s
template <bool kToAscend>
__global__ void fp4_layout_kernel(const uint32_t* __restrict__ src, uint32_t* __restrict__ dst,
                                  long long rows, int C) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;  // word index, canonical order
    const int cw = C >> 2;
    if (i >= rows * cw) return;
    const long long r = i / cw;
    const int c = (int)(i % cw) << 2;
    const long long R = r >> 6;
    const int a = (int)(r >> 4) & 3, b = (int)(r >> 3) & 1, c8 = (int)r & 7;
    const int j = c >> 7, p = (c >> 4) & 7, q = (c >> 2) & 3;
    const int J = C >> 7;
    const long long off = ((((((2 * R + b) * 4 + a) * 8 + p) * J + j) * 4 + q) * 8 + c8);
    if (kToAscend) dst[off] = src[i];
    else dst[i] = src[off];
}

// Stored ("ascend") word offset of the canonical word (row r, byte column c, c % 4 == 0) of a
// [rows, C]-byte FP4 matrix; see fp4_layout_kernel.
__device__ __forceinline__ long long ascend_word_offset(long long r, int c, int C) {
    const long long R = r >> 6;
    const int a = (int)(r >> 4) & 3, b = (int)(r >> 3) & 1, c8 = (int)r & 7;
    const int j = c >> 7, p = (c >> 4) & 7, q = (c >> 2) & 3;
    const int J = C >> 7;
    return ((((((2 * R + b) * 4 + a) * 8 + p) * J + j) * 4 + q) * 8 + c8);
}

// The reference's FP4 weight format as a standalone operator (the dequant phase of its GEMM kernel,
// grouped_gemm/op_kernel/antiquant_impl.h:23-85,146-169,210-251): codes [G*K, N/2] bytes (canonical
// or stored order), bf16 scale [G*K/16, N], out bf16 [G*K, N] = rne_bf16(e2m1 * scale) -- the product of
// two bf16 values is exact in fp32, so one bf16x2 multiply is that rounding.  One thread per 32-bit
// word: 8 codes of one k row, 16 bytes of scales in, 16 bytes out.
template <bool kAscend>
__global__ void __launch_bounds__(256)
fp4_dequant_bf16_scale_kernel(const uint32_t* __restrict__ codes, const uint4* __restrict__ scale, uint4* __restrict__ out,
                              long long rows, int C) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;  // canonical word index
    const int cw = C >> 2;
    if (i >= rows * cw) return;
    const long long r = i / cw;
    const int wcol = (int)(i % cw);
    const uint32_t w = kAscend ? __ldg(codes + ascend_word_offset(r, wcol << 2, C)) : __ldcs(codes + i);
    const uint4 sc = __ldg(scale + (r >> 4) * cw + wcol);  // 8 bf16 scales = the word's 8 columns
    uint32_t o[4];
    e2m1x8_to_bf16(w, o);
    __stcs(out + i, make_uint4(mul_bf16x2(o[0], sc.x), mul_bf16x2(o[1], sc.y), mul_bf16x2(o[2], sc.z), mul_bf16x2(o[3], sc.w)));
}

// The reference's FP8 weight format as a standalone operator (antiquant_impl.h:87-129,171-208,
// 253-266): codes uint8 [G*K, N], one fp32 scale per 128 x 128 block, out = rne_bf16(e4m3 * scale) with
// the reference's decode (no NaN: 0x7F / 0xFF are +-480).  One thread per 16 codes.
__global__ void __launch_bounds__(256)
fp8_dequant_kernel(const uint4* __restrict__ codes, const float* __restrict__ scale, uint4* __restrict__ out, long long rows,
                   int K, int N) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;  // 16-byte unit
    const int units = N >> 4;
    if (i >= rows * units) return;
    const long long r = i / units;  // g * K + k
    const int n0 = (int)(i % units) << 4;
    const long long g = r / K;
    const int k = (int)(r % K);
    const float sf = __ldg(scale + (g * (K >> 7) + (k >> 7)) * (N >> 7) + (n0 >> 7));
    const f32x2 sf2 = pack_f32x2(sf, sf);
    const uint4 q = __ldcs(codes + i);
    const uint32_t w4[4] = {q.x, q.y, q.z, q.w};
    uint32_t o[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
#pragma unroll
        for (int hp = 0; hp < 2; ++hp) {
            // bytes (2 hp, 2 hp + 1) of the word, each into the high byte of a 16-bit lane; the 4 exponent and 3
            // mantissa bits then sit under the bf16 exponent: exact after * 2^120, subnormals included
            const uint32_t t = prmt(w4[j], 0u, hp == 0 ? 0x1404u : 0x3424u);
            const uint32_t xb = ((t >> 4) & 0x07F007F0u) | (t & 0x80008000u);
            const uint32_t yb = mul_bf16x2(xb, 0x7B807B80u);
            const f32x2 f = mul_f32x2(pack_u32x2(yb << 16, yb & 0xFFFF0000u), sf2);
            o[2 * j + hp] = pack_bf16x2(f32x2_lo(f), f32x2_hi(f));
        }
    }
    __stcs(out + 2 * i, make_uint4(o[0], o[1], o[2], o[3]));
    __stcs(out + 2 * i + 1, make_uint4(o[4], o[5], o[6], o[7]));
}

// Two-level FP4 scale fold (grouped_gemm/test/python/test_group_gemm_fp4.py:86-94 and the transpose
// of :186): block scale bf16 [G, N, KB] times the expert's fp32 global scale (one per expert, or one
// for the first and one for the second half of the N rows), rounded to bf16, written [G, KB, N] --
// the scale tensor the fp4 operators take.
__global__ void fp4_scale_fold_kernel(const __nv_bfloat16* __restrict__ block, const float* __restrict__ glob,
                                      __nv_bfloat16* __restrict__ out, int N, int KB, int S, long long total) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;  // output index (g, kb, n)
    if (i >= total) return;
    const int n = (int)(i % N);
    const long long gk = i / N;
    const int kb = (int)(gk % KB);
    const long long g = gk / KB;
    const float gs = glob[g * S + ((S == 2 && n >= N / 2) ? 1 : 0)];
    out[i] = __float2bfloat16_rn(__bfloat162float(block[(g * N + n) * KB + kb]) * gs);
}

}  // namespace b200moe

using namespace b200moe;

extern "C" int b200moe_fp4_dequant_bf16_scale(const void* codes, const void* scale, void* out_bf16, int64_t G, int64_t K,
                                              int64_t N, int weight_layout, void* stream) {
    if (weight_layout != B200MOE_LAYOUT_CANONICAL && weight_layout != B200MOE_LAYOUT_ASCEND) return B200MOE_ERR_ARGUMENT;
    if (G < 0 || K < 0 || N < 0 || (K % 64) != 0 || (N % 256) != 0 || N > 0x7FFFFFF0LL) return B200MOE_ERR_SHAPE;
    if (G == 0 || K == 0 || N == 0) return B200MOE_OK;
    if (!codes || !scale || !out_bf16) return B200MOE_ERR_NULL_POINTER;
    if (!aligned16(codes) || !aligned16(scale) || !aligned16(out_bf16)) return B200MOE_ERR_ALIGNMENT;
    const long long rows = G * K;
    const int C = (int)(N / 2);
    const long long blocks = (rows * (C / 4) + 255) / 256;
    if (blocks > 0x7FFFFFFFLL) return B200MOE_ERR_SHAPE;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (weight_layout == B200MOE_LAYOUT_ASCEND)
        fp4_dequant_bf16_scale_kernel<true><<<(unsigned)blocks, 256, 0, s>>>(
            static_cast<const uint32_t*>(codes), static_cast<const uint4*>(scale), static_cast<uint4*>(out_bf16), rows, C);
    else
        fp4_dequant_bf16_scale_kernel<false><<<(unsigned)blocks, 256, 0, s>>>(
            static_cast<const uint32_t*>(codes), static_cast<const uint4*>(scale), static_cast<uint4*>(out_bf16), rows, C);
    B200MOE_CUDA_TRY(cudaGetLastError());
    return B200MOE_OK;
}

extern "C" int b200moe_fp8_dequant(const void* codes, const float* scale, void* out_bf16, int64_t G, int64_t K, int64_t N,
                                   void* stream) {
    if (G < 0 || K < 0 || N < 0 || (K % 128) != 0 || (N % 128) != 0 || N > 0x7FFFFFF0LL || K > 0x7FFFFFF0LL)
        return B200MOE_ERR_SHAPE;
    if (G == 0 || K == 0 || N == 0) return B200MOE_OK;
    if (!codes || !scale || !out_bf16) return B200MOE_ERR_NULL_POINTER;
    if (!aligned16(codes) || !aligned16(out_bf16)) return B200MOE_ERR_ALIGNMENT;
    const long long rows = G * K;
    const long long blocks = (rows * (N / 16) + 255) / 256;
    if (blocks > 0x7FFFFFFFLL) return B200MOE_ERR_SHAPE;
    fp8_dequant_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint4*>(codes), scale, static_cast<uint4*>(out_bf16), rows, (int)K, (int)N);
    B200MOE_CUDA_TRY(cudaGetLastError());
    return B200MOE_OK;
}

extern "C" int b200moe_fp4_scale_fold(const void* block_scale, const float* global_scale, void* out, int64_t G, int64_t N,
                                      int64_t KB, int64_t n_global, void* stream) {
    if (G < 0 || N < 0 || KB < 0 || (n_global != 1 && n_global != 2) || (n_global == 2 && (N % 2) != 0) ||
        N > 0x7FFFFFF0LL || KB > 0x7FFFFFF0LL)
        return B200MOE_ERR_SHAPE;
    if (G == 0 || N == 0 || KB == 0) return B200MOE_OK;
    if (!block_scale || !global_scale || !out) return B200MOE_ERR_NULL_POINTER;
    const long long total = G * N * KB;
    const long long blocks = (total + 255) / 256;
    if (blocks > 0x7FFFFFFFLL) return B200MOE_ERR_SHAPE;
    fp4_scale_fold_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(block_scale), global_scale, static_cast<__nv_bfloat16*>(out), (int)N, (int)KB,
        (int)n_global, total);
    B200MOE_CUDA_TRY(cudaGetLastError());
    return B200MOE_OK;
}

extern "C" int b200moe_fp4_dequant(const void* codes, const void* scale_e8m0, void* out_bf16, int64_t n_elems,
                                   int scale_kind, void* stream) {
    if (scale_kind != B200MOE_FP4_SCALE_NONE && scale_kind != B200MOE_FP4_SCALE_E8M0_PER32)
        return B200MOE_ERR_ARGUMENT;
    if (n_elems < 0 || (n_elems % 32) != 0) return B200MOE_ERR_SHAPE;
    if (n_elems == 0) return B200MOE_OK;
    if (codes == nullptr || out_bf16 == nullptr) return B200MOE_ERR_NULL_POINTER;
    if (scale_kind == B200MOE_FP4_SCALE_E8M0_PER32 && scale_e8m0 == nullptr) return B200MOE_ERR_NULL_POINTER;
    if (!aligned16(codes) || !aligned16(out_bf16)) return B200MOE_ERR_ALIGNMENT;
    const long long n_words = n_elems / 8;
    const long long per_block = (long long)kDqThreads * kDqUnroll;
    const long long blocks = (n_words + per_block - 1) / per_block;
    if (blocks > 0x7FFFFFFFLL) return B200MOE_ERR_SHAPE;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (scale_kind == B200MOE_FP4_SCALE_E8M0_PER32)
        fp4_dequant_kernel<true><<<(unsigned)blocks, kDqThreads, 0, s>>>(
            static_cast<const uint32_t*>(codes), static_cast<const uint8_t*>(scale_e8m0),
            static_cast<uint4*>(out_bf16), n_words);
    else
        fp4_dequant_kernel<false><<<(unsigned)blocks, kDqThreads, 0, s>>>(
            static_cast<const uint32_t*>(codes), nullptr, static_cast<uint4*>(out_bf16), n_words);
    B200MOE_CUDA_TRY(cudaGetLastError());
    return B200MOE_OK;
}

extern "C" int b200moe_fp4_layout(const void* src, void* dst, int64_t G, int64_t K, int64_t N, int to_ascend,
                                  void* stream) {
    if (G < 0 || K < 0 || N < 0 || (K % 64) != 0 || (N % 256) != 0) return B200MOE_ERR_SHAPE;
    if (G == 0 || K == 0 || N == 0) return B200MOE_OK;
    if (src == nullptr || dst == nullptr) return B200MOE_ERR_NULL_POINTER;
    if (!aligned16(src) || !aligned16(dst)) return B200MOE_ERR_ALIGNMENT;
    const long long rows = G * K;
    const int C = (int)(N / 2);
    const long long words = rows * (C / 4);
    const long long blocks = (words + 255) / 256;
    if (blocks > 0x7FFFFFFFLL) return B200MOE_ERR_SHAPE;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (to_ascend)
        fp4_layout_kernel<true><<<(unsigned)blocks, 256, 0, s>>>(static_cast<const uint32_t*>(src),
                                                                  static_cast<uint32_t*>(dst), rows, C);
    else
        fp4_layout_kernel<false><<<(unsigned)blocks, 256, 0, s>>>(static_cast<const uint32_t*>(src),
                                                                   static_cast<uint32_t*>(dst), rows, C);
    B200MOE_CUDA_TRY(cudaGetLastError());
    return B200MOE_OK;
}
