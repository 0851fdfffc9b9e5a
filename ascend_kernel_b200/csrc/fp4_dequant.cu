// Standalone FP4(e2m1) -> BF16 dequantisation and the FP4 weight layout conversion.
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

}  // namespace b200moe

using namespace b200moe;

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
