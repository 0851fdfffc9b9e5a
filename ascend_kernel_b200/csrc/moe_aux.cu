// Small bandwidth kernels the MoE layer needs around the two grouped GEMMs:
// SiLU(gate)*up, row gather (token dispatch / permutation) and the weighted combine.
#include "common.cuh"

namespace b200moe {

// h [rows, 2I] bf16 (gate columns first) -> out [rows, I]; 8 elements per thread.
__global__ void silu_mul_kernel(const uint4* __restrict__ h, uint4* __restrict__ out, long long rows, int inter8) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= rows * inter8) return;
    const long long r = i / inter8;
    const int c = (int)(i % inter8);
    const uint4 g = h[r * (2LL * inter8) + c];
    const uint4 u = h[r * (2LL * inter8) + inter8 + c];
    const uint32_t gw[4] = {g.x, g.y, g.z, g.w}, uw[4] = {u.x, u.y, u.z, u.w};
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float g0 = __uint_as_float(gw[j] << 16), g1 = __uint_as_float(gw[j] & 0xFFFF0000u);
        const float u0 = __uint_as_float(uw[j] << 16), u1 = __uint_as_float(uw[j] & 0xFFFF0000u);
        const float a0 = g0 / (1.f + __expf(-g0)), a1 = g1 / (1.f + __expf(-g1));
        o[j] = pack_bf16x2(a0 * u0, a1 * u1);
    }
    out[i] = make_uint4(o[0], o[1], o[2], o[3]);
}

// dst[i, :] = src[index[i], :]; one CTA per destination row, 16 bytes per thread per step.
__global__ void gather_rows_kernel(const uint4* __restrict__ src, const int32_t* __restrict__ index,
                                   uint4* __restrict__ dst, int width16) {
    const long long row = blockIdx.x;
    const long long from = index[row];
    for (int c = threadIdx.x; c < width16; c += blockDim.x) dst[row * width16 + c] = src[from * width16 + c];
}

// out[t, :] = bf16(sum_j weight[t, j] * y[slot[t, j], :]) in fp32; one CTA per token.
__global__ void combine_kernel(const uint4* __restrict__ y, const int32_t* __restrict__ slot,
                               const float* __restrict__ weight, uint4* __restrict__ out, int top_k, int width16) {
    const long long t = blockIdx.x;
    for (int c = threadIdx.x; c < width16; c += blockDim.x) {
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int j = 0; j < top_k; ++j) {
            const long long s = slot[t * top_k + j];
            const float w = weight[t * top_k + j];
            const uint4 v = y[s * width16 + c];
            const uint32_t vw[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                acc[2 * q] = fmaf(w, __uint_as_float(vw[q] << 16), acc[2 * q]);
                acc[2 * q + 1] = fmaf(w, __uint_as_float(vw[q] & 0xFFFF0000u), acc[2 * q + 1]);
            }
        }
        out[t * width16 + c] = make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]),
                                          pack_bf16x2(acc[4], acc[5]), pack_bf16x2(acc[6], acc[7]));
    }
}

}  // namespace b200moe

using namespace b200moe;

extern "C" int b200moe_silu_mul(const void* h, void* out, int64_t rows, int64_t inter, void* stream) {
    if (rows < 0 || inter <= 0 || (inter % 8) != 0) return B200MOE_ERR_SHAPE;
    if (rows == 0) return B200MOE_OK;
    if (!h || !out) return B200MOE_ERR_NULL_POINTER;
    if (!aligned16(h) || !aligned16(out)) return B200MOE_ERR_ALIGNMENT;
    const long long n = rows * (inter / 8);
    const long long blocks = (n + 255) / 256;
    if (blocks > 0x7FFFFFFFLL) return B200MOE_ERR_SHAPE;
    silu_mul_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint4*>(h), static_cast<uint4*>(out), rows, (int)(inter / 8));
    B200MOE_CUDA_TRY(cudaGetLastError());
    return B200MOE_OK;
}

extern "C" int b200moe_gather_rows(const void* src, const int32_t* index, void* dst, int64_t n_rows, int64_t width,
                                   void* stream) {
    if (n_rows < 0 || width <= 0 || (width % 8) != 0 || n_rows > 0x7FFFFFFFLL) return B200MOE_ERR_SHAPE;
    if (n_rows == 0) return B200MOE_OK;
    if (!src || !index || !dst) return B200MOE_ERR_NULL_POINTER;
    if (!aligned16(src) || !aligned16(dst)) return B200MOE_ERR_ALIGNMENT;
    gather_rows_kernel<<<(unsigned)n_rows, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint4*>(src), index, static_cast<uint4*>(dst), (int)(width / 8));
    B200MOE_CUDA_TRY(cudaGetLastError());
    return B200MOE_OK;
}

extern "C" int b200moe_combine(const void* y, const int32_t* slot, const float* weight, void* out, int64_t n_tokens,
                               int64_t top_k, int64_t width, void* stream) {
    if (n_tokens < 0 || top_k <= 0 || width <= 0 || (width % 8) != 0 || n_tokens > 0x7FFFFFFFLL)
        return B200MOE_ERR_SHAPE;
    if (n_tokens == 0) return B200MOE_OK;
    if (!y || !slot || !weight || !out) return B200MOE_ERR_NULL_POINTER;
    if (!aligned16(y) || !aligned16(out)) return B200MOE_ERR_ALIGNMENT;
    combine_kernel<<<(unsigned)n_tokens, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint4*>(y), slot, weight, static_cast<uint4*>(out), (int)top_k, (int)(width / 8));
    B200MOE_CUDA_TRY(cudaGetLastError());
    return B200MOE_OK;
}
