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

// dst[i, :] = src[index[i], :].  One warp per destination row at a time (grid-stride over rows); a lane keeps
// eight 16-byte loads in flight before the first store, and the next row's index is fetched while the current
// row is being copied: a copy kernel is bound by the bytes in flight, not by its instruction count.
constexpr int kRowUnroll = 8;

// kSum: also rowsum[i] = the fp32 sum of the row's elements, added up in the order of the grouped GEMM's own
// row-sum kernel (a lane takes the 16-byte chunks lane, lane + 32, ...; low + high element of each 32-bit word;
// then the xor-shuffle tree), so the bits are the ones that kernel would produce.
template <bool kSum>
__global__ void __launch_bounds__(256) gather_rows_kernel(const uint4* __restrict__ src, const int32_t* __restrict__ index,
                                                          uint4* __restrict__ dst, int width16, int n_rows,
                                                          float* __restrict__ rowsum) {
    const int lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
    const int n_warps = gridDim.x * wpb;
    int row = blockIdx.x * wpb + (threadIdx.x >> 5);
    long long from = row < n_rows ? __ldg(index + row) : 0;
    for (; row < n_rows; row += n_warps) {
        const uint4* s = src + from * width16;
        uint4* d = dst + (long long)row * width16;
        const int next = row + n_warps;
        if (next < n_rows) from = __ldg(index + next);
        float sum = 0.f;
        for (int c = lane; c < width16; c += 32 * kRowUnroll) {
            uint4 v[kRowUnroll];
#pragma unroll
            for (int u = 0; u < kRowUnroll; ++u)
                if (c + 32 * u < width16) v[u] = __ldg(s + c + 32 * u);
#pragma unroll
            for (int u = 0; u < kRowUnroll; ++u) {
                if (c + 32 * u < width16) {
                    d[c + 32 * u] = v[u];
                    if constexpr (kSum) {
                        const uint32_t w[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
                        for (int j = 0; j < 4; ++j) sum += __uint_as_float(w[j] << 16) + __uint_as_float(w[j] & 0xFFFF0000u);
                    }
                }
            }
        }
        if constexpr (kSum) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
            if (lane == 0) rowsum[row] = sum;
        }
    }
}

// out[t, :] = bf16(sum_j weight[t, j] * y[slot[t, j], :]) in fp32; one CTA per token.  The token's row indices
// and weights are read once into shared memory; a thread then has its top_k 16-byte loads of a column chunk
// in flight together.
constexpr int kCombineMaxK = 32;

__global__ void __launch_bounds__(256) combine_kernel(const uint4* __restrict__ y, const int32_t* __restrict__ slot,
                                                      const float* __restrict__ weight, uint4* __restrict__ out, int top_k,
                                                      int width16) {
    const long long t = blockIdx.x;
    __shared__ long long s_row[kCombineMaxK];
    __shared__ float s_w[kCombineMaxK];
    if ((int)threadIdx.x < top_k) {
        s_row[threadIdx.x] = (long long)slot[t * top_k + threadIdx.x] * width16;
        s_w[threadIdx.x] = weight[t * top_k + threadIdx.x];
    }
    __syncthreads();
    for (int c = threadIdx.x; c < width16; c += blockDim.x) {
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int j0 = 0; j0 < top_k; j0 += 8) {
            uint4 v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j)
                if (j0 + j < top_k) v[j] = __ldg(y + s_row[j0 + j] + c);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                if (j0 + j < top_k) {
                    const float w = s_w[j0 + j];
                    const uint32_t vw[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        acc[2 * q] = fmaf(w, __uint_as_float(vw[q] << 16), acc[2 * q]);
                        acc[2 * q + 1] = fmaf(w, __uint_as_float(vw[q] & 0xFFFF0000u), acc[2 * q + 1]);
                    }
                }
            }
        }
        out[t * width16 + c] = make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]),
                                          pack_bf16x2(acc[4], acc[5]), pack_bf16x2(acc[6], acc[7]));
    }
}

// ---- routing: softmax -> top-k -> renormalise, and the sort of (token, k) pairs by expert -------
// One warp per token.  The renormalised top-k weights of a softmax only need the k largest logits:
// w_i = exp(l_i - l_max) / sum_{j in top-k} exp(l_j - l_max).  Ties go to the lower expert index.
constexpr int kRouteMaxPerLane = 32;  // E <= 1024

__global__ void route_topk_kernel(const __nv_bfloat16* __restrict__ logits, int T, int E, int k,
                                  int32_t* __restrict__ idx, float* __restrict__ w, int32_t* __restrict__ hist) {
    const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (t >= T) return;
    float v[kRouteMaxPerLane];
    const int per = (E + 31) / 32;
#pragma unroll
    for (int i = 0; i < kRouteMaxPerLane; ++i) {
        const int e = i * 32 + lane;
        const float f = (i < per && e < E) ? __bfloat162float(logits[(size_t)t * E + e]) : -INFINITY;
        v[i] = f == f ? f : -INFINITY;  // a NaN logit ranks last instead of derailing the comparisons
    }
    float top0 = 0.f, denom = 0.f, mine = 0.f;
    int mine_idx = 0;
    for (int j = 0; j < k; ++j) {
        float best = -INFINITY;
        int bi = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < kRouteMaxPerLane; ++i) {
            const int e = i * 32 + lane;
            if (i < per && (v[i] > best || (v[i] == best && e < bi))) { best = v[i]; bi = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
        }
        if (j == 0) top0 = best;
        const float p = __expf(best - top0);
        denom += p;
        bi = bi < E ? bi : E - 1;  // unreachable with k <= E; keeps the histogram index in range regardless
        if (lane == j) { mine = p; mine_idx = bi; }
        if ((bi & 31) == lane) {
#pragma unroll
            for (int i = 0; i < kRouteMaxPerLane; ++i)
                if (i == (bi >> 5)) v[i] = -INFINITY;
        }
    }
    if (lane < k) {
        idx[(size_t)t * k + lane] = mine_idx;
        w[(size_t)t * k + lane] = mine / denom;
        atomicAdd(&hist[mine_idx], 1);
    }
}

// Single CTA: exclusive prefix of the per-expert histogram -> cursor[e] (start of expert e in the
// sorted order) and the int64 counts the grouped GEMM takes as group_list.
__global__ void route_prefix_kernel(const int32_t* __restrict__ hist, int E, int32_t* __restrict__ cursor,
                                    long long* __restrict__ counts64) {
    __shared__ int s[1024];
    const int e = threadIdx.x;
    const int c = e < E ? hist[e] : 0;
    s[e] = c;
    __syncthreads();
    for (int o = 1; o < 1024; o <<= 1) {
        const int add = e >= o ? s[e - o] : 0;
        __syncthreads();
        s[e] += add;
        __syncthreads();
    }
    if (e < E) {
        cursor[e] = s[e] - c;
        counts64[e] = c;
    }
}

// Every (token, j) pair takes the next free position of its expert.  Order inside an expert is
// arbitrary (rows are independent); slot[t, j] remembers where the pair went.
__global__ void route_scatter_kernel(const int32_t* __restrict__ idx, long long n_pairs, int k,
                                     int32_t* __restrict__ cursor, int32_t* __restrict__ token_of,
                                     int32_t* __restrict__ slot) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_pairs) return;
    const int pos = atomicAdd(&cursor[idx[i]], 1);
    token_of[pos] = (int32_t)(i / k);
    slot[i] = pos;
}

// Expert-parallel regroup: rows arrive ordered (source rank, local expert); the grouped GEMM wants
// them expert-major.  cnt[r, e] rows per block; pos[i] = expert-major position of received row i.
__global__ void regroup_index_kernel(const long long* __restrict__ cnt, int world, int e_local,
                                     int32_t* __restrict__ pos, int32_t* __restrict__ inv,
                                     long long* __restrict__ local_counts) {
    __shared__ int src_start[1024], em_start[1024], size[1024];
    const int nb = world * e_local;
    if (threadIdx.x == 0) {
        int acc = 0;
        for (int b = 0; b < nb; ++b) { size[b] = (int)cnt[b]; src_start[b] = acc; acc += size[b]; }
        acc = 0;
        for (int e = 0; e < e_local; ++e) {
            int tot = 0;
            for (int r = 0; r < world; ++r) { em_start[r * e_local + e] = acc; acc += size[r * e_local + e]; tot += size[r * e_local + e]; }
            local_counts[e] = tot;
        }
    }
    __syncthreads();
    for (int b = 0; b < nb; ++b) {
        const int s0 = src_start[b], d0 = em_start[b];
        for (int i = threadIdx.x; i < size[b]; i += blockDim.x) {
            pos[s0 + i] = d0 + i;
            inv[d0 + i] = s0 + i;
        }
    }
}

}  // namespace b200moe

using namespace b200moe;

extern "C" int b200moe_moe_route(const void* logits, int64_t n_tokens, int64_t n_experts, int64_t top_k, int32_t* idx,
                                 float* weight, int64_t* counts, int32_t* token_of, int32_t* slot, int32_t* scratch,
                                 void* stream) {
    if (n_tokens < 0 || n_experts <= 0 || n_experts > 1024 || top_k <= 0 || top_k > 32 || top_k > n_experts ||
        n_tokens * top_k > 0x7FFFFFF0LL)
        return B200MOE_ERR_SHAPE;
    if (!logits || !idx || !weight || !counts || !token_of || !slot || !scratch) return B200MOE_ERR_NULL_POINTER;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    int32_t* hist = scratch;
    int32_t* cursor = scratch + n_experts;
    B200MOE_CUDA_TRY(cudaMemsetAsync(hist, 0, sizeof(int32_t) * (size_t)n_experts, s));
    if (n_tokens > 0) {
        route_topk_kernel<<<(unsigned)((n_tokens + 7) / 8), 256, 0, s>>>(static_cast<const __nv_bfloat16*>(logits),
                                                                         (int)n_tokens, (int)n_experts, (int)top_k, idx,
                                                                         weight, hist);
        B200MOE_CUDA_TRY(cudaGetLastError());
    }
    route_prefix_kernel<<<1, 1024, 0, s>>>(hist, (int)n_experts, cursor, reinterpret_cast<long long*>(counts));
    B200MOE_CUDA_TRY(cudaGetLastError());
    const long long n_pairs = n_tokens * top_k;
    if (n_pairs > 0) {
        route_scatter_kernel<<<(unsigned)((n_pairs + 255) / 256), 256, 0, s>>>(idx, n_pairs, (int)top_k, cursor, token_of,
                                                                                slot);
        B200MOE_CUDA_TRY(cudaGetLastError());
    }
    return B200MOE_OK;
}

extern "C" int b200moe_moe_regroup_index(const int64_t* recv_counts, int64_t world, int64_t e_local, int32_t* pos,
                                         int32_t* inv, int64_t* local_counts, void* stream) {
    if (world <= 0 || e_local <= 0 || world * e_local > 1024) return B200MOE_ERR_SHAPE;
    if (!recv_counts || !pos || !inv || !local_counts) return B200MOE_ERR_NULL_POINTER;
    regroup_index_kernel<<<1, 1024, 0, static_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<const long long*>(recv_counts), (int)world, (int)e_local, pos, inv,
        reinterpret_cast<long long*>(local_counts));
    B200MOE_CUDA_TRY(cudaGetLastError());
    return B200MOE_OK;
}

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
    // eight warps per CTA, up to eight CTAs per SM: every warp copies a few rows
    const long long want = (n_rows + 7) / 8, cap = 8LL * sm_count();
    gather_rows_kernel<false><<<(unsigned)(want < cap ? want : cap), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint4*>(src), index, static_cast<uint4*>(dst), (int)(width / 8), (int)n_rows, nullptr);
    B200MOE_CUDA_TRY(cudaGetLastError());
    return B200MOE_OK;
}

extern "C" int b200moe_gather_rows_sum(const void* src, const int32_t* index, void* dst, float* rowsum, int64_t n_rows,
                                       int64_t width, void* stream) {
    if (n_rows < 0 || width <= 0 || (width % 8) != 0 || n_rows > 0x7FFFFFFFLL) return B200MOE_ERR_SHAPE;
    if (n_rows == 0) return B200MOE_OK;
    if (!src || !index || !dst || !rowsum) return B200MOE_ERR_NULL_POINTER;
    if (!aligned16(src) || !aligned16(dst)) return B200MOE_ERR_ALIGNMENT;
    const long long want = (n_rows + 7) / 8, cap = 8LL * sm_count();
    gather_rows_kernel<true><<<(unsigned)(want < cap ? want : cap), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint4*>(src), index, static_cast<uint4*>(dst), (int)(width / 8), (int)n_rows, rowsum);
    B200MOE_CUDA_TRY(cudaGetLastError());
    return B200MOE_OK;
}

extern "C" int b200moe_combine(const void* y, const int32_t* slot, const float* weight, void* out, int64_t n_tokens,
                               int64_t top_k, int64_t width, void* stream) {
    if (n_tokens < 0 || top_k <= 0 || top_k > kCombineMaxK || width <= 0 || (width % 8) != 0 || n_tokens > 0x7FFFFFFFLL)
        return B200MOE_ERR_SHAPE;
    if (n_tokens == 0) return B200MOE_OK;
    if (!y || !slot || !weight || !out) return B200MOE_ERR_NULL_POINTER;
    if (!aligned16(y) || !aligned16(out)) return B200MOE_ERR_ALIGNMENT;
    combine_kernel<<<(unsigned)n_tokens, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint4*>(y), slot, weight, static_cast<uint4*>(out), (int)top_k, (int)(width / 8));
    B200MOE_CUDA_TRY(cudaGetLastError());
    return B200MOE_OK;
}
