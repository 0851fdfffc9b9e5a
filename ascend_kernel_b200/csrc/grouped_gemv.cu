// Grouped GEMV for decode-sized expert batches (HBM-bandwidth kernel).
//
// Work item = (non-empty expert, slab of 256 output columns); persistent CTAs take items with a
// static stride.  One producer thread streams the expert's weight slab through a 4-stage
// shared-memory ring with TMA (64 k-rows x 256 columns per stage, the matching 4 x 64 slice of x
// beside it); eight consumer warps decode the packed weights in registers (128-bit shared loads,
// in-register byte / nibble unpack), multiply by the fp32-widened x rows and keep fp32
// accumulators; partial sums of the 16 half-warps are combined with one warp shuffle and one
// pass through shared memory; scale/offset are applied in the fp32 epilogue and the result is
// rounded to bf16 once.  Experts with more than 4 rows are processed 4 rows at a time.
#include "common.cuh"
#include "ptx.cuh"

namespace b200moe {

constexpr int kGvSlabN = 256;
constexpr int kGvKT = 64;
constexpr int kGvStages = 4;
constexpr int kGvWarps = 8;  // consumer warps
constexpr int kGvThreads = (kGvWarps + 1) * 32;
constexpr int kGvRows = 4;  // x rows per pass
constexpr int kGvXTileBytes = kGvRows * kGvKT * 2;

struct GemvArgs {
    const void* scale;
    const __nv_bfloat16* offset;
    const int64_t* group_list;
    __nv_bfloat16* y;
    int M, K, N, G, gl_type;
    int* status;
};

template <int MODE>
struct GvTraits {
    // bytes of one packed weight row inside a slab
    static constexpr int kRowBytes = (MODE == B200MOE_CT_FP4 || MODE == B200MOE_CT_INT4) ? kGvSlabN / 2 : kGvSlabN;
    static constexpr int kTileBytes = kRowBytes * kGvKT;
};

// Shared-memory carve-up (dynamic): [barriers | flags][row_start G+1][active G][stages][red][redx]
struct GvSmem {
    uint64_t full[kGvStages];
    uint64_t empty[kGvStages];
    int n_active;
    int abort;
};

__device__ __forceinline__ bool gv_wait(uint32_t bar, uint32_t parity, volatile int* abort, int* status, int id) {
    if (*abort) return false;
    if (ptx::mbar_wait(bar, parity)) return true;
    *abort = 1;
    if (status != nullptr) {
        atomicCAS(status, kDevOk, kDevWaitExpired);
        status[1] = id;
    }
    return false;
}

// Decode the thread's 16 columns of one weight row into fp32.
template <int MODE>
__device__ __forceinline__ void gv_decode(const uint8_t* row_ptr, int l16, float (&wv)[16], const float* sc) {
    if constexpr (MODE == B200MOE_CT_INT8) {
        const uint4 q = *reinterpret_cast<const uint4*>(row_ptr + l16 * 16);
        const uint32_t w4[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t u = w4[i] ^ 0x80808080u;  // biased byte: value + 128
#pragma unroll
            for (int b = 0; b < 4; ++b)
                wv[4 * i + b] = __uint_as_float(prmt(u, 0x4B000000u, 0x7440u | b)) - 8388736.0f;
        }
    } else if constexpr (MODE == B200MOE_CT_FP8) {
        const uint4 q = *reinterpret_cast<const uint4*>(row_ptr + l16 * 16);
        const uint32_t w4[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                // e4m3 bits moved under the fp32 exponent: value * 2^-120 (subnormals included)
                const uint32_t p = prmt(w4[i], 0u, 0x0444u | (b << 12));  // byte b -> bits 31..24
                const uint32_t d = ((p >> 4) & 0x07F00000u) | (p & 0x80000000u);
                wv[4 * i + b] = __uint_as_float(d) * 1.329227995784916e36f;  // 2^120
            }
        }
    } else {  // FP4: 8 bytes = 16 codes
        const uint2 q = *reinterpret_cast<const uint2*>(row_ptr + l16 * 8);
        const uint32_t w2[2] = {q.x, q.y};
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            uint32_t o[4];
            e2m1x8_to_bf16(w2[i], o);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                wv[8 * i + 2 * j] = __uint_as_float(o[j] << 16) * sc[8 * i + 2 * j];
                wv[8 * i + 2 * j + 1] = __uint_as_float(o[j] & 0xFFFF0000u) * sc[8 * i + 2 * j + 1];
            }
        }
    }
}

template <int MODE, int MB>
__device__ __forceinline__ void gv_consume(const GemvArgs& a, GvSmem* sm, uint8_t* stages, float* red, float* redx,
                                           uint32_t& it, int g, int r0, int rows_valid, int n0) {
    using T = GvTraits<MODE>;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int half = lane >> 4, l16 = lane & 15;
    const int unit = 2 * warp + half;  // 0..15, owns k rows 4*unit .. 4*unit+3 of every stage
    const int n_kt = a.K / kGvKT;
    const bool has_offset = (MODE == B200MOE_CT_INT8) && a.offset != nullptr;

    float acc[MB][16];
    float xsum[MB];
#pragma unroll
    for (int m = 0; m < MB; ++m) {
        xsum[m] = 0.f;
#pragma unroll
        for (int c = 0; c < 16; ++c) acc[m][c] = 0.f;
    }

    for (int kt = 0; kt < n_kt; ++kt, ++it) {
        const uint32_t s = it % kGvStages, ph = (it / kGvStages) & 1;
        if (!gv_wait(ptx::smem_u32(&sm->full[s]), ph, &sm->abort, a.status, 100 + (int)s)) break;
        const uint8_t* wt = stages + s * (T::kTileBytes + kGvXTileBytes);
        const __nv_bfloat16* xt = reinterpret_cast<const __nv_bfloat16*>(wt + T::kTileBytes);

        float xv[MB][4];
#pragma unroll
        for (int m = 0; m < MB; ++m) {
            const uint2 q = *reinterpret_cast<const uint2*>(xt + m * kGvKT + 4 * unit);
            xv[m][0] = __uint_as_float(q.x << 16);
            xv[m][1] = __uint_as_float(q.x & 0xFFFF0000u);
            xv[m][2] = __uint_as_float(q.y << 16);
            xv[m][3] = __uint_as_float(q.y & 0xFFFF0000u);
        }
        float sc[16];
        if constexpr (MODE == B200MOE_CT_FP8) {
            const int kb = (kt * kGvKT) >> 7, nb = (n0 + l16 * 16) >> 7;
            const float sf = __ldg(static_cast<const float*>(a.scale) +
                                   ((size_t)g * (a.K >> 7) + kb) * (a.N >> 7) + nb);
#pragma unroll
            for (int m = 0; m < MB; ++m)
#pragma unroll
                for (int j = 0; j < 4; ++j) xv[m][j] *= sf;
        } else if constexpr (MODE == B200MOE_CT_FP4) {
            const int kg = (kt * kGvKT + 4 * unit) >> 4;
            const uint4* sp = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(a.scale) +
                                                             ((size_t)g * (a.K >> 4) + kg) * a.N + n0 + l16 * 16);
            const uint4 s0 = __ldg(sp), s1 = __ldg(sp + 1);
            const uint32_t sw[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                sc[2 * i] = __uint_as_float(sw[i] << 16);
                sc[2 * i + 1] = __uint_as_float(sw[i] & 0xFFFF0000u);
            }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float wv[16];
            gv_decode<MODE>(wt + (4 * unit + j) * T::kRowBytes, l16, wv, sc);
#pragma unroll
            for (int m = 0; m < MB; ++m)
#pragma unroll
                for (int c = 0; c < 16; ++c) acc[m][c] = fmaf(xv[m][j], wv[c], acc[m][c]);
        }
        if (has_offset) {
#pragma unroll
            for (int m = 0; m < MB; ++m) xsum[m] += (xv[m][0] + xv[m][1]) + (xv[m][2] + xv[m][3]);
        }
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&sm->empty[s]));
    }

    // ---- combine the 16 partial sums per column -------------------------------------------------
#pragma unroll
    for (int m = 0; m < MB; ++m)
#pragma unroll
        for (int c = 0; c < 16; ++c) acc[m][c] += __shfl_xor_sync(0xffffffffu, acc[m][c], 16);
    if (half == 0) {
#pragma unroll
        for (int m = 0; m < MB; ++m) {
            float4* dst = reinterpret_cast<float4*>(red + ((warp * kGvRows + m) * kGvSlabN) + l16 * 16);
#pragma unroll
            for (int c = 0; c < 4; ++c)
                dst[c] = make_float4(acc[m][4 * c], acc[m][4 * c + 1], acc[m][4 * c + 2], acc[m][4 * c + 3]);
        }
    }
    if (l16 == 0) {
#pragma unroll
        for (int m = 0; m < MB; ++m) redx[unit * kGvRows + m] = xsum[m];
    }
    asm volatile("bar.sync 1, %0;" ::"n"(kGvWarps * 32) : "memory");
    if (!sm->abort) {
        const int t = threadIdx.x;  // column inside the slab
        const int n = n0 + t;
        float s_n = 1.f, so_n = 0.f;
        if constexpr (MODE == B200MOE_CT_INT8) {
            s_n = __bfloat162float(static_cast<const __nv_bfloat16*>(a.scale)[(size_t)g * a.N + n]);
            if (has_offset) so_n = s_n * __bfloat162float(a.offset[(size_t)g * a.N + n]);
        }
#pragma unroll
        for (int m = 0; m < MB; ++m) {
            if (m < rows_valid) {
                float v = 0.f;
#pragma unroll
                for (int w = 0; w < kGvWarps; ++w) v += red[(w * kGvRows + m) * kGvSlabN + t];
                if constexpr (MODE == B200MOE_CT_INT8) {
                    float xs = 0.f;
                    if (has_offset) {
#pragma unroll
                        for (int u = 0; u < 2 * kGvWarps; ++u) xs += redx[u * kGvRows + m];
                    }
                    v = fmaf(so_n, xs, s_n * v);
                }
                a.y[(size_t)(r0 + m) * a.N + n] = __float2bfloat16_rn(v);
            }
        }
    }
    asm volatile("bar.sync 1, %0;" ::"n"(kGvWarps * 32) : "memory");
}

template <int MODE>
__global__ void __maxnreg__(112)
grouped_gemv_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                    const GemvArgs a) {
    using T = GvTraits<MODE>;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    GvSmem* sm = reinterpret_cast<GvSmem*>(smem_raw);
    int* row_start = reinterpret_cast<int*>(smem_raw + 128);
    int* active = row_start + (a.G + 1);
    uintptr_t p = reinterpret_cast<uintptr_t>(active + a.G);
    p = (p + 1023) & ~uintptr_t(1023);
    uint8_t* stages = reinterpret_cast<uint8_t*>(p);
    float* red = reinterpret_cast<float*>(stages + kGvStages * (T::kTileBytes + kGvXTileBytes));
    float* redx = red + kGvWarps * kGvRows * kGvSlabN;

    load_row_starts(a.group_list, a.G, a.M, a.gl_type, row_start, a.status);
    if (threadIdx.x == 0) {
        int n = 0;
        for (int g = 0; g < a.G; ++g)
            if (row_start[g + 1] > row_start[g]) active[n++] = g;
        sm->n_active = n;
        sm->abort = 0;
        for (int s = 0; s < kGvStages; ++s) {
            ptx::mbar_init(ptx::smem_u32(&sm->full[s]), 1);
            ptx::mbar_init(ptx::smem_u32(&sm->empty[s]), kGvWarps);
        }
        ptx::fence_mbar_init();
        ptx::prefetch_tensormap(&tmap_w);
        ptx::prefetch_tensormap(&tmap_x);
    }
    __syncthreads();

    const int n_slabs = a.N / kGvSlabN;
    const int n_items = sm->n_active * n_slabs;
    const int n_kt = a.K / kGvKT;
    const int warp = threadIdx.x >> 5;
    uint32_t it = 0;

    if (warp == kGvWarps) {
        // ---------------- producer ----------------
        if ((threadIdx.x & 31) == 0) {
            bool ok = true;
            for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
                const int g = active[item / n_slabs];
                const int n0 = (item % n_slabs) * kGvSlabN;
                const int r0 = row_start[g], r1 = row_start[g + 1];
                for (int r = r0; r < r1 && ok; r += kGvRows) {
                    for (int kt = 0; kt < n_kt; ++kt, ++it) {
                        const uint32_t s = it % kGvStages, ph = (it / kGvStages) & 1;
                        if (it >= kGvStages &&
                            !gv_wait(ptx::smem_u32(&sm->empty[s]), ph ^ 1, &sm->abort, a.status, 200 + (int)s)) {
                            ok = false;
                            break;
                        }
                        const uint32_t bar = ptx::smem_u32(&sm->full[s]);
                        const uint32_t dst = ptx::smem_u32(stages + s * (T::kTileBytes + kGvXTileBytes));
                        ptx::mbar_arrive_expect_tx(bar, T::kTileBytes + kGvXTileBytes);
                        ptx::tma_load_2d(dst, &tmap_w, bar, n0 * T::kRowBytes / kGvSlabN, g * a.K + kt * kGvKT);
                        ptx::tma_load_2d(dst + T::kTileBytes, &tmap_x, bar, kt * kGvKT, r);
                    }
                }
            }
            if (!ok) {
                // wind down: give copies still in flight a bounded time to land before exiting
                const uint32_t issued = it;
                for (uint32_t j = (issued > kGvStages ? issued - kGvStages : 0); j < issued; ++j)
                    (void)ptx::mbar_wait(ptx::smem_u32(&sm->full[j % kGvStages]), (j / kGvStages) & 1);
            }
        }
    } else {
        // ---------------- consumers ----------------
        for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
            const int g = active[item / n_slabs];
            const int n0 = (item % n_slabs) * kGvSlabN;
            const int r0 = row_start[g], r1 = row_start[g + 1];
            for (int r = r0; r < r1; r += kGvRows) {
                const int rows = min(kGvRows, r1 - r);
                if (rows == 1) gv_consume<MODE, 1>(a, sm, stages, red, redx, it, g, r, rows, n0);
                else if (rows == 2) gv_consume<MODE, 2>(a, sm, stages, red, redx, it, g, r, rows, n0);
                else gv_consume<MODE, 4>(a, sm, stages, red, redx, it, g, r, rows, n0);
                if (sm->abort) break;
            }
            if (sm->abort) break;
        }
    }
}

template <int MODE>
static size_t gv_smem_bytes(int G) {
    using T = GvTraits<MODE>;
    size_t b = 128 + sizeof(int) * (size_t)(2 * G + 1);
    b = (b + 1023) / 1024 * 1024 + 1024;  // slack for the 1024-byte alignment of the stage ring
    b += (size_t)kGvStages * (T::kTileBytes + kGvXTileBytes);
    b += sizeof(float) * (kGvWarps * kGvRows * kGvSlabN + 2 * kGvWarps * kGvRows);
    return b;
}

template <int MODE>
static int gv_launch(const void* x, const void* w, const GemvArgs& a, cudaStream_t stream) {
    using T = GvTraits<MODE>;
    CUtensorMap tw, tx;
    const bool packed = T::kRowBytes != kGvSlabN;
    int rc = make_tensor_map_2d(&tw, w, 1, (uint64_t)a.G * a.K, packed ? a.N / 2 : a.N, kGvKT, T::kRowBytes, false);
    if (rc != B200MOE_OK) return rc;
    rc = make_tensor_map_2d(&tx, x, 2, (uint64_t)a.M, a.K, kGvRows, kGvKT, false);
    if (rc != B200MOE_OK) return rc;
    const size_t smem = gv_smem_bytes<MODE>(a.G);
    B200MOE_CUDA_TRY(cudaFuncSetAttribute(grouped_gemv_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          (int)smem));
    const int grid = 2 * sm_count();
    grouped_gemv_kernel<MODE><<<grid, kGvThreads, smem, stream>>>(tw, tx, a);
    B200MOE_CUDA_TRY(cudaGetLastError());
    return B200MOE_OK;
}

}  // namespace b200moe

using namespace b200moe;

extern "C" size_t b200moe_grouped_gemv_workspace_bytes(int64_t, int64_t K, int64_t N, int64_t G, int compute_type,
                                                       int weight_layout) {
    size_t b = B200MOE_STATUS_BYTES;
    if (compute_type == B200MOE_CT_FP4 && weight_layout == B200MOE_LAYOUT_ASCEND)
        b += (size_t)G * (size_t)K * (size_t)(N / 2);  // canonical copy of the pre-shuffled weights
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
    if ((K % kGvKT) != 0 || (N % kGvSlabN) != 0) return B200MOE_ERR_SHAPE;
    if (compute_type == B200MOE_CT_FP8 && ((K % 128) != 0 || (N % 128) != 0)) return B200MOE_ERR_SHAPE;
    if (compute_type == B200MOE_CT_INT4) return B200MOE_ERR_UNSUPPORTED;
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
    a.scale = scale;
    a.offset = static_cast<const __nv_bfloat16*>(offset);
    a.group_list = group_list;
    a.y = static_cast<__nv_bfloat16*>(y);
    a.M = (int)M; a.K = (int)K; a.N = (int)N; a.G = (int)G;
    a.gl_type = group_list_type;
    a.status = static_cast<int*>(workspace);

    const void* w = weight;
    if (compute_type == B200MOE_CT_FP4 && weight_layout == B200MOE_LAYOUT_ASCEND) {
        void* canon = static_cast<uint8_t*>(workspace) + B200MOE_STATUS_BYTES;
        int rc = b200moe_fp4_layout(weight, canon, G, K, N, 0, stream);
        if (rc != B200MOE_OK) return rc;
        w = canon;
    }
    switch (compute_type) {
        case B200MOE_CT_INT8: return gv_launch<B200MOE_CT_INT8>(x, w, a, s);
        case B200MOE_CT_FP8: return gv_launch<B200MOE_CT_FP8>(x, w, a, s);
        default: return gv_launch<B200MOE_CT_FP4>(x, w, a, s);
    }
}
