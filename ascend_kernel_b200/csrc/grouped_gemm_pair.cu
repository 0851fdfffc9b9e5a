// Antiquant grouped GEMM, CTA-pair variant: two CTAs on neighbouring SMs (a thread-block cluster
// of 2) compute one 256-row x 256-column output tile with tcgen05.mma.cta_group::2.
//
// Why a pair: with one CTA per tile the tensor core re-reads the whole 256-column bf16 weight tile
// from shared memory for every 128 rows, and the CTA has to dequantise all 256 columns itself; the
// shared-memory port and the CUDA-core dequant then bound the kernel, not the tensor core.  In a
// pair each CTA loads its own 128 rows of x, dequantises only ITS 128 weight columns, and the
// hardware feeds both tensor cores from both halves: per CTA and 64-k stage 16 KB of x arrive by
// TMA, 16 KB of bf16 weights are written by the dequant warps, 32 KB are read by the tensor core.
//
// Per CTA (24 warps):
//   warp 0      TMA producer of the CTA's x box (128 rows x 64 k, 128-byte swizzle) + L2 prefetch of
//               the packed weight tile further ahead
//   warp 2      TMEM allocation (both CTAs, collectively); in the leader CTA one lane issues the MMAs
//               for the pair and commits to the barriers of both CTAs (multicast commit)
//   warps 4-7   epilogue of the CTA's own 128 rows (accumulator double-buffered in TMEM: the
//               epilogue of tile i overlaps the main loop of tile i+1)
//   warps 8-23  dequant, two groups of 8 warps on alternate k-stages
// One ring of 6 stages, each holding the x box and the bf16 weight half-tile.  The "full" barrier
// of a stage lives in the leader CTA and collects both CTAs' TMA bytes and both CTAs' dequant
// warps (the peer's TMA names the leader's barrier, its warps arrive remotely); the "empty"
// barrier exists in both CTAs and is released by the leader's multicast commit.  All waits are bounded; on expiry a status word is set and every role
// of both CTAs winds down to the closing cluster barrier.
#include "common.cuh"
#include "gemm_args.cuh"
#include "ptx.cuh"

namespace b200moe {
namespace pair {

constexpr int kRowsCta = 128;          // rows of the tile owned by one CTA
constexpr int kTileM = 2 * kRowsCta;   // rows of the pair's tile
constexpr int kBN = 256, kBK = 64;
constexpr int kColsCta = kBN / 2;      // weight columns dequantised by one CTA
constexpr int kStages = 6;
constexpr int kPrefetch = 2;
constexpr int kL2Ahead = 8;
constexpr int kThreads = 768;
constexpr int kWarpTma = 0, kWarpMma = 2, kWarpEpi0 = 4, kWarpDq0 = 8;
constexpr int kDqGroups = 2, kDqGroupWarps = 8;
constexpr int kDqRowStep = 4 * kDqGroupWarps;  // a warp owns four k rows of the 128-column half
constexpr int kDqRows = kBK / kDqRowStep;
constexpr int kSuperRows = 8;
constexpr int kABytes = kRowsCta * kBK * 2;   // 16 KB
constexpr int kBBytes = kBK * kColsCta * 2;   // 16 KB
constexpr int kStageBytes = kABytes + kBBytes;
constexpr uint32_t kTmemCols = 512;

template <int MODE>
struct Traits {
    static constexpr bool kNibbles = (MODE == B200MOE_CT_FP4 || MODE == B200MOE_CT_INT4);
};

struct Shared {
    uint64_t full[kStages];       // leader only: TMA bytes and dequant warps of both CTAs
    uint64_t empty[kStages];      // multicast commit from the leader
    uint64_t t_full[2];           // multicast commit: accumulator ready
    uint64_t t_empty[2];          // leader only: epilogue warps of both CTAs
    uint64_t drain;
    uint32_t tmem_base;
    int abort;
    int n_tiles;
};

struct TileInfo {
    int g, row0, row_end, n0;
};

__device__ __noinline__ bool wait_slow(uint32_t bar, uint32_t parity, Shared* sh, int* status, int id, bool cluster) {
    volatile int* abort = &sh->abort;
    const uint64_t t0 = ptx::globaltimer_ns();
    uint32_t spins = 0;
    while (!(cluster ? ptx::mbar_try_wait_cluster(bar, parity) : ptx::mbar_try_wait(bar, parity))) {
        if ((++spins & 0xFF) == 0) {
            if (*abort) return false;
            if (ptx::globaltimer_ns() - t0 > ptx::kWaitLimitNs) {
                *abort = 1;
                if (status != nullptr) {
                    atomicCAS(status, kDevOk, kDevWaitExpired);
                    status[1] = id;
                }
                return false;
            }
        }
    }
    return true;
}
__device__ __forceinline__ bool wait(uint64_t* bar, uint32_t parity, Shared* sh, int* status, int id) {
    const uint32_t b = ptx::smem_u32(bar);
    if (ptx::mbar_try_wait(b, parity)) return true;
    return wait_slow(b, parity, sh, status, id, false);
}
__device__ __forceinline__ bool wait_cluster(uint64_t* bar, uint32_t parity, Shared* sh, int* status, int id) {
    const uint32_t b = ptx::smem_u32(bar);
    if (ptx::mbar_try_wait_cluster(b, parity)) return true;
    return wait_slow(b, parity, sh, status, id, true);
}

__device__ __forceinline__ TileInfo locate_tile(int t, const int* tile_prefix, const int* row_start, int G, int n_nt) {
    int lo = 0, hi = G;  // largest g with tile_prefix[g] <= t
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (tile_prefix[mid] <= t) lo = mid;
        else hi = mid;
    }
    const int g = lo;
    const int j = t - tile_prefix[g];
    const int r0 = row_start[g], r1 = row_start[g + 1];
    const int mt = (r1 - r0 + kTileM - 1) / kTileM;
    const int per_super = kSuperRows * n_nt;  // super-tiles keep x rows and the expert's weights in L2
    const int st = j / per_super;
    const int base = st * kSuperRows;
    const int h = min(kSuperRows, mt - base);
    const int jj = j - st * per_super;
    TileInfo ti;
    ti.g = g;
    ti.n0 = (jj / h) * kBN;
    ti.row0 = r0 + (base + jj % h) * kTileM;
    ti.row_end = r1;
    return ti;
}

struct StageIter {
    int t, kt;
    TileInfo ti;
    bool valid;
};
__device__ __forceinline__ void iter_start(StageIter& it, int first, int n_tiles, const int* tile_prefix,
                                           const int* row_start, int G, int n_nt) {
    it.t = first;
    it.kt = 0;
    it.valid = it.t < n_tiles;
    if (it.valid) it.ti = locate_tile(it.t, tile_prefix, row_start, G, n_nt);
}
__device__ __forceinline__ void iter_next(StageIter& it, int step, int n_kt, int n_tiles, const int* tile_prefix,
                                          const int* row_start, int G, int n_nt) {
    if (++it.kt < n_kt) return;
    it.kt = 0;
    it.t += step;
    it.valid = it.t < n_tiles;
    if (it.valid) it.ti = locate_tile(it.t, tile_prefix, row_start, G, n_nt);
}

// bf16 half-tile (MN-major, 128-byte swizzle): two blocks of 64 columns; inside a block row k
// occupies 128 bytes at k*128 and its eight 16-byte chunks are XOR-swizzled with (k & 7).
__device__ __forceinline__ uint32_t btile_offset(int k, int nchunk16) {  // nchunk16: 0..15
    return (uint32_t)((nchunk16 >> 3) * (kBK * 128) + k * 128 + (((nchunk16 & 7) ^ (k & 7)) << 4));
}

// A dequant warp owns four consecutive k rows of the 128-column half.  Each quarter-warp holds four
// lanes on an even row in one 64-column block and four lanes on the next row in the other block,
// so its 128-bit stores hit eight different 16-byte bank groups.
struct DqLane {
    int row;  // 0 .. kDqRowStep-1; the thread converts k = row + kDqRowStep * j, j < kDqRows
    int c16;  // 16-column chunk 0..7 of the CTA's half
};
__device__ __forceinline__ DqLane dq_lane(int tid) {
    const int w = tid >> 5, l = tid & 31;
    const int p = l >> 3, q = l & 7, odd = q >> 2;
    DqLane d;
    d.row = 4 * w + 2 * (p >> 1) + odd;
    d.c16 = 4 * ((p & 1) ^ odd) + (q & 3);
    return d;
}

struct PackedRegs {
    uint4 q[kDqRows];
};

template <int MODE>
__device__ __forceinline__ void load_packed(PackedRegs& r, const uint8_t* __restrict__ w, const GemmArgs& a,
                                            const TileInfo& ti, int kt, const DqLane& d, int col_base) {
    using T = Traits<MODE>;
    const size_t row_bytes = T::kNibbles ? (size_t)a.N / 2 : (size_t)a.N;
    const int col = ti.n0 + col_base + d.c16 * 16;
    const uint8_t* base = w + ((size_t)ti.g * a.K + (size_t)kt * kBK + d.row) * row_bytes + (T::kNibbles ? col >> 1 : col);
#pragma unroll
    for (int j = 0; j < kDqRows; ++j) {
        const uint8_t* p = base + (size_t)(kDqRowStep * j) * row_bytes;
        if constexpr (T::kNibbles) {
            const uint2 v = __ldg(reinterpret_cast<const uint2*>(p));
            r.q[j] = make_uint4(v.x, v.y, 0u, 0u);
        } else {
            r.q[j] = __ldg(reinterpret_cast<const uint4*>(p));
        }
    }
}

template <int MODE>
__device__ __forceinline__ void convert_stage(const PackedRegs& r, uint8_t* bt, const GemmArgs& a, const TileInfo& ti,
                                              int kt, const DqLane& d, int col_base) {
    const int c16 = d.c16;
    const int col = ti.n0 + col_base + c16 * 16;
    float sf = 1.f;
    if constexpr (MODE == B200MOE_CT_FP8) {
        sf = __ldg(static_cast<const float*>(a.scale) + ((size_t)ti.g * (a.K >> 7) + ((kt * kBK) >> 7)) * (a.N >> 7) +
                   (col >> 7));
    }
#pragma unroll
    for (int j = 0; j < kDqRows; ++j) {
        const int k = d.row + kDqRowStep * j;
        const uint4 q = r.q[j];
        uint32_t o[8];
        if constexpr (MODE == B200MOE_CT_INT8) {
            // tile columns 4i..4i+3 hold weight columns 4i, 4i+2, 4i+1, 4i+3 (undone in the epilogue)
            s8x4_to_bf16_even_odd(q.x, o[0], o[1]);
            s8x4_to_bf16_even_odd(q.y, o[2], o[3]);
            s8x4_to_bf16_even_odd(q.z, o[4], o[5]);
            s8x4_to_bf16_even_odd(q.w, o[6], o[7]);
        } else if constexpr (MODE == B200MOE_CT_FP8) {
            const uint32_t w4[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                float f[4];
#pragma unroll
                for (int b = 0; b < 4; ++b) {
                    const uint32_t p = prmt(w4[i], 0u, 0x0444u | (b << 12));
                    const uint32_t dd = ((p >> 4) & 0x07F00000u) | (p & 0x80000000u);
                    f[b] = (__uint_as_float(dd) * 1.329227995784916e36f) * sf;  // exact * 2^120, then fp32 scale
                }
                o[2 * i] = pack_bf16x2(f[0], f[1]);
                o[2 * i + 1] = pack_bf16x2(f[2], f[3]);
            }
        } else {  // FP4
            const uint4* sp = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(a.scale) +
                                                             ((size_t)ti.g * (a.K >> 4) + ((kt * kBK + k) >> 4)) * a.N + col);
            const uint4 s0 = __ldg(sp), s1 = __ldg(sp + 1);
            uint32_t v[4];
            e2m1x8_to_bf16(q.x, v);
            o[0] = mul_bf16x2(v[0], s0.x); o[1] = mul_bf16x2(v[1], s0.y);
            o[2] = mul_bf16x2(v[2], s0.z); o[3] = mul_bf16x2(v[3], s0.w);
            e2m1x8_to_bf16(q.y, v);
            o[4] = mul_bf16x2(v[0], s1.x); o[5] = mul_bf16x2(v[1], s1.y);
            o[6] = mul_bf16x2(v[2], s1.z); o[7] = mul_bf16x2(v[3], s1.w);
        }
        *reinterpret_cast<uint4*>(bt + btile_offset(k, 2 * c16)) = make_uint4(o[0], o[1], o[2], o[3]);
        *reinterpret_cast<uint4*>(bt + btile_offset(k, 2 * c16 + 1)) = make_uint4(o[4], o[5], o[6], o[7]);
    }
}

template <int MODE>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
grouped_gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
                         const uint8_t* __restrict__ weight, const GemmArgs a) {
    using T = Traits<MODE>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* ring = base;  // stage s: [x box 16 KB][bf16 weight half-tile 16 KB]
    Shared* sh = reinterpret_cast<Shared*>(ring + kStages * kStageBytes);
    int* row_start = reinterpret_cast<int*>(reinterpret_cast<uint8_t*>(sh) + 512);
    int* tile_prefix = row_start + (a.G + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = ptx::cluster_ctarank();  // 0 = leader
    const bool leader = rank == 0;
    const int pair_id = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const int n_nt = a.N / kBN;
    const int n_kt = a.K / kBK;
    const int col_base = (int)rank * kColsCta;  // this CTA's weight columns inside the tile

    load_row_starts(a.group_list, a.G, a.M, a.gl_type, row_start, leader ? a.status : nullptr);
    if (threadIdx.x == 0) {
        int acc = 0;
        tile_prefix[0] = 0;
        for (int g = 0; g < a.G; ++g) {
            acc += ((row_start[g + 1] - row_start[g] + kTileM - 1) / kTileM) * n_nt;
            tile_prefix[g + 1] = acc;
        }
        sh->n_tiles = acc;
        sh->abort = 0;
        for (int i = 0; i < kStages; ++i) {
            ptx::mbar_init(ptx::smem_u32(&sh->full[i]), 1 + 2 * kDqGroupWarps);
            ptx::mbar_init(ptx::smem_u32(&sh->empty[i]), 1);
        }
        for (int i = 0; i < 2; ++i) {
            ptx::mbar_init(ptx::smem_u32(&sh->t_full[i]), 1);
            ptx::mbar_init(ptx::smem_u32(&sh->t_empty[i]), 8);  // 4 epilogue warps of each CTA
        }
        ptx::mbar_init(ptx::smem_u32(&sh->drain), 1);
        ptx::fence_mbar_init();
        ptx::prefetch_tensormap(&tmap_x);
        ptx::prefetch_tensormap(&tmap_w);
    }
    if (warp == kWarpMma) {
        ptx::tmem_alloc_pair(ptx::smem_u32(&sh->tmem_base), kTmemCols);
        ptx::tmem_relinquish_pair();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::cluster_sync();  // both CTAs' barriers are initialised before any remote arrive / multicast commit
    ptx::tc_fence_after();

    const int n_tiles = sh->n_tiles;
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&sh->tmem_base);

    if (warp == kWarpTma) {
        // ------------------------------ x-box producer + L2 prefetch of weights ------------------------------
        if (lane == 0) {
            uint32_t s = 0, ph = 0, n = 0;
            bool ok = true;
            StageIter far;
            iter_start(far, pair_id, n_tiles, tile_prefix, row_start, a.G, n_nt);
            for (int i = 0; i < kL2Ahead && far.valid; ++i) {
                const int c = far.ti.n0 + col_base;
                ptx::tma_prefetch_l2_2d(&tmap_w, T::kNibbles ? c / 2 : c, far.ti.g * a.K + far.kt * kBK);
                iter_next(far, n_pairs, n_kt, n_tiles, tile_prefix, row_start, a.G, n_nt);
            }
            for (int t = pair_id; t < n_tiles && ok; t += n_pairs) {
                const TileInfo ti = locate_tile(t, tile_prefix, row_start, a.G, n_nt);
                for (int kt = 0; kt < n_kt; ++kt, ++n) {
                    if (n >= kStages && !wait(&sh->empty[s], ph ^ 1, sh, a.status, 10 + (int)s)) { ok = false; break; }
                    const uint32_t bar = ptx::smem_u32(&sh->full[s]);
                    if (leader) {
                        ptx::mbar_arrive_expect_tx(bar, 2 * kABytes);  // the x boxes of both CTAs
                        ptx::tma_load_2d(ptx::smem_u32(ring + s * kStageBytes), &tmap_x, bar, kt * kBK, ti.row0);
                    } else {
                        ptx::tma_load_2d_pair(ptx::smem_u32(ring + s * kStageBytes), &tmap_x, ptx::mapa(bar, 0), kt * kBK,
                                              ti.row0 + kRowsCta);
                    }
                    if (far.valid) {
                        const int c = far.ti.n0 + col_base;
                        ptx::tma_prefetch_l2_2d(&tmap_w, T::kNibbles ? c / 2 : c, far.ti.g * a.K + far.kt * kBK);
                        iter_next(far, n_pairs, n_kt, n_tiles, tile_prefix, row_start, a.G, n_nt);
                    }
                    if (++s == kStages) { s = 0; ph ^= 1; }
                }
            }
        }
    } else if (warp == kWarpMma) {
        // ------------------------------ leader CTA: MMA issue for the pair ------------------------------
        if (leader && lane == 0) {
            uint32_t idesc = ptx::umma_idesc_bf16(kTileM, kBN, true);
            // A: K-major, 8-row groups 1024 B apart, 32 B per 16 k inside the swizzle atom
            const uint64_t da0 = ptx::umma_desc_sw128(ptx::smem_u32(ring), 0, 1024);
            // B: MN-major, 64-column blocks kBK*128 B apart (LBO), 8-k groups 1024 B apart (SBO)
            const uint64_t db0 = ptx::umma_desc_sw128(ptx::smem_u32(ring + kABytes), kBK * 128, 1024);
            uint32_t s = 0, ph = 0, it = 0;
            bool ok = true;
            for (int t = pair_id; t < n_tiles && ok; t += n_pairs, ++it) {
                const uint32_t ab = it & 1, pht = (it >> 1) & 1;
                if (it >= 2 && !wait_cluster(&sh->t_empty[ab], pht ^ 1, sh, a.status, 30 + (int)ab)) { ok = false; break; }
                ptx::tc_fence_after();
                const uint32_t d_tmem = tmem_base + ab * kBN;
                uint32_t accumulate = 0;
                for (int kt = 0; kt < n_kt; ++kt) {
                    if (!wait_cluster(&sh->full[s], ph, sh, a.status, 40 + (int)s)) { ok = false; break; }
                    ptx::tc_fence_after();
                    const uint64_t off = (uint64_t)(s * (kStageBytes >> 4));
#pragma unroll
                    for (int k16 = 0; k16 < kBK / 16; ++k16) {
                        ptx::umma_bf16_pair(d_tmem, da0 + off + (uint64_t)(k16 * 2), db0 + off + (uint64_t)(k16 * 128), idesc,
                                            accumulate);
                        accumulate = 1;
                    }
                    ptx::umma_commit_pair(ptx::smem_u32(&sh->empty[s]), 3);
                    if (++s == kStages) { s = 0; ph ^= 1; }
                }
                if (ok) ptx::umma_commit_pair(ptx::smem_u32(&sh->t_full[ab]), 3);
            }
            // drain: every issued MMA must have completed before either CTA releases TMEM or exits
            ptx::umma_commit_pair(ptx::smem_u32(&sh->drain), 1);
            (void)ptx::mbar_wait(ptx::smem_u32(&sh->drain), 0);
        }
        __syncwarp();
    } else if (warp >= kWarpEpi0 && warp < kWarpEpi0 + 4) {
        // ------------------------------ epilogue of this CTA's 128 rows ------------------------------
        const int quarter = warp & 3;
        const bool per_channel = (MODE == B200MOE_CT_INT8);
        const bool has_offset = per_channel && a.offset != nullptr;
        uint32_t it = 0;
        for (int t = pair_id; t < n_tiles; t += n_pairs, ++it) {
            const TileInfo ti = locate_tile(t, tile_prefix, row_start, a.G, n_nt);
            const uint32_t ab = it & 1, pht = (it >> 1) & 1;
            if (!__all_sync(0xffffffffu, wait(&sh->t_full[ab], pht, sh, a.status, 60 + (int)ab))) break;
            ptx::tc_fence_after();
            const int row = ti.row0 + (int)rank * kRowsCta + quarter * 32 + lane;
            const bool row_ok = row < ti.row_end;
            const float rs = (has_offset && row_ok) ? __ldg(a.rowsum + row) : 0.f;
            __nv_bfloat16* yrow = a.y + (size_t)row * a.N + ti.n0;
#pragma unroll 1
            for (int c = 0; c < kBN / 32; ++c) {
                uint32_t r[32];
                ptx::tmem_ld_32x32(tmem_base + ab * kBN + c * 32 + ((uint32_t)(quarter * 32) << 16), r);
                float sv = 1.f, sov = 0.f;
                if (per_channel) {
                    const size_t ci = (size_t)ti.g * a.N + ti.n0 + c * 32 + lane;
                    sv = __bfloat162float(static_cast<const __nv_bfloat16*>(a.scale)[ci]);
                    if (has_offset) sov = sv * __bfloat162float(a.offset[ci]);
                }
                ptx::tmem_ld_wait();
                uint32_t o[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    // the int8 dequant stores columns (0,2,1,3) of every group of four
                    constexpr bool kPerm = (MODE == B200MOE_CT_INT8);
                    const int p0 = kPerm ? ((2 * j) & ~3) + (((2 * j) & 3) == 2 ? 1 : 0) : 2 * j;
                    const int p1 = kPerm ? ((2 * j) & ~3) + (((2 * j) & 3) == 2 ? 3 : 2) : 2 * j + 1;
                    float v0 = __uint_as_float(r[p0]), v1 = __uint_as_float(r[p1]);
                    if (per_channel) {
                        const float s0 = __shfl_sync(0xffffffffu, sv, 2 * j), s1 = __shfl_sync(0xffffffffu, sv, 2 * j + 1);
                        const float so0 = __shfl_sync(0xffffffffu, sov, 2 * j), so1 = __shfl_sync(0xffffffffu, sov, 2 * j + 1);
                        v0 = fmaf(so0, rs, s0 * v0);
                        v1 = fmaf(so1, rs, s1 * v1);
                    }
                    o[j] = pack_bf16x2(v0, v1);
                }
                if (row_ok) {
                    uint4* dst = reinterpret_cast<uint4*>(yrow + c * 32);
#pragma unroll
                    for (int q = 0; q < 4; ++q) dst[q] = make_uint4(o[4 * q], o[4 * q + 1], o[4 * q + 2], o[4 * q + 3]);
                }
            }
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive_cluster(ptx::mapa(ptx::smem_u32(&sh->t_empty[ab]), 0));
        }
    } else if (warp >= kWarpDq0) {
        // ------------------------------ dequant of this CTA's 128 weight columns ------------------------------
        const int dq_tid = threadIdx.x - kWarpDq0 * 32;
        const int grp = dq_tid / (kDqGroupWarps * 32);
        const DqLane d = dq_lane(dq_tid % (kDqGroupWarps * 32));
        StageIter cur, pf;
        iter_start(cur, pair_id, n_tiles, tile_prefix, row_start, a.G, n_nt);
        for (int i = 0; i < grp && cur.valid; ++i) iter_next(cur, n_pairs, n_kt, n_tiles, tile_prefix, row_start, a.G, n_nt);
        pf = cur;
        PackedRegs regs[kPrefetch];
#pragma unroll
        for (int u = 0; u < kPrefetch; ++u) {
            if (pf.valid) {
                load_packed<MODE>(regs[u], weight, a, pf.ti, pf.kt, d, col_base);
#pragma unroll
                for (int i = 0; i < kDqGroups; ++i)
                    if (pf.valid) iter_next(pf, n_pairs, n_kt, n_tiles, tile_prefix, row_start, a.G, n_nt);
            }
        }
        uint32_t ib = grp;
        bool ok = true;
        while (cur.valid && ok) {
#pragma unroll
            for (int u = 0; u < kPrefetch; ++u) {
                if (!cur.valid) break;
                const uint32_t s = ib % kStages, ph = (ib / kStages) & 1;
                bool got = true;
                if (ib >= kStages) got = wait(&sh->empty[s], ph ^ 1, sh, a.status, 80 + (int)s);
                if (!__all_sync(0xffffffffu, got)) { ok = false; break; }
                convert_stage<MODE>(regs[u], ring + s * kStageBytes + kABytes, a, cur.ti, cur.kt, d, col_base);
                ptx::fence_proxy_async_smem();  // generic-proxy writes -> visible to the tensor cores (async proxy)
                __syncwarp();
                if (lane == 0) {
                    if (leader) ptx::mbar_arrive(ptx::smem_u32(&sh->full[s]));
                    else ptx::mbar_arrive_cluster(ptx::mapa(ptx::smem_u32(&sh->full[s]), 0));
                }
                if (pf.valid) load_packed<MODE>(regs[u], weight, a, pf.ti, pf.kt, d, col_base);
#pragma unroll
                for (int i = 0; i < kDqGroups; ++i) {
                    if (pf.valid) iter_next(pf, n_pairs, n_kt, n_tiles, tile_prefix, row_start, a.G, n_nt);
                    if (cur.valid) iter_next(cur, n_pairs, n_kt, n_tiles, tile_prefix, row_start, a.G, n_nt);
                }
                ib += kDqGroups;
            }
        }
    }

    // Both CTAs stay until the pair is done: the leader's MMAs read the peer's shared memory and
    // remote arrivals must not target a CTA that has exited.
    ptx::tc_fence_before();
    __syncthreads();
    ptx::cluster_sync();
    if (warp == kWarpMma) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc_pair(tmem_base, kTmemCols);
    }
}

static size_t smem_bytes(int G) {
    return 1024 + (size_t)kStages * kStageBytes + 512 + sizeof(int) * 2 * (size_t)(G + 1);
}

template <int MODE>
static int launch(const void* x, const void* w, const GemmArgs& a, cudaStream_t stream) {
    using T = Traits<MODE>;
    CUtensorMap tx, tw;
    int rc = make_tensor_map_2d(&tx, x, 2, (uint64_t)a.M, a.K, kRowsCta, kBK, true);
    if (rc != B200MOE_OK) return rc;
    rc = make_tensor_map_2d(&tw, w, 1, (uint64_t)a.G * a.K, T::kNibbles ? a.N / 2 : a.N, kBK,
                            T::kNibbles ? kColsCta / 2 : kColsCta, false);
    if (rc != B200MOE_OK) return rc;
    const size_t smem = smem_bytes(a.G);
    B200MOE_CUDA_TRY(cudaFuncSetAttribute(grouped_gemm_pair_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          (int)smem));
    const int grid = sm_count() & ~1;
    grouped_gemm_pair_kernel<MODE><<<grid, kThreads, smem, stream>>>(tx, tw, static_cast<const uint8_t*>(w), a);
    B200MOE_CUDA_TRY(cudaGetLastError());
    return B200MOE_OK;
}

}  // namespace pair

int launch_grouped_gemm_pair(int mode, const void* x, const void* w, const GemmArgs& a, cudaStream_t stream) {
    switch (mode) {
        case B200MOE_CT_INT8: return pair::launch<B200MOE_CT_INT8>(x, w, a, stream);
        case B200MOE_CT_FP8: return pair::launch<B200MOE_CT_FP8>(x, w, a, stream);
        case B200MOE_CT_FP4: return pair::launch<B200MOE_CT_FP4>(x, w, a, stream);
        default: return B200MOE_ERR_UNSUPPORTED;
    }
}

}  // namespace b200moe
