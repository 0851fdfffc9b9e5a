// Antiquant grouped GEMM for prefill-sized expert batches: persistent, warp-specialised
// tcgen05 / TMEM kernel fed by TMA (sm_100a).
//
//   y[rows of expert g] = bf16( x[rows of expert g] @ dequant(W[g]) ),  fp32 accumulation in TMEM.
//
// One CTA per SM draws output tiles of up to 256 rows x 256 columns from a global ticket counter:
// two UMMA 128x256x16 instructions (rows 0-127 and 128-255 of the tile, one TMEM accumulator of
// 256 columns each) share every dequantised weight stage, so the CUDA-core dequant work per
// tensor-core flop is half that of a 128-row tile; tiles with at most 128 rows issue one.  The
// tile list is derived inside the kernel from the device-side group_list (prefix sum over the
// experts' tile counts kept in shared memory, binary search per tile), so there is no host
// synchronisation and no schedule in global memory.
//
// Warp roles (28 warps):
//   warp 0      TMA producer of x tiles (one or two boxes of 128 rows x 64 k, bf16, 128-byte
//               swizzle, K-major A) and L2 prefetch of the packed weight tiles further ahead
//   warp 2      TMEM allocation + tcgen05.mma issue (one elected lane)
//   warps 4-11  epilogue, four warps per accumulator: tcgen05.ld, scale/offset in fp32, bf16 stores
//   warps 12-27 dequant, two groups of 8 warps taking alternate k-stages: packed weights global ->
//               registers (128-bit coalesced loads, prefetched two of the group's stages ahead) ->
//               bf16 tile in the UMMA MN-major 128-byte-swizzle layout
// One ring of 3 stages (x boxes 32 KB + bf16 weights 32 KB), one full and one empty barrier per
// stage: the single MMA-issuing thread pays one wait and one commit per stage.  Shared-memory bandwidth bounds this kernel (the
// tensor core alone reads 48 KB per 64-k stage), so packed weights go through registers, not
// through a shared-memory staging ring, and the bf16 tile is written without bank conflicts.
// Weights never make a round trip through global memory.  Every wait is bounded; on expiry the
// kernel records an error status, all roles wind down, copies in flight are given time to land
// and TMEM is released.
#include <mutex>

#include "common.cuh"
#include "gemm_args.cuh"
#include "ptx.cuh"

namespace b200moe {

constexpr int kBM = 128, kBN = 256, kBK = 64;
constexpr int kTileM = 2 * kBM;  // rows of an output tile (two MMA row halves)
constexpr int kNS = 3;  // ring stages, each an x stage (32 KB) and a bf16 weight stage (32 KB); int4: 2 stages of 32 + 2 x 32 KB
constexpr int kPrefetch = 2;  // packed stages held in registers ahead of the one being converted
constexpr int kL2Ahead = 8;   // stages by which the L2 prefetch of packed weights leads the x-tile loads
constexpr int kGemmThreads = 896;
constexpr int kWarpA = 0, kWarpMma = 2, kWarpEpi0 = 4, kEpiWarps = 8, kWarpDq0 = 12;
// The dequant warps form kDqGroups groups; group i converts the k-stages i, i + kDqGroups, ...
// so a warp pays the barrier handshake once per kDqGroups stages and the groups overlap each
// other's waits.
constexpr int kDqGroups = 2;
constexpr int kDqGroupWarps = 8;
constexpr int kDqRows = kBK / (2 * kDqGroupWarps);  // k rows converted by a thread per stage
constexpr int kDqRowStep = 2;                        // distance between a thread's rows
constexpr int kDqWarpRows = 2 * kDqRows;             // a warp owns this many consecutive k rows
constexpr int kSuperRows = 8;  // m-tiles per L2 super-tile
// Published tiles a role may lag behind the publisher: the publisher leads the x loads by kL2Ahead
// stages, those lead the MMAs by the ring depth, the epilogue trails by at most two tiles; with one
// stage per tile that is kL2Ahead + kNS + 2 tiles.
constexpr int kTileRing = 32;
constexpr int kBarrierBytes = 512;  // shared memory reserved for GmBarriers
constexpr int kEpiScaleFloats = 2 * kBN;  // per epilogue warp: the tile's column scales and scale * offset
constexpr int kAHalfBytes = kBM * kBK * 2;   // one 128-row box
constexpr int kATileBytes = 2 * kAHalfBytes;  // an x stage holds both row halves
constexpr int kSmallRows = 32;                 // rows of the small x box (a nearly empty last row half)
constexpr int kSmallBytes = kSmallRows * kBK * 2;
constexpr int kBTileBytes = kBK * kBN * 2;
constexpr uint32_t kTmemCols = 512;

// Internal kernel mode: fp4 weights in the stored ("ascend") order, read as they are.  In that order a
// 64-row x 128-byte tile of the canonical matrix is still a 64 x 128-byte box of the same 2-D array
// (row = (b*4 + a)*8 + p, 128 bytes = [q (4)][c8 (8)][4 bytes], for canonical row 16a + 8b + c8 and
// byte column 128j + 16p + 4q + s), so tensor maps and strides are those of the canonical layout
// and only the thread -> data assignment of the dequant warps changes: a thread takes 8 rows x 8
// columns (two 16-byte loads) instead of 4 rows x 16 columns.
constexpr int kCtFp4Ascend = 16;

template <int MODE>
struct GmTraits {
    static constexpr bool kNibbles = (MODE == B200MOE_CT_FP4 || MODE == B200MOE_CT_INT4 || MODE == kCtFp4Ascend);
    // int4 with per-128-k scale/offset: (w + o) * s does not fit bf16, so every k block is fed to
    // the tensor core twice -- a stage carries two weight tiles, hi = bf16(v) and lo = bf16(v - hi),
    // multiplied with the same x block; the fp32 accumulator then holds x @ v to about 2^-16 relative.
    static constexpr int kParts = (MODE == B200MOE_CT_INT4) ? 2 : 1;
    // ring depth: 3 x (32 + 32 KB) or 2 x (32 + 64 KB), 192 KB either way
    static constexpr int kStages = (kParts == 1) ? kNS : 2;
    static constexpr int kPRowBytes = kNibbles ? kBN / 2 : kBN;
    static constexpr int kPTileBytes = kPRowBytes * kBK;
    // bf16 weights need no conversion: TMA writes the 64-column blocks of the weight tile straight
    // into the B ring (a 64 k x 128-byte box with the 128-byte swizzle is exactly one block of the
    // MN-major operand layout) and the dequant warps have nothing to do
    static constexpr bool kDirect = (MODE == B200MOE_CT_BF16);
};

struct GmBarriers {
    uint64_t full[kNS];   // TMA bytes of the x boxes + the dequant warps of the stage's group
    uint64_t empty[kNS];  // one tcgen05.commit per stage
    // accumulator hand-off, one pair per 256-column accumulator: a two-half tile uses both, a one-half
    // tile alternates between them so that its epilogue overlaps the next tile's main loop
    uint64_t t_full[2], t_empty[2];
    uint64_t drain;
    uint32_t tmem_base;
    int abort;
    int n_tiles;
    int pad;
    // Tile schedule of this CTA: tiles are drawn from a global ticket counter (status word 2) by the
    // thread that runs furthest ahead and published here, entry i % kTileRing = (i + 1) << 32 | tile.
    // Every role walks the entries in order, so all see the same sequence.
    unsigned long long tile_ring[kTileRing];
};

struct TileInfo {
    int g, row0, row_end, n0;
    int halves;  // 1: at most 128 rows in the tile, 2: more
};

// Bounded wait on a pipeline barrier.  The fast path is a single try_wait; the slow path polls,
// notices an abort raised by another role and gives up after ptx::kWaitLimitNs.
__device__ __noinline__ bool gm_wait_slow(uint32_t bar, uint32_t parity, GmBarriers* sb, int* status, int id) {
    volatile int* abort = &sb->abort;
    const uint64_t t0 = ptx::globaltimer_ns();
    uint32_t spins = 0;
    while (!ptx::mbar_try_wait(bar, parity)) {
        if ((++spins & 0xFF) == 0) {
            if (*abort) return false;
            if (ptx::globaltimer_ns() - t0 > ptx::kWaitLimitNs) {
                *abort = 1;
                report_status(status, kDevWaitExpired, id);
                return false;
            }
        }
    }
    return true;
}
__device__ __forceinline__ bool gm_wait(uint64_t* bar, uint32_t parity, GmBarriers* sb, int* status, int id) {
    const uint32_t b = ptx::smem_u32(bar);
    if (ptx::mbar_try_wait(b, parity)) return true;
    return gm_wait_slow(b, parity, sb, status, id);
}

// tile index -> expert, first row, row bound, first column.  tile_prefix has G+1 entries.
// The seq-th tile of this CTA (seq counts from 0 and is advanced), or n_tiles when the schedule has
// ended, a wait expired or another role aborted.  The publisher is always far ahead, so outside the
// first microseconds of the kernel the entry is already there.
__device__ __forceinline__ int next_tile(GmBarriers* sb, uint32_t& seq, int n_tiles, int* status) {
    const volatile unsigned long long* e = &sb->tile_ring[seq % kTileRing];
    const uint32_t want = seq + 1;
    unsigned long long v = *e;
    if ((uint32_t)(v >> 32) != want) {
        volatile int* abort = &sb->abort;
        const uint64_t t0 = ptx::globaltimer_ns();
        uint32_t spins = 0;
        while ((uint32_t)((v = *e) >> 32) != want) {
            if ((++spins & 0xFF) == 0) {
                if (*abort) return n_tiles;
                if (ptx::globaltimer_ns() - t0 > ptx::kWaitLimitNs) {
                    *abort = 1;
                    report_status(status, kDevWaitExpired, 90);
                    return n_tiles;
                }
            }
        }
    }
    ++seq;
    const int t = (int)(uint32_t)v;
    return t < n_tiles ? t : n_tiles;
}

// Tile numbering: first every tile with two row halves (more than 128 rows), expert by expert in
// super-tiles, then every tile with one row half (the last, short m-tile of an expert).  tile_prefix
// holds two prefix arrays of G + 1 entries each: two-half tiles before expert g, one-half tiles
// before expert g.
__device__ __forceinline__ TileInfo locate_tile(int t, const int* tile_prefix, const int* row_start, int G, int n_nt) {
    const int n_two = tile_prefix[G];
    const bool two = t < n_two;
    const int* pref = two ? tile_prefix : tile_prefix + (G + 1);
    const int tt = two ? t : t - n_two;
    int lo = 0, hi = G;  // largest g with pref[g] <= tt
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (pref[mid] <= tt) lo = mid;
        else hi = mid;
    }
    const int g = lo;
    const int j = tt - pref[g];
    const int r0 = row_start[g], r1 = row_start[g + 1];
    TileInfo ti;
    ti.g = g;
    ti.row_end = r1;
    if (two) {
        const int mt = (pref[g + 1] - pref[g]) / n_nt;
        // super-tiles of up to kSuperRows m-tiles x all n-tiles keep x rows and the expert's weights
        // L2-resident while they are shared by concurrently running CTAs
        const int per_super = kSuperRows * n_nt;
        const int st = j / per_super;
        const int base = st * kSuperRows;
        const int h = min(kSuperRows, mt - base);
        const int jj = j - st * per_super;
        ti.n0 = (jj / h) * kBN;
        ti.row0 = r0 + (base + jj % h) * kTileM;
        ti.halves = 2;
    } else {
        ti.n0 = j * kBN;
        ti.row0 = r0 + ((r1 - r0) / kTileM) * kTileM;
        ti.halves = 1;
    }
    return ti;
}

// ---- dequant of one packed stage into the bf16 UMMA tile --------------------------------------
// bf16 tile layout (MN-major, 128-byte swizzle): four blocks of 64 columns; inside a block row k
// occupies 128 bytes at k*128 and its eight 16-byte chunks are XOR-swizzled with (k & 7).
__device__ __forceinline__ uint32_t btile_offset(int k, int nchunk16) {  // nchunk16: 16-byte chunk 0..31
    return (uint32_t)((nchunk16 >> 3) * (kBK * 128) + k * 128 + (((nchunk16 & 7) ^ (k & 7)) << 4));
}

// Thread -> (row, 16-column chunk) assignment of the dequant warps.  A warp owns kDqWarpRows
// consecutive k rows (inside one 16-row scale group of the fp4 format) and converts them two at a
// time (an even one and the next).  Each quarter-warp holds four lanes on the even row in
// 64-column block p and four lanes on the odd row in block p^1: the 128-bit stores of a quarter
// then hit eight different 16-byte bank groups (the swizzle term k&7 differs in its low bit
// between the two rows), and the packed loads of a warp still cover both rows contiguously.
struct DqLane {
    int row;  // the thread converts k = row + kDqRowStep * j, j < kDqRows, of its stages
    int c16;  // 16-column chunk 0..15
    // stored-order fp4 only: the thread converts canonical rows k0 .. k0 + 7, columns 8 * chunk .. + 7
    int k0, chunk, src_row, src_byte;  // where its 32 bytes start inside the 64 x 128-byte box
};
template <int MODE>
__device__ __forceinline__ DqLane dq_lane(int tid) {
    const int w = tid >> 5, l = tid & 31;
    DqLane d;
    if constexpr (MODE == kCtFp4Ascend) {
        const int a = w >> 1, b = w & 1;      // warp <-> rows 16a + 8b .. + 7 (one 16-row scale group)
        d.k0 = 16 * a + 8 * b;
        d.chunk = l;                          // lane <-> 16-byte chunk of the bf16 tile row (8 columns)
        d.src_row = (b * 4 + a) * 8 + (l >> 2);
        d.src_byte = (l & 3) * 32;
        d.row = d.src_row;                    // what dq_locate adds to the stage's first row
        d.c16 = 0;
    } else {
        const int p = l >> 3, q = l & 7, odd = q >> 2;
        d.row = kDqWarpRows * w + odd;
        d.c16 = 4 * (p ^ odd) + (q & 3);
        d.k0 = d.chunk = d.src_row = d.src_byte = 0;
    }
    return d;
}

// Packed weights of one stage held by a thread: kDqRows rows x 16 columns.
template <int MODE>
struct PackedRegs {
    uint4 q[kDqRows];  // fp4 / int4 use only .x/.y of each
    uint4 s[2];        // fp4 only: the bf16 scales of the thread's 16 columns (one 16-row group)
    float sf;          // fp8 only: the fp32 scale of the thread's 128 x 128 block
};

// Position of a dequant thread in the (tile, k-stage) sequence of its CTA, with the address of the
// thread's first packed row of that stage carried along (advanced by a constant inside a tile).
struct DqIter {
    int t, kt, g, n0;
    uint32_t seq;  // tiles taken from the CTA's schedule so far
    bool valid;
    const uint8_t* wp;
};
template <int MODE>
__device__ __forceinline__ void dq_locate(DqIter& it, const uint8_t* __restrict__ w, const GemmArgs& a, const DqLane& d,
                                          int n_tiles, const int* tile_prefix, const int* row_start, int n_nt) {
    using T = GmTraits<MODE>;
    it.valid = it.t < n_tiles;
    if (!it.valid) return;
    const TileInfo ti = locate_tile(it.t, tile_prefix, row_start, a.G, n_nt);
    it.g = ti.g;
    it.n0 = ti.n0;
    const size_t row_bytes = T::kNibbles ? (size_t)a.N / 2 : (size_t)a.N;
    it.wp = w + ((size_t)ti.g * a.K + (size_t)it.kt * kBK + d.row) * row_bytes +
            (MODE == kCtFp4Ascend ? (ti.n0 >> 1) + d.src_byte
             : T::kNibbles        ? (ti.n0 >> 1) + d.c16 * 8
                                  : ti.n0 + d.c16 * 16);
}
template <int MODE>
__device__ __forceinline__ void dq_advance(DqIter& it, int step, const uint8_t* __restrict__ w, const GemmArgs& a,
                                           const DqLane& d, int n_kt, int n_tiles, const int* tile_prefix,
                                           const int* row_start, int n_nt, GmBarriers* sb) {
    using T = GmTraits<MODE>;
    it.kt += step;
    if (it.kt < n_kt) {
        it.wp += (size_t)step * kBK * (T::kNibbles ? (size_t)a.N / 2 : (size_t)a.N);
        return;
    }
    do {
        it.kt -= n_kt;
        it.t = next_tile(sb, it.seq, n_tiles, a.status);
    } while (it.kt >= n_kt && it.t < n_tiles);
    dq_locate<MODE>(it, w, a, d, n_tiles, tile_prefix, row_start, n_nt);
}

template <int MODE>
__device__ __forceinline__ void load_packed(PackedRegs<MODE>& r, const DqIter& it, const GemmArgs& a, const DqLane& d) {
    using T = GmTraits<MODE>;
    if constexpr (MODE == kCtFp4Ascend) {
        // 32 consecutive bytes = rows c8 = 0..7 of the thread's 8 columns, 4 bytes each; one scale
        // vector (8 columns of the rows' 16-row group)
        r.q[0] = __ldg(reinterpret_cast<const uint4*>(it.wp));
        r.q[1] = __ldg(reinterpret_cast<const uint4*>(it.wp + 16));
        r.s[0] = __ldg(reinterpret_cast<const uint4*>(
            static_cast<const __nv_bfloat16*>(a.scale) +
            ((size_t)it.g * (a.K >> 4) + ((it.kt * kBK + d.k0) >> 4)) * a.N + it.n0 + d.chunk * 8));
        return;
    }
    const size_t row_bytes = T::kNibbles ? (size_t)a.N / 2 : (size_t)a.N;
#pragma unroll
    for (int j = 0; j < kDqRows; ++j) {
        const uint8_t* p = it.wp + (size_t)(kDqRowStep * j) * row_bytes;
        if constexpr (T::kNibbles) {
            const uint2 v = __ldg(reinterpret_cast<const uint2*>(p));
            r.q[j] = make_uint4(v.x, v.y, 0u, 0u);
        } else if (MODE != B200MOE_CT_FP8 || it.n0 + d.c16 * 16 < a.N) {
            r.q[j] = __ldg(reinterpret_cast<const uint4*>(p));
        } else {
            r.q[j] = make_uint4(0u, 0u, 0u, 0u);  // columns past N in the 128-column last tile of an fp8 matrix
        }
    }
    if constexpr (MODE == B200MOE_CT_FP8) {
        r.sf = it.n0 + d.c16 * 16 < a.N
                   ? __ldg(static_cast<const float*>(a.scale) + ((size_t)it.g * (a.K >> 7) + ((it.kt * kBK) >> 7)) * (a.N >> 7) +
                           ((it.n0 + d.c16 * 16) >> 7))
                   : 0.f;
    }
    if constexpr (MODE == B200MOE_CT_FP4) {
        const uint4* sp = reinterpret_cast<const uint4*>(
            static_cast<const __nv_bfloat16*>(a.scale) +
            ((size_t)it.g * (a.K >> 4) + ((it.kt * kBK + d.row) >> 4)) * a.N + it.n0 + d.c16 * 16);
        r.s[0] = __ldg(sp);
        r.s[1] = __ldg(sp + 1);
    }
}

// 16-byte shared-memory store at a 32-bit shared address.
__device__ __forceinline__ void sts128(uint32_t addr, uint32_t x, uint32_t y, uint32_t z, uint32_t w) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}
// Shared address of the thread's chunk pair in its row j, from the address `sa` of the pair in its
// row 0: the thread's rows are k = row0 + 2j with row0 & 7 in {0, 1}, so the swizzle term changes by
// XOR with 2j (bits 5..6 of the address) and the row offset by j * 256 bytes.  The second chunk of
// the pair is at the returned address ^ 16.
__device__ __forceinline__ uint32_t dq_row_addr(uint32_t sa, int j) { return (sa ^ (uint32_t)(j << 5)) + (uint32_t)(j * 256); }

// Stored-order fp4: eight rows of eight columns; `sa` is the shared address of the thread's chunk in
// its first row (a multiple of 8, so row i flips the chunk's swizzle bits by i and adds i * 128).
__device__ __forceinline__ void convert_stage_fp4_ascend(const PackedRegs<kCtFp4Ascend>& r, uint32_t sa) {
    const uint4 sc = r.s[0];
    const uint32_t w8[8] = {r.q[0].x, r.q[0].y, r.q[0].z, r.q[0].w, r.q[1].x, r.q[1].y, r.q[1].z, r.q[1].w};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        uint32_t v[4];
        e2m1x8_to_bf16(w8[i], v);
        sts128((sa ^ (uint32_t)(i << 4)) + (uint32_t)(i * 128), mul_bf16x2(v[0], sc.x), mul_bf16x2(v[1], sc.y),
               mul_bf16x2(v[2], sc.z), mul_bf16x2(v[3], sc.w));
    }
}

template <int MODE>
__device__ __forceinline__ void convert_stage(const PackedRegs<MODE>& r, uint32_t sa) {
    const float sf = (MODE == B200MOE_CT_FP8) ? r.sf : 1.f;
    const f32x2 sf2 = pack_f32x2(sf, sf);
#pragma unroll
    for (int j = 0; j < kDqRows; ++j) {
        const uint4 q = r.q[j];
        uint32_t o[8];
        if constexpr (MODE == B200MOE_CT_INT8) {
            // tile columns 4i..4i+3 hold weight columns 4i, 4i+2, 4i+1, 4i+3 (undone in the epilogue)
            s8x4_to_bf16_even_odd(q.x, o[0], o[1]);
            s8x4_to_bf16_even_odd(q.y, o[2], o[3]);
            s8x4_to_bf16_even_odd(q.z, o[4], o[5]);
            s8x4_to_bf16_even_odd(q.w, o[6], o[7]);
        } else if constexpr (MODE == B200MOE_CT_FP8) {
            // e4m3 byte -> bf16 with the 4 exponent and 3 mantissa bits placed under the bf16 exponent
            // (exact after * 2^120, subnormals included), two values per instruction; widened to fp32,
            // scaled with the block's fp32 scale and rounded once to bf16.
            const uint32_t w4[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
#pragma unroll
                for (int hp = 0; hp < 2; ++hp) {
                    const uint32_t t = prmt(w4[i], 0u, hp == 0 ? 0x1404u : 0x3424u);
                    const uint32_t xb = ((t >> 4) & 0x07F007F0u) | (t & 0x80008000u);
                    const uint32_t yb = mul_bf16x2(xb, 0x7B807B80u);  // * 2^120
                    const f32x2 f = mul_f32x2(pack_u32x2(yb << 16, yb & 0xFFFF0000u), sf2);
                    o[2 * i + hp] = pack_bf16x2(f32x2_lo(f), f32x2_hi(f));
                }
            }
        } else {  // FP4: 8 bytes = 16 codes; the thread's rows share one 16-row scale group
            const uint4 s0 = r.s[0], s1 = r.s[1];
            uint32_t v[4];
            e2m1x8_to_bf16(q.x, v);
            o[0] = mul_bf16x2(v[0], s0.x); o[1] = mul_bf16x2(v[1], s0.y);
            o[2] = mul_bf16x2(v[2], s0.z); o[3] = mul_bf16x2(v[3], s0.w);
            e2m1x8_to_bf16(q.y, v);
            o[4] = mul_bf16x2(v[0], s1.x); o[5] = mul_bf16x2(v[1], s1.y);
            o[6] = mul_bf16x2(v[2], s1.z); o[7] = mul_bf16x2(v[3], s1.w);
        }
        const uint32_t aj = dq_row_addr(sa, j);
        sts128(aj, o[0], o[1], o[2], o[3]);
        sts128(aj ^ 16u, o[4], o[5], o[6], o[7]);
    }
}

// int4 with per-128-k scale / offset: one pass over a k block produces both stages it feeds to the
// tensor core, hi = bf16(v) and lo = bf16(v - hi) with v = w * s + o * s in fp32.  The thread's
// rows lie in the same 128-k group, so its 16 scales and offsets are loaded once per k block
// (before the wait for the stage, so that their latency is hidden by it).
struct Int4Scales {
    uint4 s[2], o[2];
};
__device__ __forceinline__ Int4Scales load_int4_scales(const GemmArgs& a, int g, int n0, int kb, const DqLane& d) {
    const size_t so = ((size_t)g * (a.K >> 7) + ((kb * kBK) >> 7)) * a.N + n0 + d.c16 * 16;
    const uint4* sp = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(a.scale) + so);
    Int4Scales r;
    r.s[0] = __ldg(sp);
    r.s[1] = __ldg(sp + 1);
    if (a.offset != nullptr) {
        const uint4* op = reinterpret_cast<const uint4*>(a.offset + so);
        r.o[0] = __ldg(op);
        r.o[1] = __ldg(op + 1);
    } else {
        r.o[0] = r.o[1] = make_uint4(0u, 0u, 0u, 0u);
    }
    return r;
}

__device__ __forceinline__ void convert_block_int4(const PackedRegs<B200MOE_CT_INT4>& r, const Int4Scales& sc,
                                                   uint32_t sa_hi, uint32_t sa_lo) {
    const f32x2 kMagic = pack_f32x2(8388616.0f, 8388616.0f);  // 2^23 + 8
#pragma unroll
    for (int h = 0; h < 2; ++h) {  // columns 8h .. 8h+7: one 16-byte chunk of the bf16 tile per row
        const uint32_t sw[4] = {sc.s[h].x, sc.s[h].y, sc.s[h].z, sc.s[h].w};
        const uint32_t ow[4] = {sc.o[h].x, sc.o[h].y, sc.o[h].z, sc.o[h].w};
        uint32_t lo_n[kDqRows], hi_n[kDqRows];
#pragma unroll
        for (int j = 0; j < kDqRows; ++j) {
            const uint32_t word = (h == 0 ? r.q[j].x : r.q[j].y) ^ 0x88888888u;  // nibble + 8, unsigned
            lo_n[j] = word & 0x0F0F0F0Fu;         // even columns, one per byte
            hi_n[j] = (word >> 4) & 0x0F0F0F0Fu;  // odd columns
        }
        uint32_t hi[kDqRows][4], lo[kDqRows][4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {  // column pair 8h + 2i, 8h + 2i + 1 = byte i of the word
            const f32x2 s2 = pack_f32x2(__uint_as_float(sw[i] << 16), __uint_as_float(sw[i] & 0xFFFF0000u));
            const f32x2 t2 = mul_f32x2(pack_f32x2(__uint_as_float(ow[i] << 16), __uint_as_float(ow[i] & 0xFFFF0000u)), s2);
#pragma unroll
            for (int j = 0; j < kDqRows; ++j) {
                // byte i under the fp32 pattern of 2^23: the float 2^23 + nibble + 8
                const f32x2 wm = pack_u32x2(prmt(lo_n[j], 0x4B000000u, 0x7440u + i), prmt(hi_n[j], 0x4B000000u, 0x7440u + i));
                const f32x2 v = fma_f32x2(sub_f32x2(wm, kMagic), s2, t2);
                const uint32_t hh = pack_bf16x2(f32x2_lo(v), f32x2_hi(v));
                hi[j][i] = hh;
                const f32x2 l = sub_f32x2(v, pack_u32x2(hh << 16, hh & 0xFFFF0000u));
                lo[j][i] = pack_bf16x2(f32x2_lo(l), f32x2_hi(l));
            }
        }
#pragma unroll
        for (int j = 0; j < kDqRows; ++j) {
            sts128(dq_row_addr(sa_hi, j) ^ (uint32_t)(h << 4), hi[j][0], hi[j][1], hi[j][2], hi[j][3]);
            sts128(dq_row_addr(sa_lo, j) ^ (uint32_t)(h << 4), lo[j][0], lo[j][1], lo[j][2], lo[j][3]);
        }
    }
}

// Position of the x producer's L2 prefetch in the (tile, k-stage) sequence of its CTA.
struct StageIter {
    int t, kt;
    TileInfo ti;
    bool valid;
};

// SILU (int8 only): the weight columns come as blocks of 128 gate columns followed by the 128 up
// columns of the same indices, and the epilogue writes bf16(silu(gate) * up), [M, N/2], instead of
// the [M, N] product (gate and up are rounded to bf16 first, as the unfused operators would).
template <int MODE, bool SILU>
__global__ void __launch_bounds__(kGemmThreads, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_xs,
                    const __grid_constant__ CUtensorMap tmap_w, const uint8_t* __restrict__ weight, const GemmArgs a) {
    using T = GmTraits<MODE>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* a_ring = base;
    constexpr int NS = T::kStages, P = T::kParts;
    uint8_t* b_ring = a_ring + NS * kATileBytes;
    GmBarriers* sb = reinterpret_cast<GmBarriers*>(b_ring + NS * P * kBTileBytes);
    static_assert(sizeof(GmBarriers) <= kBarrierBytes, "barrier block");
    float* epi_scale = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(sb) + kBarrierBytes);
    int* row_start = reinterpret_cast<int*>(epi_scale + kEpiWarps * kEpiScaleFloats);
    int* tile_prefix = row_start + (a.G + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_nt = (a.N + kBN - 1) / kBN;  // (fp8 only: the last tile may hold 128 columns)
    const int n_kt = a.K / kBK;  // stages per tile

    load_row_starts(a.group_list, a.G, a.M, a.gl_type, row_start, a.status);
    if (threadIdx.x == 0) {
        int acc = 0, acc1 = 0;
        int* pref1 = tile_prefix + (a.G + 1);
        tile_prefix[0] = 0;
        pref1[0] = 0;
        for (int g = 0; g < a.G; ++g) {
            const int rows = row_start[g + 1] - row_start[g], tail = rows % kTileM;
            acc += (rows / kTileM + (tail > kBM ? 1 : 0)) * n_nt;    // tiles with two row halves
            acc1 += ((tail >= 1 && tail <= kBM) ? 1 : 0) * n_nt;      // the short last m-tile, if any
            tile_prefix[g + 1] = acc;
            pref1[g + 1] = acc1;
        }
        acc += acc1;
        sb->n_tiles = acc;
        sb->abort = 0;
        for (int i = 0; i < kTileRing; ++i) sb->tile_ring[i] = 0ull;
        for (int i = 0; i < NS; ++i) {
            ptx::mbar_init(ptx::smem_u32(&sb->full[i]), T::kDirect ? 1 : 1 + kDqGroupWarps);
            ptx::mbar_init(ptx::smem_u32(&sb->empty[i]), 1);
        }
        for (int i = 0; i < 2; ++i) {
            ptx::mbar_init(ptx::smem_u32(&sb->t_full[i]), 1);
            ptx::mbar_init(ptx::smem_u32(&sb->t_empty[i]), kEpiWarps / 2);
        }
        ptx::mbar_init(ptx::smem_u32(&sb->drain), 1);
        ptx::fence_mbar_init();
        ptx::prefetch_tensormap(&tmap_x);
        ptx::prefetch_tensormap(&tmap_xs);
        ptx::prefetch_tensormap(&tmap_w);
    }
    if (warp == kWarpMma) {
        ptx::tmem_alloc(ptx::smem_u32(&sb->tmem_base), kTmemCols);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();

    const int n_tiles = sb->n_tiles;
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&sb->tmem_base);

    if (warp == kWarpA) {
        // ------------------------------ x-tile producer ------------------------------
        // Also pulls the packed weight tile of the stage kL2Ahead further on into L2 (a TMA
        // prefetch has no shared-memory destination), so the dequant warps' register loads, which
        // can only run a stage or two ahead, find their data in L2 instead of waiting on HBM.
        if (lane == 0) {
            uint32_t ia = 0, seq = 0, published = 0;
            bool ok = true;
            // This thread runs furthest ahead (its L2 prefetch leads everything else), so it draws the
            // tiles.  One ticket is always held in hand, so the atomic's latency is off the path.
            int* ticket = a.status + 2;  // zeroed by the host before the launch
            int held = atomicAdd(ticket, 1);
            auto publish = [&]() -> int {
                const int t = held < n_tiles ? held : n_tiles;
                *reinterpret_cast<volatile unsigned long long*>(&sb->tile_ring[published % kTileRing]) =
                    ((unsigned long long)(published + 1) << 32) | (uint32_t)t;
                ++published;
                if (t < n_tiles) held = atomicAdd(ticket, 1);
                return t;
            };
            StageIter far;
            far.t = publish();
            far.kt = 0;
            far.valid = far.t < n_tiles;
            if (far.valid) far.ti = locate_tile(far.t, tile_prefix, row_start, a.G, n_nt);
            auto far_step = [&]() {
                if constexpr (!T::kDirect)
                    ptx::tma_prefetch_l2_2d(&tmap_w, T::kNibbles ? far.ti.n0 / 2 : far.ti.n0, far.ti.g * a.K + far.kt * kBK);
                if (++far.kt < n_kt) return;
                far.kt = 0;
                far.t = publish();
                far.valid = far.t < n_tiles;
                if (far.valid) far.ti = locate_tile(far.t, tile_prefix, row_start, a.G, n_nt);
            };
            for (int i = 0; i < kL2Ahead && far.valid; ++i) far_step();
            for (;;) {
                const int t = next_tile(sb, seq, n_tiles, a.status);
                if (t >= n_tiles || !ok) break;
                const TileInfo ti = locate_tile(t, tile_prefix, row_start, a.G, n_nt);
                // The last row half of a tile often holds only a few rows of the expert (a second half
                // of a dozen rows when an expert has a little over 128): a box of kSmallRows rows then
                // replaces the 128-row box.  The MMA still reads 128 rows; what the rows beyond the box
                // hold is left over from earlier stages and lands in accumulator rows that are never
                // stored.
                const int last_rows = ti.row_end - (ti.row0 + (ti.halves - 1) * kBM);
                const bool small_last = last_rows <= kSmallRows;
                const uint32_t stage_bytes = (uint32_t)((ti.halves - 1) * kAHalfBytes + (small_last ? kSmallBytes : kAHalfBytes));
                const CUtensorMap* last_map = small_last ? &tmap_xs : &tmap_x;
                for (int kt = 0; kt < n_kt; ++kt, ++ia) {
                    const uint32_t s = ia % NS, ph = (ia / NS) & 1;
                    if (ia >= NS && !gm_wait(&sb->empty[s], ph ^ 1, sb, a.status, 10 + (int)s)) { ok = false; break; }
                    const uint32_t bar = ptx::smem_u32(&sb->full[s]);
                    const int kx = kt * kBK;
                    ptx::mbar_arrive_expect_tx(bar, stage_bytes + (T::kDirect ? (uint32_t)kBTileBytes : 0u));
                    if constexpr (T::kDirect) {
#pragma unroll
                        for (int blk = 0; blk < kBN / 64; ++blk)
                            ptx::tma_load_2d(ptx::smem_u32(b_ring + s * kBTileBytes + blk * (kBK * 128)), &tmap_w, bar,
                                             ti.n0 + blk * 64, ti.g * a.K + kx);
                    }
                    if (ti.halves == 2) {
                        ptx::tma_load_2d(ptx::smem_u32(a_ring + s * kATileBytes), &tmap_x, bar, kx, ti.row0);
                        ptx::tma_load_2d(ptx::smem_u32(a_ring + s * kATileBytes + kAHalfBytes), last_map, bar, kx,
                                         ti.row0 + kBM);
                    } else {
                        ptx::tma_load_2d(ptx::smem_u32(a_ring + s * kATileBytes), last_map, bar, kx, ti.row0);
                    }
                    if (far.valid) far_step();
                }
            }
            if (!ok)
                for (uint32_t j = (ia > NS ? ia - NS : 0); j < ia; ++j)
                    (void)ptx::mbar_wait(ptx::smem_u32(&sb->full[j % NS]), (j / NS) & 1);
        }
    } else if (warp == kWarpMma) {
        // ------------------------------ MMA issuer ------------------------------
        // One thread feeds the tensor core; its per-stage instruction count bounds the MMA rate, so
        // ring positions and parities are carried incrementally and the shared-memory descriptors
        // are a 64-bit base plus a small stage / k offset.
        if (lane == 0) {
            const uint32_t idesc = ptx::umma_idesc_bf16(kBM, kBN, true);
            // A: K-major, 8-row groups 1024 B apart, 32 B per 16 k inside the swizzle atom
            const uint64_t da0 = ptx::umma_desc_sw128(ptx::smem_u32(a_ring), 0, 1024);
            // B: MN-major, 64-column blocks kBK*128 B apart (LBO), 8-k groups 1024 B apart (SBO)
            const uint64_t db0 = ptx::umma_desc_sw128(ptx::smem_u32(b_ring), kBK * 128, 1024);
            uint32_t sa = 0, pha = 0;
            uint32_t uses[2] = {0, 0}, next1 = 0;
            bool ok = true;
            uint32_t seq = 0;
            for (;;) {
                const int t = next_tile(sb, seq, n_tiles, a.status);
                if (t >= n_tiles || !ok) break;
                const TileInfo ti = locate_tile(t, tile_prefix, row_start, a.G, n_nt);
                // accumulators of this tile: both for two halves, else the one used less recently;
                // the epilogue of their previous tile must have drained them
                const uint32_t b0 = ti.halves == 2 ? 0u : next1, b1 = ti.halves == 2 ? 2u : next1 + 1u;
                if (ti.halves == 1) next1 ^= 1u;
                for (uint32_t b = b0; b < b1 && ok; ++b)
                    if (uses[b] >= 1 && !gm_wait(&sb->t_empty[b], (uses[b] - 1) & 1, sb, a.status, 30 + (int)b)) ok = false;
                if (!ok) break;
                const uint32_t acc0 = tmem_base + b0 * kBN;
                ptx::tc_fence_after();
                uint32_t accumulate = 0;
                for (int kt = 0; kt < n_kt; ++kt) {
                    if (!gm_wait(&sb->full[sa], pha, sb, a.status, 40 + (int)sa)) { ok = false; break; }
                    ptx::tc_fence_after();
                    const uint64_t da = da0 + (uint64_t)(sa * (kATileBytes >> 4));
#pragma unroll
                    for (int p = 0; p < P; ++p) {  // int4: the hi tile, then the lo tile, against the same x stage
                        const uint64_t db = db0 + (uint64_t)((sa * P + p) * (kBTileBytes >> 4));
#pragma unroll
                        for (int k16 = 0; k16 < kBK / 16; ++k16)
                            ptx::umma_bf16(acc0, da + (uint64_t)(k16 * 2), db + (uint64_t)(k16 * 128), idesc,
                                           accumulate | (uint32_t)(k16 + p));
                        if (ti.halves == 2) {
#pragma unroll
                            for (int k16 = 0; k16 < kBK / 16; ++k16)
                                ptx::umma_bf16(acc0 + kBN, da + (uint64_t)((kAHalfBytes >> 4) + k16 * 2),
                                               db + (uint64_t)(k16 * 128), idesc, accumulate | (uint32_t)(k16 + p));
                        }
                    }
                    accumulate = 1;
                    ptx::umma_commit(ptx::smem_u32(&sb->empty[sa]));
                    if (++sa == NS) { sa = 0; pha ^= 1; }
                }
                if (ok)
                    for (uint32_t b = b0; b < b1; ++b) {
                        ptx::umma_commit(ptx::smem_u32(&sb->t_full[b]));
                        ++uses[b];
                    }
            }
            // drain: every issued MMA must have completed before TMEM is released
            ptx::umma_commit(ptx::smem_u32(&sb->drain));
            (void)ptx::mbar_wait(ptx::smem_u32(&sb->drain), 0);
        }
        __syncwarp();
    } else if (warp >= kWarpEpi0 && warp < kWarpEpi0 + kEpiWarps) {
        // ------------------------------ epilogue ------------------------------
        const int quarter = warp & 3;                 // TMEM lanes 32*quarter .. +31 are the ones this warp may read
        const int grp = (warp - kWarpEpi0) >> 2;      // which accumulator this warp drains
        const bool per_channel = (MODE == B200MOE_CT_INT8);
        const bool has_offset = per_channel && a.offset != nullptr;
        uint32_t use = 0, next1 = 0, seq = 0;
        for (;;) {
            const int t = next_tile(sb, seq, n_tiles, a.status);
            if (t >= n_tiles) break;
            const TileInfo ti = locate_tile(t, tile_prefix, row_start, a.G, n_nt);
            // a two-half tile: this group takes row half `grp`; a one-half tile sits in one accumulator
            bool mine = true;
            int half = grp;
            if (ti.halves == 1) {
                mine = (int)next1 == grp;
                half = 0;
                next1 ^= 1u;
            }
            if (!mine) continue;
            // int8: every thread needs the scale (and scale * offset) of all 256 columns of the tile; the
            // warp stages them in its own shared-memory strip while the tile is still being accumulated
            float* es = epi_scale + (warp - kWarpEpi0) * kEpiScaleFloats;
            if (per_channel) {
                const size_t c0 = (size_t)ti.g * a.N + ti.n0;
#pragma unroll
                for (int i = 0; i < kBN / 32; ++i) {
                    const int col = i * 32 + lane;
                    const float sv = __bfloat162float(static_cast<const __nv_bfloat16*>(a.scale)[c0 + col]);
                    es[col] = sv;
                    es[kBN + col] = has_offset ? sv * __bfloat162float(a.offset[c0 + col]) : 0.f;
                }
                __syncwarp();
            }
            if (!__all_sync(0xffffffffu, gm_wait(&sb->t_full[grp], use & 1, sb, a.status, 60 + grp))) break;
            ++use;
            ptx::tc_fence_after();
            {
                const int row = ti.row0 + half * kBM + quarter * 32 + lane;
                const bool row_ok = row < ti.row_end;
                const float rs = (has_offset && row_ok) ? __ldg(a.rowsum + row) : 0.f;
                if constexpr (SILU) {
                    __nv_bfloat16* arow = a.y + (size_t)row * (a.N >> 1) + (ti.n0 >> 1);
                    const uint32_t acc = tmem_base + grp * kBN + ((uint32_t)(quarter * 32) << 16);
#pragma unroll 1
                    for (int c = 0; c < kBN / 32; ++c) {  // 16 activation columns per step
                        uint32_t rg[16], ru[16];
                        ptx::tmem_ld_32x16(acc + c * 16, rg);
                        ptx::tmem_ld_32x16(acc + kBN / 2 + c * 16, ru);
                        ptx::tmem_ld_wait();
                        uint32_t o[8];
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            const float4 sg = *reinterpret_cast<const float4*>(es + c * 16 + 4 * q);
                            const float4 og = *reinterpret_cast<const float4*>(es + kBN + c * 16 + 4 * q);
                            const float4 su = *reinterpret_cast<const float4*>(es + kBN / 2 + c * 16 + 4 * q);
                            const float4 ou = *reinterpret_cast<const float4*>(es + kBN + kBN / 2 + c * 16 + 4 * q);
                            // accumulator positions (0,2,1,3) of a group of four hold columns 0..3
                            const uint32_t g01 = pack_bf16x2(fmaf(og.x, rs, sg.x * __uint_as_float(rg[4 * q])),
                                                             fmaf(og.y, rs, sg.y * __uint_as_float(rg[4 * q + 2])));
                            const uint32_t g23 = pack_bf16x2(fmaf(og.z, rs, sg.z * __uint_as_float(rg[4 * q + 1])),
                                                             fmaf(og.w, rs, sg.w * __uint_as_float(rg[4 * q + 3])));
                            const uint32_t u01 = pack_bf16x2(fmaf(ou.x, rs, su.x * __uint_as_float(ru[4 * q])),
                                                             fmaf(ou.y, rs, su.y * __uint_as_float(ru[4 * q + 2])));
                            const uint32_t u23 = pack_bf16x2(fmaf(ou.z, rs, su.z * __uint_as_float(ru[4 * q + 1])),
                                                             fmaf(ou.w, rs, su.w * __uint_as_float(ru[4 * q + 3])));
                            const uint32_t gw[2] = {g01, g23}, uw[2] = {u01, u23};
#pragma unroll
                            for (int i = 0; i < 2; ++i) {
                                const float g0 = __uint_as_float(gw[i] << 16), g1 = __uint_as_float(gw[i] & 0xFFFF0000u);
                                const float u0 = __uint_as_float(uw[i] << 16), u1 = __uint_as_float(uw[i] & 0xFFFF0000u);
                                o[2 * q + i] = pack_bf16x2(g0 / (1.f + __expf(-g0)) * u0, g1 / (1.f + __expf(-g1)) * u1);
                            }
                        }
                        if (row_ok) {
                            uint4* dst = reinterpret_cast<uint4*>(arow + c * 16);
                            dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
                            dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
                        }
                    }
                } else {
                __nv_bfloat16* yrow = a.y + (size_t)row * a.N + ti.n0;
#pragma unroll 1
                for (int c = 0; c < kBN / 32; ++c) {
                    if (MODE == B200MOE_CT_FP8 && ti.n0 + c * 32 >= a.N) break;  // 128-column last tile
                    uint32_t r[32];
                    ptx::tmem_ld_32x32(tmem_base + grp * kBN + c * 32 + ((uint32_t)(quarter * 32) << 16), r);
                    ptx::tmem_ld_wait();
                    uint32_t o[16];
#pragma unroll
                    for (int q = 0; q < 8; ++q) {  // output columns 4q .. 4q+3 of the chunk
                        float4 s4 = make_float4(1.f, 1.f, 1.f, 1.f), o4 = make_float4(0.f, 0.f, 0.f, 0.f);
                        if (per_channel) {
                            s4 = *reinterpret_cast<const float4*>(es + c * 32 + 4 * q);
                            o4 = *reinterpret_cast<const float4*>(es + kBN + c * 32 + 4 * q);
                        }
                        // the int8 dequant stores columns (0,2,1,3) of every group of four, so output
                        // column 4q + i sits at accumulator position 4q + (0,2,1,3)[i]
                        constexpr bool kPerm = (MODE == B200MOE_CT_INT8);
                        float v0 = __uint_as_float(r[4 * q]), v1 = __uint_as_float(r[4 * q + (kPerm ? 2 : 1)]);
                        float v2 = __uint_as_float(r[4 * q + (kPerm ? 1 : 2)]), v3 = __uint_as_float(r[4 * q + 3]);
                        if (per_channel) {
                            v0 = fmaf(o4.x, rs, s4.x * v0);
                            v1 = fmaf(o4.y, rs, s4.y * v1);
                            v2 = fmaf(o4.z, rs, s4.z * v2);
                            v3 = fmaf(o4.w, rs, s4.w * v3);
                        }
                        o[2 * q] = pack_bf16x2(v0, v1);
                        o[2 * q + 1] = pack_bf16x2(v2, v3);
                    }
                    if (row_ok) {
                        uint4* dst = reinterpret_cast<uint4*>(yrow + c * 32);
#pragma unroll
                        for (int q = 0; q < 4; ++q) dst[q] = make_uint4(o[4 * q], o[4 * q + 1], o[4 * q + 2], o[4 * q + 3]);
                    }
                }
                }
            }
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&sb->t_empty[grp]));
        }
    } else if (warp >= kWarpDq0 && !T::kDirect) {
        // ------------------------------ dequant ------------------------------
        // A unit of work is one stage (one k block); for int4 it holds the hi and the lo tile.  These
        // warps bound the kernel when tiles are small, so the loop carries as little bookkeeping as it
        // can: a stage counter, one iterator (for the loads, kPrefetch units ahead) whose global address
        // advances by a constant inside a tile, and shared addresses derived from one per-thread offset.
        const int dq_tid = threadIdx.x - kWarpDq0 * 32;
        const int grp = dq_tid / (kDqGroupWarps * 32);
        const DqLane d = dq_lane<MODE>(dq_tid % (kDqGroupWarps * 32));
        DqIter pf;
        pf.seq = 0;
        pf.t = next_tile(sb, pf.seq, n_tiles, a.status);
        pf.kt = 0;
        dq_locate<MODE>(pf, weight, a, d, n_tiles, tile_prefix, row_start, n_nt);
        if (grp > 0 && pf.valid) dq_advance<MODE>(pf, grp, weight, a, d, n_kt, n_tiles, tile_prefix, row_start, n_nt, sb);
        DqIter cur = pf;  // int4 only: the stage being converted (its scales are loaded late)
        PackedRegs<MODE> regs[kPrefetch];
        bool loaded[kPrefetch];
#pragma unroll
        for (int u = 0; u < kPrefetch; ++u) {
            loaded[u] = pf.valid;
            if (pf.valid) {
                load_packed<MODE>(regs[u], pf, a, d);
                dq_advance<MODE>(pf, kDqGroups, weight, a, d, n_kt, n_tiles, tile_prefix, row_start, n_nt, sb);
            }
        }
        const uint32_t sa0 = ptx::smem_u32(b_ring) + (MODE == kCtFp4Ascend ? btile_offset(d.k0, d.chunk)
                                                                            : btile_offset(d.row, 2 * d.c16));
        uint32_t ib = grp;
        bool ok = true;
        while (ok) {
#pragma unroll
            for (int u = 0; u < kPrefetch; ++u) {
                if (!loaded[u]) { ok = false; break; }  // the schedule has ended
                const uint32_t slot = ib % NS;
                Int4Scales sc4;
                if constexpr (MODE == B200MOE_CT_INT4) sc4 = load_int4_scales(a, cur.g, cur.n0, cur.kt, d);
                bool got = true;
                if (ib >= NS) got = gm_wait(&sb->empty[slot], ((ib / NS) & 1) ^ 1, sb, a.status, 80 + (int)slot);
                if (!__all_sync(0xffffffffu, got)) { ok = false; break; }
                const uint32_t sa = sa0 + slot * (uint32_t)(P * kBTileBytes);
                if constexpr (MODE == B200MOE_CT_INT4)
                    convert_block_int4(regs[u], sc4, sa, sa + kBTileBytes);
                else if constexpr (MODE == kCtFp4Ascend)
                    convert_stage_fp4_ascend(regs[u], sa);
                else
                    convert_stage<MODE>(regs[u], sa);
                ptx::fence_proxy_async_smem();  // generic-proxy writes -> visible to the tensor core (async proxy)
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&sb->full[slot]));
                loaded[u] = pf.valid;
                if (pf.valid) {
                    load_packed<MODE>(regs[u], pf, a, d);
                    dq_advance<MODE>(pf, kDqGroups, weight, a, d, n_kt, n_tiles, tile_prefix, row_start, n_nt, sb);
                }
                if constexpr (MODE == B200MOE_CT_INT4)
                    dq_advance<MODE>(cur, kDqGroups, weight, a, d, n_kt, n_tiles, tile_prefix, row_start, n_nt, sb);
                ib += kDqGroups;
            }
        }
    }

    ptx::tc_fence_before();
    __syncthreads();
    if (warp == kWarpMma) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc(tmem_base, kTmemCols);
    }
}

// Row sums of x in fp32 (the offset term of the int8 epilogue): one warp per row.  Rows past the
// last group are skipped (a caller may pass a buffer sized for the worst case as x).
__global__ void rowsum_kernel(const __nv_bfloat16* __restrict__ x, float* __restrict__ out, int M, int K,
                              const long long* __restrict__ group_list, int G, int gl_type) {
    // rows in use = end of the last group (clamped to M): a warp-level reduction, then one shared
    // atomic per warp
    __shared__ int s_used;
    if (threadIdx.x == 0) s_used = 0;
    __syncthreads();
    long long v = 0;
    for (int g = threadIdx.x; g < G; g += blockDim.x) {
        const long long c = group_list[g];
        if (gl_type == B200MOE_GROUP_LIST_COUNTS) v += c > 0 ? c : 0; else v = c > v ? c : v;
    }
    v = v > M ? M : v;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const long long other = __shfl_xor_sync(0xffffffffu, v, o);
        if (gl_type == B200MOE_GROUP_LIST_COUNTS) v += other; else v = other > v ? other : v;
    }
    v = v > M ? M : v;
    if ((threadIdx.x & 31) == 0 && v > 0) {
        if (gl_type == B200MOE_GROUP_LIST_COUNTS) atomicAdd(&s_used, (int)v); else atomicMax(&s_used, (int)v);
    }
    __syncthreads();
    const int used = (s_used < 0 || s_used > M) ? M : s_used;  // (a sum of eight clamped parts could wrap)
    const int wpb = blockDim.x >> 5;
    for (int row = blockIdx.x * wpb + (threadIdx.x >> 5); row < used; row += gridDim.x * wpb) {
        const uint4* p = reinterpret_cast<const uint4*>(x + (size_t)row * K);
        float s = 0.f;
        for (int i = threadIdx.x & 31; i < K / 8; i += 32) {
            const uint4 q = __ldg(p + i);
            const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) s += __uint_as_float(w[j] << 16) + __uint_as_float(w[j] & 0xFFFF0000u);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        if ((threadIdx.x & 31) == 0) out[row] = s;
    }
}

// Grid of the row-sum kernel: one warp per row up to a few CTAs per multiprocessor, then a stride
// (every CTA first reduces the group list, which should not be repeated thousands of times).
static unsigned rowsum_blocks(int64_t M) {
    const int64_t want = (M + 7) / 8, cap = 16LL * sm_count();
    return (unsigned)(want < 1 ? 1 : (want < cap ? want : cap));
}

void launch_rowsum(const void* x, float* out, int64_t M, int64_t K, const int64_t* group_list, int64_t G, int gl_type,
                   cudaStream_t stream) {
    rowsum_kernel<<<rowsum_blocks(M), 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(x), out, (int)M, (int)K,
                                                        reinterpret_cast<const long long*>(group_list), (int)G, gl_type);
}

static size_t gm_smem_bytes(int G) {
    return 1024 + (size_t)kNS * (kATileBytes + kBTileBytes) + kBarrierBytes + sizeof(float) * kEpiWarps * kEpiScaleFloats +
           sizeof(int) * 3 * (size_t)(G + 1);
}

template <int MODE, bool SILU = false>
static int gm_launch(const void* x, const void* w, const GemmArgs& a, cudaStream_t stream) {
    using T = GmTraits<MODE>;
    CUtensorMap tx, txs, tw;
    int rc = make_tensor_map_2d(&tx, x, 2, (uint64_t)a.M, a.K, kBM, kBK, true);
    if (rc != B200MOE_OK) return rc;
    rc = make_tensor_map_2d(&txs, x, 2, (uint64_t)a.M, a.K, kSmallRows, kBK, true);
    if (rc != B200MOE_OK) return rc;
    if (T::kDirect)
        rc = make_tensor_map_2d(&tw, w, 2, (uint64_t)a.G * a.K, a.N, kBK, 64, true);
    else
        rc = make_tensor_map_2d(&tw, w, 1, (uint64_t)a.G * a.K, T::kNibbles ? a.N / 2 : a.N, kBK,
                                a.N < kBN ? (uint32_t)(T::kNibbles ? a.N / 2 : a.N) : (uint32_t)T::kPRowBytes, false);
    if (rc != B200MOE_OK) return rc;
    const size_t smem = gm_smem_bytes(a.G);
    B200MOE_CUDA_TRY(cudaFuncSetAttribute(grouped_gemm_kernel<MODE, SILU>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          (int)smem));
    grouped_gemm_kernel<MODE, SILU><<<sm_count(), kGemmThreads, smem, stream>>>(tx, txs, tw, static_cast<const uint8_t*>(w), a);
    B200MOE_CUDA_TRY(cudaGetLastError());
    return B200MOE_OK;
}

static size_t align256(size_t v) { return (v + 255) & ~size_t(255); }

}  // namespace b200moe

using namespace b200moe;

extern "C" size_t b200moe_grouped_gemm_workspace_bytes(int64_t M, int64_t K, int64_t N, int64_t G, int compute_type,
                                                       int weight_layout) {
    size_t b = B200MOE_STATUS_BYTES;
    if (compute_type == B200MOE_CT_INT8) b += align256((size_t)M * sizeof(float));
    (void)K; (void)N; (void)G; (void)weight_layout;  // stored-order fp4 weights are read in place
    return b;
}

extern "C" int b200moe_grouped_gemm(const void* x, const void* weight, const void* scale, const void* offset,
                                    const int64_t* group_list, void* y, int64_t M, int64_t K, int64_t N, int64_t G,
                                    int compute_type, int group_list_type, int weight_layout, void* workspace,
                                    size_t workspace_bytes, void* stream) {
    if (compute_type < B200MOE_CT_FP8 || compute_type > B200MOE_CT_BF16) return B200MOE_ERR_COMPUTE_TYPE;
    if (group_list_type != B200MOE_GROUP_LIST_CUMSUM && group_list_type != B200MOE_GROUP_LIST_COUNTS)
        return B200MOE_ERR_ARGUMENT;
    if (weight_layout != B200MOE_LAYOUT_CANONICAL && weight_layout != B200MOE_LAYOUT_ASCEND)
        return B200MOE_ERR_ARGUMENT;
    if (M < 0 || K <= 0 || N <= 0 || G <= 0 || G > kMaxExperts || M > 0x7FFFFFF0LL || K > 0x7FFFFFF0LL ||
        N > 0x7FFFFFF0LL || G * K > 0x7FFFFFF0LL)
        return B200MOE_ERR_SHAPE;
    // fp8: what the reference takes (K and N multiples of its 128 x 128 scale block: a last tile of
    // 128 columns); the other modes work on whole 256-column tiles
    if (compute_type == B200MOE_CT_FP8 ? ((K % 128) != 0 || (N % 128) != 0) : ((K % kBK) != 0 || (N % kBN) != 0))
        return B200MOE_ERR_SHAPE;
    if (compute_type == B200MOE_CT_INT4 && (K % 128) != 0) return B200MOE_ERR_SHAPE;
    if (M == 0) return B200MOE_OK;
    const bool needs_scale = compute_type != B200MOE_CT_BF16;
    if (!x || !weight || (needs_scale && !scale) || !group_list || !y) return B200MOE_ERR_NULL_POINTER;
    if (!aligned16(x) || !aligned16(weight) || (scale && !aligned16(scale)) || !aligned16(y) || (offset && !aligned16(offset)))
        return B200MOE_ERR_ALIGNMENT;
    const size_t need = b200moe_grouped_gemm_workspace_bytes(M, K, N, G, compute_type, weight_layout);
    if (workspace == nullptr || workspace_bytes < need || !aligned16(workspace)) return B200MOE_ERR_WORKSPACE;

    cudaStream_t s = static_cast<cudaStream_t>(stream);
    B200MOE_CUDA_TRY(cudaMemsetAsync(workspace, 0, 16, s));
    uint8_t* ws = static_cast<uint8_t*>(workspace) + B200MOE_STATUS_BYTES;
    GemmArgs a;
    a.scale = scale;
    a.offset = nullptr;
    a.rowsum = nullptr;
    a.group_list = group_list;
    a.y = static_cast<__nv_bfloat16*>(y);
    a.M = (int)M; a.K = (int)K; a.N = (int)N; a.G = (int)G;
    a.gl_type = group_list_type;
    a.status = static_cast<int*>(workspace);

    if (compute_type == B200MOE_CT_INT8) {
        float* rowsum = reinterpret_cast<float*>(ws);
        ws += align256((size_t)M * sizeof(float));
        if (offset != nullptr) {
            rowsum_kernel<<<rowsum_blocks(M), 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x), rowsum, (int)M,
                                                                   (int)K, reinterpret_cast<const long long*>(group_list),
                                                                   (int)G, group_list_type);
            B200MOE_CUDA_TRY(cudaGetLastError());
            a.offset = static_cast<const __nv_bfloat16*>(offset);
            a.rowsum = rowsum;
        }
        return gm_launch<B200MOE_CT_INT8>(x, weight, a, s);
    }
    if (compute_type == B200MOE_CT_INT4) {
        a.offset = static_cast<const __nv_bfloat16*>(offset);  // folded into the weights by the dequant warps
        return gm_launch<B200MOE_CT_INT4>(x, weight, a, s);
    }
    if (compute_type == B200MOE_CT_FP8) return gm_launch<B200MOE_CT_FP8>(x, weight, a, s);
    if (compute_type == B200MOE_CT_BF16) return gm_launch<B200MOE_CT_BF16>(x, weight, a, s);
    // the stored ("ascend") order is read in place by the dequant warps
    if (weight_layout == B200MOE_LAYOUT_ASCEND) return gm_launch<kCtFp4Ascend>(x, weight, a, s);
    return gm_launch<B200MOE_CT_FP4>(x, weight, a, s);
}

extern "C" int b200moe_grouped_gemm_int8_silu(const void* x, const void* weight, const void* scale, const void* offset,
                                              const int64_t* group_list, void* out, int64_t M, int64_t K, int64_t N,
                                              int64_t G, int group_list_type, void* workspace, size_t workspace_bytes,
                                              void* stream) {
    if (group_list_type != B200MOE_GROUP_LIST_CUMSUM && group_list_type != B200MOE_GROUP_LIST_COUNTS)
        return B200MOE_ERR_ARGUMENT;
    if (M < 0 || K <= 0 || N <= 0 || G <= 0 || G > kMaxExperts || M > 0x7FFFFFF0LL || K > 0x7FFFFFF0LL ||
        N > 0x7FFFFFF0LL || G * K > 0x7FFFFFF0LL)
        return B200MOE_ERR_SHAPE;
    if ((K % kBK) != 0 || (N % kBN) != 0) return B200MOE_ERR_SHAPE;
    if (M == 0) return B200MOE_OK;
    if (!x || !weight || !scale || !group_list || !out) return B200MOE_ERR_NULL_POINTER;
    if (!aligned16(x) || !aligned16(weight) || !aligned16(scale) || !aligned16(out) || (offset && !aligned16(offset)))
        return B200MOE_ERR_ALIGNMENT;
    const size_t need = b200moe_grouped_gemm_workspace_bytes(M, K, N, G, B200MOE_CT_INT8, B200MOE_LAYOUT_CANONICAL);
    if (workspace == nullptr || workspace_bytes < need || !aligned16(workspace)) return B200MOE_ERR_WORKSPACE;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    B200MOE_CUDA_TRY(cudaMemsetAsync(workspace, 0, 16, s));
    GemmArgs a;
    a.scale = scale;
    a.offset = nullptr;
    a.rowsum = nullptr;
    a.group_list = group_list;
    a.y = static_cast<__nv_bfloat16*>(out);
    a.M = (int)M; a.K = (int)K; a.N = (int)N; a.G = (int)G;
    a.gl_type = group_list_type;
    a.status = static_cast<int*>(workspace);
    if (offset != nullptr) {
        float* rowsum = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + B200MOE_STATUS_BYTES);
        rowsum_kernel<<<rowsum_blocks(M), 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x), rowsum, (int)M, (int)K,
                                                       reinterpret_cast<const long long*>(group_list), (int)G,
                                                       group_list_type);
        B200MOE_CUDA_TRY(cudaGetLastError());
        a.offset = static_cast<const __nv_bfloat16*>(offset);
        a.rowsum = rowsum;
    }
    return gm_launch<B200MOE_CT_INT8, true>(x, weight, a, s);
}

// ---------------------------------------------------------------------------------------------
// Allocation-free variant for callers that cannot allocate device memory
// ---------------------------------------------------------------------------------------------
// Some hosts of these kernels may not call cudaMalloc at all: a plug-in that runs inside another
// framework's execution step, where every device allocation is owned by that framework's arena and
// a foreign cudaMalloc would fragment or deadlock it; a real-time serving loop that forbids
// allocation after start-up.  The regular
// entry point asks such callers for a workspace they have no way to provide.  This one keeps the
// kernel's scratch (two status words and one fp32 row sum per row of x) in a fixed array that is
// part of the loaded library image, so the caller passes inputs and outputs only.
namespace b200moe {

constexpr long long kNoAllocMaxRows = 65536;
static __device__ __align__(256) unsigned char g_noalloc_scratch[B200MOE_STATUS_BYTES + kNoAllocMaxRows * sizeof(float)];

// Device address of the scratch array on the current device, resolved once per device.  The array's
// name is only a host-side handle: a kernel must be given the address cudaGetSymbolAddress returns.
// This lookup and the first launch of the kernel on a device (the driver loads the kernel image, with
// the array in it, at that point) are the set-up a warm-up call gets out of the way: callers make one
// call per device before their allocation-free phase and before any stream capture.  The cached
// address is valid for the life of the process, not across a device reset.
static int noalloc_scratch(void** out) {
    static void* addr[64];
    static std::mutex mu;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return B200MOE_ERR_CUDA;
    std::lock_guard<std::mutex> lock(mu);
    if (addr[dev] == nullptr) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_noalloc_scratch) != cudaSuccess || p == nullptr) {
            (void)cudaGetLastError();
            return B200MOE_ERR_CUDA;
        }
        addr[dev] = p;
    }
    *out = addr[dev];
    return B200MOE_OK;
}

}  // namespace b200moe

extern "C" int64_t b200moe_grouped_gemm_int8_noalloc_max_rows(void) { return kNoAllocMaxRows; }

extern "C" int b200moe_grouped_gemm_int8_noalloc(const void* x, const void* weight, const void* scale,
                                                 const void* offset, const int64_t* group_list, void* y, int64_t M,
                                                 int64_t K, int64_t N, int64_t G, int group_list_type, void* stream) {
    if (group_list_type != B200MOE_GROUP_LIST_CUMSUM && group_list_type != B200MOE_GROUP_LIST_COUNTS)
        return B200MOE_ERR_ARGUMENT;
    if (M < 0 || K <= 0 || N <= 0 || G <= 0 || G > kMaxExperts || K > 0x7FFFFFF0LL || N > 0x7FFFFFF0LL ||
        G * K > 0x7FFFFFF0LL)
        return B200MOE_ERR_SHAPE;
    if (M > kNoAllocMaxRows) return B200MOE_ERR_NOALLOC_LIMIT;
    if ((K % kBK) != 0 || (N % kBN) != 0) return B200MOE_ERR_SHAPE;
    if (M == 0) return B200MOE_OK;
    if (!x || !weight || !scale || !group_list || !y) return B200MOE_ERR_NULL_POINTER;
    if (!aligned16(x) || !aligned16(weight) || !aligned16(scale) || !aligned16(y) || (offset && !aligned16(offset)))
        return B200MOE_ERR_ALIGNMENT;

    void* scratch = nullptr;
    const int rc = noalloc_scratch(&scratch);
    if (rc != B200MOE_OK) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // the array keeps whatever the previous call left: the status words must start at zero
    B200MOE_CUDA_TRY(cudaMemsetAsync(scratch, 0, 16, s));
    GemmArgs a;
    a.scale = scale;
    a.offset = nullptr;
    a.rowsum = nullptr;
    a.group_list = group_list;
    a.y = static_cast<__nv_bfloat16*>(y);
    a.M = (int)M; a.K = (int)K; a.N = (int)N; a.G = (int)G;
    a.gl_type = group_list_type;
    a.status = static_cast<int*>(scratch);
    if (offset != nullptr) {
        float* rowsum = reinterpret_cast<float*>(static_cast<unsigned char*>(scratch) + B200MOE_STATUS_BYTES);
        rowsum_kernel<<<rowsum_blocks(M), 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x), rowsum, (int)M, (int)K,
                                                              reinterpret_cast<const long long*>(group_list), (int)G,
                                                              group_list_type);
        B200MOE_CUDA_TRY(cudaGetLastError());
        a.offset = static_cast<const __nv_bfloat16*>(offset);
        a.rowsum = rowsum;
    }
    return gm_launch<B200MOE_CT_INT8>(x, weight, a, s);
}

extern "C" int b200moe_noalloc_read_status(int32_t out[2], void* stream) {
    if (out == nullptr) return B200MOE_ERR_NULL_POINTER;
    void* scratch = nullptr;
    const int rc = noalloc_scratch(&scratch);
    if (rc != B200MOE_OK) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    B200MOE_CUDA_TRY(cudaMemcpyAsync(out, scratch, 2 * sizeof(int32_t), cudaMemcpyDeviceToHost, s));
    B200MOE_CUDA_TRY(cudaStreamSynchronize(s));
    return B200MOE_OK;
}
