// Antiquant grouped GEMM on int8 weights in a tile-packed order, for callers that keep the expert
// weights resident and can repack them once (the MoE layer): persistent, warp-specialised
// tcgen05 kernel in which the dequantised weights never touch shared memory.
//
//   y^T[weight columns, rows of expert g] = W[g]^T @ x[rows of expert g]^T
//
// The operands are swapped against the generic kernel (grouped_gemm.cu): the 128 lanes of an MMA
// are weight columns and its N extent is the tile's token rows rounded up to 16 (16 .. 160), so an
// expert with 137 rows costs 144 columns of tensor-core time instead of two 128-row halves, and the
// A operand (bf16 weights) is written by the dequant warps straight into tensor memory
// (tcgen05.st) and read from there by the MMA.  Shared memory carries only the x tile (TMA, K-major,
// 128-byte swizzle; the B operand): per 64-k stage of a 144-row tile 37 KB of operand reads and
// 20 KB of TMA writes, against 160 KB for a two-half tile of the generic kernel, whose bound is the
// shared-memory port.
//
// Packed order (b200moe_pack_weight_int8 writes it): [G][N / 256 tiles][K / 64 stages][8 warp
// blocks][4 k-chunks][32 lanes][16 bytes].  A tile is 256 weight columns = two MMA halves of 128
// (with gate_up: 128 gate columns and the 128 up columns of the same indices); warp block 4 h + q holds
// columns 32 q .. 32 q + 31 of half h, one lane per column; a lane's 16 bytes are 16 consecutive k
// of its column in the byte order (k0, k2, k1, k3) per 32-bit word, which the two-bytes-at-a-time
// int8 -> bf16 conversion turns into the (k, k + 1) pairs a tensor-memory column holds.  A dequant
// warp therefore reads 512 contiguous bytes per load instruction and 2 KB contiguous per stage.
//
// Warp roles (28 warps): warp 0 x-tile producer, tile tickets and L2 prefetch of packed weights;
// warp 2 TMEM allocation and MMA issue; warps 4-11 epilogue (lane = weight column: per-channel
// scale and offset are per-thread scalars, a warp stores 64 contiguous bytes of one output row
// per instruction); warps 12-27 dequant in two groups on alternate stages.  TMEM: accumulators of
// the two halves at columns 0 and 160, the A ring (3 stages x 2 halves x 32 columns) from column
// 320.  The x ring has its own barriers and twice the depth: an x box takes 700 to 800 cycles from
// issue to arrival, more than a stage lasts, and shared memory has the room that tensor memory lacks.
// The MMA warp's loop is serial and every step of it costs tens of cycles, so it sees ONE barrier
// pair: a relay lane of the dequant group (which has slack) waits for the stage's x tile before the
// group reports the stage full, and hands the x slot back to the producer when it observes the
// completion of the MMAs that read it.  Every wait is bounded.
#include <atomic>

#include "common.cuh"
#include "gemm_args.cuh"
#include "ptx.cuh"

namespace b200moe {
namespace pk {

// SMs the persistent kernels of this file leave to other kernels (b200moe_set_gemm_reserved_sms)
static std::atomic<int> g_reserved_sms{0};
static unsigned grid_ctas() {
    const int sms = sm_count();
    int r = g_reserved_sms.load(std::memory_order_relaxed);
    r = r < 0 ? 0 : (r > sms - 1 ? sms - 1 : r);
    return (unsigned)(sms - r);
}

constexpr int kBK = 64;        // k per stage
constexpr int kTileN = 256;    // weight columns per tile: two MMA halves of 128
constexpr int kMaxR = 160;     // token rows per tile (the MMA's N extent), a multiple of 32
constexpr int kStages = 3;     // A ring (tensor memory), 64 k per stage
constexpr int kXStages = 6;    // x ring (shared memory), 64 k per stage (120 KB; 80 KB more hold the epilogue's staging tile)
constexpr int kThreads = 896;
constexpr int kWarpProd = 0, kWarpMma = 2, kWarpEpi0 = 4, kEpiWarps = 8, kWarpDq0 = 12;
constexpr int kDqGroups = 2, kDqGroupWarps = 8;
constexpr int kPrefetch = 2;    // packed stages a dequant thread holds in registers ahead of the conversion
constexpr int kL2Ahead = 4;     // stages by which the L2 prefetch of packed weights leads the x loads
constexpr int kSuperRows = 8;   // m-tiles per L2 super-tile
constexpr int kTileRing = 32;
constexpr int kXSlotBytes = kMaxR * kBK * 2;  // 20 KB, a multiple of 1024
constexpr int kStageWBytes = kBK * kTileN;    // packed bytes of one stage
constexpr int kBigBox = 128, kSmallBox = 32;  // rows of the two x boxes
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kACol = 2 * kMaxR;          // first column of the A ring
constexpr uint32_t kAStageCols = 64;           // 2 halves x 32 columns (64 k as bf16 pairs)
constexpr int kBarrierBytes = 1024;
constexpr int kEpiStripBytes = kMaxR * 4;  // per epilogue warp: the row sums of the tile's rows
constexpr int kStageTileBytes = kMaxR * kTileN * 2;  // the epilogue's bf16 staging tile (80 KB)
static_assert(kACol + kStages * kAStageCols <= kTmemCols, "tensor memory budget");

struct TileInfo {
    int g, row0, rows;  // expert, first row, rows of the expert inside the tile (1 .. kMaxR)
    int j;              // tile column index (256 weight columns each)
};

struct Barriers {
    uint64_t x_full[kXStages];   // x ring: TMA bytes; waited for by the relay lane of the stage's dequant group
    uint64_t x_empty[kXStages];  // x ring: one arrive by the relay lane once the stage's MMAs have completed
    uint64_t full[kStages];   // the 8 dequant warps of the stage's group: A slot written AND x tile landed
    uint64_t empty[kStages];  // one tcgen05.commit per stage
    uint64_t t_full, t_empty; // accumulator hand-off with the epilogue
    uint64_t stage_full, stage_free;  // the epilogue warps among themselves: staging tile written / stored
    uint64_t drain;
    uint32_t tmem_base;
    int abort;
    int n_tiles;
    int pad;
    // The published tiles, resolved once by the publisher: entry i % kTileRing = {i + 1, first row,
    // expert | rows << 16 (rows 0 = end of the schedule), tile column}, written and read as one aligned
    // 16-byte vector, so a reader sees the sequence number and the tile together.  Every other role reads
    // the entry instead of repeating the search and the divisions at each tile switch.
    uint4 tile_ring[kTileRing];
};
static_assert(sizeof(Barriers) <= kBarrierBytes, "barrier block");


__device__ __noinline__ bool wait_slow(uint32_t bar, uint32_t parity, Barriers* sb, int* status, int id) {
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
__device__ __forceinline__ bool pk_wait(uint64_t* bar, uint32_t parity, Barriers* sb, int* status, int id) {
    const uint32_t b = ptx::smem_u32(bar);
    if (ptx::mbar_try_wait(b, parity)) return true;
    return wait_slow(b, parity, sb, status, id);
}

__device__ __forceinline__ uint4 ring_load(const uint4* e) {
    uint4 v;
    asm volatile("ld.volatile.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "r"(ptx::smem_u32(e)));
    return v;
}

// The seq-th tile of this CTA (seq is advanced) into `ti`; false when the schedule has ended, a wait
// expired or another role aborted.
__device__ __forceinline__ bool next_tile(Barriers* sb, uint32_t& seq, TileInfo& ti, int* status) {
    const uint4* e = &sb->tile_ring[seq % kTileRing];
    const uint32_t want = seq + 1;
    uint4 v = ring_load(e);
    if (v.x != want) {
        volatile int* abort = &sb->abort;
        const uint64_t t0 = ptx::globaltimer_ns();
        uint32_t spins = 0;
        while ((v = ring_load(e)).x != want) {
            if ((++spins & 0xFF) == 0) {
                if (*abort) return false;
                if (ptx::globaltimer_ns() - t0 > ptx::kWaitLimitNs) {
                    *abort = 1;
                    report_status(status, kDevWaitExpired, 90);
                    return false;
                }
            }
        }
    }
    ++seq;
    ti.row0 = (int)v.y;
    ti.g = (int)(v.z & 0xFFFFu);
    ti.rows = (int)(v.z >> 16);
    ti.j = (int)v.w;
    return ti.rows != 0;
}

// Rows of an m-tile of an expert with `rows` rows: the expert is cut into the fewest tiles of at
// most kMaxR rows, of equal size rounded up to 16 (a short last tile would still pay a full
// dequantisation of the weight tile).
__device__ __forceinline__ int tile_rows_of(int rows) {
    const int n_mt = (rows + kMaxR - 1) / kMaxR;
    return n_mt == 0 ? kMaxR : ((((rows + n_mt - 1) / n_mt) + 15) & ~15);
}

// tile index -> expert, rows, tile column.  tile_prefix has G + 1 entries.  Inside an expert the
// tiles run in super-tiles of up to kSuperRows m-tiles x all tile columns, m fastest, so that
// concurrently running CTAs share a weight tile and the expert's x rows in L2.
__device__ __forceinline__ TileInfo locate_tile(int t, const int* tile_prefix, const int* row_start, int G, int n_nt) {
    int lo = 0, hi = G;  // largest g with tile_prefix[g] <= t
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (tile_prefix[mid] <= t) lo = mid;
        else hi = mid;
    }
    const int g = lo, j = t - tile_prefix[g];
    const int r0 = row_start[g], rows = row_start[g + 1] - r0;
    const int mt = (tile_prefix[g + 1] - tile_prefix[g]) / n_nt;
    const int tr = tile_rows_of(rows);
    const int per_super = kSuperRows * n_nt;
    const int st = j / per_super, base = st * kSuperRows;
    const int h = min(kSuperRows, mt - base);
    const int jj = j - st * per_super;
    const int m = base + jj % h;
    TileInfo ti;
    ti.g = g;
    ti.j = jj / h;
    ti.row0 = r0 + m * tr;
    ti.rows = min(tr, rows - m * tr);
    return ti;
}

// Position of a dequant thread in the (tile, stage) sequence of its CTA; wp = the thread's 16 bytes
// of k-chunk 0 of that stage.
struct DqIter {
    int kt;
    uint32_t seq;
    bool valid;
    TileInfo ti;
    const uint8_t* wp;
};
__device__ __forceinline__ void dq_locate(DqIter& it, const uint8_t* __restrict__ w, int thread_off, int n_kt, int n_nt) {
    if (!it.valid) return;
    it.wp = w + (((size_t)it.ti.g * n_nt + it.ti.j) * n_kt + it.kt) * (size_t)kStageWBytes + thread_off;
}
__device__ __forceinline__ void dq_advance(DqIter& it, int step, const uint8_t* __restrict__ w, const GemmArgs& a,
                                           int thread_off, int n_kt, int n_nt, Barriers* sb) {
    it.kt += step;
    if (it.kt < n_kt) {
        it.wp += (size_t)step * kStageWBytes;
        return;
    }
    do {
        it.kt -= n_kt;
        it.valid = next_tile(sb, it.seq, it.ti, a.status);
    } while (it.kt >= n_kt && it.valid);
    dq_locate(it, w, thread_off, n_kt, n_nt);
}

// GATE_UP: a tile's half 0 holds 128 gate columns and half 1 the up columns of the same indices; the
// epilogue writes bf16(silu(gate) * up), [M, N / 2] (gate and up are rounded to bf16 first, as the
// unfused operators would).
template <bool GATE_UP>
__global__ void __launch_bounds__(kThreads, 1)
grouped_gemm_packed_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_xs,
                           const uint8_t* __restrict__ weight, const GemmArgs a) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* x_ring = base;
    uint8_t* epi_stage = x_ring + kXStages * kXSlotBytes;
    Barriers* sb = reinterpret_cast<Barriers*>(epi_stage + kStageTileBytes);
    __shared__ __nv_bfloat16* s_dst_base[8];  // scatter mode: the destination tensors (indexed per row)
    if (threadIdx.x < 8) s_dst_base[threadIdx.x] = a.dst_base[threadIdx.x];
    float* epi_rowsum = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(sb) + kBarrierBytes);
    int* row_start = reinterpret_cast<int*>(reinterpret_cast<uint8_t*>(epi_rowsum) + kEpiWarps * kEpiStripBytes);
    int* tile_prefix = row_start + (a.G + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_nt = a.N / kTileN;
    const int n_kt = a.K / kBK;

    load_row_starts(a.group_list, a.G, a.M, a.gl_type, row_start, a.status);
    if (threadIdx.x == 0) {
        int acc = 0;
        tile_prefix[0] = 0;
        for (int g = 0; g < a.G; ++g) {
            const int rows = row_start[g + 1] - row_start[g];
            acc += ((rows + kMaxR - 1) / kMaxR) * n_nt;
            tile_prefix[g + 1] = acc;
        }
        sb->n_tiles = acc;
        sb->abort = 0;
        for (int i = 0; i < kTileRing; ++i) sb->tile_ring[i] = make_uint4(0u, 0u, 0u, 0u);
        for (int i = 0; i < kXStages; ++i) {
            ptx::mbar_init(ptx::smem_u32(&sb->x_full[i]), 1);
            ptx::mbar_init(ptx::smem_u32(&sb->x_empty[i]), 1);
        }
        for (int i = 0; i < kStages; ++i) {
            ptx::mbar_init(ptx::smem_u32(&sb->full[i]), kDqGroupWarps);
            ptx::mbar_init(ptx::smem_u32(&sb->empty[i]), 1);
        }
        ptx::mbar_init(ptx::smem_u32(&sb->t_full), 1);
        ptx::mbar_init(ptx::smem_u32(&sb->t_empty), kEpiWarps);
        ptx::mbar_init(ptx::smem_u32(&sb->stage_full), kEpiWarps);
        ptx::mbar_init(ptx::smem_u32(&sb->stage_free), kEpiWarps);
        ptx::mbar_init(ptx::smem_u32(&sb->drain), 1);
        ptx::fence_mbar_init();
        ptx::prefetch_tensormap(&tmap_x);
        ptx::prefetch_tensormap(&tmap_xs);
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

    if (warp == kWarpProd) {
        // ------------------------------ x-tile producer ------------------------------
        if (lane == 0) {
            uint32_t ia = 0, seq = 0, published = 0;
            bool ok = true;
            int* ticket = a.status + 2;  // zeroed by the host before the launch
            int held = atomicAdd(ticket, 1);
            TileInfo far_ti;  // the tile published last, resolved
            auto publish = [&]() -> bool {
                const bool live = held < n_tiles;
                uint4 entry = make_uint4(published + 1, 0u, 0u, 0u);  // rows 0: the schedule has ended
                if (live) {
                    far_ti = locate_tile(held, tile_prefix, row_start, a.G, n_nt);
                    entry.y = (uint32_t)far_ti.row0;
                    entry.z = (uint32_t)far_ti.g | ((uint32_t)far_ti.rows << 16);
                    entry.w = (uint32_t)far_ti.j;
                }
                asm volatile("st.volatile.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(
                                 ptx::smem_u32(&sb->tile_ring[published % kTileRing])),
                             "r"(entry.x), "r"(entry.y), "r"(entry.z), "r"(entry.w)
                             : "memory");
                ++published;
                if (live) held = atomicAdd(ticket, 1);
                return live;
            };
            // L2 prefetch of the packed stage kL2Ahead further on (a stage is 16 KB contiguous)
            bool far_live = publish();
            int far_kt = 0;
            const uint8_t* far_p = nullptr;
            auto far_locate = [&]() {
                if (far_live) far_p = weight + ((size_t)far_ti.g * n_nt + far_ti.j) * n_kt * (size_t)kStageWBytes;
            };
            far_locate();
            auto far_step = [&]() {
                ptx::bulk_prefetch_l2(far_p + (size_t)far_kt * kStageWBytes, kStageWBytes);
                if (++far_kt < n_kt) return;
                far_kt = 0;
                far_live = publish();
                far_locate();
            };
            for (int i = 0; i < kL2Ahead && far_live; ++i) far_step();
            for (;;) {
                TileInfo ti;
                if (!next_tile(sb, seq, ti, a.status) || !ok) break;
                // the tile's rows rounded up to the small box; rows past the expert's end belong to the
                // next expert (or are zero-filled past M) and land in accumulator columns never stored
                const int r32 = (ti.rows + kSmallBox - 1) & ~(kSmallBox - 1);
                const int n_big = r32 / kBigBox, n_small = (r32 % kBigBox) / kSmallBox;
                const uint32_t stage_bytes = (uint32_t)(r32 * kBK * 2);
                for (int kt = 0; kt < n_kt; ++kt, ++ia) {
                    const uint32_t s = ia % kXStages, ph = (ia / kXStages) & 1;
                    if (ia >= kXStages && !pk_wait(&sb->x_empty[s], ph ^ 1, sb, a.status, 10 + (int)s)) { ok = false; break; }
                    const uint32_t bar = ptx::smem_u32(&sb->x_full[s]);
                    const uint32_t dst = ptx::smem_u32(x_ring + s * kXSlotBytes);
                    const int kx = kt * kBK;
                    ptx::mbar_arrive_expect_tx(bar, stage_bytes);
                    if (n_big) ptx::tma_load_2d(dst, &tmap_x, bar, kx, ti.row0);
                    for (int b = 0; b < n_small; ++b)
                        ptx::tma_load_2d(dst + (uint32_t)((n_big * kBigBox + b * kSmallBox) * kBK * 2), &tmap_xs, bar, kx,
                                         ti.row0 + n_big * kBigBox + b * kSmallBox);
                    if (far_live) far_step();
                }
            }
            if (!ok)
                for (uint32_t j = (ia > kXStages ? ia - kXStages : 0); j < ia; ++j)
                    (void)ptx::mbar_wait(ptx::smem_u32(&sb->x_full[j % kXStages]), (j / kXStages) & 1);
        }
    } else if (warp == kWarpMma) {
        // ------------------------------ MMA issuer ------------------------------
        // The whole warp walks the loop (waits, tile lookup, descriptor arithmetic stay warp-uniform,
        // which keeps them off the per-thread path); one elected lane issues the tcgen05 instructions.
        // An MMA of this kernel lasts 64 to 80 cycles, so the issuing lane's instruction count per MMA
        // matters: every operand is a loop-invariant base plus a compile-time offset.
        {
            const bool leader = ptx::elect_one();
            // B: the x tile, K-major, 8-row groups 1024 B apart, 32 B per 16 k inside the swizzle atom
            const uint64_t db0 = ptx::umma_desc_sw128(ptx::smem_u32(x_ring), 0, 1024);
            const uint32_t ta0 = tmem_base + kACol;
            uint32_t s = 0, ph = 0, xs = 0, tiles_done = 0, seq = 0;
            bool ok = true;
            // whether the next stage's barrier has been seen complete already: polled (non-blocking) right
            // after a stage's MMAs are issued, so that the poll's latency runs beside the commit's
            bool ready = false;
            for (;;) {
                TileInfo ti;
                if (!next_tile(sb, seq, ti, a.status) || !ok) break;
                const uint32_t idesc = ptx::umma_idesc_bf16(128, (ti.rows + 15) & ~15, false);
                // the epilogue must have drained the previous tile's accumulators
                if (tiles_done >= 1 && !pk_wait(&sb->t_empty, (tiles_done - 1) & 1, sb, a.status, 30)) { ok = false; break; }
                ptx::tc_fence_after();
                uint32_t accumulate = 0;
                for (int kt = 0; kt < n_kt; ++kt) {
                    if (!ready && !pk_wait(&sb->full[s], ph, sb, a.status, 40 + (int)s)) { ok = false; break; }
                    ptx::tc_fence_after();
                    const uint64_t db = db0 + (uint64_t)(xs * (kXSlotBytes >> 4));
                    const uint32_t ta = ta0 + s * kAStageCols;
                    const uint32_t s_next = (s + 1 == kStages) ? 0u : s + 1, ph_next = (s + 1 == kStages) ? ph ^ 1u : ph;
                    if (leader) {
#pragma unroll
                        for (int h = 0; h < 2; ++h)
#pragma unroll
                            for (int k16 = 0; k16 < kBK / 16; ++k16)
                                ptx::umma_bf16_ta(tmem_base + h * kMaxR, ta + h * 32 + k16 * 8, db + (uint64_t)(k16 * 2), idesc,
                                                  accumulate | (uint32_t)k16);
                    }
                    ready = ptx::mbar_test_wait(ptx::smem_u32(&sb->full[s_next]), ph_next);
                    if (leader) ptx::umma_commit(ptx::smem_u32(&sb->empty[s]));
                    ready = __all_sync(0xffffffffu, ready);
                    accumulate = 1;
                    s = s_next;
                    ph = ph_next;
                    if (++xs == kXStages) xs = 0;
                }
                if (!ok) break;
                if (leader) ptx::umma_commit(ptx::smem_u32(&sb->t_full));
                __syncwarp();
                ++tiles_done;
            }
            // drain: every issued MMA must have completed before TMEM is released
            if (leader) {
                ptx::umma_commit(ptx::smem_u32(&sb->drain));
                (void)ptx::mbar_wait(ptx::smem_u32(&sb->drain), 0);
            }
        }
        __syncwarp();
    } else if (warp >= kWarpEpi0 && warp < kWarpEpi0 + kEpiWarps) {
        // ------------------------------ epilogue ------------------------------
        // Lane = weight column (TMEM lane 32 * quarter + lane of a half), accumulator columns = token
        // rows.  Two phases per tile.  A: TMEM -> registers -> scale / offset (and SiLU(gate) * up) -> bf16
        // into a [rows][tile columns] staging tile in shared memory; plain: warp (quarter, half) drains its
        // half, GATE_UP: both warps of a quarter read both accumulators and share the 16-row chunks.  The
        // accumulators are handed back to the MMA warp as soon as a warp's own reads are done.  B: the
        // eight warps store the staged rows, a whole row segment (512 or 256 contiguous bytes, 16 per lane)
        // per instruction -- to y, or in scatter mode to each row's own destination, which may be another
        // GPU's memory -- while the next tile is already being accumulated.
        const int ew = warp - kWarpEpi0, quarter = warp & 3, second = ew >> 2;
        const bool has_offset = a.offset != nullptr;
        const uint32_t lane_sel = (uint32_t)(quarter * 32) << 16;
        constexpr int kRowBytes = GATE_UP ? 256 : 512;  // bytes of a staged row
        const uint32_t stage_u32 = ptx::smem_u32(epi_stage);
        // the thread's column in the staging tile
        const uint32_t my_col_bytes = (uint32_t)(((GATE_UP ? 0 : second * 128) + quarter * 32 + lane) * 2);
        uint32_t use = 0, seq = 0;
        bool scattered = false;
        for (;;) {
            TileInfo ti;
            if (!next_tile(sb, seq, ti, a.status)) break;
            const int ci = quarter * 32 + lane;  // column inside a half
            const __nv_bfloat16* sp = static_cast<const __nv_bfloat16*>(a.scale) + (size_t)ti.g * a.N;
            const __nv_bfloat16* op = has_offset ? a.offset + (size_t)ti.g * a.N : nullptr;
            float s0, so0 = 0.f, s1 = 0.f, so1 = 0.f;
            if constexpr (GATE_UP) {
                const int cg = ti.j * 128 + ci, cu = (a.N >> 1) + cg;
                s0 = __bfloat162float(sp[cg]);
                s1 = __bfloat162float(sp[cu]);
                if (has_offset) { so0 = s0 * __bfloat162float(op[cg]); so1 = s1 * __bfloat162float(op[cu]); }
            } else {
                const int c = ti.j * kTileN + second * 128 + ci;
                s0 = __bfloat162float(sp[c]);
                if (has_offset) so0 = s0 * __bfloat162float(op[c]);
            }
            const int ld_out = GATE_UP ? (a.N >> 1) : a.N;
            const int n_chunks = (ti.rows + 15) >> 4;
            // row sums of the tile's rows into the warp's strip while the tile is still being accumulated
            float* rsum = epi_rowsum + ew * kMaxR;
            if (has_offset) {
                __syncwarp();
                for (int i = lane; i < ti.rows; i += 32) rsum[i] = __ldg(a.rowsum + ti.row0 + i);
                __syncwarp();
            }
            if (!__all_sync(0xffffffffu, pk_wait(&sb->t_full, use & 1, sb, a.status, 60))) break;
            // every warp has stored the previous tile's rows: the staging tile may be overwritten
            if (use >= 1 && !__all_sync(0xffffffffu, pk_wait(&sb->stage_free, (use - 1) & 1, sb, a.status, 62))) break;
            ptx::tc_fence_after();
            // ---- phase A ----
            for (int c = GATE_UP ? second : 0; c < n_chunks; c += GATE_UP ? 2 : 1) {
                uint32_t v0[16], v1[16];
                if constexpr (GATE_UP) {
                    ptx::tmem_ld_32x16(tmem_base + lane_sel + c * 16, v0);
                    ptx::tmem_ld_32x16(tmem_base + lane_sel + kMaxR + c * 16, v1);
                } else {
                    ptx::tmem_ld_32x16(tmem_base + lane_sel + second * kMaxR + c * 16, v0);
                }
                ptx::tmem_ld_wait();
                // passes over the chunk's 16 rows (loads, arithmetic, stores), so that the rows' dependent
                // chains overlap instead of running one after the other
                float rs[16];
#pragma unroll
                for (int i = 0; i < 4; ++i) {  // (the strip is kMaxR long: a ragged last chunk reads stale, unused values)
                    const float4 r4 = has_offset ? reinterpret_cast<const float4*>(rsum + c * 16)[i] : make_float4(0.f, 0.f, 0.f, 0.f);
                    rs[4 * i] = r4.x; rs[4 * i + 1] = r4.y; rs[4 * i + 2] = r4.z; rs[4 * i + 3] = r4.w;
                }
                unsigned short ob[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    float o = fmaf(so0, rs[i], s0 * __uint_as_float(v0[i]));
                    if constexpr (GATE_UP) {
                        const float g = __bfloat162float(__float2bfloat16_rn(o));
                        const float u = __bfloat162float(__float2bfloat16_rn(fmaf(so1, rs[i], s1 * __uint_as_float(v1[i]))));
                        o = __fdividef(g, 1.f + __expf(-g)) * u;
                    }
                    ob[i] = __bfloat16_as_ushort(__float2bfloat16_rn(o));
                }
                const uint32_t sa = stage_u32 + (uint32_t)(c * 16 * kRowBytes) + my_col_bytes;
#pragma unroll
                for (int i = 0; i < 16; ++i)
                    asm volatile("st.shared.b16 [%0], %1;" ::"r"(sa + (uint32_t)(i * kRowBytes)), "h"(ob[i]) : "memory");
            }
            // this warp's reads of the accumulators are done: hand them back, report the staging written
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                ptx::mbar_arrive(ptx::smem_u32(&sb->t_empty));
                ptx::mbar_arrive(ptx::smem_u32(&sb->stage_full));
            }
            if (!__all_sync(0xffffffffu, pk_wait(&sb->stage_full, use & 1, sb, a.status, 64))) break;
            ++use;
            // ---- phase B ----
            constexpr int kLanesPerRow = kRowBytes / 16, kRowsPerStep = 32 / kLanesPerRow;  // 32 / 1 or 16 / 2
            const int lr = lane / kLanesPerRow, lc = lane % kLanesPerRow;
            const size_t col0 = (size_t)ti.j * (GATE_UP ? 128 : kTileN) + (size_t)lc * 8;  // first of the lane's 8 columns
            for (int r = ew * kRowsPerStep + lr; r < ti.rows; r += kEpiWarps * kRowsPerStep) {
                uint4 v;
                asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                             : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                             : "r"(stage_u32 + (uint32_t)(r * kRowBytes + lc * 16)));
                __nv_bfloat16* dst;
                if (GATE_UP || a.row_code == nullptr) {
                    dst = a.y + (size_t)(ti.row0 + r) * ld_out;
                } else {
                    // scatter mode: the row's own destination (a code naming none is skipped)
                    const long long code = __ldg(a.row_code + ti.row0 + r);
                    const unsigned int bi = (unsigned int)(code >> 32), ri = (unsigned int)code;
                    if ((int)bi >= a.n_base || (long long)ri >= a.dst_rows) continue;
                    dst = s_dst_base[bi] + (size_t)ri * ld_out;
                    scattered = true;
                }
                *reinterpret_cast<uint4*>(dst + col0) = v;
            }
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&sb->stage_free));
        }
        // rows stored into other GPUs' memory must be visible there before a later kernel signals them
        if (scattered) __threadfence_system();
    } else if (warp >= kWarpDq0) {
        // ------------------------------ dequant ------------------------------
        const int dq_tid = threadIdx.x - kWarpDq0 * 32;
        const int grp = dq_tid / (kDqGroupWarps * 32);
        const int wb = (dq_tid / 32) % kDqGroupWarps;  // warp block 4 h + q; q equals warp index % 4
        const int thread_off = wb * 2048 + lane * 16;
        const bool relay = (dq_tid % (kDqGroupWarps * 32)) == 0;  // lane 0 of the group's first warp
        const uint32_t ta0 = tmem_base + kACol + (uint32_t)((wb >> 2) * 32) + ((uint32_t)((wb & 3) * 32) << 16);
        DqIter pf;
        pf.seq = 0;
        pf.valid = next_tile(sb, pf.seq, pf.ti, a.status);
        pf.kt = 0;
        dq_locate(pf, weight, thread_off, n_kt, n_nt);
        if (grp > 0 && pf.valid) dq_advance(pf, grp, weight, a, thread_off, n_kt, n_nt, sb);
        uint4 regs[kPrefetch][4];
        bool loaded[kPrefetch];
#pragma unroll
        for (int u = 0; u < kPrefetch; ++u) {
            loaded[u] = pf.valid;
            if (pf.valid) {
#pragma unroll
                for (int i = 0; i < 4; ++i) regs[u][i] = __ldg(reinterpret_cast<const uint4*>(pf.wp + i * 512));
                dq_advance(pf, kDqGroups, weight, a, thread_off, n_kt, n_nt, sb);
            }
        }
        uint32_t ib = grp;
        bool ok = true;
        while (ok) {
#pragma unroll
            for (int u = 0; u < kPrefetch; ++u) {
                if (!loaded[u]) { ok = false; break; }  // the schedule has ended
                const uint32_t slot = ib % kStages;
                bool got = true;
                if (ib >= kStages) {
                    got = pk_wait(&sb->empty[slot], ((ib / kStages) & 1) ^ 1, sb, a.status, 80 + (int)slot);
                    // the MMAs of stage ib - kStages have completed: their x slot goes back to the producer
                    if (relay && got) ptx::mbar_arrive(ptx::smem_u32(&sb->x_empty[(ib - kStages) % kXStages]));
                }
                if (!__all_sync(0xffffffffu, got)) { ok = false; break; }
                ptx::tc_fence_after();
                // The relay lane will report the stage full only when its x tile has landed as well.  The tile
                // was requested kXStages stages ago, so this wait is over before the conversion is; its
                // result is consumed after the stores.
                bool x_ok = true;
                if (relay) x_ok = pk_wait(&sb->x_full[ib % kXStages], (ib / kXStages) & 1, sb, a.status, 50);
                const uint32_t ta = ta0 + slot * kAStageCols;
#pragma unroll
                for (int i = 0; i < 4; ++i) {  // 16 k = 8 columns per chunk
                    const uint4 q = regs[u][i];
                    uint32_t o[8];
                    s8x4_to_bf16_even_odd(q.x, o[0], o[1]);
                    s8x4_to_bf16_even_odd(q.y, o[2], o[3]);
                    s8x4_to_bf16_even_odd(q.z, o[4], o[5]);
                    s8x4_to_bf16_even_odd(q.w, o[6], o[7]);
                    ptx::tmem_st_32x8(ta + i * 8, o);
                }
                ptx::tmem_st_wait();
                ptx::tc_fence_before();
                if (!__all_sync(0xffffffffu, x_ok)) { ok = false; break; }
                if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&sb->full[slot]));
                loaded[u] = pf.valid;
                if (pf.valid) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) regs[u][i] = __ldg(reinterpret_cast<const uint4*>(pf.wp + i * 512));
                    dq_advance(pf, kDqGroups, weight, a, thread_off, n_kt, n_nt, sb);
                }
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

// [G, K, N] int8 -> the packed order.  One thread writes one lane's 16 bytes of a k-chunk.
__global__ void pack_weight_int8_kernel(const int8_t* __restrict__ w, uint4* __restrict__ out, int K, int N, int gate_up,
                                        long long n_units) {
    const long long u = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (u >= n_units) return;
    const int lane = (int)(u & 31), i = (int)(u >> 5) & 3, wb = (int)(u >> 7) & 7;
    const long long stage = u >> 10;  // (g * n_nt + j) * n_kt + kt
    const int n_kt = K / kBK, n_nt = N / kTileN;
    const int kt = (int)(stage % n_kt);
    const long long gj = stage / n_kt;
    const int j = (int)(gj % n_nt);
    const long long g = gj / n_nt;
    const int h = wb >> 2, ci = (wb & 3) * 32 + lane;
    const int col = gate_up ? (h ? N / 2 : 0) + j * 128 + ci : j * kTileN + h * 128 + ci;
    const int8_t* src = w + ((size_t)g * K + (size_t)kt * kBK + i * 16) * N + col;
    uint32_t word[4];
#pragma unroll
    for (int wd = 0; wd < 4; ++wd) {
        const uint32_t b0 = (uint8_t)src[(size_t)(4 * wd) * N], b1 = (uint8_t)src[(size_t)(4 * wd + 1) * N];
        const uint32_t b2 = (uint8_t)src[(size_t)(4 * wd + 2) * N], b3 = (uint8_t)src[(size_t)(4 * wd + 3) * N];
        word[wd] = b0 | (b2 << 8) | (b1 << 16) | (b3 << 24);  // byte order (k0, k2, k1, k3)
    }
    out[u] = make_uint4(word[0], word[1], word[2], word[3]);
}

}  // namespace pk

}  // namespace b200moe

using namespace b200moe;

extern "C" int b200moe_set_gemm_reserved_sms(int n) { return pk::g_reserved_sms.exchange(n < 0 ? 0 : n); }

extern "C" int b200moe_pack_weight_int8(const void* weight, void* packed, int64_t G, int64_t K, int64_t N, int gate_up,
                                        void* stream) {
    if (G < 0 || K < 0 || N < 0 || (K % pk::kBK) != 0 || (N % pk::kTileN) != 0) return B200MOE_ERR_SHAPE;
    if (G == 0 || K == 0 || N == 0) return B200MOE_OK;
    if (weight == nullptr || packed == nullptr) return B200MOE_ERR_NULL_POINTER;
    if (!aligned16(weight) || !aligned16(packed)) return B200MOE_ERR_ALIGNMENT;
    const long long n_units = (long long)G * K * N / 16;
    const long long blocks = (n_units + 255) / 256;
    if (K > 0x7FFFFFF0LL || N > 0x7FFFFFF0LL || blocks > 0x7FFFFFFFLL) return B200MOE_ERR_SHAPE;
    pk::pack_weight_int8_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const int8_t*>(weight), static_cast<uint4*>(packed), (int)K, (int)N, gate_up != 0, n_units);
    B200MOE_CUDA_TRY(cudaGetLastError());
    return B200MOE_OK;
}

static int packed_launch(const void* x, const void* packed, const void* scale, const void* offset,
                         const float* x_rowsum, const int64_t* group_list, void* y, const int64_t* row_code,
                         void* const* dst_base, int64_t n_base,
                         int64_t dst_rows, int64_t M, int64_t K, int64_t N, int64_t G, int group_list_type, int gate_up_silu,
                         void* workspace, size_t workspace_bytes, void* stream) {
    if (group_list_type != B200MOE_GROUP_LIST_CUMSUM && group_list_type != B200MOE_GROUP_LIST_COUNTS)
        return B200MOE_ERR_ARGUMENT;
    if (M < 0 || K <= 0 || N <= 0 || G <= 0 || G > kMaxExperts || M > 0x7FFFFFF0LL || K > 0x7FFFFFF0LL ||
        N > 0x7FFFFFF0LL || G * (N / pk::kTileN) * (M / 16 + 2) > 0x7FFFFFF0LL)
        return B200MOE_ERR_SHAPE;
    if ((K % pk::kBK) != 0 || (N % pk::kTileN) != 0) return B200MOE_ERR_SHAPE;
    if (row_code != nullptr && (gate_up_silu || n_base < 1 || n_base > 8 || dst_rows < 0 || dst_base == nullptr))
        return B200MOE_ERR_ARGUMENT;
    if (M == 0) return B200MOE_OK;
    if (!x || !packed || !scale || !group_list || (!y && !row_code)) return B200MOE_ERR_NULL_POINTER;
    if (!aligned16(x) || !aligned16(packed) || !aligned16(scale) || (y && !aligned16(y)) || (offset && !aligned16(offset)))
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
    a.y = static_cast<__nv_bfloat16*>(y);
    a.M = (int)M; a.K = (int)K; a.N = (int)N; a.G = (int)G;
    a.gl_type = group_list_type;
    a.status = static_cast<int*>(workspace);
    if (row_code != nullptr) {
        a.row_code = reinterpret_cast<const long long*>(row_code);
        a.n_base = (int)n_base;
        a.dst_rows = dst_rows;
        for (int i = 0; i < (int)n_base; ++i) {
            if (dst_base[i] == nullptr) return B200MOE_ERR_NULL_POINTER;
            if (!aligned16(dst_base[i])) return B200MOE_ERR_ALIGNMENT;
            a.dst_base[i] = static_cast<__nv_bfloat16*>(dst_base[i]);
        }
    }
    if (offset != nullptr) {
        a.offset = static_cast<const __nv_bfloat16*>(offset);
        if (x_rowsum != nullptr) {
            a.rowsum = x_rowsum;  // the caller already has the fp32 sums of the rows of x (e.g. from the row gather)
        } else {
            float* rowsum = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + B200MOE_STATUS_BYTES);
            launch_rowsum(x, rowsum, M, K, group_list, G, group_list_type, s);
            B200MOE_CUDA_TRY(cudaGetLastError());
            a.rowsum = rowsum;
        }
    }
    CUtensorMap tx, txs;
    int rc = make_tensor_map_2d(&tx, x, 2, (uint64_t)M, (uint64_t)K, pk::kBigBox, pk::kBK, true);
    if (rc != B200MOE_OK) return rc;
    rc = make_tensor_map_2d(&txs, x, 2, (uint64_t)M, (uint64_t)K, pk::kSmallBox, pk::kBK, true);
    if (rc != B200MOE_OK) return rc;
    const size_t smem = 1024 + (size_t)pk::kXStages * pk::kXSlotBytes + pk::kStageTileBytes + pk::kBarrierBytes +
                        (size_t)pk::kEpiWarps * pk::kEpiStripBytes + sizeof(int) * 2 * (size_t)(G + 1);
    if (gate_up_silu) {
        B200MOE_CUDA_TRY(cudaFuncSetAttribute(pk::grouped_gemm_packed_kernel<true>,
                                              cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        pk::grouped_gemm_packed_kernel<true><<<pk::grid_ctas(), pk::kThreads, smem, s>>>(tx, txs, static_cast<const uint8_t*>(packed), a);
    } else {
        B200MOE_CUDA_TRY(cudaFuncSetAttribute(pk::grouped_gemm_packed_kernel<false>,
                                              cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        pk::grouped_gemm_packed_kernel<false><<<pk::grid_ctas(), pk::kThreads, smem, s>>>(tx, txs, static_cast<const uint8_t*>(packed), a);
    }
    B200MOE_CUDA_TRY(cudaGetLastError());
    return B200MOE_OK;
}

extern "C" int b200moe_grouped_gemm_int8_packed(const void* x, const void* packed, const void* scale, const void* offset,
                                                const int64_t* group_list, void* y, int64_t M, int64_t K, int64_t N,
                                                int64_t G, int group_list_type, int gate_up_silu, void* workspace,
                                                size_t workspace_bytes, void* stream) {
    return packed_launch(x, packed, scale, offset, nullptr, group_list, y, nullptr, nullptr, 0, 0, M, K, N, G, group_list_type,
                         gate_up_silu, workspace, workspace_bytes, stream);
}

extern "C" int b200moe_grouped_gemm_int8_packed_rowsum(const void* x, const void* packed, const void* scale,
                                                       const void* offset, const float* x_rowsum, const int64_t* group_list,
                                                       void* y, int64_t M, int64_t K, int64_t N, int64_t G,
                                                       int group_list_type, int gate_up_silu, void* workspace,
                                                       size_t workspace_bytes, void* stream) {
    if (offset != nullptr && x_rowsum == nullptr) return B200MOE_ERR_NULL_POINTER;
    return packed_launch(x, packed, scale, offset, x_rowsum, group_list, y, nullptr, nullptr, 0, 0, M, K, N, G,
                         group_list_type, gate_up_silu, workspace, workspace_bytes, stream);
}

extern "C" int b200moe_grouped_gemm_int8_packed_scatter(const void* x, const void* packed, const void* scale,
                                                        const void* offset, const int64_t* group_list,
                                                        const int64_t* row_code, void* const* dst_base, int64_t n_base,
                                                        int64_t dst_rows, int64_t M, int64_t K, int64_t N, int64_t G,
                                                        int group_list_type, void* workspace, size_t workspace_bytes,
                                                        void* stream) {
    if (row_code == nullptr) return B200MOE_ERR_NULL_POINTER;
    return packed_launch(x, packed, scale, offset, nullptr, group_list, nullptr, row_code, dst_base, n_base, dst_rows, M, K, N, G,
                         group_list_type, 0, workspace, workspace_bytes, stream);
}
