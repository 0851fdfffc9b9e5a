// Expert-parallel token exchange over NVLink peer memory.
//
// Every rank owns four buffers that all ranks of the node can address (CUDA IPC mappings): a
// receive buffer for token rows, a result buffer for the rows its experts produced, a table of
// per-(source rank, expert) row counts and a few signal words.  A step is
//
//   post_counts   my per-expert row counts -> every rank's table, then a signal
//   dispatch      wait for all counts; every CTA derives, for each expert, where this rank's rows
//                 start in the owner's receive buffer (rows land expert-major, ordered by source
//                 rank inside an expert, so the grouped GEMM reads them without a regroup pass);
//                 one warp per row stores it straight into the owner's memory (16-byte stores over
//                 NVLink); the last CTA signals every rank
//   wait_rows     until every source rank has signalled
//   ... grouped GEMM, SiLU*up, grouped GEMM into the result buffer ...
//   post_results  signal every rank that this rank's results are complete
//   combine       wait for every owner; out[t] = sum_j w[t,j] * result row of (t,j), read from the
//                 owner's result buffer with 16-byte loads over NVLink
//
// No host synchronisation, no staging copy, and no collective library call inside a step.  Signals
// are 64-bit step numbers that only grow, so nothing is ever reset.  The count exchange of step
// n+1 doubles as the barrier that makes it safe to overwrite the buffers of step n: a rank posts
// its counts only after its own combine of step n, and nobody writes rows before it has seen the
// counts of every rank.
//
// Every wait is bounded (ptx::kWaitLimitNs): on expiry the kernel records status 2, stores no rows into
// any rank's buffers (dispatch) or treats the missing results as absent rows (combine), and still posts
// its own signals; all addresses are computed locally and clamped to the buffer capacity, so a
// missing peer can produce wrong numbers on the rank that waited but never a fault, a hang, or
// overwritten buffers on a healthy rank.  Peer memory is only
// touched with plain loads and stores (no TMA, no multicast).
#include <cstring>

#include "common.cuh"
#include "ptx.cuh"

namespace b200moe {

struct EpComm {
    int world, rank, n_experts, e_local;
    long long cap_rows;
    int width16;  // 16-byte vectors per row
    uint4* recv_x[B200MOE_EP_MAX_WORLD];
    const uint4* y[B200MOE_EP_MAX_WORLD];
    int32_t* counts[B200MOE_EP_MAX_WORLD];             // [world, n_experts] on every rank
    unsigned long long* signal[B200MOE_EP_MAX_WORLD];  // [3, B200MOE_EP_MAX_WORLD] on every rank
    int dispatch_ctas;                                 // 0, or the most CTAs the dispatch kernel may use
    int* status;                                       // local: two status words
    unsigned long long* step_counter;                  // local: the step number when the host passes 0
    long long* ret_code[B200MOE_EP_MAX_WORLD];         // optional: where each delivered row's result returns to
    float* recv_sum[B200MOE_EP_MAX_WORLD];             // optional: fp32 sum of each delivered row, beside it
};

constexpr int kSigCounts = 0, kSigRows = 1, kSigResults = 2;

__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(unsigned long long* p, unsigned long long v) {
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

// Thread s < world waits until rank s has signalled `step` in this rank's own signal block.
// Returns (to every thread) whether all arrived in time.
__device__ __forceinline__ bool ep_wait_all(const EpComm& c, int which, unsigned long long step, int id) {
    __shared__ int s_ok;
    if (threadIdx.x == 0) s_ok = 1;
    __syncthreads();
    if ((int)threadIdx.x < c.world) {
        const unsigned long long* p = c.signal[c.rank] + which * B200MOE_EP_MAX_WORLD + threadIdx.x;
        const uint64_t t0 = ptx::globaltimer_ns();
        while (ld_acquire_sys(p) < step) {
            __nanosleep(64);
            if (ptx::globaltimer_ns() - t0 > ptx::kWaitLimitNs) {
                s_ok = 0;
                if (atomicCAS(c.status, kDevOk, kDevWaitExpired) == kDevOk) c.status[1] = id * 100 + (int)threadIdx.x;
                break;
            }
        }
    }
    __syncthreads();
    return s_ok != 0;
}

// All threads' earlier writes (to any rank's memory) become visible system-wide, then thread d
// signals rank d.
__device__ __forceinline__ void ep_signal_all(const EpComm& c, int which, unsigned long long step) {
    __threadfence_system();
    __syncthreads();
    if ((int)threadIdx.x < c.world)
        st_release_sys(c.signal[threadIdx.x] + which * B200MOE_EP_MAX_WORLD + c.rank, step);
}

// The host may pass step 0: the step number then lives on the device (the counts kernel opens a
// step by incrementing it, the other kernels read it), which keeps the arguments of a whole layer
// pass constant from step to step.
__device__ __forceinline__ unsigned long long ep_step(const EpComm& c, unsigned long long step) {
    return step != 0 ? step : *c.step_counter;
}

__global__ void ep_post_counts_kernel(EpComm c, const long long* __restrict__ counts, unsigned long long step) {
    __shared__ unsigned long long s_step;
    if (threadIdx.x == 0) {
        if (step == 0) {
            step = *c.step_counter + 1;
            *c.step_counter = step;
        }
        s_step = step;
    }
    __syncthreads();
    step = s_step;
    for (int e = threadIdx.x; e < c.n_experts; e += blockDim.x) {
        const int v = (int)counts[e];
        for (int d = 0; d < c.world; ++d) c.counts[d][c.rank * c.n_experts + e] = v;
    }
    ep_signal_all(c, kSigCounts, step);
}

__global__ void ep_post_kernel(EpComm c, int which, unsigned long long step) { ep_signal_all(c, which, ep_step(c, step)); }

__global__ void ep_wait_kernel(EpComm c, int which, unsigned long long step) {
    (void)ep_wait_all(c, which, ep_step(c, step), 10 + which);
}

// The plan every CTA derives from the count table (E <= 1024):
//   s_start[e]  first of this rank's sorted rows that belongs to expert e (s_start[E] = all rows)
//   s_base[e]   position, in the owner's receive buffer, of this rank's first row of expert e
__global__ void __launch_bounds__(1024)
ep_dispatch_kernel(EpComm c, const uint4* __restrict__ x, const int32_t* __restrict__ token_of, int n_rows,
                   unsigned long long step, int32_t* __restrict__ remote_pos, long long* __restrict__ local_counts,
                   long long* __restrict__ n_recv, int* __restrict__ done_counter) {
    __shared__ int s_start[kMaxExperts + 1], s_base[kMaxExperts], s_tot[kMaxExperts], s_before[kMaxExperts];
    step = ep_step(c, step);
    // If the counts of some rank never arrive the plan below would be built from a stale table: no row is
    // stored anywhere then (a healthy peer's buffers must not be overwritten by a rank that is out of step);
    // the local outputs are still written and the rows signal is still posted, so nobody waits for this rank.
    const bool counts_ok = ep_wait_all(c, kSigCounts, step, 1);
    const int E = c.n_experts;
    const int32_t* tab = c.counts[c.rank];
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        int tot = 0, before = 0;
        for (int s = 0; s < c.world; ++s) {
            int v = tab[s * E + e];
            v = v < 0 ? 0 : v;
            tot += v;
            if (s < c.rank) before += v;
        }
        s_tot[e] = tot;
        s_before[e] = before;
        int mine = tab[c.rank * E + e];
        s_start[e + 1] = mine < 0 ? 0 : mine;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int acc = 0, run = 0;
        s_start[0] = 0;
        for (int e = 0; e < E; ++e) {
            if (e % c.e_local == 0) acc = 0;  // first expert of the next owner
            s_base[e] = acc + s_before[e];
            acc += s_tot[e];
            run += s_start[e + 1];
            s_start[e + 1] = run;
        }
    }
    __syncthreads();
    if (blockIdx.x == 0) {
        // the group list of this rank's own experts and the number of rows it receives
        long long total = 0;
        for (int e = threadIdx.x; e < c.e_local; e += blockDim.x) local_counts[e] = s_tot[c.rank * c.e_local + e];
        if (threadIdx.x == 0) {
            for (int e = 0; e < c.e_local; ++e) total += s_tot[c.rank * c.e_local + e];
            *n_recv = total < c.cap_rows ? total : c.cap_rows;
        }
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
    for (int i = blockIdx.x * wpb + warp; i < n_rows; i += gridDim.x * wpb) {
        // expert of sorted row i: the last e with s_start[e] <= i
        int lo = 0, hi = E;
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (s_start[mid] <= i) lo = mid; else hi = mid;
        }
        const int e = lo, d = e / c.e_local;
        const long long pos = (long long)s_base[e] + (i - s_start[e]);
        const bool fits = counts_ok && i < s_start[E] && pos < c.cap_rows;
        if (lane == 0) {
            remote_pos[i] = fits ? (int32_t)(d * c.cap_rows + pos) : -1;
            // the return address of the row's result: this rank, sorted position i
            if (fits && c.ret_code[d] != nullptr) c.ret_code[d][pos] = ((long long)c.rank << 32) | (unsigned int)i;
        }
        if (!fits) {
            if (counts_ok && lane == 0 && atomicCAS(c.status, kDevOk, kDevBadGroupList) == kDevOk) c.status[1] = e;
            continue;
        }
        const uint4* src = x + (long long)token_of[i] * c.width16;
        uint4* dst = c.recv_x[d] + pos * c.width16;
        // the row's fp32 sum travels with it (the owner's gate/up GEMM needs it for the offset term): added up
        // in the order of that GEMM's own row-sum pass, so the bits are the same
        float sum = 0.f;
        for (int v = lane; v < c.width16; v += 32) {
            const uint4 q = __ldg(src + v);
            dst[v] = q;
            const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) sum += __uint_as_float(w[j] << 16) + __uint_as_float(w[j] & 0xFFFF0000u);
        }
        if (c.recv_sum[d] != nullptr) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
            if (lane == 0) c.recv_sum[d][pos] = sum;
        }
    }
    // completion: the last CTA to finish signals every rank
    __threadfence_system();
    __syncthreads();
    __shared__ int s_last;
    if (threadIdx.x == 0) s_last = (atomicAdd(done_counter, 1) == (int)gridDim.x - 1);
    __syncthreads();
    if (s_last) {
        if (threadIdx.x == 0) *done_counter = 0;
        ep_signal_all(c, kSigRows, step);
    }
}

// The end of a step whose results were PUSHED to their source ranks, in one kernel: CTA 0 signals that this rank's
// own pushes (made by an earlier kernel on the stream) are complete, every CTA waits for all ranks' signals, then
// out[t, :] = bf16(sum_j weight[t, j] * ret[slot[t, j], :]) over this rank's own return buffer.  (Signal kernel,
// wait kernel and weighted-sum kernel in one launch.)  An expired wait is recorded; the sum then runs over what
// the buffer holds.
__global__ void __launch_bounds__(256) ep_finish_kernel(EpComm c, const uint4* __restrict__ ret, const int32_t* __restrict__ slot,
                                                        const float* __restrict__ weight, uint4* __restrict__ out, int top_k,
                                                        unsigned long long step) {
    step = ep_step(c, step);
    if (blockIdx.x == 0) ep_signal_all(c, kSigResults, step);
    (void)ep_wait_all(c, kSigResults, step, 3);
    const long long t = blockIdx.x;
    __shared__ long long s_off[32];
    __shared__ float s_w[32];
    if ((int)threadIdx.x < top_k) {
        s_off[threadIdx.x] = (long long)slot[t * top_k + threadIdx.x] * c.width16;
        s_w[threadIdx.x] = weight[t * top_k + threadIdx.x];
    }
    __syncthreads();
    for (int v = threadIdx.x; v < c.width16; v += blockDim.x) {
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int j0 = 0; j0 < top_k; j0 += 8) {
            uint4 q[8];
#pragma unroll
            for (int j = 0; j < 8; ++j)
                if (j0 + j < top_k) q[j] = ret[s_off[j0 + j] + v];  // (plain loads: the rows were written by other GPUs)
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                if (j0 + j < top_k) {
                    const float w = s_w[j0 + j];
                    const uint32_t vw[4] = {q[j].x, q[j].y, q[j].z, q[j].w};
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        acc[2 * k] = fmaf(w, __uint_as_float(vw[k] << 16), acc[2 * k]);
                        acc[2 * k + 1] = fmaf(w, __uint_as_float(vw[k] & 0xFFFF0000u), acc[2 * k + 1]);
                    }
                }
            }
        }
        out[t * c.width16 + v] = make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]),
                                            pack_bf16x2(acc[4], acc[5]), pack_bf16x2(acc[6], acc[7]));
    }
}

// out[t, :] = bf16(sum_j weight[t, j] * result row of pair (t, j)), the row read from its owner.
__global__ void ep_combine_kernel(EpComm c, const int32_t* __restrict__ remote_pos, const int32_t* __restrict__ slot,
                                  const float* __restrict__ weight, uint4* __restrict__ out, int top_k,
                                  unsigned long long step) {
    // results that were never signalled complete are not read: their rows count as absent
    const bool results_ok = ep_wait_all(c, kSigResults, ep_step(c, step), 2);
    const long long t = blockIdx.x;
    __shared__ const uint4* s_row[32];
    __shared__ float s_w[32];
    if ((int)threadIdx.x < top_k) {
        const int rp = remote_pos[slot[t * top_k + threadIdx.x]];
        s_row[threadIdx.x] = (rp < 0 || !results_ok) ? nullptr : c.y[rp / c.cap_rows] + (rp % c.cap_rows) * c.width16;
        s_w[threadIdx.x] = weight[t * top_k + threadIdx.x];
    }
    __syncthreads();
    for (int v = threadIdx.x; v < c.width16; v += blockDim.x) {
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        // the loads cross NVLink: eight are issued before the first is consumed
        for (int j0 = 0; j0 < top_k; j0 += 8) {
            uint4 q[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                q[j] = make_uint4(0u, 0u, 0u, 0u);
                if (j0 + j < top_k && s_row[j0 + j] != nullptr) q[j] = s_row[j0 + j][v];
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float w = j0 + j < top_k ? s_w[j0 + j] : 0.f;
                const uint32_t vw[4] = {q[j].x, q[j].y, q[j].z, q[j].w};
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    acc[2 * k] = fmaf(w, __uint_as_float(vw[k] << 16), acc[2 * k]);
                    acc[2 * k + 1] = fmaf(w, __uint_as_float(vw[k] & 0xFFFF0000u), acc[2 * k + 1]);
                }
            }
        }
        out[t * c.width16 + v] = make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]),
                                            pack_bf16x2(acc[4], acc[5]), pack_bf16x2(acc[6], acc[7]));
    }
}

// SiLU(gate) * up over the first *n_rows rows only (the receive buffer is sized for the worst case).
__global__ void silu_mul_dyn_kernel(const uint4* __restrict__ h, uint4* __restrict__ out,
                                    const long long* __restrict__ n_rows, int inter8) {
    const long long n = *n_rows * inter8;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / inter8;
        const int col = (int)(i % inter8);
        const uint4 g = h[r * (2LL * inter8) + col];
        const uint4 u = h[r * (2LL * inter8) + inter8 + col];
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
}

static int to_comm(const b200moe_ep_comm* h, EpComm* c) {
    if (h == nullptr) return B200MOE_ERR_NULL_POINTER;
    if (h->world < 1 || h->world > B200MOE_EP_MAX_WORLD || h->rank < 0 || h->rank >= h->world || h->n_experts < 1 ||
        h->n_experts > kMaxExperts || h->n_experts % h->world != 0 || h->cap_rows < 1 || h->hidden < 8 ||
        h->hidden % 8 != 0 || h->cap_rows * (long long)h->world > 0x7FFFFFF0LL)
        return B200MOE_ERR_SHAPE;
    c->world = h->world;
    c->rank = h->rank;
    c->n_experts = h->n_experts;
    c->e_local = h->n_experts / h->world;
    c->cap_rows = h->cap_rows;
    c->width16 = (int)(h->hidden / 8);
    c->dispatch_ctas = h->dispatch_ctas;
    for (int r = 0; r < h->world; ++r) {
        if (!h->peer_recv_x[r] || !h->peer_y[r] || !h->peer_counts[r] || !h->peer_signal[r]) return B200MOE_ERR_NULL_POINTER;
        if (!aligned16(h->peer_recv_x[r]) || !aligned16(h->peer_y[r])) return B200MOE_ERR_ALIGNMENT;
        c->recv_x[r] = static_cast<uint4*>(h->peer_recv_x[r]);
        c->y[r] = static_cast<const uint4*>(h->peer_y[r]);
        c->counts[r] = h->peer_counts[r];
        c->signal[r] = reinterpret_cast<unsigned long long*>(h->peer_signal[r]);
        c->ret_code[r] = reinterpret_cast<long long*>(h->peer_ret_code[r]);
        c->recv_sum[r] = h->peer_recv_sum[r];
    }
    for (int r = h->world; r < B200MOE_EP_MAX_WORLD; ++r) {
        c->ret_code[r] = nullptr;
        c->recv_sum[r] = nullptr;
    }
    if (!h->status || !h->step_counter) return B200MOE_ERR_NULL_POINTER;
    c->status = h->status;
    c->step_counter = reinterpret_cast<unsigned long long*>(h->step_counter);
    return B200MOE_OK;
}

}  // namespace b200moe

using namespace b200moe;

extern "C" int b200moe_ep_post_counts(const b200moe_ep_comm* comm, const int64_t* counts, uint64_t step, void* stream) {
    EpComm c;
    int rc = to_comm(comm, &c);
    if (rc != B200MOE_OK) return rc;
    if (!counts) return B200MOE_ERR_NULL_POINTER;
    ep_post_counts_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(c, reinterpret_cast<const long long*>(counts),
                                                                            (unsigned long long)step);
    B200MOE_CUDA_TRY(cudaGetLastError());
    return B200MOE_OK;
}

extern "C" int b200moe_ep_dispatch(const b200moe_ep_comm* comm, const void* x, const int32_t* token_of, int64_t n_rows,
                                   uint64_t step, int32_t* remote_pos, int64_t* local_counts, int64_t* n_recv,
                                   int32_t* done_counter, void* stream) {
    EpComm c;
    int rc = to_comm(comm, &c);
    if (rc != B200MOE_OK) return rc;
    if (n_rows < 0 || n_rows > 0x7FFFFFF0LL) return B200MOE_ERR_SHAPE;
    if (!x || !token_of || !remote_pos || !local_counts || !n_recv || !done_counter) return B200MOE_ERR_NULL_POINTER;
    if (!aligned16(x)) return B200MOE_ERR_ALIGNMENT;
    // one warp per row, 32 warps per CTA; at least one CTA so that the plan and the signal happen
    long long blocks = (n_rows + 31) / 32;
    const long long cap = c.dispatch_ctas > 0 ? (long long)c.dispatch_ctas : 4LL * sm_count();
    blocks = blocks < 1 ? 1 : (blocks > cap ? cap : blocks);
    ep_dispatch_kernel<<<(unsigned)blocks, 1024, 0, static_cast<cudaStream_t>(stream)>>>(
        c, static_cast<const uint4*>(x), token_of, (int)n_rows, (unsigned long long)step, remote_pos,
        reinterpret_cast<long long*>(local_counts), reinterpret_cast<long long*>(n_recv), done_counter);
    B200MOE_CUDA_TRY(cudaGetLastError());
    return B200MOE_OK;
}

extern "C" int b200moe_ep_wait(const b200moe_ep_comm* comm, int which, uint64_t step, void* stream) {
    EpComm c;
    int rc = to_comm(comm, &c);
    if (rc != B200MOE_OK) return rc;
    if (which < 0 || which > 2) return B200MOE_ERR_ARGUMENT;
    ep_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(c, which, (unsigned long long)step);
    B200MOE_CUDA_TRY(cudaGetLastError());
    return B200MOE_OK;
}

extern "C" int b200moe_ep_post(const b200moe_ep_comm* comm, int which, uint64_t step, void* stream) {
    EpComm c;
    int rc = to_comm(comm, &c);
    if (rc != B200MOE_OK) return rc;
    if (which < 0 || which > 2) return B200MOE_ERR_ARGUMENT;
    ep_post_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(c, which, (unsigned long long)step);
    B200MOE_CUDA_TRY(cudaGetLastError());
    return B200MOE_OK;
}

extern "C" int b200moe_ep_combine(const b200moe_ep_comm* comm, const int32_t* remote_pos, const int32_t* slot,
                                  const float* weight, void* out, int64_t n_tokens, int64_t top_k, uint64_t step,
                                  void* stream) {
    EpComm c;
    int rc = to_comm(comm, &c);
    if (rc != B200MOE_OK) return rc;
    if (n_tokens < 0 || n_tokens > 0x7FFFFFFFLL || top_k < 1 || top_k > 32) return B200MOE_ERR_SHAPE;
    if (!remote_pos || !slot || !weight || !out) return B200MOE_ERR_NULL_POINTER;
    if (!aligned16(out)) return B200MOE_ERR_ALIGNMENT;
    if (n_tokens == 0) {
        // nothing to combine, but the results signal must still be consumed in step order
        return b200moe_ep_wait(comm, kSigResults, step, stream);
    }
    ep_combine_kernel<<<(unsigned)n_tokens, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        c, remote_pos, slot, weight, static_cast<uint4*>(out), (int)top_k, (unsigned long long)step);
    B200MOE_CUDA_TRY(cudaGetLastError());
    return B200MOE_OK;
}

extern "C" int b200moe_ep_finish(const b200moe_ep_comm* comm, const void* ret, const int32_t* slot, const float* weight,
                                 void* out, int64_t n_tokens, int64_t top_k, uint64_t step, void* stream) {
    EpComm c;
    int rc = to_comm(comm, &c);
    if (rc != B200MOE_OK) return rc;
    if (n_tokens <= 0 || top_k <= 0 || top_k > 32 || n_tokens > 0x7FFFFFFFLL) return B200MOE_ERR_SHAPE;
    if (!ret || !slot || !weight || !out) return B200MOE_ERR_NULL_POINTER;
    if (!aligned16(ret) || !aligned16(out)) return B200MOE_ERR_ALIGNMENT;
    ep_finish_kernel<<<(unsigned)n_tokens, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        c, static_cast<const uint4*>(ret), slot, weight, static_cast<uint4*>(out), (int)top_k, (unsigned long long)step);
    B200MOE_CUDA_TRY(cudaGetLastError());
    return B200MOE_OK;
}

extern "C" int b200moe_silu_mul_dyn(const void* h, void* out, const int64_t* n_rows, int64_t inter, void* stream) {
    if (inter <= 0 || (inter % 8) != 0) return B200MOE_ERR_SHAPE;
    if (!h || !out || !n_rows) return B200MOE_ERR_NULL_POINTER;
    if (!aligned16(h) || !aligned16(out)) return B200MOE_ERR_ALIGNMENT;
    silu_mul_dyn_kernel<<<(unsigned)(8 * sm_count()), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint4*>(h), static_cast<uint4*>(out), reinterpret_cast<const long long*>(n_rows),
        (int)(inter / 8));
    B200MOE_CUDA_TRY(cudaGetLastError());
    return B200MOE_OK;
}

// ---- buffers other processes of the node can map (CUDA IPC) ------------------------------------
extern "C" int b200moe_ipc_alloc(size_t bytes, void** ptr, unsigned char handle[B200MOE_IPC_HANDLE_BYTES]) {
    static_assert(sizeof(cudaIpcMemHandle_t) == B200MOE_IPC_HANDLE_BYTES, "IPC handle size");
    if (!ptr || !handle || bytes == 0) return B200MOE_ERR_NULL_POINTER;
    void* p = nullptr;
    B200MOE_CUDA_TRY(cudaMalloc(&p, bytes));
    if (cudaMemset(p, 0, bytes) != cudaSuccess) {
        (void)cudaGetLastError();
        (void)cudaFree(p);
        return B200MOE_ERR_CUDA;
    }
    cudaIpcMemHandle_t h;
    if (cudaIpcGetMemHandle(&h, p) != cudaSuccess) {
        (void)cudaGetLastError();
        (void)cudaFree(p);
        return B200MOE_ERR_CUDA;
    }
    memcpy(handle, &h, sizeof(h));
    *ptr = p;
    return B200MOE_OK;
}

extern "C" int b200moe_ipc_open(const unsigned char handle[B200MOE_IPC_HANDLE_BYTES], void** ptr) {
    if (!ptr || !handle) return B200MOE_ERR_NULL_POINTER;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof(h));
    B200MOE_CUDA_TRY(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
    return B200MOE_OK;
}

extern "C" int b200moe_ipc_close(void* ptr) {
    if (!ptr) return B200MOE_ERR_NULL_POINTER;
    B200MOE_CUDA_TRY(cudaIpcCloseMemHandle(ptr));
    return B200MOE_OK;
}

extern "C" int b200moe_ipc_free(void* ptr) {
    if (!ptr) return B200MOE_ERR_NULL_POINTER;
    B200MOE_CUDA_TRY(cudaFree(ptr));
    return B200MOE_OK;
}
