/*
 * b200moe.h -- C ABI of the B200 (sm_100a) MoE expert-GEMM hot path.
 *
 * Drop-in boundary for the three operators the chitu engine calls through the reference's
 * `cinfer_ascendc` extension.  Every entry point takes plain device pointers and sizes, launches
 * asynchronously on the given CUDA stream (a `cudaStream_t` passed as `void*`; NULL = default
 * stream), never synchronises, never allocates device memory (the caller passes a workspace),
 * and returns 0 on success or a B200MOE_ERR_* code when the arguments are rejected (nothing is
 * launched in that case).  Outputs are caller-allocated and written in place; output rows owned
 * by no expert are left untouched, exactly as the reference operators do.
 *
 * Reference interfaces replaced (paths inside the reference project):
 *   b200moe_grouped_gemm       grouped_gemm/src/grouped_gemm.h:12-16 (GroupedGemm), which calls
 *                              aclnnGroupedMatmulAntiquantGetWorkspaceSize + aclnnGroupedMatmulAntiquant
 *                              (grouped_gemm/src/grouped_gemm.cpp:145-159); python name
 *                              `grouped_gemm` in pybind.cpp:17-19
 *   b200moe_grouped_gemm_workspace_bytes
 *                              the workspace half of that two-phase call
 *                              (grouped_gemm/op_host/grouped_matmul_antiquant_tiling.cpp:413-460)
 *   b200moe_grouped_gemv       grouped_soft_gemv/src/grouped_soft_gemv.h:12-14 (GroupedSoftGemv),
 *                              python name `grouped_soft_gemv` in pybind.cpp:14-16
 *   b200moe_fp4_dequant        the dequant phase of the GEMM kernel
 *                              (grouped_gemm/op_kernel/antiquant_impl.h:210-251) as a standalone op
 *   b200moe_fp4_layout         weight pre-shuffle the reference tests apply on the host
 *                              (grouped_gemm/test/python/test_group_gemm_fp4.py:129-142)
 */
#ifndef B200MOE_H_
#define B200MOE_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ---------------------------------------------------------------------- */
enum {
    B200MOE_OK = 0,
    B200MOE_ERR_COMPUTE_TYPE = 1, /* not one of the B200MOE_CT_* values                     */
    B200MOE_ERR_NULL_POINTER = 2, /* a required pointer is NULL                              */
    B200MOE_ERR_SHAPE = 3,        /* negative size, or K/N not a multiple the mode requires:
                                     fp8 K % 128 and N % 128 (as the reference); fp4 / int8 / bf16
                                     K % 64 and N % 256; int4 K % 128 and N % 256                */
    B200MOE_ERR_ALIGNMENT = 4,    /* a pointer is not 16-byte aligned                        */
    B200MOE_ERR_WORKSPACE = 5,    /* workspace missing or smaller than *_workspace_bytes()   */
    B200MOE_ERR_ARGUMENT = 6,     /* invalid enum value (group_list_type, layout, ...)       */
    B200MOE_ERR_CUDA = 7,         /* a CUDA runtime / driver call failed at launch           */
    B200MOE_ERR_UNSUPPORTED = 8,  /* valid request this build does not implement             */
    B200MOE_ERR_NOALLOC_LIMIT = 9 /* more rows than the allocation-free entry point can hold  */
};

/* ---- compute types (the reference's `computeType` string) ------------------------------- */
enum {
    B200MOE_CT_FP8 = 0,  /* "fp8": uint8 e4m3 codes [G,K,N], fp32 scale [G,K/128,N/128]      */
    B200MOE_CT_FP4 = 1,  /* "fp4": e2m1 pairs [G,K,N/2] (low nibble = even n), bf16 scale
                                   [G,K/16,N]                                                */
    B200MOE_CT_INT8 = 2, /* "int8": int8 [G,K,N], bf16 scale/offset [G,N]: (W+offset)*scale  */
    B200MOE_CT_INT4 = 3, /* "int4": two's-complement pairs [G,K,N/2], bf16 scale/offset
                                   [G,K/128,N]                                               */
    B200MOE_CT_BF16 = 4  /* "bf16": bf16 weights [G,K,N], no scale (grouped GEMM only): the
                                   matmul phase of the reference kernel on its own,
                                   grouped_gemm/op_kernel/grouped_matmul.h:409-463            */
};

enum { B200MOE_GROUP_LIST_CUMSUM = 0, B200MOE_GROUP_LIST_COUNTS = 1 };
/* fp4 weights only: CANONICAL = [G,K,N/2], low nibble = even column; ASCEND = the reference's
 * pre-shuffled stored order (b200moe_fp4_layout converts).  Both kernels read either in place. */
enum { B200MOE_LAYOUT_CANONICAL = 0, B200MOE_LAYOUT_ASCEND = 1 };
enum { B200MOE_FP4_SCALE_NONE = 0, B200MOE_FP4_SCALE_E8M0_PER32 = 1 };

/* Device-side status words live in the first 256 bytes of every workspace:
 *   word 0: 0 = ok; 1 = group_list invalid (not monotone / exceeds M; rows were clamped);
 *           2 = a bounded pipeline wait expired inside a kernel (results are incomplete)
 *   word 1: detail (expert index or barrier id)
 *   words 2, 3: used by the kernels
 *   words 4, 5: the first non-zero (word 0, word 1) of any call that used this workspace since the
 *           caller last zeroed them.  Every entry point zeroes words 0 to 3 before its launch and never
 *           words 4, 5: a binding that reuses one workspace reads them at its own synchronisation points
 *           (b200moe_read_sticky_status) instead of after every call. */
#define B200MOE_STATUS_BYTES 256

/* Grouped GEMM for prefill-sized expert batches:
 *   y[r0_g:r1_g, :] = bf16( x[r0_g:r1_g, :] @ dequant(weight[g]) ), fp32 accumulation.
 * x: bf16 [M,K] row-major; y: bf16 [M,N] row-major; group_list: int64 [G] on the device,
 * cumulative row boundaries (type 0, reference behaviour) or per-expert counts (type 1).
 * fp8/fp4: dequantised weights are rounded to bf16 before the product (reference semantics),
 * `offset` is accepted and ignored.  int8: exact integer weights on the tensor cores, scale and
 * offset applied in the fp32 epilogue; offset may be NULL (= 0). */
int b200moe_grouped_gemm(const void* x, const void* weight, const void* scale, const void* offset,
                         const int64_t* group_list, void* y, int64_t M, int64_t K, int64_t N, int64_t G,
                         int compute_type, int group_list_type, int weight_layout, void* workspace,
                         size_t workspace_bytes, void* stream);

size_t b200moe_grouped_gemm_workspace_bytes(int64_t M, int64_t K, int64_t N, int64_t G, int compute_type,
                                            int weight_layout);

/* Gate / up projection of a gated FFN with SiLU(gate) * up fused into the epilogue (int8 weights;
 * no reference counterpart: the reference ships the GEMM only and chitu applies the activation in a
 * separate operator).  weight int8 [G, K, N] with N = 2 * I and the gate and up columns interleaved
 * in blocks of 128: columns [256 b, 256 b + 128) are gate columns [128 b, 128 b + 128) and columns
 * [256 b + 128, 256 b + 256) the up columns of the same indices; scale / offset [G, N] in the same
 * order.  out bf16 [M, I]: out[m, j] = bf16(silu(g) * u) with g, u the bf16-rounded products
 * b200moe_grouped_gemm would have written for gate column j and up column j, so the result equals
 * b200moe_grouped_gemm followed by b200moe_silu_mul bit for bit.  Workspace as for
 * b200moe_grouped_gemm with compute_type int8. */
int b200moe_grouped_gemm_int8_silu(const void* x, const void* weight, const void* scale, const void* offset,
                                   const int64_t* group_list, void* out, int64_t M, int64_t K, int64_t N, int64_t G,
                                   int group_list_type, void* workspace, size_t workspace_bytes, void* stream);

/* Int8 grouped GEMM on weights repacked once into a tile order (no reference counterpart: the
 * reference reads [G, K, N] on every call; a caller that keeps expert weights resident, like the MoE
 * layer, repacks them at load time).  In the packed order every dequantised weight tile is written by
 * the kernel straight into tensor memory as the MMA's A operand (lanes = weight columns), the token
 * rows of an expert are the MMA's N extent (rounded up to 16, at most 160 per tile), and shared memory
 * carries only the x tiles.
 *   b200moe_pack_weight_int8: weight int8 [G, K, N] -> packed, G*K*N bytes, K % 64 == 0,
 *     N % 256 == 0.  gate_up != 0: N = 2 * I with the gate columns first; a tile then pairs 128 gate
 *     columns with the up columns of the same indices.  src and dst must not overlap.
 *   b200moe_grouped_gemm_int8_packed: same results as b200moe_grouped_gemm with compute_type int8
 *     (gate_up_silu == 0, packed with gate_up == 0; y bf16 [M, N]) or as b200moe_grouped_gemm
 *     followed by b200moe_silu_mul (gate_up_silu != 0, packed with gate_up != 0; y bf16 [M, N / 2]).
 *     scale / offset bf16 [G, N] in the ORIGINAL column order.  Workspace as for
 *     b200moe_grouped_gemm with compute_type int8. */
int b200moe_pack_weight_int8(const void* weight, void* packed, int64_t G, int64_t K, int64_t N, int gate_up,
                             void* stream);
int b200moe_grouped_gemm_int8_packed(const void* x, const void* packed, const void* scale, const void* offset,
                                     const int64_t* group_list, void* y, int64_t M, int64_t K, int64_t N, int64_t G,
                                     int group_list_type, int gate_up_silu, void* workspace, size_t workspace_bytes,
                                     void* stream);
/* The same for a caller that already holds x_rowsum fp32 [M], the sum of each row of x (needed for the offset
 * term; b200moe_gather_rows_sum produces it while it gathers the rows): the launch then makes no pass of its
 * own over x.  x_rowsum may be NULL only when offset is.  (No reference counterpart.) */
int b200moe_grouped_gemm_int8_packed_rowsum(const void* x, const void* packed, const void* scale, const void* offset,
                                            const float* x_rowsum, const int64_t* group_list, void* y, int64_t M,
                                            int64_t K, int64_t N, int64_t G, int group_list_type, int gate_up_silu,
                                            void* workspace, size_t workspace_bytes, void* stream);

/* b200moe_grouped_gemm_int8_packed (gate_up_silu == 0) whose result rows go where a table says instead of
 * into one [M, N] tensor (no reference counterpart; it is the down projection of an expert-parallel layer
 * handing each row straight back to the rank the token came from, over NVLink, while the GEMM is still
 * running): row r of the product is stored at dst_base[row_code[r] >> 32] + (row_code[r] & 0xffffffff) * N
 * elements.  row_code int64 [M] on the device; dst_base: n_base (<= 8) device pointers, each to bf16
 * [dst_rows, N], which may be another GPU's memory mapped into this process (plain 2-byte stores, 64
 * contiguous bytes per warp; no TMA, no multicast).  A code whose base index is >= n_base or whose row
 * index is >= dst_rows is skipped.  Every thread issues a system-scope fence after the stores of a tile,
 * so a signal posted by a later kernel on the stream covers them. */
int b200moe_grouped_gemm_int8_packed_scatter(const void* x, const void* packed, const void* scale, const void* offset,
                                             const int64_t* group_list, const int64_t* row_code, void* const* dst_base,
                                             int64_t n_base, int64_t dst_rows, int64_t M, int64_t K, int64_t N, int64_t G,
                                             int group_list_type, void* workspace, size_t workspace_bytes, void* stream);

/* Number of multiprocessors the persistent packed-weight GEMM kernels leave free (default 0: one CTA on
 * every SM).  For callers that run other kernels BESIDE a grouped GEMM -- the expert-parallel layer stores
 * the next step's tokens into their owners' memory on a second stream while the current step's GEMMs run;
 * a persistent CTA fills an SM's register file, so those kernels need SMs of their own.  Process-wide,
 * takes effect for launches made after the call; values outside [0, SM count - 1] are clamped.  Returns
 * the previous value.  (No reference counterpart.) */
int b200moe_set_gemm_reserved_sms(int n);

/* Allocation-free int8 grouped GEMM.  (No counterpart in the reference: its host binding always
 * obtains a workspace with aclrtMalloc.)  For callers that must not allocate device memory -- a
 * plug-in running inside another framework's step whose allocator owns all device memory, or a
 * serving loop that forbids allocation after start-up -- and so cannot hand the regular entry
 * point a workspace.  Same arguments and results as
 * b200moe_grouped_gemm with compute_type int8 and the canonical layout, minus the workspace: the
 * scratch (status words, one fp32 row sum per row of x) lives in a fixed array inside the library,
 * 256 B + 4 B x b200moe_grouped_gemm_int8_noalloc_max_rows() = 256.25 KiB held on every GPU that
 * loads the library, until the process exits.  M beyond that limit returns
 * B200MOE_ERR_NOALLOC_LIMIT and launches nothing.  The call performs no cudaMalloc / cudaFree and
 * uses no allocating library routine.  The FIRST call on each device does set-up work that is not
 * allocation-free: it looks up the array's device address (cudaGetSymbolAddress) and, being the
 * first launch of the kernel there, makes the driver load the kernel image (with the array in it),
 * which takes device memory.  So make one warm-up call per device before the phase in which nothing
 * may be allocated, and before any stream capture begins.  The looked-up address is cached per
 * device for the life of the process; it does not survive a device reset.  All calls
 * share the one array: calls that overlap on the GPU (different streams) race on it; serialise
 * them.  The device status words of the last call can be read with b200moe_noalloc_read_status. */
int b200moe_grouped_gemm_int8_noalloc(const void* x, const void* weight, const void* scale, const void* offset,
                                      const int64_t* group_list, void* y, int64_t M, int64_t K, int64_t N,
                                      int64_t G, int group_list_type, void* stream);
int64_t b200moe_grouped_gemm_int8_noalloc_max_rows(void);
/* Copies the two device status words left by the last allocation-free call on the current device to
 * the host (synchronises the stream). */
int b200moe_noalloc_read_status(int32_t out[2], void* stream);

/* Grouped GEMV for decode-sized expert batches (any number of rows per expert is accepted;
 * it is bandwidth-optimal up to 4 rows per expert).  Dequantised weights stay fp32, x is
 * widened to fp32, one final round to bf16.  `offset` only for int8/int4 (may be NULL).
 * fp4: a short first kernel writes x as f16 into the workspace, each row scaled by a power of two, and the
 * multiply-adds then run on the tensor core -- for the rows where that copy is exact (every element within about
 * 2^-32 of the row's largest; x' * e2m1 products are then exact, as in fp32); other rows, and rows with an infinity
 * or a NaN, go through fp32 multiply-adds in a second kernel.  Same results either way up to summation order. */
int b200moe_grouped_gemv(const void* x, const void* weight, const void* scale, const void* offset,
                         const int64_t* group_list, void* y, int64_t M, int64_t K, int64_t N, int64_t G,
                         int compute_type, int group_list_type, int weight_layout, void* workspace,
                         size_t workspace_bytes, void* stream);

size_t b200moe_grouped_gemv_workspace_bytes(int64_t M, int64_t K, int64_t N, int64_t G, int compute_type,
                                            int weight_layout);

/* Standalone FP4(e2m1) -> BF16.  codes: n_elems/2 bytes, low nibble = even element; scale:
 * one e8m0 byte per 32 consecutive elements (scale_kind 1) or NULL (scale_kind 0);
 * out: n_elems bf16.  n_elems must be a multiple of 32.  Bit-exact. */
int b200moe_fp4_dequant(const void* codes, const void* scale_e8m0, void* out_bf16, int64_t n_elems,
                        int scale_kind, void* stream);

/* The reference's two weight formats dequantised on their own: the dequant phase of its GEMM kernel
 * (grouped_gemm/op_kernel/grouped_matmul_antiquant.h:632-654 writes exactly these bf16 weights to
 * its workspace), bit-exact against the reference's Python goldens.
 *   fp4: codes [G,K,N/2] (canonical or stored order), bf16 scale [G,K/16,N]:
 *        out[g,k,n] = rne_bf16(e2m1(code) * scale[g,k/16,n])        antiquant_impl.h:23-85,146-169,210-251
 *   fp8: uint8 codes [G,K,N], fp32 scale [G,K/128,N/128]:
 *        out[g,k,n] = rne_bf16(e4m3(code) * scale[g,k/128,n/128])   antiquant_impl.h:87-129,171-208,253-266
 * out: bf16 [G,K,N].  fp4: K % 64 == 0, N % 256 == 0; fp8: K % 128 == 0, N % 128 == 0. */
int b200moe_fp4_dequant_bf16_scale(const void* codes, const void* scale, void* out_bf16, int64_t G, int64_t K, int64_t N,
                                   int weight_layout, void* stream);
int b200moe_fp8_dequant(const void* codes, const float* scale, void* out_bf16, int64_t G, int64_t K, int64_t N,
                        void* stream);

/* Two-level FP4 scale fold, the preparation the reference's test applies on the host
 * (grouped_gemm/test/python/test_group_gemm_fp4.py:86-94 and the transpose of :186): block_scale bf16
 * [G, N, KB] (one per 16 k, KB = K/16) times the expert's fp32 global scale -- global_scale fp32
 * [G, n_global], n_global 1 (whole expert) or 2 (first / second half of the N rows, i.e. gate / up) --
 * rounded to bf16 and written [G, KB, N], the scale tensor the fp4 operators take. */
int b200moe_fp4_scale_fold(const void* block_scale, const float* global_scale, void* out, int64_t G, int64_t N, int64_t KB,
                           int64_t n_global, void* stream);

/* FP4 weight layout conversion, [G,K,N/2] bytes: to_ascend != 0 canonical -> stored ("ascend")
 * order, 0 the inverse.  src and dst must not overlap. */
int b200moe_fp4_layout(const void* src, void* dst, int64_t G, int64_t K, int64_t N, int to_ascend, void* stream);

/* Small kernels the MoE layer needs around the two GEMMs (no reference counterpart: the
 * reference ships only the two operators; these belong to the benchmark's layer configuration). */
/* out[r, i] = bf16( silu(h[r, i]) * h[r, I + i] ), h bf16 [rows, 2I], out bf16 [rows, I]. */
int b200moe_silu_mul(const void* h, void* out, int64_t rows, int64_t inter, void* stream);
/* dst[i, :] = src[index[i], :] for i < n_rows (bf16 rows of `width` elements, int32 index). */
int b200moe_gather_rows(const void* src, const int32_t* index, void* dst, int64_t n_rows, int64_t width,
                        void* stream);
/* The same, and rowsum[i] = the fp32 sum of row i's elements, bit for bit what the int8 grouped GEMMs compute for
 * their offset term (b200moe_grouped_gemm_int8_packed_rowsum takes it and skips that pass over x). */
int b200moe_gather_rows_sum(const void* src, const int32_t* index, void* dst, float* rowsum, int64_t n_rows,
                            int64_t width, void* stream);
/* out[t, :] = bf16( sum_j weight[t, j] * y[slot[t, j], :] ), y bf16 [*, width], slot int32 [T, top_k],
 * weight fp32 [T, top_k]; top_k <= 32. */
int b200moe_combine(const void* y, const int32_t* slot, const float* weight, void* out, int64_t n_tokens,
                    int64_t top_k, int64_t width, void* stream);

/* Router of the MoE layer: softmax over the experts -> top_k -> weights renormalised to sum 1
 * (ties go to the lower expert index), and the sort of the (token, j) pairs by expert.
 * logits bf16 [T, E] (E <= 1024); outputs: idx int32 [T, top_k], weight fp32 [T, top_k],
 * counts int64 [E] (rows per expert, usable as a counts group_list), token_of int32 [T*top_k]
 * (source token of each sorted row), slot int32 [T, top_k] (sorted position of each pair; the order
 * inside an expert is arbitrary).  scratch: 2*E int32. */
int b200moe_moe_route(const void* logits, int64_t n_tokens, int64_t n_experts, int64_t top_k, int32_t* idx,
                      float* weight, int64_t* counts, int32_t* token_of, int32_t* slot, int32_t* scratch, void* stream);
/* Expert-parallel regroup index: recv_counts int64 [world, e_local] = rows received per (source
 * rank, local expert), in arrival order; pos[i] = expert-major position of received row i, inv its
 * inverse, local_counts int64 [e_local] the rows per local expert.  world*e_local <= 1024. */
int b200moe_moe_regroup_index(const int64_t* recv_counts, int64_t world, int64_t e_local, int32_t* pos, int32_t* inv,
                              int64_t* local_counts, void* stream);

/* ---- expert-parallel token exchange over NVLink peer memory ----------------------------------
 * (No reference counterpart: the reference ships the two operators only; chitu exchanges tokens
 * with its own collectives.  These entry points are the exchange steps of the benchmark's MoE layer
 * written as kernels that store token rows into, and load result rows from, the memory of the rank
 * that owns the expert -- no collective library call, staging copy or host synchronisation inside a
 * step.)  Every rank of one node owns four buffers that all ranks can address (b200moe_ipc_*):
 *   recv_x  bf16 [cap_rows, hidden]   rows routed to this rank's experts, expert-major
 *   y       bf16 [cap_rows, hidden]   the rows its experts produced, same positions
 *   counts  int32 [world, n_experts]  rows per (source rank, expert)
 *   signal  uint64 [3, B200MOE_EP_MAX_WORLD]  step numbers: counts / rows / results, one per source
 * `step` is a number that grows by one per layer pass, starting at 1 (the buffers start zeroed).
 * A caller that wants identical arguments in every pass (to record the pass once and replay it)
 * passes step 0 everywhere: b200moe_ep_post_counts then opens a step by incrementing
 * *step_counter on the device and the other calls read it.
 * Waits inside the kernels are bounded (2 s): on expiry status word 0 of `status` becomes 2 and the
 * kernels carry on without faulting.  world <= B200MOE_EP_MAX_WORLD, n_experts % world == 0,
 * n_experts <= 1024, cap_rows * world < 2^31. */
#define B200MOE_EP_MAX_WORLD 8
#define B200MOE_IPC_HANDLE_BYTES 64
typedef struct b200moe_ep_comm {
    int32_t world, rank, n_experts;
    int32_t dispatch_ctas;  /* 0 = as many CTAs as the rows call for (up to 4 per SM); > 0 = at most this many, for
                             * a dispatch that runs beside a grouped GEMM on the SMs that kernel leaves free */
    int64_t cap_rows, hidden;
    void* peer_recv_x[B200MOE_EP_MAX_WORLD];
    void* peer_y[B200MOE_EP_MAX_WORLD];
    int32_t* peer_counts[B200MOE_EP_MAX_WORLD];
    uint64_t* peer_signal[B200MOE_EP_MAX_WORLD];
    int32_t* status;        /* local device memory, >= 2 words, zeroed by the caller */
    uint64_t* step_counter; /* local device memory, one word, zeroed by the caller (see `step`) */
    /* Optional (all NULL = not used): results pushed back by the owner's down projection instead of being
     * fetched by b200moe_ep_combine.  Every rank owns
     *   ret       bf16 [cap_send, hidden]  one row per (token, j) pair this rank dispatched, in its sorted order
     *   ret_code  int64 [cap_rows]         for the row at each position of this rank's recv_x: the source rank
     *                                      << 32 | the row's index in the source's sorted order
     * b200moe_ep_dispatch fills ret_code next to every row it delivers; b200moe_grouped_gemm_int8_packed_scatter
     * stores each result row at ret[index] of its source rank; the source then combines locally
     * (b200moe_ep_wait for the results signal, b200moe_combine over its own ret). */
    void* peer_ret[B200MOE_EP_MAX_WORLD];
    int64_t* peer_ret_code[B200MOE_EP_MAX_WORLD];
    int64_t cap_send;
    /* Optional (all NULL = not used): recv_sum fp32 [cap_rows] on every rank; b200moe_ep_dispatch stores the fp32 sum
     * of every row it delivers at the row's position (the bits b200moe_grouped_gemm_int8_packed_rowsum wants as
     * x_rowsum), so the owner's gate/up GEMM makes no pass of its own over the received rows. */
    float* peer_recv_sum[B200MOE_EP_MAX_WORLD];
} b200moe_ep_comm;
enum { B200MOE_EP_SIG_COUNTS = 0, B200MOE_EP_SIG_ROWS = 1, B200MOE_EP_SIG_RESULTS = 2 };

/* counts int64 [n_experts] (this rank's rows per expert, as b200moe_moe_route returns them) ->
 * row `rank` of every rank's count table, then the counts signal. */
int b200moe_ep_post_counts(const b200moe_ep_comm* comm, const int64_t* counts, uint64_t step, void* stream);
/* Waits for every rank's counts, then stores row x[token_of[i], :] of each of this rank's n_rows
 * sorted rows into the owner's recv_x and signals every rank.  Outputs (local): remote_pos int32
 * [n_rows] = owner * cap_rows + position (-1 if the owner's buffer is full), local_counts int64
 * [n_experts / world] = rows per own expert (a counts group_list), n_recv int64 [1] = their sum.
 * done_counter: int32 [1], zero before the first call. */
int b200moe_ep_dispatch(const b200moe_ep_comm* comm, const void* x, const int32_t* token_of, int64_t n_rows,
                        uint64_t step, int32_t* remote_pos, int64_t* local_counts, int64_t* n_recv,
                        int32_t* done_counter, void* stream);
/* One small kernel that waits until every rank has signalled `which` for `step`. */
int b200moe_ep_wait(const b200moe_ep_comm* comm, int which, uint64_t step, void* stream);
/* Signals `which` for `step` to every rank (everything this stream wrote before is visible first). */
int b200moe_ep_post(const b200moe_ep_comm* comm, int which, uint64_t step, void* stream);
/* The end of a step whose results were pushed (b200moe_grouped_gemm_int8_packed_scatter), in one launch: signals
 * this rank's results for `step` (its pushes, made earlier on the stream, are complete), waits for every rank's
 * results signal, then out[t, :] = bf16(sum_j weight[t, j] * ret[slot[t, j], :]) over this rank's own return
 * buffer `ret` -- b200moe_ep_post + b200moe_ep_wait + b200moe_combine.  n_tokens >= 1 (the launch carries the
 * signal), top_k <= 32. */
int b200moe_ep_finish(const b200moe_ep_comm* comm, const void* ret, const int32_t* slot, const float* weight, void* out,
                      int64_t n_tokens, int64_t top_k, uint64_t step, void* stream);
/* Waits for every rank's results signal, then out[t, :] = bf16(sum_j weight[t, j] * y_owner[pos, :])
 * with (owner, pos) = remote_pos[slot[t, j]]. */
int b200moe_ep_combine(const b200moe_ep_comm* comm, const int32_t* remote_pos, const int32_t* slot,
                       const float* weight, void* out, int64_t n_tokens, int64_t top_k, uint64_t step, void* stream);
/* b200moe_silu_mul over the first *n_rows rows, the count read on the device. */
int b200moe_silu_mul_dyn(const void* h, void* out, const int64_t* n_rows, int64_t inter, void* stream);

/* Device buffers that other processes of the node can map.  alloc: cudaMalloc + zero fill + IPC
 * handle; open / close: map / unmap another process's buffer (peer access is enabled on demand);
 * free: release an own buffer.  These four are the only entry points that allocate. */
int b200moe_ipc_alloc(size_t bytes, void** ptr, unsigned char handle[B200MOE_IPC_HANDLE_BYTES]);
int b200moe_ipc_open(const unsigned char handle[B200MOE_IPC_HANDLE_BYTES], void** ptr);
int b200moe_ipc_close(void* ptr);
int b200moe_ipc_free(void* ptr);

/* Copies the two device status words of a workspace to the host (synchronises the stream). */
int b200moe_read_status(const void* workspace, int32_t out[2], void* stream);
/* Copies words 4, 5 (the first finding since they were last zeroed) to the host (synchronises the
 * stream); clear != 0 zeroes them afterwards. */
int b200moe_read_sticky_status(void* workspace, int32_t out[2], int clear, void* stream);

const char* b200moe_strerror(int code);
/* "major.minor" of this ABI; a binding can refuse to run against another major. */
const char* b200moe_version(void);

#ifdef __cplusplus
}
#endif
#endif /* B200MOE_H_ */
