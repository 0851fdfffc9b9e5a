// Shared device/host helpers of the b200moe kernels (sm_100a only).
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/b200moe.h"

#if defined(__CUDA_ARCH__) && (__CUDA_ARCH__ < 1000)
#error "b200moe kernels are written for sm_100a"
#endif

namespace b200moe {

// Device status words (first 16 bytes of a workspace).
constexpr int kDevOk = 0;
constexpr int kDevBadGroupList = 1;
constexpr int kDevWaitExpired = 2;

// Records a device-side finding in the status words of a workspace: words 0 / 1 (zeroed by every
// entry point before its launch) hold the code and detail of the current call, words 4 / 5 keep the
// first finding of ANY call that used this workspace since the caller last zeroed them -- a binding
// that reuses one workspace can check them at its own synchronisation points.
__device__ __forceinline__ void report_status(int* status, int code, int detail) {
    if (status == nullptr) return;
    if (atomicCAS(status, 0, code) == 0) status[1] = detail;
    if (atomicCAS(status + 4, 0, code) == 0) status[5] = detail;
}

// Largest expert count the kernels keep in shared memory.
constexpr int kMaxExperts = 1024;

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

#define B200MOE_CUDA_TRY(expr)                      \
    do {                                            \
        cudaError_t e__ = (expr);                   \
        if (e__ != cudaSuccess) {                   \
            (void)cudaGetLastError();               \
            return B200MOE_ERR_CUDA;                \
        }                                           \
    } while (0)

// Multiprocessor count of the current device (cached per device).
int sm_count();

// ---- tensor maps (driver entry point fetched through the runtime, no libcuda link) ---------
// 2-D row-major tensor [rows, cols] of `elem_bytes`-byte elements, box [box_rows, box_cols].
// swizzle128: 128-byte swizzle (box_cols * elem_bytes must be 128), else no swizzle.
int make_tensor_map_2d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t rows, uint64_t cols,
                       uint32_t box_rows, uint32_t box_cols, bool swizzle128);

// ---- small device utilities ---------------------------------------------------------------
__device__ __forceinline__ float bf16_bits_to_float(uint32_t b) { return __uint_as_float(b << 16); }

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}

__device__ __forceinline__ uint32_t mul_bf16x2(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}

// Two fp32 values in one 64-bit register for the two-wide FP32 instructions of sm_100.
typedef unsigned long long f32x2;
__device__ __forceinline__ f32x2 pack_u32x2(uint32_t lo, uint32_t hi) {
    f32x2 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
    return r;
}
__device__ __forceinline__ f32x2 pack_f32x2(float lo, float hi) {
    return pack_u32x2(__float_as_uint(lo), __float_as_uint(hi));
}
__device__ __forceinline__ float f32x2_lo(f32x2 v) { return __uint_as_float((uint32_t)v); }
__device__ __forceinline__ float f32x2_hi(f32x2 v) { return __uint_as_float((uint32_t)(v >> 32)); }
__device__ __forceinline__ f32x2 mul_f32x2(f32x2 a, f32x2 b) {
    f32x2 r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ f32x2 sub_f32x2(f32x2 a, f32x2 b) {
    f32x2 r;
    asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ f32x2 fma_f32x2(f32x2 a, f32x2 b, f32x2 c) {
    f32x2 r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}

__device__ __forceinline__ uint32_t fma_bf16x2(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t r;
    asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
    return r;
}

__device__ __forceinline__ uint32_t add_bf16x2(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("add.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}

// Eight packed FP4 e2m1 codes (nibble i = element i) -> eight bf16 values, in element order.
// The three magnitude bits of a code are dropped into bf16 bits [8:6] (two exponent LSBs and the
// mantissa MSB); read as bf16 that is value * 2^-126 including the subnormal code 0.5, so one
// exact multiply by 2^126 yields the e2m1 value.  Codes i and i+4 sit 16 bits apart and share
// one bf16x2 lane pair, which makes the sign and magnitude moves two shifts and two logic ops.
__device__ __forceinline__ void e2m1x8_to_bf16(uint32_t w, uint32_t out[4]) {
    constexpr uint32_t kTwo126 = 0x7E807E80u;
    uint32_t r[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t m = (i < 2) ? (w << (6 - 4 * i)) : (w >> (4 * i - 6));
        const uint32_t s = w << (12 - 4 * i);
        r[i] = mul_bf16x2((m & 0x01C001C0u) | (s & 0x80008000u), kTwo126);
    }
    out[0] = prmt(r[0], r[1], 0x5410);
    out[1] = prmt(r[2], r[3], 0x5410);
    out[2] = prmt(r[0], r[1], 0x7632);
    out[3] = prmt(r[2], r[3], 0x7632);
}

// Four signed int8 (one 32-bit word, byte i = element i) -> four bf16, exact.
// byte = 16*hs + lo with hs the signed high nibble; 0x4300|n is the bf16 128+n.
__device__ __forceinline__ void s8x4_to_bf16(uint32_t w, uint32_t& o01, uint32_t& o23) {
    const uint32_t lo = w & 0x0F0F0F0Fu;
    const uint32_t hi = ((w >> 4) & 0x0F0F0F0Fu) ^ 0x08080808u;  // high nibble + 8, 0..15
    const uint32_t k43 = 0x43434343u;
    const uint32_t lo01 = prmt(lo, k43, 0x4140), lo23 = prmt(lo, k43, 0x4342);
    const uint32_t hi01 = prmt(hi, k43, 0x4140), hi23 = prmt(hi, k43, 0x4342);
    // (128+h')*16 - 2304 = 16*(h'-8) - 128 ; + (128+lo) = 16*hs + lo
    constexpr uint32_t k16 = 0x41804180u;    // 16.0
    constexpr uint32_t kneg = 0xC510C510u;   // -2304.0
    o01 = add_bf16x2(fma_bf16x2(hi01, k16, kneg), lo01);
    o23 = add_bf16x2(fma_bf16x2(hi23, k16, kneg), lo23);
}

// Four signed int8 (one 32-bit word) -> four bf16, exact, in seven instructions.
// byte = low7 - 128*sign: (w & 0x7F) | 0x4300 is the bf16 128+low7 and (w & 0x80) | 0x4300 is the
// bf16 128 or 256, so one bf16x2 subtraction per two bytes yields the value.  The masks pick
// bytes 0 and 2 of the word (and 1 and 3 after a shift): `o02` holds elements (0, 2), `o13`
// elements (1, 3).
__device__ __forceinline__ void s8x4_to_bf16_even_odd(uint32_t w, uint32_t& o02, uint32_t& o13) {
    uint32_t lo, sg;
    asm("lop3.b32 %0, %1, 0x007F007F, 0x43004300, 0xEA;" : "=r"(lo) : "r"(w));  // (w & m) | c
    asm("lop3.b32 %0, %1, 0x00800080, 0x43004300, 0xEA;" : "=r"(sg) : "r"(w));
    asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(o02) : "r"(lo), "r"(sg));
    const uint32_t v = w >> 8;
    asm("lop3.b32 %0, %1, 0x007F007F, 0x43004300, 0xEA;" : "=r"(lo) : "r"(v));
    asm("lop3.b32 %0, %1, 0x00800080, 0x43004300, 0xEA;" : "=r"(sg) : "r"(v));
    asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(o13) : "r"(lo), "r"(sg));
}

// Row boundaries of every expert from the device-side group_list, clamped into [0, M] and made
// monotone so no later index can leave the tensors; a violation is reported in the status words.
// Executed by a whole CTA; row_start has G+1 entries in shared memory.  G <= kMaxExperts.
__device__ __forceinline__ void load_row_starts(const int64_t* __restrict__ gl, int G, int M, int gl_type,
                                                int* row_start, int* status) {
    // every thread fetches one entry (clamped into int range), then one thread makes the list
    // monotone: G is a few hundred and this runs once per CTA
    for (int g = threadIdx.x; g < G; g += blockDim.x) {
        long long v = gl[g];
        row_start[g + 1] = (int)(v < -1 ? -1 : (v > (long long)M + 1 ? (long long)M + 1 : v));
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int prev = 0;
        row_start[0] = 0;
        bool bad = false;
        int bad_at = 0;
        for (int g = 0; g < G; ++g) {
            const int v = row_start[g + 1];
            int end = (gl_type == B200MOE_GROUP_LIST_COUNTS) ? prev + v : v;
            if (v < 0 || end < prev || end > M) {
                if (!bad) bad_at = g;
                bad = true;
                end = (v < 0 || end < prev) ? prev : M;
            }
            row_start[g + 1] = end;
            prev = end;
        }
        if (bad) report_status(status, kDevBadGroupList, bad_at);
    }
    __syncthreads();
}

}  // namespace b200moe
