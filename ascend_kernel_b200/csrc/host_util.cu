// Host-side helpers: status strings, SM count, tensor-map encoding, status read-back.
#include <cudaTypedefs.h>

#include <mutex>

#include "common.cuh"

namespace b200moe {

int sm_count() {
    static int cached[64];
    static std::mutex mu;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    std::lock_guard<std::mutex> lock(mu);
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

static PFN_cuTensorMapEncodeTiled_v12000 encode_fn() {
    static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess) {
            fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
        } else {
            (void)cudaGetLastError();
        }
    });
    return fn;
}

int make_tensor_map_2d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t rows, uint64_t cols,
                       uint32_t box_rows, uint32_t box_cols, bool swizzle128) {
    auto fn = encode_fn();
    if (fn == nullptr) return B200MOE_ERR_CUDA;
    CUtensorMapDataType dt = elem_bytes == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {cols * (uint64_t)elem_bytes};
    cuuint32_t box[2] = {box_cols, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(out, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? B200MOE_OK : B200MOE_ERR_CUDA;
}

}  // namespace b200moe

extern "C" {

const char* b200moe_strerror(int code) {
    switch (code) {
        case B200MOE_OK: return "ok";
        case B200MOE_ERR_COMPUTE_TYPE: return "invalid compute type (expected fp8, fp4, int8 or int4)";
        case B200MOE_ERR_NULL_POINTER: return "a required pointer is NULL";
        case B200MOE_ERR_SHAPE: return "invalid shape for this compute type";
        case B200MOE_ERR_ALIGNMENT: return "pointer not 16-byte aligned";
        case B200MOE_ERR_WORKSPACE: return "workspace missing or too small";
        case B200MOE_ERR_ARGUMENT: return "invalid argument";
        case B200MOE_ERR_CUDA: return "CUDA call failed";
        case B200MOE_ERR_UNSUPPORTED: return "not implemented for this combination";
        case B200MOE_ERR_NOALLOC_LIMIT: return "too many rows for the allocation-free entry point (see b200moe_grouped_gemm_int8_noalloc_max_rows)";
        default: return "unknown b200moe status";
    }
}

const char* b200moe_version(void) { return "1.1"; }

int b200moe_read_status(const void* workspace, int32_t out[2], void* stream) {
    if (workspace == nullptr || out == nullptr) return B200MOE_ERR_NULL_POINTER;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    B200MOE_CUDA_TRY(cudaMemcpyAsync(out, workspace, 2 * sizeof(int32_t), cudaMemcpyDeviceToHost, s));
    B200MOE_CUDA_TRY(cudaStreamSynchronize(s));
    return B200MOE_OK;
}

int b200moe_read_sticky_status(void* workspace, int32_t out[2], int clear, void* stream) {
    if (workspace == nullptr || out == nullptr) return B200MOE_ERR_NULL_POINTER;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    B200MOE_CUDA_TRY(cudaMemcpyAsync(out, static_cast<const uint8_t*>(workspace) + 16, 2 * sizeof(int32_t),
                                     cudaMemcpyDeviceToHost, s));
    if (clear) B200MOE_CUDA_TRY(cudaMemsetAsync(static_cast<uint8_t*>(workspace) + 16, 0, 8, s));
    B200MOE_CUDA_TRY(cudaStreamSynchronize(s));
    return B200MOE_OK;
}

}  // extern "C"
