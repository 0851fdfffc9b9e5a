// Arguments shared by the grouped-GEMM kernels.
#pragma once

#include "common.cuh"

namespace b200moe {

struct GemmArgs {
    const void* scale;
    const __nv_bfloat16* offset;
    const float* rowsum;  // [M] sum_k x[m,k]; only read when offset != nullptr
    const int64_t* group_list;
    __nv_bfloat16* y;
    int M, K, N, G, gl_type;
    int* status;
};

// out[m] = sum_k x[m, k] in fp32 for the rows the group list uses (grouped_gemm.cu).
void launch_rowsum(const void* x, float* out, int64_t M, int64_t K, const int64_t* group_list, int64_t G, int gl_type,
                   cudaStream_t stream);

}  // namespace b200moe
