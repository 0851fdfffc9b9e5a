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
    // packed kernel only, optional: result row r goes to dst_base[row_code[r] >> 32] + (low 32 bits) * N
    // instead of y + r * N (rows handed back to the ranks they came from)
    const long long* row_code = nullptr;
    __nv_bfloat16* dst_base[8] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
    int n_base = 0;
    long long dst_rows = 0;
};

// out[m] = sum_k x[m, k] in fp32 for the rows the group list uses (grouped_gemm.cu).
void launch_rowsum(const void* x, float* out, int64_t M, int64_t K, const int64_t* group_list, int64_t G, int gl_type,
                   cudaStream_t stream);

}  // namespace b200moe
