// Arguments shared by the grouped-GEMM kernels and the launcher of the CTA-pair variant.
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

// CTA-pair (cta_group::2) kernel, grouped_gemm_pair.cu.  mode is a B200MOE_CT_* value.
int launch_grouped_gemm_pair(int mode, const void* x, const void* w, const GemmArgs& a, cudaStream_t stream);

}  // namespace b200moe
