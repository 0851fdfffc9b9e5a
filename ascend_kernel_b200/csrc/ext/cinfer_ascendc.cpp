// Python module `cinfer_ascendc`: the operator names and keyword arguments of the reference's
// extension (pybind.cpp:13-32 of the reference; GroupedGemm at grouped_gemm/src/grouped_gemm.h:12-16,
// GroupedSoftGemv at grouped_soft_gemv/src/grouped_soft_gemv.h:12-14), bound to the B200 kernels
// through the C ABI of include/b200moe.h.  This file only unpacks tensors: device/dtype/shape
// checks, the current CUDA stream, a workspace from torch's caching allocator, status -> exception.
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/extension.h>

#include <cstdio>
#include <stdexcept>
#include <string>

#include "../../../include/b200moe.h"

namespace {

int compute_type_of(const std::string& s) {
    if (s == "fp8") return B200MOE_CT_FP8;
    if (s == "fp4") return B200MOE_CT_FP4;
    if (s == "int8") return B200MOE_CT_INT8;
    if (s == "int4") return B200MOE_CT_INT4;
    // same report as the reference binding for an unknown computeType
    std::printf("Invalid compute type: %s. Supported: \"fp4\", \"fp8\", \"int8\", \"int4\"\n", s.c_str());
    throw std::runtime_error("Host tiling failed!");
}

int layout_of(const std::string& s) {
    if (s == "ascend") return B200MOE_LAYOUT_ASCEND;
    if (s == "canonical") return B200MOE_LAYOUT_CANONICAL;
    throw std::runtime_error("weight_layout must be \"ascend\" or \"canonical\"");
}

void check_tensor(const at::Tensor& t, const char* name) {
    TORCH_CHECK(t.defined(), name, " is undefined");
    TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor (there is no CPU path)");
    TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
}

void raise_on(int rc, const char* what) {
    if (rc != B200MOE_OK) {
        std::printf("%s failed. ERROR: %d (%s)\n", what, rc, b200moe_strerror(rc));
        throw std::runtime_error(std::string(what) + ": " + b200moe_strerror(rc));
    }
}

struct Dims {
    int64_t M, K, N, G;
};

Dims dims_of(const at::Tensor& x, const at::Tensor& weight, const at::Tensor& group_list, const at::Tensor& output,
             int ct) {
    TORCH_CHECK(x.scalar_type() == at::kBFloat16 && output.scalar_type() == at::kBFloat16,
                "x and output must be bfloat16");
    TORCH_CHECK(group_list.scalar_type() == at::kLong, "group_list must be int64");
    TORCH_CHECK(x.dim() == 2 && weight.dim() == 3 && output.dim() == 2, "expected x [M,K], weight [G,K,N], output [M,N]");
    TORCH_CHECK(weight.element_size() == 1, "weight must be a 1-byte container (uint8 / int8)");
    Dims d{x.size(0), x.size(1), weight.size(2), weight.size(0)};
    if (ct == B200MOE_CT_FP4 || ct == B200MOE_CT_INT4) d.N *= 2;  // two codes per byte
    TORCH_CHECK(weight.size(1) == d.K && output.size(0) == d.M && output.size(1) == d.N && group_list.numel() == d.G,
                "shape mismatch between x, weight, output and group_list");
    return d;
}

void check_scale(const at::Tensor& s, int ct, const Dims& d, const char* name) {
    if (ct == B200MOE_CT_FP8) {
        TORCH_CHECK(s.scalar_type() == at::kFloat && s.numel() == d.G * (d.K / 128) * (d.N / 128), name,
                    " must be float32 [G, K/128, N/128]");
    } else if (ct == B200MOE_CT_FP4) {
        TORCH_CHECK(s.scalar_type() == at::kBFloat16 && s.numel() == d.G * (d.K / 16) * d.N, name,
                    " must be bfloat16 [G, K/16, N]");
    } else if (ct == B200MOE_CT_INT8) {
        TORCH_CHECK(s.scalar_type() == at::kBFloat16 && s.numel() == d.G * d.N, name, " must be bfloat16 [G, N]");
    } else {
        TORCH_CHECK(s.scalar_type() == at::kBFloat16 && s.numel() == d.G * (d.K / 128) * d.N, name,
                    " must be bfloat16 [G, K/128, N]");
    }
}

void GroupedGemm(at::Tensor x, at::Tensor weight, at::Tensor antiquantScaleOptional,
                 at::Tensor antiquantOffsetOptional, at::Tensor groupListOptional, const std::string& computeType,
                 at::Tensor output, int64_t group_list_type, const std::string& weight_layout) {
    const int ct = compute_type_of(computeType);
    const int layout = layout_of(weight_layout);
    check_tensor(x, "x"); check_tensor(weight, "weight"); check_tensor(antiquantScaleOptional, "antiquantScaleOptional");
    check_tensor(groupListOptional, "groupListOptional"); check_tensor(output, "output");
    const Dims d = dims_of(x, weight, groupListOptional, output, ct);
    check_scale(antiquantScaleOptional, ct, d, "antiquantScaleOptional");
    const void* offset = nullptr;  // fp8 / fp4: accepted and ignored, as in the reference kernel
    if ((ct == B200MOE_CT_INT8 || ct == B200MOE_CT_INT4) && antiquantOffsetOptional.defined() &&
        antiquantOffsetOptional.numel() > 0) {
        check_tensor(antiquantOffsetOptional, "antiquantOffsetOptional");
        check_scale(antiquantOffsetOptional, ct, d, "antiquantOffsetOptional");
        offset = antiquantOffsetOptional.data_ptr();
    }
    c10::cuda::CUDAGuard guard(x.device());
    auto stream = c10::cuda::getCurrentCUDAStream();
    const size_t ws_bytes = b200moe_grouped_gemm_workspace_bytes(d.M, d.K, d.N, d.G, ct, layout);
    at::Tensor ws = at::empty({(int64_t)ws_bytes}, x.options().dtype(at::kByte));
    raise_on(b200moe_grouped_gemm(x.data_ptr(), weight.data_ptr(), antiquantScaleOptional.data_ptr(), offset,
                                  groupListOptional.data_ptr<int64_t>(), output.data_ptr(), d.M, d.K, d.N, d.G, ct,
                                  (int)group_list_type, layout, ws.data_ptr(), ws_bytes, stream.stream()),
             "grouped_gemm");
}

void GroupedSoftGemv(at::Tensor x, at::Tensor weight, at::Tensor scale, at::Tensor groupList,
                     const std::string& computeType, at::Tensor output, int64_t group_list_type,
                     const std::string& weight_layout, c10::optional<at::Tensor> offset_opt) {
    const int ct = compute_type_of(computeType);
    const int layout = layout_of(weight_layout);
    check_tensor(x, "x"); check_tensor(weight, "weight"); check_tensor(scale, "scale");
    check_tensor(groupList, "groupList"); check_tensor(output, "output");
    const Dims d = dims_of(x, weight, groupList, output, ct);
    check_scale(scale, ct, d, "scale");
    const void* offset = nullptr;
    if (offset_opt.has_value() && offset_opt->defined()) {
        TORCH_CHECK(ct == B200MOE_CT_INT8 || ct == B200MOE_CT_INT4, "offset is only defined for int8 / int4");
        check_tensor(*offset_opt, "offset");
        check_scale(*offset_opt, ct, d, "offset");
        offset = offset_opt->data_ptr();
    }
    c10::cuda::CUDAGuard guard(x.device());
    auto stream = c10::cuda::getCurrentCUDAStream();
    const size_t ws_bytes = b200moe_grouped_gemv_workspace_bytes(d.M, d.K, d.N, d.G, ct, layout);
    at::Tensor ws = at::empty({(int64_t)ws_bytes}, x.options().dtype(at::kByte));
    raise_on(b200moe_grouped_gemv(x.data_ptr(), weight.data_ptr(), scale.data_ptr(), offset,
                                  groupList.data_ptr<int64_t>(), output.data_ptr(), d.M, d.K, d.N, d.G, ct,
                                  (int)group_list_type, layout, ws.data_ptr(), ws_bytes, stream.stream()),
             "grouped_soft_gemv");
}

void Fp4Dequant(at::Tensor codes, c10::optional<at::Tensor> scale, at::Tensor output) {
    check_tensor(codes, "codes"); check_tensor(output, "output");
    TORCH_CHECK(codes.element_size() == 1 && output.scalar_type() == at::kBFloat16 &&
                output.numel() == 2 * codes.numel(), "codes: bytes [..., L/2]; output: bfloat16 [..., L]");
    const void* sp = nullptr;
    if (scale.has_value() && scale->defined()) {
        check_tensor(*scale, "scale");
        TORCH_CHECK(scale->element_size() == 1 && scale->numel() * 32 == output.numel(),
                    "scale: one e8m0 byte per 32 elements");
        sp = scale->data_ptr();
    }
    c10::cuda::CUDAGuard guard(codes.device());
    raise_on(b200moe_fp4_dequant(codes.data_ptr(), sp, output.data_ptr(), output.numel(),
                                 sp ? B200MOE_FP4_SCALE_E8M0_PER32 : B200MOE_FP4_SCALE_NONE,
                                 c10::cuda::getCurrentCUDAStream().stream()),
             "fp4_dequant");
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    using namespace pybind11::literals;
    m.def("grouped_soft_gemv", &GroupedSoftGemv, "x"_a, "weight"_a, "scale"_a, "groupList"_a, "computeType"_a,
          "output"_a, "group_list_type"_a = 0, "weight_layout"_a = "ascend", "offset"_a = pybind11::none(),
          "GROUP GEMV.");
    m.def("grouped_gemm", &GroupedGemm, "x"_a, "weight"_a, "antiquantScaleOptional"_a, "antiquantOffsetOptional"_a,
          "groupListOptional"_a, "computeType"_a, "output"_a, "group_list_type"_a = 0, "weight_layout"_a = "ascend",
          "GROUP GEMM.");
    m.def("fp4_dequant", &Fp4Dequant, "codes"_a, "scale"_a, "output"_a, "FP4(e2m1) -> BF16.");
}
