// Python module `cinfer_ascendc`: the operator names and keyword arguments of the reference's
// extension (pybind.cpp:13-32 of the reference; GroupedGemm at grouped_gemm/src/grouped_gemm.h:12-16,
// GroupedSoftGemv at grouped_soft_gemv/src/grouped_soft_gemv.h:12-14), bound to the B200 kernels
// through the C ABI of include/b200moe.h.  This file only unpacks tensors: device/dtype/shape
// checks, the current CUDA stream, a workspace from torch's caching allocator, status -> exception.
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <cuda_runtime_api.h>
#include <torch/extension.h>

#include <cstdio>
#include <map>
#include <mutex>
#include <stdexcept>
#include <string>
#include <utility>

#include "../../../include/b200moe.h"

namespace {

int compute_type_of(const std::string& s) {
    if (s == "fp8") return B200MOE_CT_FP8;
    if (s == "fp4") return B200MOE_CT_FP4;
    if (s == "int8") return B200MOE_CT_INT8;
    if (s == "int4") return B200MOE_CT_INT4;
    if (s == "bf16") return B200MOE_CT_BF16;
    // same report as the reference binding for an unknown computeType
    std::printf("Invalid compute type: %s. Supported: \"fp4\", \"fp8\", \"int8\", \"int4\", \"bf16\"\n", s.c_str());
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

// One persistent workspace per (device, stream).  The reference binding keeps a process-wide,
// never-freed workspace map as well (grouped_gemm/src/grouped_gemm.cpp:91-120); this one is guarded by
// a mutex, and it exists for a second reason: words 4 / 5 of a workspace keep the first device-side
// finding (invalid group list, expired wait) of every call that used it, so last_status() can report
// at the caller's synchronisation point what no asynchronous call can report by itself.
std::mutex g_ws_mutex;
std::map<std::pair<int, void*>, at::Tensor> g_workspaces;

at::Tensor workspace_for(const at::Tensor& like, size_t bytes, void* stream) {
    std::lock_guard<std::mutex> lock(g_ws_mutex);
    const auto key = std::make_pair((int)like.get_device(), stream);
    auto it = g_workspaces.find(key);
    if (it == g_workspaces.end() || (size_t)it->second.numel() < bytes) {
        at::Tensor fresh = at::zeros({(int64_t)std::max<size_t>(bytes, size_t(1) << 20)}, like.options().dtype(at::kByte));
        if (it != g_workspaces.end()) fresh.slice(0, 16, 24).copy_(it->second.slice(0, 16, 24));
        g_workspaces[key] = fresh;
        return fresh;
    }
    return it->second;
}

std::pair<int, int> LastStatus(bool clear) {
    std::lock_guard<std::mutex> lock(g_ws_mutex);
    int dev = 0;
    TORCH_CHECK(cudaGetDevice(&dev) == cudaSuccess, "cudaGetDevice failed");
    std::pair<int, int> found{0, 0};
    for (auto& kv : g_workspaces) {
        if (kv.first.first != dev) continue;
        int32_t out[2] = {0, 0};
        const int rc = b200moe_read_sticky_status(kv.second.data_ptr(), out, clear ? 1 : 0, kv.first.second);
        TORCH_CHECK(rc == B200MOE_OK, "read_sticky_status: ", b200moe_strerror(rc));
        if (found.first == 0 && out[0] != 0) found = {out[0], out[1]};
    }
    return found;
}

void CheckStatus() {
    const auto st = LastStatus(true);
    if (st.first != 0)
        throw std::runtime_error("b200moe device status " + std::to_string(st.first) + " (detail " +
                                 std::to_string(st.second) + "): " +
                                 (st.first == 1 ? "a group_list was invalid, rows were clamped"
                                                : "a bounded wait inside a kernel expired, results are incomplete"));
}

Dims dims_of(const at::Tensor& x, const at::Tensor& weight, const at::Tensor& group_list, const at::Tensor& output,
             int ct) {
    TORCH_CHECK(x.scalar_type() == at::kBFloat16 && output.scalar_type() == at::kBFloat16,
                "x and output must be bfloat16");
    TORCH_CHECK(group_list.scalar_type() == at::kLong, "group_list must be int64");
    TORCH_CHECK(x.dim() == 2 && weight.dim() == 3 && output.dim() == 2, "expected x [M,K], weight [G,K,N], output [M,N]");
    if (ct == B200MOE_CT_BF16) {
        TORCH_CHECK(weight.scalar_type() == at::kBFloat16, "weight must be bfloat16 for computeType bf16");
    } else {
        TORCH_CHECK(weight.element_size() == 1, "weight must be a 1-byte container (uint8 / int8)");
    }
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
    check_tensor(x, "x"); check_tensor(weight, "weight");
    check_tensor(groupListOptional, "groupListOptional"); check_tensor(output, "output");
    const Dims d = dims_of(x, weight, groupListOptional, output, ct);
    const void* scale_ptr = nullptr;  // bf16: the matmul phase alone, no scale
    if (ct != B200MOE_CT_BF16) {
        check_tensor(antiquantScaleOptional, "antiquantScaleOptional");
        check_scale(antiquantScaleOptional, ct, d, "antiquantScaleOptional");
        scale_ptr = antiquantScaleOptional.data_ptr();
    }
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
    at::Tensor ws = workspace_for(x, ws_bytes, stream.stream());
    raise_on(b200moe_grouped_gemm(x.data_ptr(), weight.data_ptr(), scale_ptr, offset,
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
    at::Tensor ws = workspace_for(x, ws_bytes, stream.stream());
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

void Fp4DequantBf16Scale(at::Tensor codes, at::Tensor scale, at::Tensor output, const std::string& weight_layout) {
    check_tensor(codes, "codes"); check_tensor(scale, "scale"); check_tensor(output, "output");
    TORCH_CHECK(codes.dim() == 3 && codes.element_size() == 1, "codes: bytes [G, K, N/2]");
    const int64_t G = codes.size(0), K = codes.size(1), N = 2 * codes.size(2);
    TORCH_CHECK(scale.scalar_type() == at::kBFloat16 && scale.numel() == G * (K / 16) * N, "scale: bfloat16 [G, K/16, N]");
    TORCH_CHECK(output.scalar_type() == at::kBFloat16 && output.numel() == G * K * N, "output: bfloat16 [G, K, N]");
    c10::cuda::CUDAGuard guard(codes.device());
    raise_on(b200moe_fp4_dequant_bf16_scale(codes.data_ptr(), scale.data_ptr(), output.data_ptr(), G, K, N,
                                            layout_of(weight_layout), c10::cuda::getCurrentCUDAStream().stream()),
             "fp4_dequant_bf16_scale");
}

void Fp8Dequant(at::Tensor codes, at::Tensor scale, at::Tensor output) {
    check_tensor(codes, "codes"); check_tensor(scale, "scale"); check_tensor(output, "output");
    TORCH_CHECK(codes.dim() == 3 && codes.element_size() == 1, "codes: uint8 [G, K, N]");
    const int64_t G = codes.size(0), K = codes.size(1), N = codes.size(2);
    TORCH_CHECK(scale.scalar_type() == at::kFloat && scale.numel() == G * (K / 128) * (N / 128),
                "scale: float32 [G, K/128, N/128]");
    TORCH_CHECK(output.scalar_type() == at::kBFloat16 && output.numel() == G * K * N, "output: bfloat16 [G, K, N]");
    c10::cuda::CUDAGuard guard(codes.device());
    raise_on(b200moe_fp8_dequant(codes.data_ptr(), scale.data_ptr<float>(), output.data_ptr(), G, K, N,
                                 c10::cuda::getCurrentCUDAStream().stream()),
             "fp8_dequant");
}

at::Tensor PackWeightInt8(at::Tensor weight, bool gate_up) {
    check_tensor(weight, "weight");
    TORCH_CHECK(weight.dim() == 3 && weight.element_size() == 1, "weight: int8 [G, K, N]");
    at::Tensor out = at::empty_like(weight);
    c10::cuda::CUDAGuard guard(weight.device());
    raise_on(b200moe_pack_weight_int8(weight.data_ptr(), out.data_ptr(), weight.size(0), weight.size(1), weight.size(2),
                                      gate_up ? 1 : 0, c10::cuda::getCurrentCUDAStream().stream()),
             "pack_weight_int8");
    return out;
}

// grouped_gemm with computeType "int8" on weights from pack_weight_int8 (same keyword names; scale / offset in
// the original column order; gate_up_silu: output [M, N/2] = bf16(silu(gate) * up)).
void GroupedGemmPacked(at::Tensor x, at::Tensor weight, at::Tensor antiquantScaleOptional,
                       c10::optional<at::Tensor> antiquantOffsetOptional, at::Tensor groupListOptional, at::Tensor output,
                       int64_t group_list_type, bool gate_up_silu) {
    check_tensor(x, "x"); check_tensor(weight, "weight"); check_tensor(antiquantScaleOptional, "antiquantScaleOptional");
    check_tensor(groupListOptional, "groupListOptional"); check_tensor(output, "output");
    TORCH_CHECK(x.scalar_type() == at::kBFloat16 && output.scalar_type() == at::kBFloat16, "x and output must be bfloat16");
    TORCH_CHECK(groupListOptional.scalar_type() == at::kLong, "group_list must be int64");
    TORCH_CHECK(x.dim() == 2 && weight.dim() == 3 && weight.element_size() == 1, "expected x [M,K], packed weight [G,K,N]");
    Dims d{x.size(0), x.size(1), weight.size(2), weight.size(0)};
    TORCH_CHECK(weight.size(1) == d.K && output.size(0) == d.M && output.size(1) == (gate_up_silu ? d.N / 2 : d.N) &&
                groupListOptional.numel() == d.G, "shape mismatch between x, weight, output and group_list");
    check_scale(antiquantScaleOptional, B200MOE_CT_INT8, d, "antiquantScaleOptional");
    const void* offset = nullptr;
    if (antiquantOffsetOptional.has_value() && antiquantOffsetOptional->defined() && antiquantOffsetOptional->numel() > 0) {
        check_tensor(*antiquantOffsetOptional, "antiquantOffsetOptional");
        check_scale(*antiquantOffsetOptional, B200MOE_CT_INT8, d, "antiquantOffsetOptional");
        offset = antiquantOffsetOptional->data_ptr();
    }
    c10::cuda::CUDAGuard guard(x.device());
    auto stream = c10::cuda::getCurrentCUDAStream();
    const size_t ws_bytes = b200moe_grouped_gemm_workspace_bytes(d.M, d.K, d.N, d.G, B200MOE_CT_INT8, B200MOE_LAYOUT_CANONICAL);
    at::Tensor ws = workspace_for(x, ws_bytes, stream.stream());
    raise_on(b200moe_grouped_gemm_int8_packed(x.data_ptr(), weight.data_ptr(), antiquantScaleOptional.data_ptr(), offset,
                                              groupListOptional.data_ptr<int64_t>(), output.data_ptr(), d.M, d.K, d.N, d.G,
                                              (int)group_list_type, gate_up_silu ? 1 : 0, ws.data_ptr(), ws_bytes,
                                              stream.stream()),
             "grouped_gemm_packed");
}

at::Tensor Fp4ScaleFold(at::Tensor block_scale, at::Tensor global_scale) {
    check_tensor(block_scale, "block_scale"); check_tensor(global_scale, "global_scale");
    TORCH_CHECK(block_scale.dim() == 3 && block_scale.scalar_type() == at::kBFloat16, "block_scale: bfloat16 [G, N, K/16]");
    const int64_t G = block_scale.size(0), N = block_scale.size(1), KB = block_scale.size(2);
    TORCH_CHECK(global_scale.scalar_type() == at::kFloat && G > 0 &&
                (global_scale.numel() == G || global_scale.numel() == 2 * G), "global_scale: float32 [G, 1 or 2, 1]");
    at::Tensor out = at::empty({G, KB, N}, block_scale.options());
    c10::cuda::CUDAGuard guard(block_scale.device());
    raise_on(b200moe_fp4_scale_fold(block_scale.data_ptr(), global_scale.data_ptr<float>(), out.data_ptr(), G, N, KB,
                                    global_scale.numel() / G, c10::cuda::getCurrentCUDAStream().stream()),
             "fp4_scale_fold");
    return out;
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
    m.def("fp4_dequant_bf16_scale", &Fp4DequantBf16Scale, "codes"_a, "scale"_a, "output"_a, "weight_layout"_a = "ascend",
          "FP4(e2m1) x bf16 scale per 16 k -> BF16 weights.");
    m.def("fp8_dequant", &Fp8Dequant, "codes"_a, "scale"_a, "output"_a, "FP8(e4m3) x fp32 scale per 128x128 -> BF16 weights.");
    m.def("pack_weight_int8", &PackWeightInt8, "weight"_a, "gate_up"_a = false,
          "int8 [G,K,N] -> the tile-packed order grouped_gemm_packed reads.");
    m.def("grouped_gemm_packed", &GroupedGemmPacked, "x"_a, "weight"_a, "antiquantScaleOptional"_a,
          "antiquantOffsetOptional"_a, "groupListOptional"_a, "output"_a, "group_list_type"_a = 0, "gate_up_silu"_a = false,
          "GROUP GEMM on int8 weights repacked once.");
    m.def("fp4_scale_fold", &Fp4ScaleFold, "block_scale"_a, "global_scale"_a, "Two-level FP4 scale fold.");
    m.def("last_status", [](bool clear) { return LastStatus(clear); }, "clear"_a = false,
          "(code, detail) of the first device-side finding since the status was last cleared.");
    m.def("check_status", &CheckStatus, "Raises if an operator call left a device-side finding (and clears it).");
}
