// Runtime knobs: the counterpart of csrc/apis/runtime.hpp:12-80 (same names and argument names).
#pragma once

#include <map>

#include "common.hpp"

namespace dg_host {

// Per-device flag that the scale-factor transform sets when it meets an FP32 scale that is negative or not a power of
// two (the reference asserts on the device, deep_gemm/include/deep_gemm/transform_sf.hpp:13-21). Reported by
// device_status(), or at once when DG_JIT_DEBUG is set.
constexpr int kStatusInvalidScaleFactor = 201;
inline std::mutex& host_mutex() { static std::mutex mu; return mu; }
inline std::map<int, torch::Tensor>& sf_flags() { static std::map<int, torch::Tensor> m; return m; }
inline torch::Tensor sf_invalid_flag(const torch::Device& device) {
    std::lock_guard<std::mutex> lock(host_mutex());
    auto& flags = sf_flags();
    auto it = flags.find(device.index());
    if (it == flags.end())
        it = flags.emplace(device.index(), torch::zeros({1}, torch::TensorOptions().dtype(torch::kInt32).device(device))).first;
    return it->second;
}

// Zero-initialised split-K scratch, one per (device, stream); the library leaves it zeroed after every launch.
inline std::map<std::pair<int, void*>, torch::Tensor>& workspaces() { static std::map<std::pair<int, void*>, torch::Tensor> m; return m; }
inline torch::Tensor workspace(const torch::Device& device, void* stream, int64_t nbytes) {
    std::lock_guard<std::mutex> lock(host_mutex());
    auto& ws = workspaces();
    const auto key = std::make_pair((int)device.index(), stream);
    auto it = ws.find(key);
    if (it == ws.end() || it->second.numel() < nbytes) {
        auto t = torch::zeros({std::max<int64_t>(nbytes, 1 << 22)}, torch::TensorOptions().dtype(torch::kUInt8).device(device));
        ws[key] = t;
        return t;
    }
    return it->second;
}
inline void drop_workspaces(int device_index) {
    std::lock_guard<std::mutex> lock(host_mutex());
    auto& ws = workspaces();
    for (auto it = ws.begin(); it != ws.end();)
        it = it->first.first == device_index ? ws.erase(it) : std::next(it);
}

// 0, or the code of the first problem a kernel recorded since the last call: 101..107 = a bounded wait inside a GEMM
// kernel gave up, 201 = a scale-factor transform met an invalid FP32 scale. Synchronises the device.
inline int device_status() {
    int32_t code = 0;
    check(dg_device_status(&code));
    const int device = at::cuda::current_device();
    if (code != 0) drop_workspaces(device);
    torch::Tensor flag;
    {
        std::lock_guard<std::mutex> lock(host_mutex());
        auto it = sf_flags().find(device);
        if (it != sf_flags().end()) flag = it->second;
    }
    if (flag.defined() && flag.item<int32_t>() != 0) {
        flag.zero_();
        if (code == 0) code = kStatusInvalidScaleFactor;
    }
    return code;
}

inline void register_runtime_apis(py::module_& m) {
    m.def("get_num_sms", []() -> int { return dg_get_num_sms(); });
    m.def("set_num_sms", [](const int& n) { check(dg_set_num_sms(n)); });
    m.def("set_npu_arch", [](const int& arch) { runtime().arch = arch; });
    m.def("get_npu_arch", []() -> int { return runtime().arch; });
    m.def("set_mk_alignment_for_contiguous_layout", [](const int& value) {
        host_assert(value == kMkAlignment, "mk alignment for the contiguous layout is fixed at " + std::to_string(kMkAlignment));
    });
    m.def("get_mk_alignment_for_contiguous_layout", []() -> int { return kMkAlignment; });
    m.def("get_theoretical_mk_alignment_for_contiguous_layout", []() -> int { return kMkAlignment; });
    m.def("init", [](const std::string& version, const std::string& library_root_path) {
        // The reference points its JIT at the installed headers here; this build has no JIT. Only the ABI is checked
        // (no device is touched, so callers can still fork after importing).
        host_assert(dg_abi_version() == DG_B200_ABI_VERSION, "libdg_b200.so has an unexpected ABI version");
    }, py::arg("version") = "", py::arg("library_root_path") = "");
    m.def("set_dry_run", [](const bool value) { runtime().dry_run = value; });
    m.def("get_dry_run", []() -> bool { return runtime().dry_run; });
    m.def("use_deterministic_algorithms", [](const bool enabled) { runtime().deterministic = enabled; }, py::arg("enabled"));
    m.def("get_deterministic_algorithms", []() -> bool { return runtime().deterministic; });
    m.def("npu_sleep", [](const int64_t& sleep_cycles, const uint32_t& marker) {
        if (runtime().dry_run) return;
        check(dg_sleep_launch(sleep_cycles, marker, dg_get_num_sms(),
                              static_cast<void*>(at::cuda::getCurrentCUDAStream().stream())));
    }, py::arg("sleep_cycles"), py::kw_only(), py::arg("marker") = 0);
    m.def("device_status", &device_status);
    m.def("_drop_workspaces", &drop_workspaces, py::arg("device_index"));
}

}  // namespace dg_host
