// Helpers shared by the binding headers: host assertions that surface in Python as RuntimeError with the reference's
// message text, tensor unpacking (pointers, majors, strides), the named-axis shape inference of
// csrc/utils/layout.hpp:140-219, the current CUDA stream, and checked calls into the C ABI.
#pragma once

#include <ATen/cuda/CUDAContext.h>
#include <torch/extension.h>

#include <atomic>
#include <cstdint>
#include <cstdlib>
#include <mutex>
#include <optional>
#include <sstream>
#include <stdexcept>
#include <string>
#include <tuple>
#include <utility>
#include <vector>

#include "../../../include/dg_b200.h"

namespace dg_host {

namespace py = pybind11;

constexpr auto kPackedFp4 = torch::kInt8;          // csrc/utils/dtype.hpp:9
constexpr int kMkAlignment = 256;                   // csrc/jit/jit.hpp:59-73

inline void host_assert(bool cond, const std::string& msg = "Assertion failed") {
    if (!cond) throw std::runtime_error(msg);
}

inline void check(int rc) {
    if (rc != DG_OK) {
        const char* msg = dg_last_error();
        throw std::runtime_error(msg != nullptr && msg[0] != 0 ? std::string(msg) : "libdg_b200 error " + std::to_string(rc));
    }
}

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }
inline int64_t align_up(int64_t a, int64_t b) { return ceil_div(a, b) * b; }

// Meta tensors (dry run) have no address; validation only needs something 32-byte aligned.
inline void* ptr_of(const torch::Tensor& t) { return t.is_meta() ? reinterpret_cast<void*>(0x1000) : t.data_ptr(); }

inline void* stream_of(const torch::Tensor& t) {
    return static_cast<void*>(at::cuda::getCurrentCUDAStream(t.device().index()).stream());
}

// ---- process-wide knobs (csrc/jit/jit.hpp:18-76)
struct Runtime {
    std::atomic<bool> dry_run{false}, deterministic{false};
    std::atomic<int> arch{100};
    const bool debug = [] { const char* e = getenv("DG_JIT_DEBUG"); return e != nullptr && e[0] != 0 && std::string(e) != "0"; }();
};
inline Runtime& runtime() { static Runtime r; return r; }

// ---- majors (csrc/utils/layout.hpp:37-52,88-99)
inline void major_check(const torch::Tensor& t) {
    const auto d = t.dim();
    if (t.stride(d - 2) == 1 && t.stride(d - 1) == 1) {
        std::ostringstream os;
        os << "Ambiguous major axis, the tensor has both last two dimensions contiguous, strides=" << t.strides();
        throw std::runtime_error(os.str());
    }
    host_assert(t.stride(d - 2) == 1 || t.stride(d - 1) == 1);
}
inline int major_ab(const torch::Tensor& t) {
    major_check(t);
    return t.stride(t.dim() - 1) == 1 ? DG_MAJOR_K : DG_MAJOR_MN;
}
inline int64_t outer_stride(const torch::Tensor& t, int major) {
    return major == DG_MAJOR_K ? t.stride(t.dim() - 2) : t.stride(t.dim() - 1);
}

// ---- named-axis shape inference with conflict diagnostics (csrc/utils/layout.hpp:140-219). A packed-FP4 tensor
// counts double along its contiguous axis.
using ShapeSpec = std::pair<std::string, const torch::Tensor*>;
inline std::vector<int64_t> shape_by_spec(const std::string& out_dims, const std::vector<ShapeSpec>& specs) {
    std::vector<int> majors;
    for (size_t idx = 0; idx < specs.size(); ++idx) {
        const auto& [dims, t] = specs[idx];
        if (t->dim() != (int64_t)dims.size())
            throw std::runtime_error("Shape mismatch: tensor #" + std::to_string(idx) + ", annotation=\"" + dims + "\"");
        int major = -1;
        for (int i = 0; i < t->dim(); ++i)
            if (t->stride(i) == 1) { major = i; break; }
        if (major < 0) {
            std::ostringstream os;
            os << "Tensor #" << idx << " annotation=\"" << dims << "\" doesn't have major axis, strides=" << t->strides();
            throw std::runtime_error(os.str());
        }
        majors.push_back(major);
    }
    std::vector<int64_t> result;
    for (char name : out_dims) {
        bool found = false;
        int64_t value = 0;
        size_t f_idx = 0;
        int f_axis = 0;
        for (size_t idx = 0; idx < specs.size(); ++idx) {
            const auto& [dims, t] = specs[idx];
            for (int axis = 0; axis < (int)dims.size(); ++axis) {
                if (dims[axis] != name) continue;
                const int64_t v = t->size(axis) * ((t->scalar_type() == kPackedFp4 && axis == majors[idx]) ? 2 : 1);
                if (!found) {
                    found = true; value = v; f_idx = idx; f_axis = axis;
                } else if (value != v) {
                    std::ostringstream os;
                    os << "Conflicting shape dimension '" << name << "': tensor #" << idx << " annotation=\"" << dims << "\" axis=" << axis
                       << " gives " << v << ", but tensor #" << f_idx << " annotation=\"" << specs[f_idx].first << "\" axis=" << f_axis
                       << " gives " << value;
                    throw std::runtime_error(os.str());
                }
            }
        }
        result.push_back(found ? value : 0);
    }
    return result;
}

inline int dtype_code(const torch::Tensor& t) {
    switch (t.scalar_type()) {
        case torch::kFloat8_e4m3fn: return DG_E4M3;
        case torch::kInt8: return DG_E2M1X2;
        case torch::kBFloat16: return DG_BF16;
        case torch::kFloat32: return DG_F32;
        default: throw std::runtime_error("Unsupported operand dtypes");
    }
}

}  // namespace dg_host
