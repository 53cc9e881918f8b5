// Epilogue selectors of the `epilogue=` argument: the counterpart of csrc/jit_kernels/epilogue_class.hpp:14-128 and of
// the pybind table csrc/apis/epilogue_class.hpp:10-21 (submodule `epilogue` with Epilogue, Identity, Alpha,
// FP8Quantization, BF16StochasticRounding).
#pragma once

#include <memory>

#include "common.hpp"

namespace dg_host {

struct EpilogueClass {
    virtual ~EpilogueClass() = default;
    virtual int kind() const { return DG_EPILOGUE_IDENTITY; }
    virtual void check(const std::optional<torch::Tensor>& c, const torch::Tensor& d) const {
        host_assert(d.scalar_type() == torch::kBFloat16 || d.scalar_type() == torch::kFloat32);
    }
};

struct IdentityEpilogue : EpilogueClass {};

struct AlphaEpilogue : EpilogueClass {
    float alpha;
    explicit AlphaEpilogue(const float& a) : alpha(a) {}
    int kind() const override { return DG_EPILOGUE_ALPHA; }
};

// The [1, N] bias of a dense GEMM (not constructible from Python: it is what a separate `c` resolves to).
struct BiasEpilogue : EpilogueClass {
    torch::Tensor bias;
    explicit BiasEpilogue(torch::Tensor b) : bias(std::move(b)) {}
    int kind() const override { return DG_EPILOGUE_BIAS; }
};

// FP32 accumulator -> BF16 by stochastic rounding with the reference's hash (operators.hpp:224-343).
struct BF16StochasticRoundingEpilogue : EpilogueClass {
    int kind() const override { return DG_EPILOGUE_STOCHASTIC_BF16; }
    void check(const std::optional<torch::Tensor>& c, const torch::Tensor& d) const override {
        host_assert(!c.has_value() && d.scalar_type() == torch::kBFloat16, "Stochastic rounding requires a direct BF16 output");
    }
};

// E4M3 output with one UE8M0 scale per row per 32 columns written to `sfd` (int16 [M, batches * N / 64], MN-major);
// csrc/jit_kernels/epilogue_class.hpp:80-108.
struct FP8QuantizationEpilogue : EpilogueClass {
    torch::Tensor sfd;
    explicit FP8QuantizationEpilogue(const torch::Tensor& s) : sfd(s) {}
    int kind() const override { return DG_EPILOGUE_FP8_QUANT; }
    void check(const std::optional<torch::Tensor>& c, const torch::Tensor& d) const override {
        host_assert(!c.has_value() && d.scalar_type() == torch::kFloat8_e4m3fn, "FP8 quantization requires a direct E4M3 output");
        host_assert(d.dim() == 2 || d.dim() == 3);
        const int64_t m = d.size(-2), n = d.size(-1), batches = d.dim() == 3 ? d.size(0) : 1;
        host_assert(n % 128 == 0, "FP8 output requires N to be a multiple of 128");
        host_assert(d.stride(-1) == 1 && (d.dim() == 2 || d.stride(0) == n),
                    "FP8 output must be contiguous in N and, when batched, hold the batches side by side in a row");
        host_assert(sfd.scalar_type() == torch::kInt16 && sfd.dim() == 2 && sfd.device() == d.device(),
                    "sfd must be a 2-D int16 tensor on the output device");
        host_assert(sfd.size(0) == m && sfd.size(1) == batches * n / 64, "sfd must have shape [M, batches * N / 64]");
        host_assert((sfd.stride(0) == 1 || m == 1) && sfd.stride(1) == m, "sfd must be MN-major");
    }
};

// csrc/jit_kernels/epilogue_class.hpp:110-128: the epilogue object, `alpha` and the FP8 output pair are exclusive.
inline std::shared_ptr<EpilogueClass> resolve_epilogue(const std::shared_ptr<EpilogueClass>& epilogue,
                                                       const std::optional<torch::Tensor>& c, const torch::Tensor& d,
                                                       const std::optional<float>& alpha = std::nullopt,
                                                       const std::optional<torch::Tensor>& sfd = std::nullopt) {
    host_assert((epilogue != nullptr) + alpha.has_value() + sfd.has_value() <= 1,
                "The epilogue class, alpha and the FP8 output pair are exclusive");
    std::shared_ptr<EpilogueClass> resolved;
    if (alpha.has_value()) resolved = std::make_shared<AlphaEpilogue>(alpha.value());
    else if (sfd.has_value()) resolved = std::make_shared<FP8QuantizationEpilogue>(sfd.value());
    else resolved = epilogue != nullptr ? epilogue : std::make_shared<IdentityEpilogue>();
    resolved->check(c, d);
    return resolved;
}

inline void register_epilogue_apis(py::module_& m) {
    auto sub = m.def_submodule("epilogue", "GEMM epilogue classes");
    py::class_<EpilogueClass, std::shared_ptr<EpilogueClass>>(sub, "Epilogue");
    py::class_<IdentityEpilogue, EpilogueClass, std::shared_ptr<IdentityEpilogue>>(sub, "Identity").def(py::init<>());
    py::class_<AlphaEpilogue, EpilogueClass, std::shared_ptr<AlphaEpilogue>>(sub, "Alpha")
        .def(py::init<const float&>(), py::arg("alpha"))
        .def_readonly("alpha", &AlphaEpilogue::alpha);
    py::class_<FP8QuantizationEpilogue, EpilogueClass, std::shared_ptr<FP8QuantizationEpilogue>>(sub, "FP8Quantization")
        .def(py::init<const torch::Tensor&>(), py::arg("sfd"))
        .def_readonly("sfd", &FP8QuantizationEpilogue::sfd);
    py::class_<BF16StochasticRoundingEpilogue, EpilogueClass, std::shared_ptr<BF16StochasticRoundingEpilogue>>(sub, "BF16StochasticRounding")
        .def(py::init<>());
}

}  // namespace dg_host
