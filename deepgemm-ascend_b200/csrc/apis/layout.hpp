// Scale-factor layout: the counterpart of csrc/apis/layout.hpp:37-128 (check_sf_layout, transform_sf_into_required_layout,
// transform_k_grouped_sf_into_required_layout, get_recipe) and of the launcher csrc/jit_kernels/transform_sf.hpp:15-105.
#pragma once

#include "common.hpp"
#include "runtime.hpp"

namespace dg_host {

using Recipe3 = std::tuple<int, int, int>;
using Recipe2 = std::tuple<int, int>;

// (gran_m, gran_n, gran_k_a, gran_k_b). The reference requires both gran_k to be 32 (csrc/apis/layout.hpp:55,125); here
// each may be 32 or 128 because a per-128 scale is expanded to the per-32 layout by the transform.
inline std::tuple<int, int, int, int> get_recipe(const std::optional<Recipe3>& recipe, const std::optional<Recipe2>& recipe_a,
                                                 const std::optional<Recipe2>& recipe_b) {
    host_assert(!(recipe.has_value() && (recipe_a.has_value() || recipe_b.has_value())),
                "recipe and recipe_a / recipe_b are mutually exclusive");
    if (recipe.has_value()) {
        const auto [gm, gn, gk] = recipe.value();
        return {gm, gn, gk, gk};
    }
    const auto [gm, gka] = recipe_a.value_or(Recipe2{1, 32});
    const auto [gn, gkb] = recipe_b.value_or(Recipe2{1, 32});
    return {gm, gn, gka, gkb};
}

// csrc/apis/layout.hpp:37-65. True when `sf` already is the required layout.
inline bool check_sf_layout(const torch::Tensor& sf, int64_t mn, int64_t k, int gran_mn, int gran_k,
                            const std::optional<int>& num_groups) {
    host_assert(sf.scalar_type() == torch::kFloat32 || sf.scalar_type() == torch::kInt16,
                "SF must be float32 or int16 (packed ue8m0x2)");
    host_assert(sf.dim() == (num_groups.has_value() ? 1 : 0) + 2, "SF has the wrong number of dimensions");
    host_assert(sf.stride(-1) == 1 || sf.stride(-2) == 1 || sf.size(-1) == 1 || sf.size(-2) == 1,
                "SF input must be contiguous in either the last or second-to-last dimension");
    if (num_groups.has_value()) host_assert(sf.size(-3) == num_groups.value());
    host_assert(gran_k == 32 || gran_k == 128, "gran_k must be 32 (or 128, expanded by the transform)");
    const int64_t div_k = sf.scalar_type() == torch::kFloat32 ? gran_k : gran_k * 2;
    host_assert(sf.size(-2) == ceil_div(mn, gran_mn),
                "SF rows: expected " + std::to_string(ceil_div(mn, gran_mn)) + ", got " + std::to_string(sf.size(-2)));
    host_assert(sf.size(-1) == ceil_div(k, div_k),
                "SF columns: expected " + std::to_string(ceil_div(k, div_k)) + ", got " + std::to_string(sf.size(-1)));
    if (sf.scalar_type() == torch::kInt16 && gran_mn == 1 && gran_k == 32 && sf.stride(-2) == 1 && sf.stride(-1) == sf.size(-2))
        return !num_groups.has_value() || sf.stride(-3) == sf.size(-2) * sf.size(-1);
    return false;
}

inline int check_psum_layout(const torch::Tensor& psum_layout, const torch::Tensor& sf) {
    host_assert(psum_layout.device() == sf.device(), "grouped_layout must be on the same device as the SF input");
    host_assert(psum_layout.scalar_type() == torch::kInt32 && psum_layout.dim() == 1 && psum_layout.is_contiguous(),
                "grouped_layout must be a contiguous 1D int32 tensor");
    host_assert(psum_layout.numel() > 0, "grouped_layout must contain at least one group");
    return (int)psum_layout.numel();
}

// csrc/jit_kernels/transform_sf.hpp:15-105. With `tma_aligned` the column stride of the result is rounded up to 8
// elements (what the GEMM's tensor map needs); the public entry point never does that. `psum_layout` pads along MN
// (m-grouped operands), `k_psum_layout` along K (k-grouped operands).
inline torch::Tensor launch_transform_sf(torch::Tensor sf, int64_t mn, int64_t k, int gran_mn, int gran_k,
                                         const std::optional<torch::Tensor>& psum_layout, bool tma_aligned,
                                         const std::optional<torch::Tensor>& k_psum_layout = std::nullopt) {
    const bool squeeze = sf.dim() == 2;
    if (squeeze) sf = sf.unsqueeze(0);
    host_assert(sf.dim() == 3, "Transform SF input must have 2 or 3 dimensions, but got " + std::to_string(sf.dim() - (squeeze ? 1 : 0)));
    host_assert(gran_mn >= 1 && gran_mn <= 128 && (gran_mn & (gran_mn - 1)) == 0, "gran_mn only support a power of two in [1, 128]");
    const int64_t batches = sf.size(0);
    int num_groups = 0, num_k_groups = 0;
    if (psum_layout.has_value()) {
        host_assert(batches == 1, "Grouped transform SF requires one logical batch and grouped_layout");
        num_groups = check_psum_layout(psum_layout.value(), sf);
    }
    if (k_psum_layout.has_value()) {
        host_assert(batches == 1 && !psum_layout.has_value(), "Grouped transform SF requires one logical batch and grouped_layout");
        host_assert(gran_k == 32, "K-grouped transform SF requires gran_k = 32");
        num_k_groups = check_psum_layout(k_psum_layout.value(), sf);
    }
    const bool is_fp32 = sf.scalar_type() == torch::kFloat32;
    const int64_t k32 = ceil_div(k, 32);
    const int64_t dst_cols = (!is_fp32 && gran_k == 32) ? sf.size(-1) : ceil_div(k32, 2);
    const int64_t col_stride = tma_aligned ? align_up(mn, 8) : mn;
    auto storage = torch::empty({batches, dst_cols, col_stride}, sf.options().dtype(torch::kInt16));
    auto out = storage.slice(2, 0, mn).transpose(-2, -1);
    if (out.numel() != 0 && !runtime().dry_run && !sf.is_meta()) {
        torch::Tensor flag;
        if (is_fp32) flag = sf_invalid_flag(sf.device());
        check(dg_transform_sf_launch(
            sf.data_ptr(), is_fp32 ? 1 : 0, (uint64_t)sf.stride(-2), (uint64_t)sf.stride(-1), (uint64_t)sf.stride(0),
            (uint32_t)sf.size(-2), (uint32_t)sf.size(-1), static_cast<int16_t*>(storage.data_ptr()), (uint64_t)col_stride,
            (uint64_t)(dst_cols * col_stride), (uint32_t)mn, (uint32_t)k32, (uint32_t)gran_mn, (uint32_t)(gran_k / 32),
            (uint32_t)batches, psum_layout.has_value() ? static_cast<const int32_t*>(psum_layout->data_ptr()) : nullptr,
            (uint32_t)num_groups, (uint32_t)kMkAlignment, flag.defined() ? static_cast<int32_t*>(flag.data_ptr()) : nullptr,
            k_psum_layout.has_value() ? static_cast<const int32_t*>(k_psum_layout->data_ptr()) : nullptr,
            (uint32_t)num_k_groups, stream_of(sf)));
        if (flag.defined() && runtime().debug && flag.item<int32_t>() != 0) {
            flag.zero_();
            throw std::runtime_error("Float32 SF must be non-negative and can't have non-zero mantissa");
        }
    }
    return squeeze ? out.squeeze(0) : out;
}

inline torch::Tensor transform_sf(const torch::Tensor& sf, int64_t mn, int64_t k, int gran_mn, int gran_k,
                                  const std::optional<int>& num_groups, bool disable_ue8m0_cast,
                                  const std::optional<torch::Tensor>& psum_layout, bool tma_aligned,
                                  const std::optional<torch::Tensor>& k_psum_layout = std::nullopt) {
    if (check_sf_layout(sf, mn, k, gran_mn, gran_k, num_groups)) {
        if (!tma_aligned || mn % 8 == 0 || sf.is_meta()) return sf;
    } else if (sf.scalar_type() == torch::kFloat32) {
        host_assert(!disable_ue8m0_cast, "Float32 SF must be converted into ue8m0, but disable_ue8m0_cast is set true");
    }
    return launch_transform_sf(sf, mn, k, gran_mn, gran_k, psum_layout, tma_aligned, k_psum_layout);
}

// csrc/apis/layout.hpp:68-92. Returns int16 [..., MN, ceil(K/64)], MN-major; returns `sf` itself when it already has
// that layout. `recipe` has three (gran_m, gran_n, gran_k; `is_sfa` selects) or two (gran_mn, gran_k) elements.
inline torch::Tensor transform_sf_into_required_layout(const torch::Tensor& sf, const int& mn, const int& k,
                                                       const std::vector<int>& recipe, const std::optional<int>& num_groups,
                                                       const std::optional<bool>& is_sfa, const bool& disable_ue8m0_cast,
                                                       const std::optional<torch::Tensor>& psum_layout) {
    int gran_mn, gran_k;
    if (recipe.size() == 3) {
        host_assert(is_sfa.has_value(), "is_sfa must be set for a 3-element recipe");
        gran_mn = is_sfa.value() ? recipe[0] : recipe[1];
        gran_k = recipe[2];
    } else {
        host_assert(recipe.size() == 2, "recipe must have 2 or 3 elements");
        gran_mn = recipe[0];
        gran_k = recipe[1];
    }
    return transform_sf(sf, mn, k, gran_mn, gran_k, num_groups, disable_ue8m0_cast, psum_layout, false);
}

// csrc/apis/layout.hpp:94-111: scale factors of a k-grouped operand ([MN, K] with K holding the groups in psum layout):
// same result layout, with every K unit inside a group's padding set to 0.
inline torch::Tensor transform_k_grouped_sf_into_required_layout(const torch::Tensor& sf, const int& mn, const int& k,
                                                                 const std::vector<int>& recipe, const std::optional<bool>& is_sfa,
                                                                 const torch::Tensor& psum_layout) {
    host_assert(is_sfa.has_value(), "is_sfa must be set");
    host_assert(recipe.size() == 3, "recipe must have 3 elements");
    return transform_sf(sf, mn, k, is_sfa.value() ? recipe[0] : recipe[1], recipe[2], std::nullopt, false, std::nullopt, false, psum_layout);
}

inline void register_layout_apis(py::module_& m) {
    m.def("transform_sf_into_required_layout", &transform_sf_into_required_layout,
          py::arg("sf"), py::arg("mn"), py::arg("k"), py::arg("recipe"),
          py::arg("num_groups") = std::nullopt, py::arg("is_sfa") = std::nullopt,
          py::arg("disable_ue8m0_cast") = false, py::arg("psum_layout") = std::nullopt);
    m.def("transform_k_grouped_sf_into_required_layout", &transform_k_grouped_sf_into_required_layout,
          py::arg("sf"), py::arg("mn"), py::arg("k"), py::arg("recipe"), py::arg("is_sfa"), py::arg("psum_layout"));
    m.def("get_recipe", [](const std::optional<Recipe3>& recipe, const std::optional<Recipe2>& recipe_a,
                           const std::optional<Recipe2>& recipe_b) { return get_recipe(recipe, recipe_a, recipe_b); },
          py::arg("recipe"), py::arg("recipe_a"), py::arg("recipe_b"));
}

}  // namespace dg_host
