// GEMM entry points: the counterpart of csrc/apis/gemm.hpp (get_gemm_desc :60-197, fp8_fp4_gemm :225-256, m-grouped
// contiguous :289-324, k-grouped :325-410, BF16 family :412-560, registrations :552-678) and of csrc/apis/einsum.hpp
// (fp8_bmm :37-71, fp8_einsum :161-216). Tensors are only unpacked here (pointers, sizes, strides); validation of the
// problem, the tiling heuristic, the tensor maps and the launches live behind the C ABI (include/dg_b200.h).
#pragma once

#include <Python.h>

#include "common.hpp"
#include "epilogue_class.hpp"
#include "layout.hpp"
#include "runtime.hpp"

namespace dg_host {

using TensorPair = std::pair<torch::Tensor, torch::Tensor>;
using OptTensor = std::optional<torch::Tensor>;
using OptConfig = std::optional<py::dict>;

// csrc/apis/gemm.hpp:105-106: meta and empty tensors have no address, so compare storage identity.
inline bool same_buffer(const torch::Tensor& c, const torch::Tensor& d) {
    if (c.is_same(d)) return true;
    if (d.is_meta() || d.numel() == 0)
        return c.storage().unsafeGetStorageImpl() == d.storage().unsafeGetStorageImpl() && c.storage_offset() == d.storage_offset();
    return c.data_ptr() == d.data_ptr();
}

// csrc/utils/layout.hpp:54-86. True: nothing is left to launch.
inline bool gemm_early_return(int64_t m, int64_t n, int64_t k, const torch::Tensor& d, const OptTensor& c, bool with_bias) {
    if (m == 0 || n == 0) return true;
    const bool is_cd_same = c.has_value() && same_buffer(c.value(), d);
    if (is_cd_same) host_assert(c->sizes() == d.sizes() && c->strides() == d.strides());
    host_assert(d.scalar_type() == torch::kBFloat16 || d.scalar_type() == torch::kFloat32 || d.scalar_type() == torch::kFloat8_e4m3fn);
    if (c.has_value()) {
        host_assert(c->dim() >= 2 && c->stride(-1) == 1);
        host_assert(d.scalar_type() == c->scalar_type());
    }
    if (k == 0) {
        if (!is_cd_same && !d.is_meta()) {
            if (c.has_value()) d.copy_(c->expand_as(d)); else d.zero_();
        }
        return true;
    }
    if (c.has_value() && !is_cd_same && !with_bias && !d.is_meta()) d.copy_(c.value());
    return false;
}

// TMA needs a 16-byte aligned base and 16-byte multiples for every stride but the contiguous one. Operands that do not
// satisfy this (K or MN not a multiple of 16, odd views) are copied once into a padded buffer.
inline torch::Tensor tma_ready_operand(const torch::Tensor& t, int major) {
    if (t.is_meta()) return t;
    const int64_t es = (int64_t)t.element_size();
    bool lead_ok = true;
    for (int i = 0; i + 2 < t.dim(); ++i) lead_ok = lead_ok && t.stride(i) * es % 16 == 0;
    if (reinterpret_cast<uintptr_t>(t.data_ptr()) % 16 == 0 && outer_stride(t, major) * es % 16 == 0 && lead_ok) return t;
    const auto src = major == DG_MAJOR_K ? t : t.transpose(-2, -1);
    const int64_t rows = src.size(-2), cols = src.size(-1) * es, pitch = align_up(cols, 16);       // (columns in bytes)
    host_assert(src.dim() == 2 || src.dim() == 3, "operands have at most one leading (group) dimension");
    std::vector<int64_t> shape(src.sizes().begin(), src.sizes().end());
    shape.back() = pitch;
    auto buf = torch::empty(shape, t.options().dtype(torch::kUInt8));
    void* stream = stream_of(t);
    const int64_t groups = src.dim() == 3 ? src.size(0) : 1;
    for (int64_t g = 0; g < groups; ++g) {
        const auto s = src.dim() == 3 ? src[g] : src;
        const auto b = src.dim() == 3 ? buf[g] : buf;
        check(dg_pad_rows_launch(s.data_ptr(), (uint64_t)(s.stride(0) * es), b.data_ptr(), (uint64_t)pitch, (uint64_t)rows, (uint64_t)cols, stream));
    }
    auto view = buf.slice(-1, 0, cols).view(t.scalar_type());
    return major == DG_MAJOR_K ? view : view.transpose(-2, -1);
}

// Packed E2M1 operand (int8, two codes per byte along its contiguous axis) -> the same logical matrix as E4M3 bytes,
// exactly, with the same major: for packed operands whose base, strides or extent break the rules of TMA's 4-bit
// unpacking where the kernel has no decoder (dg_fp4_expansion_needed).
inline torch::Tensor expand_fp4_operand(const torch::Tensor& t, int major) {
    const auto src = major == DG_MAJOR_K ? t : t.transpose(-2, -1);
    host_assert(src.dim() == 2 || src.dim() == 3, "operands have at most one leading (group) dimension");
    const int64_t rows = src.size(-2), cols = src.size(-1), pitch = align_up(2 * cols, 32);
    std::vector<int64_t> shape(src.sizes().begin(), src.sizes().end());
    shape.back() = pitch;
    auto buf = torch::empty(shape, t.options().dtype(torch::kUInt8));
    if (!t.is_meta()) {
        void* stream = stream_of(t);
        const int64_t groups = src.dim() == 3 ? src.size(0) : 1;
        for (int64_t g = 0; g < groups; ++g) {
            const auto s = src.dim() == 3 ? src[g] : src;
            const auto b = src.dim() == 3 ? buf[g] : buf;
            check(dg_expand_fp4_launch(s.data_ptr(), (uint64_t)s.stride(0), b.data_ptr(), (uint64_t)pitch, (uint64_t)rows, (uint64_t)cols, stream));
        }
    }
    auto view = buf.slice(-1, 0, 2 * cols).view(torch::kFloat8_e4m3fn);
    return major == DG_MAJOR_K ? view : view.transpose(-2, -1);
}

inline void apply_config_override(const OptConfig& config, dg_gemm_config_t& cfg) {
    memset(&cfg, 0, sizeof(cfg));
    for (auto item : config.value()) {
        const auto key = item.first.cast<std::string>();
        const auto value = item.second.cast<int64_t>();
        if (key == "block_m") cfg.block_m = (uint32_t)value;
        else if (key == "block_n") cfg.block_n = (uint32_t)value;
        else if (key == "block_k") cfg.block_k = (uint32_t)value;
        else if (key == "num_stages") cfg.num_stages = (uint32_t)value;
        else if (key == "cta_group") cfg.cta_group = (uint32_t)value;
        else if (key == "split_k") cfg.split_k = (uint32_t)value;
        else if (key == "store_bufs") cfg.reserved[1] = (uint32_t)value;
        else if (key == "k_stagger") cfg.reserved[2] = (uint32_t)value;
        else if (key == "cluster_split") cfg.reserved[3] = (uint32_t)value;
        else if (key == "raster_group") cfg.reserved[4] = (uint32_t)value;
        else if (key == "epilogue_warps") {
            host_assert(value == 4 || value == 8, "epilogue_warps must be 4 or 8");
            cfg.reserved[5] = value == 8 ? 2u : 1u;
        } else throw std::runtime_error("unknown config key '" + key + "'");
    }
}

// csrc/apis/gemm.hpp:60-197 followed by the dispatch of :22-33. `a`, `b` are the logical [.., MN, K] views.
inline void run_gemm(int gemm_type, const torch::Tensor& a, const torch::Tensor& b, const torch::Tensor& d, const OptTensor& c,
                     std::shared_ptr<EpilogueClass> epilogue, const OptTensor& sfa_in, const OptTensor& sfb_in,
                     const std::optional<Recipe3>& recipe, const std::optional<Recipe2>& recipe_a, const std::optional<Recipe2>& recipe_b,
                     const OptTensor& grouped_layout, bool disable_ue8m0_cast, int64_t expected_m, const OptConfig& config) {
    const int major_a = major_ab(a), major_b = major_ab(b);
    int64_t g = 0, m = 0, n = 0, k = 0;
    const auto take = [&](const std::vector<int64_t>& v) { if (v.size() == 3) { m = v[0]; n = v[1]; k = v[2]; } else { g = v[0]; m = v[1]; n = v[2]; k = v[3]; } };
    if (gemm_type == DG_GEMM_NORMAL) {
        take(shape_by_spec("mnk", {{"mk", &a}, {"nk", &b}, {"mn", &d}}));
    } else if (gemm_type == DG_GEMM_M_GROUPED_PSUM) {
        take(shape_by_spec("gmnk", {{"mk", &a}, {"gnk", &b}, {"mn", &d}, {"g", &grouped_layout.value()}}));
        host_assert(major_a == DG_MAJOR_K, "A must be K-major for the m-grouped contiguous layout");
    } else if (gemm_type == DG_GEMM_M_GROUPED_MASKED) {
        take(shape_by_spec("gmnk", {{"gmk", &a}, {"gnk", &b}, {"gmn", &d}, {"g", &grouped_layout.value()}}));
        host_assert(major_a == DG_MAJOR_K, "A must be K-major for the m-grouped masked layout");
    } else if (gemm_type == DG_GEMM_K_GROUPED_PSUM) {
        take(shape_by_spec("gmnk", {{"mk", &a}, {"nk", &b}, {"gmn", &d}, {"g", &grouped_layout.value()}}));
        host_assert(major_a == DG_MAJOR_MN, "A must be MN-major for the k-grouped layout");
        host_assert(major_b == DG_MAJOR_MN, "B must be MN-major for the k-grouped layout");
    } else if (gemm_type == DG_GEMM_BATCHED) {
        take(shape_by_spec("bmnk", {{"bmk", &a}, {"bnk", &b}, {"bmn", &d}}));
    } else {
        throw std::runtime_error("Unsupported gemm type");
    }
    host_assert(d.dim() >= 2 && d.stride(-1) == 1, "D must be contiguous in its last dimension");
    if (grouped_layout.has_value()) {
        host_assert(grouped_layout->is_contiguous(), "grouped_layout must be contiguous");
        host_assert(grouped_layout->scalar_type() == torch::kInt32, "grouped_layout must be int32");
    }

    const bool is_cd_same = c.has_value() && same_buffer(c.value(), d);
    const bool with_bias = gemm_type == DG_GEMM_NORMAL && c.has_value() && !is_cd_same;
    if (gemm_type == DG_GEMM_NORMAL && c.has_value()) {
        host_assert(c->dim() == 2 && c->size(0) == (with_bias ? 1 : m) && c->size(1) == n,
                    "C must match D's pointer and shape for accumulation, or be a separate [1, N] bias");
        host_assert(c->device() == d.device(), "C and D must be on the same device");
    }
    if (with_bias) {
        host_assert(c->is_contiguous(), "Bias must be contiguous");
        host_assert(epilogue->kind() != DG_EPILOGUE_ALPHA, "alpha and bias cannot be used together");
    }
    if (gemm_early_return(m, n, k, d, c, with_bias)) return;
    if (with_bias) epilogue = std::make_shared<BiasEpilogue>(c.value());

    const bool masked = gemm_type == DG_GEMM_M_GROUPED_MASKED || gemm_type == DG_GEMM_BATCHED;   // A, SFA and D carry the group dimension
    const bool bf16 = a.scalar_type() == torch::kBFloat16 && b.scalar_type() == torch::kBFloat16;   // no scale factors (csrc/apis/gemm.hpp:412-433)
    host_assert(bf16 || (sfa_in.has_value() && sfb_in.has_value()), "Unsupported operand dtypes");
    torch::Tensor sfa, sfb;
    if (!bf16) {
        const auto [gran_m, gran_n, gran_k_a, gran_k_b] = get_recipe(recipe, recipe_a, recipe_b);
        if (gemm_type == DG_GEMM_K_GROUPED_PSUM) {
            sfa = transform_sf(sfa_in.value(), m, k, gran_m, gran_k_a, std::nullopt, false, std::nullopt, true, grouped_layout);
            sfb = transform_sf(sfb_in.value(), n, k, gran_n, gran_k_b, std::nullopt, false, std::nullopt, true, grouped_layout);
        } else {
            sfa = transform_sf(sfa_in.value(), m, k, gran_m, gran_k_a, masked ? std::optional<int>((int)g) : std::nullopt, disable_ue8m0_cast,
                               gemm_type == DG_GEMM_M_GROUPED_PSUM ? grouped_layout : std::nullopt, true);
            sfb = transform_sf(sfb_in.value(), n, k, gran_n, gran_k_b, gemm_type != DG_GEMM_NORMAL ? std::optional<int>((int)g) : std::nullopt,
                               disable_ue8m0_cast, std::nullopt, true);
        }
    }
    dg_gemm_desc_t desc;
    memset(&desc, 0, sizeof(desc));
    desc.a_dtype = dtype_code(a);
    desc.b_dtype = dtype_code(b);
    desc.d_dtype = d.scalar_type() == torch::kFloat8_e4m3fn ? DG_E4M3 : dtype_code(d);
    auto a_use = tma_ready_operand(a, major_a);
    auto b_use = tma_ready_operand(b, major_b);
    desc.a = ptr_of(a_use);
    desc.b = ptr_of(b_use);
    desc.d = ptr_of(d);
    if (!bf16) {
        desc.sfa = static_cast<const int16_t*>(ptr_of(sfa));
        desc.sfb = static_cast<const int16_t*>(ptr_of(sfb));
        desc.sfa_stride = (uint64_t)sfa.stride(-1);
        desc.sfb_stride = (uint64_t)sfb.stride(-1);
        desc.sfa_group_stride = sfa.dim() == 3 ? (uint64_t)sfa.stride(0) : 0;
        desc.sfb_group_stride = sfb.dim() == 3 ? (uint64_t)sfb.stride(0) : 0;
    }
    desc.m = (uint32_t)m; desc.n = (uint32_t)n; desc.k = (uint32_t)k;
    desc.major_a = major_a; desc.major_b = major_b;
    desc.outer_stride_a = (uint64_t)outer_stride(a_use, major_a);
    desc.outer_stride_b = (uint64_t)outer_stride(b_use, major_b);
    desc.outer_stride_d = (uint64_t)d.stride(-2);
    desc.group_stride_a = masked ? (uint64_t)a_use.stride(0) : 0;
    desc.group_stride_b = b_use.dim() == 3 ? (uint64_t)b_use.stride(0) : 0;
    desc.group_stride_d = (masked || gemm_type == DG_GEMM_K_GROUPED_PSUM) ? (uint64_t)d.stride(0) : 0;
    desc.gemm_type = gemm_type;
    if (!bf16 && (a.scalar_type() == kPackedFp4 || b.scalar_type() == kPackedFp4)) {
        // packed operands the kernels cannot read as they are become E4M3 first (exact)
        int expand_a = 0, expand_b = 0;
        check(dg_fp4_expansion_needed(&desc, &expand_a, &expand_b));
        if (expand_a) {
            a_use = expand_fp4_operand(a_use, major_a);
            desc.a = ptr_of(a_use); desc.a_dtype = DG_E4M3;
            desc.outer_stride_a = (uint64_t)outer_stride(a_use, major_a);
            desc.group_stride_a = masked ? (uint64_t)a_use.stride(0) : 0;
        }
        if (expand_b) {
            b_use = expand_fp4_operand(b_use, major_b);
            desc.b = ptr_of(b_use); desc.b_dtype = DG_E4M3;
            desc.outer_stride_b = (uint64_t)outer_stride(b_use, major_b);
            desc.group_stride_b = b_use.dim() == 3 ? (uint64_t)b_use.stride(0) : 0;
        }
    }
    desc.accumulate = (c.has_value() && !with_bias) ? 1 : 0;
    desc.grouped_layout = grouped_layout.has_value() ? static_cast<const int32_t*>(ptr_of(grouped_layout.value())) : nullptr;
    desc.num_groups = (uint32_t)g;
    // (for the k-grouped layout `expected_m` carries the expected K of one group, csrc/apis/gemm.hpp:35-43)
    desc.expected_m = (uint32_t)(expected_m > 0 ? expected_m : (gemm_type == DG_GEMM_M_GROUPED_PSUM && g ? m / g : m));
    desc.epilogue = epilogue->kind();
    if (auto* alpha = dynamic_cast<AlphaEpilogue*>(epilogue.get())) desc.alpha = alpha->alpha;
    if (auto* bias = dynamic_cast<BiasEpilogue*>(epilogue.get())) desc.bias = ptr_of(bias->bias);
    if (auto* quant = dynamic_cast<FP8QuantizationEpilogue*>(epilogue.get())) {
        desc.sfd = static_cast<int16_t*>(ptr_of(quant->sfd));
        desc.sfd_stride = (uint64_t)quant->sfd.stride(1);
    }
    desc.deterministic = runtime().deterministic ? 1 : 0;

    dg_gemm_config_t cfg;
    const dg_gemm_config_t* cfg_ptr = nullptr;
    if (config.has_value()) {
        apply_config_override(config, cfg);
        cfg_ptr = &cfg;
    }
    if (runtime().dry_run || d.is_meta()) {
        check(dg_gemm_dry_run(&desc, cfg_ptr));
        return;
    }
    void* stream = stream_of(d);
    const size_t ws_bytes = dg_gemm_workspace_bytes(&desc, cfg_ptr);
    torch::Tensor ws;
    if (ws_bytes != 0) ws = workspace(d.device(), stream, (int64_t)ws_bytes);
    check(dg_gemm_launch(&desc, cfg_ptr, ws.defined() ? ws.data_ptr() : nullptr, ws.defined() ? (size_t)ws.numel() : 0, stream));
    // a_use / b_use / sfa / sfb may be temporaries: the caching allocator keeps them valid for work already enqueued on
    // this stream, exactly as the reference relies on (csrc/jit_kernels/gemm_config.hpp:77-78).
}

inline TensorPair transposed(const TensorPair& p, bool enable, int d0, int d1) {
    return enable ? TensorPair{p.first.transpose(d0, d1), p.second.transpose(d0, d1)} : p;
}

// ---- dense FP8 / FP8 x FP4 (csrc/apis/gemm.hpp:199-256)
template <bool kTransA, bool kTransB>
static void fp8_fp4_gemm(const TensorPair& a, const TensorPair& b, const torch::Tensor& d, const OptTensor& c,
                         const std::optional<Recipe3>& recipe, const std::optional<Recipe2>& recipe_a,
                         const std::optional<Recipe2>& recipe_b, const std::string& compiled_dims, const bool& disable_ue8m0_cast,
                         const std::optional<float>& alpha, const std::shared_ptr<EpilogueClass>& epilogue, const OptConfig& config) {
    const auto at = transposed(a, kTransA, 0, 1), bt = transposed(b, kTransB, 0, 1);
    host_assert(d.scalar_type() == torch::kBFloat16 || d.scalar_type() == torch::kFloat32, "D must be bf16 or fp32");
    run_gemm(DG_GEMM_NORMAL, at.first, bt.first, d, c, resolve_epilogue(epilogue, c, d, alpha), at.second, bt.second,
             recipe, recipe_a, recipe_b, std::nullopt, disable_ue8m0_cast, 0, config);
}

// ---- m-grouped contiguous (csrc/apis/gemm.hpp:258-324)
template <bool kTransB>
static void m_grouped_fp8_fp4_gemm_contiguous(const TensorPair& a, const TensorPair& b, const torch::Tensor& d, const torch::Tensor& grouped_layout,
                                              const std::optional<Recipe3>& recipe, const std::optional<Recipe2>& recipe_a,
                                              const std::optional<Recipe2>& recipe_b, const std::string& compiled_dims,
                                              const bool& disable_ue8m0_cast, const bool& use_psum_layout, const bool& ensure_zero_padding,
                                              const std::optional<int>& expected_m_for_psum_layout,
                                              const std::shared_ptr<EpilogueClass>& epilogue, const OptConfig& config) {
    const auto bt = transposed(b, kTransB, 1, 2);
    const auto ok = [](const torch::Tensor& t) { return t.scalar_type() == torch::kFloat8_e4m3fn || t.scalar_type() == kPackedFp4; };
    host_assert(ok(a.first) && ok(bt.first), "Unsupported operand dtypes");
    host_assert(d.scalar_type() == torch::kBFloat16 || d.scalar_type() == torch::kFloat32, "D must be bf16 or fp32");
    host_assert(use_psum_layout, "use_psum_layout must be True");
    run_gemm(DG_GEMM_M_GROUPED_PSUM, a.first, bt.first, d, std::nullopt, resolve_epilogue(epilogue, std::nullopt, d), a.second, bt.second,
             recipe, recipe_a, recipe_b, grouped_layout, disable_ue8m0_cast, expected_m_for_psum_layout.value_or(0), config);
}

// ---- m-grouped masked. The reference only names this entry point (csrc/apis/gemm.hpp:606,630); the signature follows
// its contiguous sibling. A [G, max_m, K], B [G, N, K], D [G, max_m, N], masked_m int32 [G] read on the device.
static void m_grouped_fp8_fp4_gemm_nt_masked(const TensorPair& a, const TensorPair& b, const torch::Tensor& d, const torch::Tensor& masked_m,
                                             const int& expected_m, const std::optional<Recipe3>& recipe,
                                             const std::optional<Recipe2>& recipe_a, const std::optional<Recipe2>& recipe_b,
                                             const std::string& compiled_dims, const bool& disable_ue8m0_cast,
                                             const std::shared_ptr<EpilogueClass>& epilogue, const OptConfig& config) {
    host_assert(d.scalar_type() == torch::kBFloat16 || d.scalar_type() == torch::kFloat32, "D must be bf16 or fp32");
    run_gemm(DG_GEMM_M_GROUPED_MASKED, a.first, b.first, d, std::nullopt, resolve_epilogue(epilogue, std::nullopt, d), a.second, b.second,
             recipe, recipe_a, recipe_b, masked_m, disable_ue8m0_cast, expected_m, config);
}

// `ks_cpu` (the host's copy of the group sizes) only feeds the tiling heuristic; None or an empty list is accepted.
inline int64_t expected_k_of(const std::optional<std::vector<int>>& ks_cpu, int64_t k, int64_t g) {
    if (!ks_cpu.has_value() || ks_cpu->empty()) return g ? k / g : k;
    int64_t sum = 0;
    for (int v : ks_cpu.value()) sum += v;
    return std::max<int64_t>(1, sum / (int64_t)ks_cpu->size());
}

// ---- k-grouped (csrc/apis/gemm.hpp:325-410): a = (A [K, M], sfA [ceil(K/32), M]), b = (B [K, N], sfB), K holding G
// groups in psum layout; D[g] = A[group g]^T @ B[group g] (+ C[g] when `c` is D itself).
static void k_grouped_fp8_gemm_tn_contiguous(const TensorPair& a, const TensorPair& b, const torch::Tensor& d, const std::optional<std::vector<int>>& ks_cpu,
                                             const torch::Tensor& grouped_layout, const OptTensor& c, const Recipe3& recipe,
                                             const std::string& compiled_dims, const bool& use_psum_layout,
                                             const std::shared_ptr<EpilogueClass>& epilogue, const OptConfig& config) {
    const auto at = transposed(a, true, 0, 1), bt = transposed(b, true, 0, 1);
    const auto ok = [](const torch::Tensor& t) { return t.scalar_type() == torch::kFloat8_e4m3fn || t.scalar_type() == kPackedFp4; };
    host_assert(ok(at.first) && ok(bt.first), "Unsupported operand dtypes");
    host_assert(d.scalar_type() == torch::kBFloat16 || d.scalar_type() == torch::kFloat32);
    host_assert(use_psum_layout);
    run_gemm(DG_GEMM_K_GROUPED_PSUM, at.first, bt.first, d, c, resolve_epilogue(epilogue, c, d), at.second, bt.second, recipe, std::nullopt,
             std::nullopt, grouped_layout, false, expected_k_of(ks_cpu, at.first.size(-1), grouped_layout.numel()), config);
}

static void k_grouped_fp8_gemm_nt_contiguous(const TensorPair& a, const TensorPair& b, const torch::Tensor& d, const std::optional<std::vector<int>>& ks_cpu,
                                             const torch::Tensor& grouped_layout, const OptTensor& c, const Recipe3& recipe,
                                             const std::string& compiled_dims, const bool& use_psum_layout,
                                             const std::shared_ptr<EpilogueClass>& epilogue, const OptConfig& config) {
    // csrc/apis/gemm.hpp:386-410: deprecated, takes A [M, K] and B [N, K] and forwards their transposes.
    PyErr_WarnEx(PyExc_DeprecationWarning,
                 "Calling k_grouped_fp8_gemm_nt_contiguous is deprecated, please transpose a, b into [k, m] and [k, n] "
                 "shape and call `k_grouped_fp8_gemm_tn_contiguous` instead", 1);
    k_grouped_fp8_gemm_tn_contiguous(transposed(a, true, 0, 1), transposed(b, true, 0, 1), d, ks_cpu, grouped_layout, c, recipe,
                                     compiled_dims, use_psum_layout, epilogue, config);
}

// ---- BF16 family (csrc/apis/gemm.hpp:412-560): same kernels with kind::f16 MMAs and no scale factors
template <bool kTransA, bool kTransB>
static void bf16_gemm(const torch::Tensor& a, const torch::Tensor& b, const torch::Tensor& d, const OptTensor& c,
                      const std::string& compiled_dims, const std::optional<float>& alpha,
                      const std::shared_ptr<EpilogueClass>& epilogue, const OptConfig& config) {
    const auto at = kTransA ? a.transpose(0, 1) : a, bt = kTransB ? b.transpose(0, 1) : b;
    host_assert(at.scalar_type() == torch::kBFloat16 && bt.scalar_type() == torch::kBFloat16, "A and B must be bfloat16");
    host_assert(d.scalar_type() == torch::kBFloat16 || d.scalar_type() == torch::kFloat32, "D must be bf16 or fp32");
    run_gemm(DG_GEMM_NORMAL, at, bt, d, c, resolve_epilogue(epilogue, c, d, alpha), std::nullopt, std::nullopt, std::nullopt,
             std::nullopt, std::nullopt, std::nullopt, false, 0, config);
}

template <bool kTransB>
static void m_grouped_bf16_gemm_contiguous(const torch::Tensor& a, const torch::Tensor& b, const torch::Tensor& d, const torch::Tensor& grouped_layout,
                                           const std::string& compiled_dims, const bool& use_psum_layout, const bool& ensure_zero_padding,
                                           const std::optional<int>& expected_m_for_psum_layout,
                                           const std::shared_ptr<EpilogueClass>& epilogue, const OptConfig& config) {
    const auto bt = kTransB ? b.transpose(1, 2) : b;
    host_assert(a.scalar_type() == torch::kBFloat16 && bt.scalar_type() == torch::kBFloat16, "A and B must be bfloat16");
    host_assert(d.scalar_type() == torch::kBFloat16 || d.scalar_type() == torch::kFloat32, "D must be bf16 or fp32");
    host_assert(use_psum_layout, "use_psum_layout must be True");
    run_gemm(DG_GEMM_M_GROUPED_PSUM, a, bt, d, std::nullopt, resolve_epilogue(epilogue, std::nullopt, d), std::nullopt, std::nullopt,
             std::nullopt, std::nullopt, std::nullopt, grouped_layout, true, expected_m_for_psum_layout.value_or(0), config);
}

static void k_grouped_bf16_gemm_tn_contiguous(const torch::Tensor& a, const torch::Tensor& b, const torch::Tensor& d, const std::optional<std::vector<int>>& ks_cpu,
                                              const torch::Tensor& grouped_layout, const OptTensor& c, const std::string& compiled_dims,
                                              const bool& use_psum_layout, const std::shared_ptr<EpilogueClass>& epilogue, const OptConfig& config) {
    const auto at = a.transpose(0, 1), bt = b.transpose(0, 1);
    host_assert(at.scalar_type() == torch::kBFloat16 && bt.scalar_type() == torch::kBFloat16, "A and B must be bfloat16");
    host_assert(d.scalar_type() == torch::kBFloat16 || d.scalar_type() == torch::kFloat32);
    host_assert(use_psum_layout);
    run_gemm(DG_GEMM_K_GROUPED_PSUM, at, bt, d, c, resolve_epilogue(epilogue, c, d), std::nullopt, std::nullopt, std::nullopt, std::nullopt,
             std::nullopt, grouped_layout, false, expected_k_of(ks_cpu, at.size(-1), grouped_layout.numel()), config);
}

// ---- batched GEMM and the three einsum forms (csrc/apis/einsum.hpp:37-71,161-216). `d` is a tensor or a (D, SFD) pair
// for E4M3 output with UE8M0 scales per 1x32.
static void fp8_bmm(const TensorPair& a, const TensorPair& b, const py::object& d, const OptTensor& c, const Recipe3& recipe,
                    const std::string& compiled_dims, const std::shared_ptr<EpilogueClass>& epilogue, const OptConfig& config) {
    torch::Tensor d_t;
    OptTensor sfd;
    if (py::isinstance<py::tuple>(d) || py::isinstance<py::list>(d)) {
        const auto seq = d.cast<py::sequence>();
        d_t = seq[0].cast<torch::Tensor>();
        sfd = seq[1].cast<torch::Tensor>();
    } else {
        d_t = d.cast<torch::Tensor>();
    }
    host_assert(a.first.scalar_type() == torch::kFloat8_e4m3fn && b.first.scalar_type() == torch::kFloat8_e4m3fn, "fp8_bmm operands must be E4M3");
    host_assert(d_t.dim() == 3 && d_t.stride(-1) == 1, "D must be [B, M, N] and contiguous in N");
    if (a.first.size(0) == 0) return;
    auto resolved = resolve_epilogue(epilogue, c, d_t, std::nullopt, sfd);
    if (auto* quant = dynamic_cast<FP8QuantizationEpilogue*>(resolved.get())) {
        if (a.first.size(-2) == 0 || b.first.size(-2) == 0 || a.first.size(-1) == 0) {
            if (!d_t.is_meta()) { d_t.zero_(); quant->sfd.zero_(); }
            return;
        }
    }
    run_gemm(DG_GEMM_BATCHED, a.first, b.first, d_t, c, resolved, a.second, b.second, recipe, std::nullopt, std::nullopt, std::nullopt,
             false, 0, config);
}

static void fp8_einsum(const std::string& expr, const TensorPair& a, const TensorPair& b, const py::object& d, const OptTensor& c,
                       const Recipe3& recipe, const std::shared_ptr<EpilogueClass>& epilogue, const OptConfig& config) {
    // expression -> permutations of (A, B, D / C) and compiled_dims
    struct Spec { std::vector<int64_t> pa, pb, pd; const char* dims; };
    Spec spec;
    if (expr == "bhr,hdr->bhd") spec = {{1, 0, 2}, {}, {1, 0, 2}, "nk"};
    else if (expr == "bhd,hdr->bhr") spec = {{1, 0, 2}, {0, 2, 1}, {1, 0, 2}, "nk"};
    else if (expr == "bhd,bhr->hdr") spec = {{1, 2, 0}, {1, 2, 0}, {}, "mn"};
    else throw std::runtime_error("Unsupported einsum expression");
    const auto perm = [](const torch::Tensor& t, const std::vector<int64_t>& p) { return p.empty() ? t : t.permute(p); };
    const bool is_pair = py::isinstance<py::tuple>(d) || py::isinstance<py::list>(d);
    host_assert(!is_pair || expr == "bhr,hdr->bhd", "only the forward expression accepts a (D, SFD) pair");
    py::object d_arg;
    if (is_pair) {
        const auto seq = d.cast<py::sequence>();
        d_arg = py::make_tuple(perm(seq[0].cast<torch::Tensor>(), spec.pd), seq[1]);
    } else {
        d_arg = py::cast(perm(d.cast<torch::Tensor>(), spec.pd));
    }
    const OptTensor c_arg = c.has_value() ? OptTensor(perm(c.value(), spec.pd)) : std::nullopt;
    fp8_bmm({perm(a.first, spec.pa), perm(a.second, spec.pa)}, {perm(b.first, spec.pb), perm(b.second, spec.pb)}, d_arg, c_arg, recipe,
            spec.dims, epilogue, config);
}

// ---- BF16 batched GEMM and einsum (csrc/apis/einsum.hpp:73-145): the batched scheduler with kind::f16 MMAs
static void bf16_bmm(const torch::Tensor& a, const torch::Tensor& b, const torch::Tensor& d, const OptTensor& c,
                     const std::string& compiled_dims, const std::shared_ptr<EpilogueClass>& epilogue, const OptConfig& config) {
    host_assert(a.scalar_type() == torch::kBFloat16 && b.scalar_type() == torch::kBFloat16, "A and B must be bfloat16");
    host_assert(d.scalar_type() == torch::kBFloat16 || d.scalar_type() == torch::kFloat32, "D must be bf16 or fp32");
    host_assert(d.dim() == 3 && d.stride(-1) == 1, "D must be [B, M, N] and contiguous in N");
    if (a.size(0) == 0) return;
    run_gemm(DG_GEMM_BATCHED, a, b, d, c, resolve_epilogue(epilogue, c, d), std::nullopt, std::nullopt, std::nullopt, std::nullopt,
             std::nullopt, std::nullopt, false, 0, config);
}

static void einsum(const std::string& expr, const torch::Tensor& a, const torch::Tensor& b, const torch::Tensor& d, const OptTensor& c,
                   const bool& use_cublaslt, const std::shared_ptr<EpilogueClass>& epilogue, const OptConfig& config) {
    host_assert(!use_cublaslt, "einsum: use_cublaslt is not implemented (csrc/apis/einsum.hpp:128-130)");
    const auto perm = [](const torch::Tensor& t, std::vector<int64_t> p) { return p.empty() ? t : t.permute(p); };
    const auto perm_c = [&](std::vector<int64_t> p) { return c.has_value() ? OptTensor(perm(c.value(), p)) : std::nullopt; };
    if (expr == "bhr,hdr->bhd") bf16_bmm(perm(a, {1, 0, 2}), b, perm(d, {1, 0, 2}), perm_c({1, 0, 2}), "nk", epilogue, config);
    else if (expr == "bhd,hdr->bhr") bf16_bmm(perm(a, {1, 0, 2}), perm(b, {0, 2, 1}), perm(d, {1, 0, 2}), perm_c({1, 0, 2}), "nk", epilogue, config);
    else if (expr == "bhd,bhr->hdr") bf16_bmm(perm(a, {1, 2, 0}), perm(b, {1, 2, 0}), d, c, "mn", epilogue, config);
    else throw std::runtime_error("Unsupported einsum expression");
}

inline void register_gemm_apis(py::module_& m) {
#define DG_DENSE_ARGS(dims)                                                                                            \
    py::arg("a"), py::arg("b"), py::arg("d"), py::arg("c") = std::nullopt, py::arg("recipe") = std::nullopt,           \
    py::arg("recipe_a") = std::nullopt, py::arg("recipe_b") = std::nullopt, py::arg("compiled_dims") = dims,           \
    py::arg("disable_ue8m0_cast") = false, py::arg("alpha") = std::nullopt, py::arg("epilogue") = nullptr,             \
    py::kw_only(), py::arg("config") = std::nullopt
    m.def("fp8_fp4_gemm_nt", &fp8_fp4_gemm<false, false>, DG_DENSE_ARGS("nk"));
    m.def("fp8_fp4_gemm_nn", &fp8_fp4_gemm<false, true>, DG_DENSE_ARGS("nk"));
    m.def("fp8_fp4_gemm_tn", &fp8_fp4_gemm<true, true>, DG_DENSE_ARGS("mn"));
    m.def("fp8_fp4_gemm_tt", &fp8_fp4_gemm<true, false>, DG_DENSE_ARGS("mn"));
#undef DG_DENSE_ARGS
#define DG_M_GROUPED_ARGS                                                                                              \
    py::arg("a"), py::arg("b"), py::arg("d"), py::arg("grouped_layout"), py::arg("recipe") = std::nullopt,            \
    py::arg("recipe_a") = std::nullopt, py::arg("recipe_b") = std::nullopt, py::arg("compiled_dims") = "nk",           \
    py::arg("disable_ue8m0_cast") = false, py::arg("use_psum_layout") = true, py::arg("ensure_zero_padding") = true,    \
    py::arg("expected_m_for_psum_layout") = std::nullopt, py::arg("epilogue") = nullptr,                               \
    py::kw_only(), py::arg("config") = std::nullopt
    m.def("m_grouped_fp8_fp4_gemm_nt_contiguous", &m_grouped_fp8_fp4_gemm_contiguous<false>, DG_M_GROUPED_ARGS);
    m.def("m_grouped_fp8_fp4_gemm_nn_contiguous", &m_grouped_fp8_fp4_gemm_contiguous<true>, DG_M_GROUPED_ARGS);
#undef DG_M_GROUPED_ARGS
    m.def("m_grouped_fp8_fp4_gemm_nt_masked", &m_grouped_fp8_fp4_gemm_nt_masked,
          py::arg("a"), py::arg("b"), py::arg("d"), py::arg("masked_m"), py::arg("expected_m"), py::arg("recipe") = std::nullopt,
          py::arg("recipe_a") = std::nullopt, py::arg("recipe_b") = std::nullopt, py::arg("compiled_dims") = "nk",
          py::arg("disable_ue8m0_cast") = false, py::arg("epilogue") = nullptr, py::kw_only(), py::arg("config") = std::nullopt);
#define DG_K_GROUPED_ARGS                                                                                              \
    py::arg("a"), py::arg("b"), py::arg("d"), py::arg("ks_cpu"), py::arg("grouped_layout"), py::arg("c") = std::nullopt, \
    py::arg("recipe") = std::make_tuple(1, 1, 32), py::arg("compiled_dims") = "mn", py::arg("use_psum_layout") = true,  \
    py::arg("epilogue") = nullptr, py::kw_only(), py::arg("config") = std::nullopt
    m.def("k_grouped_fp8_gemm_tn_contiguous", &k_grouped_fp8_gemm_tn_contiguous, DG_K_GROUPED_ARGS);
    m.def("k_grouped_fp8_gemm_nt_contiguous", &k_grouped_fp8_gemm_nt_contiguous, DG_K_GROUPED_ARGS);
#undef DG_K_GROUPED_ARGS
    m.attr("fp8_gemm_nt") = m.attr("fp8_fp4_gemm_nt");
    m.attr("fp8_gemm_nn") = m.attr("fp8_fp4_gemm_nn");
    m.attr("fp8_gemm_tn") = m.attr("fp8_fp4_gemm_tn");
    m.attr("fp8_gemm_tt") = m.attr("fp8_fp4_gemm_tt");
    m.attr("m_grouped_fp8_gemm_nt_contiguous") = m.attr("m_grouped_fp8_fp4_gemm_nt_contiguous");
    m.attr("m_grouped_fp8_gemm_nn_contiguous") = m.attr("m_grouped_fp8_fp4_gemm_nn_contiguous");
    m.attr("m_grouped_fp8_gemm_nt_masked") = m.attr("m_grouped_fp8_fp4_gemm_nt_masked");

#define DG_BF16_ARGS(dims)                                                                                             \
    py::arg("a"), py::arg("b"), py::arg("d"), py::arg("c") = std::nullopt, py::arg("compiled_dims") = dims,            \
    py::arg("alpha") = std::nullopt, py::arg("epilogue") = nullptr, py::kw_only(), py::arg("config") = std::nullopt
    m.def("bf16_gemm_nt", &bf16_gemm<false, false>, DG_BF16_ARGS("nk"));
    m.def("bf16_gemm_nn", &bf16_gemm<false, true>, DG_BF16_ARGS("nk"));
    m.def("bf16_gemm_tn", &bf16_gemm<true, true>, DG_BF16_ARGS("mn"));
    m.def("bf16_gemm_tt", &bf16_gemm<true, false>, DG_BF16_ARGS("mn"));
#undef DG_BF16_ARGS
#define DG_M_GROUPED_BF16_ARGS                                                                                         \
    py::arg("a"), py::arg("b"), py::arg("d"), py::arg("grouped_layout"), py::arg("compiled_dims") = "nk",              \
    py::arg("use_psum_layout") = true, py::arg("ensure_zero_padding") = true,                                          \
    py::arg("expected_m_for_psum_layout") = std::nullopt, py::arg("epilogue") = nullptr,                               \
    py::kw_only(), py::arg("config") = std::nullopt
    m.def("m_grouped_bf16_gemm_nt_contiguous", &m_grouped_bf16_gemm_contiguous<false>, DG_M_GROUPED_BF16_ARGS);
    m.def("m_grouped_bf16_gemm_nn_contiguous", &m_grouped_bf16_gemm_contiguous<true>, DG_M_GROUPED_BF16_ARGS);
#undef DG_M_GROUPED_BF16_ARGS
    m.def("k_grouped_bf16_gemm_tn_contiguous", &k_grouped_bf16_gemm_tn_contiguous,
          py::arg("a"), py::arg("b"), py::arg("d"), py::arg("ks_cpu"), py::arg("grouped_layout"), py::arg("c") = std::nullopt,
          py::arg("compiled_dims") = "mn", py::arg("use_psum_layout") = true, py::arg("epilogue") = nullptr,
          py::kw_only(), py::arg("config") = std::nullopt);

    m.def("fp8_bmm", &fp8_bmm, py::arg("a"), py::arg("b"), py::arg("d"), py::arg("c") = std::nullopt,
          py::arg("recipe") = std::make_tuple(1, 1, 32), py::arg("compiled_dims") = "nk", py::arg("epilogue") = nullptr,
          py::kw_only(), py::arg("config") = std::nullopt);
    m.def("bf16_bmm", &bf16_bmm, py::arg("a"), py::arg("b"), py::arg("d"), py::arg("c") = std::nullopt, py::arg("compiled_dims") = "nk",
          py::arg("epilogue") = nullptr, py::kw_only(), py::arg("config") = std::nullopt);
    m.def("einsum", &einsum, py::arg("expr"), py::arg("a"), py::arg("b"), py::arg("d"), py::arg("c") = std::nullopt,
          py::arg("use_cublaslt") = false, py::arg("epilogue") = nullptr, py::kw_only(), py::arg("config") = std::nullopt);
    m.def("fp8_einsum", &fp8_einsum, py::arg("expr"), py::arg("a"), py::arg("b"), py::arg("d"), py::arg("c") = std::nullopt,
          py::arg("recipe") = std::make_tuple(1, 1, 32), py::arg("epilogue") = nullptr, py::kw_only(), py::arg("config") = std::nullopt);
}

}  // namespace dg_host
