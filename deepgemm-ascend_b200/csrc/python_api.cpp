// The `_C` torch extension of deep_gemm for B200: the same module table as the reference's csrc/python_api.cpp:29-42
// (runtime knobs, epilogue classes, GEMM entry points, scale-factor layout), with the host logic of csrc/apis in C++
// on top of the C ABI of libdg_b200.so. Nothing here computes: every launch goes through include/dg_b200.h.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>
#include <torch/python.h>

#include <map>

#include "apis/runtime.hpp"
#include "apis/epilogue_class.hpp"
#include "apis/layout.hpp"
#include "apis/gemm.hpp"

#ifndef TORCH_EXTENSION_NAME
#define TORCH_EXTENSION_NAME _C
#endif

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.doc() = "deep_gemm host layer for NVIDIA B200 (sm_100a)";
    dg_host::register_runtime_apis(m);
    dg_host::register_epilogue_apis(m);
    dg_host::register_gemm_apis(m);
    dg_host::register_layout_apis(m);
    m.attr("STATUS_INVALID_SCALE_FACTOR") = dg_host::kStatusInvalidScaleFactor;
}
