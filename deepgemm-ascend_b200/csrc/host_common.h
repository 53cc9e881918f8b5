// Host-side helpers shared by the translation units of libdg_b200.so: the status codes of the C ABI,
// the per-thread error message, and argument / CUDA checks that return instead of throwing.
#pragma once

#include <cuda_runtime.h>
#include <cstdarg>
#include <cstdio>

#include "../../include/dg_b200.h"

namespace dg {

void set_last_error(const char* fmt, ...);
void count_kernel_launch(unsigned n = 1);

}  // namespace dg

#define DG_CHECK_ARG(cond, ...)                      \
    do {                                             \
        if (!(cond)) {                               \
            dg::set_last_error(__VA_ARGS__);         \
            return DG_ERR_INVALID;                   \
        }                                            \
    } while (0)

#define DG_UNSUPPORTED(cond, ...)                    \
    do {                                             \
        if (cond) {                                  \
            dg::set_last_error(__VA_ARGS__);         \
            return DG_ERR_UNSUPPORTED;               \
        }                                            \
    } while (0)

#define DG_CHECK_CUDA(expr)                                                                  \
    do {                                                                                     \
        cudaError_t err__ = (expr);                                                          \
        if (err__ != cudaSuccess) {                                                          \
            dg::set_last_error("CUDA error %d (%s) at %s:%d", (int)err__,                    \
                               cudaGetErrorString(err__), __FILE__, __LINE__);               \
            return DG_ERR_CUDA;                                                              \
        }                                                                                    \
    } while (0)
