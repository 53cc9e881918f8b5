// Busy-wait marker kernel: the counterpart of the reference's sleep_impl (deep_gemm/include/deep_gemm/sleep.hpp:5-15,
// launched by npu_sleep, csrc/apis/runtime.hpp:64-79). Benchmarks enqueue it in front of a timed region so that the
// host can queue the launches that follow while the device is still busy, and with marker 1 / 2 as begin / end marks
// a profiler can find by kernel name.
#include <cuda_runtime.h>
#include <cstdint>

#include "host_common.h"

namespace dg {

// One block per SM spins on its SM clock until `cycles` have passed. The wait is bounded by the argument check on the
// host (at most kMaxSleepCycles, about two seconds), so the kernel always ends by itself.
constexpr int64_t kMaxSleepCycles = 4000000000ll;

template <uint32_t kMarker>
__global__ void sleep_kernel(int64_t cycles) {
    const int64_t start = clock64();
    while (clock64() - start < cycles) {
        #pragma unroll
        for (int i = 0; i < 4; ++i) asm volatile("nanosleep.u32 32;");
    }
}

}  // namespace dg

extern "C" int dg_sleep_launch(int64_t sleep_cycles, uint32_t marker, int num_blocks, void* stream) {
    DG_CHECK_ARG(sleep_cycles >= 0 && sleep_cycles <= dg::kMaxSleepCycles, "sleep_cycles must be in [0, %lld]",
                 (long long)dg::kMaxSleepCycles);
    DG_CHECK_ARG(num_blocks > 0 && num_blocks <= 65535, "num_blocks out of range");
    auto s = static_cast<cudaStream_t>(stream);
    // The marker only selects the kernel's name (sleep_kernel<0>, <1>, <2>; others share <3>).
    switch (marker) {
        case 0: dg::sleep_kernel<0><<<num_blocks, 32, 0, s>>>(sleep_cycles); break;
        case 1: dg::sleep_kernel<1><<<num_blocks, 32, 0, s>>>(sleep_cycles); break;
        case 2: dg::sleep_kernel<2><<<num_blocks, 32, 0, s>>>(sleep_cycles); break;
        default: dg::sleep_kernel<3><<<num_blocks, 32, 0, s>>>(sleep_cycles); break;
    }
    DG_CHECK_CUDA(cudaGetLastError());
    dg::count_kernel_launch();
    return DG_OK;
}
