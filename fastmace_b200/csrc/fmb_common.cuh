// Shared helpers of the fmb200 CUDA sources: error plumbing, block scans and deterministic reductions.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/fmb200.h"

namespace fmb {

void set_error(const char* what, cudaError_t err, const char* file, int line);
void count_launch();
void set_error_text(const char* text);
// Raises a kernel's dynamic shared-memory limit on the CURRENT device, once per (device, kernel): the attribute is
// per device, so a process that drives several GPUs sets it on each of them.
cudaError_t opt_in_shared_memory(const void* kernel, int bytes);

#define FMB_CUDA_CHECK(expr)                                            \
    do {                                                                \
        cudaError_t err__ = (expr);                                     \
        if (err__ != cudaSuccess) {                                     \
            ::fmb::set_error(#expr, err__, __FILE__, __LINE__);         \
            return FMB_ERR_CUDA;                                        \
        }                                                               \
    } while (0)

#define FMB_LAUNCH_CHECK()                  \
    do {                                    \
        ::fmb::count_launch();              \
        FMB_CUDA_CHECK(cudaGetLastError()); \
    } while (0)

#define FMB_REQUIRE(cond, text)                  \
    do {                                         \
        if (!(cond)) {                           \
            ::fmb::set_error_text(text);         \
            return FMB_ERR_ARG;                  \
        }                                        \
    } while (0)

constexpr int kC = 128;          // channels
constexpr int kNSH = 16;         // spherical-harmonic components, l <= 3
constexpr int kRadial = 64;      // radial MLP width
constexpr int kBessel = 8;
constexpr int kScanBlock = 1024;
constexpr int kScanItems = 4;    // items per thread
constexpr int kScanTile = kScanBlock * kScanItems;

static inline int ceil_div(long long a, long long b) { return (int)((a + b - 1) / b); }

// Exclusive scan of `in[0..n)` into `out[0..n]` (out[n] = total). `scratch` holds >= 2 * ceil(n / 4096) + 2 ints.
// If `flag` is non-null the kernels return at once when *flag == 0.
int exclusive_scan(const int32_t* in, int32_t* out, int n, int32_t* scratch, const int32_t* flag, cudaStream_t stream);

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ int warp_sum(int v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

}  // namespace fmb
