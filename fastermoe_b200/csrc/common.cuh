// Shared helpers of libfmoe_b200: error reporting, dtype helpers, launch math.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cstdint>
#include <cstdio>
#include <cstdarg>
#include "../../include/fmoe_b200.h"

namespace fmoe {

// Thread-local text of the last failure; returned by fmoe_last_error_string().
void set_error(const char* fmt, ...);

inline int fail(int code, const char* fmt, ...) __attribute__((format(printf, 2, 3)));
inline int fail(int code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    set_error("%s", buf);
    return code;
}

#define FMOE_CUDA_TRY(expr)                                                         \
    do {                                                                            \
        cudaError_t err__ = (expr);                                                 \
        if (err__ != cudaSuccess) {                                                 \
            (void)cudaGetLastError(); /* do not leave the error for the next call */\
            return ::fmoe::fail(FMOE_ERR_CUDA, "%s failed: %s (%s:%d)", #expr,      \
                                cudaGetErrorString(err__), __FILE__, __LINE__);     \
        }                                                                           \
    } while (0)

#define FMOE_CHECK_LAUNCH() FMOE_CUDA_TRY(cudaGetLastError())

#define FMOE_REQUIRE(cond, ...)                                                     \
    do {                                                                            \
        if (!(cond)) return ::fmoe::fail(FMOE_ERR_INVALID, __VA_ARGS__);            \
    } while (0)

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

inline int dtype_size(int dtype) {
    switch (dtype) {
        case FMOE_F32: return 4;
        case FMOE_F16: return 2;
        case FMOE_BF16: return 2;
        default: return 0;
    }
}

// Number of SMs of the current device (cached per device).
int sm_count();

template <typename T> __device__ __forceinline__ float to_float(T v);
template <> __device__ __forceinline__ float to_float<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_float<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_float<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float apply_act(float v, int act) {
    if (act == FMOE_ACT_RELU) return v > 0.f ? v : 0.f;
    if (act == FMOE_ACT_GELU) return 0.5f * v * (1.f + erff(v * 0.70710678118654752440f));
    return v;
}
// d act(v) / dv, for the exact (erf) GELU that torch.nn.GELU() computes and for
// ReLU with the reference's convention that the gradient is zero where the
// activation output is <= 0 (cuda/fused_compute.cuh:36-44).
__device__ __forceinline__ float act_grad(float v, int act) {
    if (act == FMOE_ACT_RELU) return v > 0.f ? 1.f : 0.f;
    if (act == FMOE_ACT_GELU) {
        float cdf = 0.5f * (1.f + erff(v * 0.70710678118654752440f));
        float pdf = 0.39894228040143267794f * __expf(-0.5f * v * v);
        return cdf + v * pdf;
    }
    return 1.f;
}

// Factor that the backward multiplies into the input gradient, from the buffer the
// forward saved: for ReLU the buffer is the activation output (gradient is zero where
// it is <= 0, cuda/fused_compute.cuh:36-44); for GELU it is the derivative itself.
__device__ __forceinline__ float saved_act_grad(float saved, int act) {
    if (act == FMOE_ACT_RELU) return saved > 0.f ? 1.f : 0.f;
    if (act == FMOE_ACT_GELU) return saved;
    return 1.f;
}

}  // namespace fmoe
