// Gate top-k: the k largest logits of every token and their expert indices, and the
// backward of that selection.  Replaces the torch.topk call of the reference's gates
// (fmoe/gates/naive_gate.py:31-34, gshard_gate.py / switch_gate.py through NaiveGate)
// and the scatter its autograd runs in the backward pass.
//
// One warp per token.  Each lane keeps the best k of the logits it strides over in
// registers (descending value, ascending expert index among equal values; NaN ranks
// above every number, as in torch.topk), then k rounds of a warp arg-max pick the
// winners in order.  Values are copied, never rounded.
#include "common.cuh"
#include <algorithm>
#include <climits>
#include <cmath>

namespace fmoe {
namespace {

constexpr int kTopKMax = 8;

// (a, ia) ranks before (b, ib)
__device__ __forceinline__ bool ranks_before(float a, int ia, float b, int ib) {
    const bool na = a != a, nb = b != b;
    if (na != nb) return na;
    if (!na && a != b) return a > b;
    return ia < ib;
}

template <typename T>
__global__ void __launch_bounds__(256)
topk_forward_kernel(const T* __restrict__ logits, int64_t n_tokens, int n_expert, int k, T* __restrict__ values,
                    int64_t* __restrict__ indices) {
    const int lane = threadIdx.x & 31;
    const int64_t tok = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (tok >= n_tokens) return;
    const T* row = logits + tok * n_expert;
    float best[kTopKMax];
    int best_i[kTopKMax];
#pragma unroll
    for (int j = 0; j < kTopKMax; ++j) { best[j] = -INFINITY; best_i[j] = INT_MAX; }
    for (int e = lane; e < n_expert; e += 32) {
        float v = to_float(row[e]);
        int vi = e;
        // insertion into the lane's sorted list (entries past k are never read)
#pragma unroll
        for (int j = 0; j < kTopKMax; ++j) {
            if (j < k && ranks_before(v, vi, best[j], best_i[j])) {
                const float tv = best[j]; const int ti = best_i[j];
                best[j] = v; best_i[j] = vi;
                v = tv; vi = ti;
            }
        }
    }
    for (int j = 0; j < k; ++j) {
        float v = best[0];
        int vi = best_i[0];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, v, off);
            const int oi = __shfl_xor_sync(0xffffffffu, vi, off);
            if (ranks_before(ov, oi, v, vi)) { v = ov; vi = oi; }
        }
        if (best_i[0] == vi) {  // this lane owned the winner: drop it
#pragma unroll
            for (int q = 0; q + 1 < kTopKMax; ++q) { best[q] = best[q + 1]; best_i[q] = best_i[q + 1]; }
            best[kTopKMax - 1] = -INFINITY; best_i[kTopKMax - 1] = INT_MAX;
        }
        if (lane == 0) {
            values[tok * k + j] = row[vi];
            indices[tok * k + j] = vi;
        }
    }
}

// Few experts (<= 32): one THREAD per token; a warp then reads 32 consecutive rows, i.e. one
// contiguous stretch of the logits, and no lane idles.  Same order as the warp kernel.
template <typename T>
__global__ void __launch_bounds__(256)
topk_forward_small_kernel(const T* __restrict__ logits, int64_t n_tokens, int n_expert, int k, T* __restrict__ values,
                          int64_t* __restrict__ indices) {
    const int64_t tok = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (tok >= n_tokens) return;
    const T* row = logits + tok * n_expert;
    float best[kTopKMax];
    int best_i[kTopKMax];
#pragma unroll
    for (int j = 0; j < kTopKMax; ++j) { best[j] = -INFINITY; best_i[j] = INT_MAX; }
    for (int e = 0; e < n_expert; ++e) {
        float v = to_float(row[e]);
        int vi = e;
#pragma unroll
        for (int j = 0; j < kTopKMax; ++j) {
            if (j < k && ranks_before(v, vi, best[j], best_i[j])) {
                const float tv = best[j]; const int ti = best_i[j];
                best[j] = v; best_i[j] = vi;
                v = tv; vi = ti;
            }
        }
    }
#pragma unroll
    for (int j = 0; j < kTopKMax; ++j) {
        if (j < k) {
            values[tok * k + j] = row[best_i[j]];
            indices[tok * k + j] = best_i[j];
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(256)
topk_backward_kernel(const T* __restrict__ grad_values, const int64_t* __restrict__ indices, int64_t n_tokens,
                     int n_expert, int k, T* __restrict__ grad_logits) {
    const int64_t total = n_tokens * n_expert;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t tok = i / n_expert;
        const int e = (int)(i - tok * n_expert);
        float g = 0.f;
        for (int j = 0; j < k; ++j)
            if (indices[tok * k + j] == e) g += to_float(grad_values[tok * k + j]);
        grad_logits[i] = from_float<T>(g);
    }
}

}  // namespace
}  // namespace fmoe

using namespace fmoe;

extern "C" int fmoe_gate_topk(const void* logits, int64_t n_tokens, int32_t n_expert_total, int32_t k, int32_t dtype,
                              void* values, int64_t* indices, fmoe_stream_t stream) {
    FMOE_REQUIRE(n_tokens >= 0 && n_expert_total > 0, "gate_topk: n_tokens=%lld n_expert_total=%d", (long long)n_tokens,
                 n_expert_total);
    FMOE_REQUIRE(k >= 1 && k <= kTopKMax && k <= n_expert_total, "gate_topk: k=%d (1..%d, <= n_expert_total)", k, kTopKMax);
    FMOE_REQUIRE(dtype_size(dtype) > 0, "gate_topk: unknown dtype %d", dtype);
    if (n_tokens == 0) return 0;
    FMOE_REQUIRE(logits && values && indices, "gate_topk: null pointer");
    cudaStream_t st = (cudaStream_t)stream;
    if (n_expert_total <= 32) {
        const unsigned nb = (unsigned)ceil_div(n_tokens, 256);
        switch (dtype) {
            case FMOE_F32: topk_forward_small_kernel<float><<<nb, 256, 0, st>>>((const float*)logits, n_tokens, n_expert_total, k, (float*)values, indices); break;
            case FMOE_F16: topk_forward_small_kernel<__half><<<nb, 256, 0, st>>>((const __half*)logits, n_tokens, n_expert_total, k, (__half*)values, indices); break;
            default: topk_forward_small_kernel<__nv_bfloat16><<<nb, 256, 0, st>>>((const __nv_bfloat16*)logits, n_tokens, n_expert_total, k, (__nv_bfloat16*)values, indices); break;
        }
        FMOE_CHECK_LAUNCH();
        return 0;
    }
    const unsigned blocks = (unsigned)ceil_div(n_tokens, 8);
    switch (dtype) {
        case FMOE_F32: topk_forward_kernel<float><<<blocks, 256, 0, st>>>((const float*)logits, n_tokens, n_expert_total, k, (float*)values, indices); break;
        case FMOE_F16: topk_forward_kernel<__half><<<blocks, 256, 0, st>>>((const __half*)logits, n_tokens, n_expert_total, k, (__half*)values, indices); break;
        default: topk_forward_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>((const __nv_bfloat16*)logits, n_tokens, n_expert_total, k, (__nv_bfloat16*)values, indices); break;
    }
    FMOE_CHECK_LAUNCH();
    return 0;
}

extern "C" int fmoe_gate_topk_backward(const void* grad_values, const int64_t* indices, int64_t n_tokens,
                                       int32_t n_expert_total, int32_t k, int32_t dtype, void* grad_logits,
                                       fmoe_stream_t stream) {
    FMOE_REQUIRE(n_tokens >= 0 && n_expert_total > 0 && k >= 1 && k <= kTopKMax, "gate_topk_backward: bad sizes");
    FMOE_REQUIRE(dtype_size(dtype) > 0, "gate_topk_backward: unknown dtype %d", dtype);
    if (n_tokens == 0) return 0;
    FMOE_REQUIRE(grad_values && indices && grad_logits, "gate_topk_backward: null pointer");
    cudaStream_t st = (cudaStream_t)stream;
    const unsigned blocks = (unsigned)std::min<int64_t>(ceil_div(n_tokens * n_expert_total, 256), 148 * 16);
    switch (dtype) {
        case FMOE_F32: topk_backward_kernel<float><<<blocks, 256, 0, st>>>((const float*)grad_values, indices, n_tokens, n_expert_total, k, (float*)grad_logits); break;
        case FMOE_F16: topk_backward_kernel<__half><<<blocks, 256, 0, st>>>((const __half*)grad_values, indices, n_tokens, n_expert_total, k, (__half*)grad_logits); break;
        default: topk_backward_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>((const __nv_bfloat16*)grad_values, indices, n_tokens, n_expert_total, k, (__nv_bfloat16*)grad_logits); break;
    }
    FMOE_CHECK_LAUNCH();
    return 0;
}
