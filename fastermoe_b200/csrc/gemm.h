// Argument blocks shared by the grouped-GEMM back ends (FFMA and tcgen05).
#pragma once
#include <cuda_runtime.h>
#include <cstdint>

namespace fmoe {

// Expert row ranges known on the host (the smart schedule's per-step micro-batches):
// expert e owns rows [lo[e], hi[e]).  Passed to the kernels by value.
constexpr int kMaxHostSegs = 64;
struct HostSegs {
    int n;  // 0: unused, read the device offsets instead
    int lo[kMaxHostSegs];
    int hi[kMaxHostSegs];
};

struct LinearArgs {
    const void* x;       // [n_rows, in_feat]
    const void* weight;  // [n_expert, out_feat, in_feat]
    const void* bias;    // [n_expert, out_feat] or null
    const int64_t* seg_offsets;  // device, [n_expert + 1]
    void* y;             // [n_rows, out_feat]
    void* pre_act;       // [n_rows, out_feat] or null: receives activation'(pre-activation) (GELU)
    int64_t n_rows, in_feat, out_feat;
    int n_expert, dtype, activation;
    const HostSegs* host_segs = nullptr;  // when set, replaces seg_offsets
};

struct LinearBwdArgs {
    const void* grad_y;  // [n_rows, out_feat]
    const void* x;       // [n_rows, in_feat]
    const void* weight;  // [n_expert, out_feat, in_feat]
    const int64_t* seg_offsets;
    const void* act_pre;  // [n_rows, in_feat] or null: ReLU: activation output; GELU: saved derivative
    void* grad_x;         // [n_rows, in_feat] or null
    void* grad_w;         // [n_expert, out_feat, in_feat] or null
    void* grad_b;         // [n_expert, out_feat] or null
    int64_t n_rows, in_feat, out_feat;
    int n_expert, dtype, activation, accumulate;
    void* scratch;
    const HostSegs* host_segs = nullptr;
    // [n_expert, in_feat] or null: per-expert column sums of grad_x (what the bias gradient of
    // the layer that produced x is, when grad_x is the gradient of its output)
    void* grad_x_colsum = nullptr;
};

int simt_linear_forward(const LinearArgs& a, cudaStream_t st);
int simt_linear_backward(const LinearBwdArgs& a, cudaStream_t st);

// Picks the tensor-core kernels when the shapes allow it, else the FFMA kernels.
int dispatch_linear_forward(const LinearArgs& a, cudaStream_t st);
int dispatch_linear_backward(const LinearBwdArgs& a, cudaStream_t st);

// tcgen05 back end.  *_supported() tells whether the shapes/dtype/alignment fit
// its tiles; callers fall back to the FFMA kernels otherwise.
bool tc_forward_supported(const LinearArgs& a);
bool tc_backward_supported(const LinearBwdArgs& a);
int tc_linear_forward(const LinearArgs& a, cudaStream_t st);
int tc_linear_backward(const LinearBwdArgs& a, cudaStream_t st);
size_t tc_backward_scratch_bytes(int64_t n_rows, int64_t in_feat, int64_t out_feat, int n_expert, int dtype);

}  // namespace fmoe
