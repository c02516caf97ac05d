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

#ifdef __CUDACC__
// Row range [lo, hi) of expert e, made safe for buffers of n_rows rows: the offsets come from
// device memory that no host code has looked at, so a range is clamped to start no earlier than
// the previous expert's end and to end no later than n_rows.  Valid offsets (non-decreasing,
// last one <= n_rows) pass through unchanged.  Returns true when something had to be clamped.
__device__ __forceinline__ bool safe_seg_range(const int64_t* __restrict__ off, const HostSegs& hs, int e, int64_t n_rows,
                                               int64_t& lo, int64_t& hi) {
    int64_t prev_hi = 0;
    bool clamped = false;
    for (int j = 0; j <= e; ++j) {
        const int64_t raw_lo = hs.n ? (int64_t)hs.lo[j] : off[j], raw_hi = hs.n ? (int64_t)hs.hi[j] : off[j + 1];
        lo = raw_lo < prev_hi ? prev_hi : raw_lo;
        if (lo > n_rows) lo = n_rows;
        hi = raw_hi < lo ? lo : raw_hi;
        if (hi > n_rows) hi = n_rows;
        clamped |= lo != raw_lo || hi != raw_hi;
        prev_hi = hi;
    }
    return clamped;
}
#endif

// Rows of the ragged-side input that are still arriving from other GPUs (see ArrivalWait in exchange.h;
// the struct is repeated here in plain form so that the GEMM code does not depend on the exchange code).
struct GemmArrival {
    const unsigned long long* flags;   // [2][64][256]: flags[(parity * 64 + source) * 256 + expert] >= epoch: rows are there
    const unsigned long long* seq;     // epoch word: the rows belong to epoch *seq + 1
    const int* src_off;                // [n_expert * world + 1]: first row of (expert, source)
    int world;
    int reserve_sms;                   // SMs left to the kernel that delivers the rows
};

// Per-expert completion of a product's output rows, for a kernel that forwards them while the
// product is still running: every epilogue warp adds 1 to done[e] when its part of a tile of expert e
// is stored; block 0 writes expected[e] (the count at which expert e is complete) and then *ready = 1.
struct GemmDone {
    int* done;       // [n_expert], zero before the launch
    int* expected;   // [n_expert]
    int* ready;      // [1], zero before the launch
    int reserve_sms;
};

// Output rows that go straight to the GPUs that own the tokens (the global_gather that would follow
// the product, done by the product's own epilogue with plain stores into peer memory): row r of
// this GPU's expert-side order belongs to block (expert i, source j), src_off[i*W+j] <= r <
// src_off[i*W+j+1], and lands at row dst_off[i*W+j] + (r - src_off[i*W+j]) of rank j's buffer, which
// starts at base[j] + the offset rank j announced for this epoch in this GPU's header.
constexpr int kRemoteMaxWorld = 32;
struct GemmRemoteOut {
    char* base[kRemoteMaxWorld];       // landing areas of all ranks as mapped here (own one at [rank])
    const unsigned long long* header;  // this GPU's header: flag arrays at the byte offsets below, [2][stride] u64 each
    const unsigned long long* seq;     // epoch word: this exchange is epoch *seq + 1
    const int* src_off;                // [n_expert * world + 1]
    const int* dst_off;                // [n_expert * world]
    unsigned int* counter;             // zero before the launch: CTAs that have finished
    unsigned long long my_dest;        // where this GPU receives (byte offset in its own area)
    unsigned long long min_dest;       // announcements below this offset point into the flag header: rejected
    unsigned long long timeout_cycles;
    int arrived_at, ann_at, dest_at, stride;   // header layout
    int world, rank;
    int enabled;
};

// The global_scatter that delivers a product's ragged-side input, done by the product itself: the two
// spare warps of every CTA move this GPU's token-side rows to the GPUs that own their experts (plain
// stores into peer memory, the push list of the exchange plan in expert-major order) and raise the
// per-(source, expert) arrival flags that the TMA producer warps -- here and on the peers -- wait on
// (GemmArrival).  The peer context (mapped areas, announcements, completion) is a GemmRemoteOut with
// enabled = 2.  Rows may be formed on the way: token-side row i is src[row_of[i] / row_div], times
// scale[row_of[i]] when scale is set (row_of null: row i of src).
struct GemmPushIn {
    const void* src;
    const int64_t* row_of;
    const void* scale;                 // same element type as the rows
    int64_t src_rows;
    int row_div;
    const int* prefix;                 // push list: [n_slots + 1] first row of each segment in token-side order ...
    const int* seg_sel;                //   [n_slots] destination rank (local_sel: this GPU)
    const int* seg_src;                //   [n_slots] first token-side row
    const int* seg_dst;                //   [n_slots] first row in the destination's expert-side buffer
    int* seg_done;                     // [n_slots] rows stored so far, zero before the launch (the last CTA clears it)
    const int64_t* expert_rows;        // rows this GPU receives / sends in this exchange (device words of the plan)
    const int64_t* token_rows;
    int64_t in_rows, out_rows;         // capacity of the token-side source / the expert-side buffer
    int64_t row_vecs;                  // 16-byte pieces per row
    int n_slots, n_expert, local_sel;
    int flags_at, flag_sources, flag_experts;   // arrival flags in a header: u64 [2][flag_sources][flag_experts] at byte flags_at
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
    const GemmArrival* arrival = nullptr;  // x is still being filled by an exchange
    const GemmDone* done = nullptr;        // y is forwarded expert by expert while the product runs
    const GemmRemoteOut* remote = nullptr; // y is not stored here at all: its rows go to their owners
    const GemmPushIn* push = nullptr;      // x is delivered by this product's own spare warps (with remote->enabled == 2)
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
    // grad_y is still being filled by an exchange: the input-gradient product waits tile by tile;
    // after_input_grad (called once, before anything that needs all of grad_y) closes the exchange
    const GemmArrival* arrival = nullptr;
    int (*after_input_grad)(void*) = nullptr;
    void* after_ctx = nullptr;
    const GemmDone* done = nullptr;        // grad_x is forwarded expert by expert while its product runs
    const GemmRemoteOut* remote = nullptr; // grad_x is not stored here at all: its rows go to their owners
    const GemmPushIn* push = nullptr;      // grad_y is delivered by the input-gradient product's own spare warps
};

int simt_linear_forward(const LinearArgs& a, cudaStream_t st);
int simt_linear_backward(const LinearBwdArgs& a, cudaStream_t st);

// Current FMOE_GEMM_* form (see fmoe_gemm_set_form).
int gemm_form();

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
