// fmoe_linear entry points: argument checks and back-end selection.
#include "common.cuh"
#include "exchange.h"
#include "gemm.h"
#include <cstdlib>

using namespace fmoe;

namespace {

// FMOE_GEMM_SIMT forces the FFMA kernels (used by tests to cross-check the tensor-core
// kernels); anything else lets the shape decide.
bool force_simt() { return gemm_form() == FMOE_GEMM_SIMT; }

int check_common(int64_t n_rows, int64_t in_feat, int64_t out_feat, int n_expert, int dtype, int act,
                 const int64_t* seg) {
    FMOE_REQUIRE(n_rows >= 0 && in_feat > 0 && out_feat > 0 && n_expert > 0,
                 "linear: bad sizes rows=%lld in=%lld out=%lld experts=%d", (long long)n_rows,
                 (long long)in_feat, (long long)out_feat, n_expert);
    FMOE_REQUIRE(dtype_size(dtype) != 0, "linear: unknown dtype %d", dtype);
    FMOE_REQUIRE(act >= FMOE_ACT_NONE && act <= FMOE_ACT_GELU, "linear: unknown activation %d", act);
    FMOE_REQUIRE(seg != nullptr, "linear: seg_offsets pointer is null");
    return 0;
}

// out[e, c] = sum of grad_x[r, c] over the rows of expert e (plain kernel for the FFMA path).
template <typename T>
__global__ void colsum_rows_kernel(const T* __restrict__ gx, const int64_t* __restrict__ seg, const HostSegs hs,
                                   T* __restrict__ out, int64_t n_rows, int64_t n_cols) {
    const int e = blockIdx.y;
    const int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= n_cols) return;
    int64_t lo, hi;
    safe_seg_range(seg, hs, e, n_rows, lo, hi);
    float s = 0.f;
    for (int64_t r = lo; r < hi; ++r) s += to_float<T>(gx[r * n_cols + c]);
    out[(int64_t)e * n_cols + c] = from_float<T>(s);
}

int colsum_rows(const LinearBwdArgs& a, cudaStream_t st) {
    static const HostSegs none = {};
    const HostSegs& hs = a.host_segs ? *a.host_segs : none;
    dim3 grid((unsigned)ceil_div(a.in_feat, 128), (unsigned)a.n_expert);
    switch (a.dtype) {
        case FMOE_F32: colsum_rows_kernel<float><<<grid, 128, 0, st>>>((const float*)a.grad_x, a.seg_offsets, hs, (float*)a.grad_x_colsum, a.n_rows, a.in_feat); break;
        case FMOE_F16: colsum_rows_kernel<__half><<<grid, 128, 0, st>>>((const __half*)a.grad_x, a.seg_offsets, hs, (__half*)a.grad_x_colsum, a.n_rows, a.in_feat); break;
        default: colsum_rows_kernel<__nv_bfloat16><<<grid, 128, 0, st>>>((const __nv_bfloat16*)a.grad_x, a.seg_offsets, hs, (__nv_bfloat16*)a.grad_x_colsum, a.n_rows, a.in_feat); break;
    }
    FMOE_CHECK_LAUNCH();
    return 0;
}

}  // namespace

namespace fmoe {
int dispatch_linear_forward(const LinearArgs& a, cudaStream_t st) {
    if (a.n_rows == 0) return 0;
    if (!force_simt() && tc_forward_supported(a)) return tc_linear_forward(a, st);
    return simt_linear_forward(a, st);
}
int dispatch_linear_backward(const LinearBwdArgs& a, cudaStream_t st) {
    if (a.grad_x_colsum) FMOE_REQUIRE(a.grad_x, "linear_backward: column sums of grad_x requested without grad_x");
    if (!force_simt() && tc_backward_supported(a) && a.n_rows > 0) return tc_linear_backward(a, st);
    if (int rc = simt_linear_backward(a, st)) return rc;
    if (a.grad_x_colsum) return colsum_rows(a, st);   // the tensor-core kernel produces them itself
    return 0;
}
}  // namespace fmoe

extern "C" size_t fmoe_linear_scratch_bytes(int64_t n_rows, int64_t in_feat, int64_t out_feat,
                                            int32_t n_expert, int32_t dtype) {
    return tc_backward_scratch_bytes(n_rows, in_feat, out_feat, n_expert, dtype);
}

extern "C" int fmoe_linear_forward(const void* x, const void* weight, const void* bias,
                                   const int64_t* seg_offsets, void* y, void* pre_act, int64_t n_rows,
                                   int64_t in_feat, int64_t out_feat, int32_t n_expert, int32_t dtype,
                                   int32_t activation, fmoe_stream_t stream) {
    if (int rc = check_common(n_rows, in_feat, out_feat, n_expert, dtype, activation, seg_offsets)) return rc;
    if (n_rows == 0) return 0;
    FMOE_REQUIRE(x && weight && y, "linear_forward: null pointer");
    LinearArgs a{x, weight, bias, seg_offsets, y, pre_act, n_rows, in_feat, out_feat, n_expert, dtype, activation};
    return dispatch_linear_forward(a, (cudaStream_t)stream);
}

extern "C" int fmoe_linear_backward(const void* grad_y, const void* x, const void* weight,
                                    const int64_t* seg_offsets, const void* act_pre, void* grad_x,
                                    void* grad_w, void* grad_b, int64_t n_rows, int64_t in_feat,
                                    int64_t out_feat, int32_t n_expert, int32_t dtype,
                                    int32_t activation, int32_t accumulate, void* scratch,
                                    fmoe_stream_t stream) {
    if (int rc = check_common(n_rows, in_feat, out_feat, n_expert, dtype, activation, seg_offsets)) return rc;
    FMOE_REQUIRE(n_rows == 0 || (grad_y && weight), "linear_backward: null pointer");
    FMOE_REQUIRE(!grad_w || x || n_rows == 0, "linear_backward: weight gradient needs the forward input");
    LinearBwdArgs a{grad_y, x, weight, seg_offsets, act_pre, grad_x, grad_w, grad_b, n_rows, in_feat,
                    out_feat, n_expert, dtype, activation, accumulate, scratch};
    return dispatch_linear_backward(a, (cudaStream_t)stream);
}

extern "C" int fmoe_linear_backward_colsum(const void* grad_y, const void* x, const void* weight,
                                           const int64_t* seg_offsets, const void* act_pre, void* grad_x,
                                           void* grad_w, void* grad_b, void* grad_x_colsum, int64_t n_rows,
                                           int64_t in_feat, int64_t out_feat, int32_t n_expert, int32_t dtype,
                                           int32_t activation, int32_t accumulate, void* scratch,
                                           fmoe_stream_t stream) {
    if (int rc = check_common(n_rows, in_feat, out_feat, n_expert, dtype, activation, seg_offsets)) return rc;
    FMOE_REQUIRE(n_rows == 0 || (grad_y && weight), "linear_backward: null pointer");
    FMOE_REQUIRE(!grad_w || x || n_rows == 0, "linear_backward: weight gradient needs the forward input");
    LinearBwdArgs a{grad_y, x, weight, seg_offsets, act_pre, grad_x, grad_w, grad_b, n_rows, in_feat,
                    out_feat, n_expert, dtype, activation, accumulate, scratch};
    a.grad_x_colsum = grad_x_colsum;
    return dispatch_linear_backward(a, (cudaStream_t)stream);
}


// ---- the same products on rows that an exchange is still delivering, or that one forwards at once --
namespace {
struct FinishCtx { const fmoe_arrival_t* arrival; fmoe_stream_t stream; };
// Closes an exchange whose rows a product has waited for tile by tile (and, for the handle of a scatter
// fused into that product, has also delivered: the handle is marked so before it is closed).
int finish_consumed(const fmoe_arrival_t* arrival, fmoe_stream_t stream) {
    fmoe_arrival_t h = *arrival;
    if (h.gather == 3) h.use = 1;
    return fmoe_peer_arrival_finish(&h, stream);
}
int finish_arrival(void* ctx) {
    FinishCtx* f = (FinishCtx*)ctx;
    return finish_consumed(f->arrival, f->stream);
}
int gemm_arrival_of(const fmoe_arrival_t* arrival, GemmArrival* g, bool* pending) {
    ArrivalWait w;
    *pending = false;
    if (!arrival || (arrival->gather != 0 && arrival->gather != 3)) return 0;
    if (int rc = arrival_wait_of(arrival, &w)) return rc;
    *pending = w.flags != nullptr;
    g->flags = w.flags; g->seq = w.seq; g->src_off = w.src_off; g->world = w.world; g->reserve_sms = w.reserve_sms;
    return 0;
}
int gemm_done_of(const fmoe_arrival_t* departure, GemmDone* g, bool* pending) {
    *pending = false;
    if (int rc = done_words_of(departure, &g->done, &g->expected, &g->ready, &g->reserve_sms)) return rc;
    *pending = g->done != nullptr;
    return 0;
}
}  // namespace

extern "C" int fmoe_linear_forward_overlapped(const void* x, const void* weight, const void* bias,
                                              const int64_t* seg_offsets, void* y, void* pre_act, int64_t n_rows,
                                              int64_t in_feat, int64_t out_feat, int32_t n_expert, int32_t dtype,
                                              int32_t activation, const fmoe_arrival_t* arrival,
                                              const fmoe_arrival_t* departure, fmoe_stream_t stream) {
    if (int rc = check_common(n_rows, in_feat, out_feat, n_expert, dtype, activation, seg_offsets)) return rc;
    GemmArrival ga;
    GemmDone gd;
    bool arriving = false, leaving = false;
    if (int rc = gemm_arrival_of(arrival, &ga, &arriving)) return rc;
    if (int rc = gemm_done_of(departure, &gd, &leaving)) return rc;
    GemmRemoteOut ro;
    if (int rc = remote_out_of(departure, &ro)) return rc;
    if (n_rows > 0) FMOE_REQUIRE(x && weight && (y || ro.enabled), "linear_forward: null pointer");
    LinearArgs a{x, weight, bias, seg_offsets, y, pre_act, n_rows, in_feat, out_feat, n_expert, dtype, activation};
    // only the tensor-core kernel can start on rows that are still arriving / report finished experts
    const bool tc = n_rows > 0 && !force_simt() && tc_forward_supported(a);
    FMOE_REQUIRE(!(leaving || ro.enabled) || (tc && n_expert == departure->n_expert),
                 "linear_forward: an overlapped gather was started for a product the tensor-core kernels do not take");
    if (ro.enabled) a.remote = &ro;
    const bool overlap = arriving && tc && n_expert == arrival->n_expert;
    if (arriving && !overlap) {
        if (int rc = fmoe_peer_arrival_finish(arrival, stream)) return rc;
    }
    if (overlap) a.arrival = &ga;
    GemmRemoteOut pin;
    GemmPushIn ps;
    if (overlap && arrival->gather == 3) {       // the product delivers its own input rows
        FMOE_REQUIRE(!ro.enabled, "linear_forward: a product cannot both deliver its input and send away its output");
        if (int rc = push_in_of(arrival, &pin, &ps)) return rc;
        a.remote = &pin;
        a.push = &ps;
    }
    if (leaving) a.done = &gd;
    if (n_rows > 0) {
        if (int rc = dispatch_linear_forward(a, (cudaStream_t)stream)) return rc;
    }
    return overlap ? finish_consumed(arrival, stream) : 0;
}

extern "C" int fmoe_linear_backward_overlapped(const void* grad_y, const void* x, const void* weight,
                                               const int64_t* seg_offsets, const void* act_pre, void* grad_x,
                                               void* grad_w, void* grad_b, void* grad_x_colsum, int64_t n_rows,
                                               int64_t in_feat, int64_t out_feat, int32_t n_expert, int32_t dtype,
                                               int32_t activation, int32_t accumulate, void* scratch,
                                               const fmoe_arrival_t* arrival, const fmoe_arrival_t* departure,
                                               fmoe_stream_t stream) {
    if (int rc = check_common(n_rows, in_feat, out_feat, n_expert, dtype, activation, seg_offsets)) return rc;
    FMOE_REQUIRE(n_rows == 0 || (grad_y && weight), "linear_backward: null pointer");
    FMOE_REQUIRE(!grad_w || x || n_rows == 0, "linear_backward: weight gradient needs the forward input");
    GemmArrival ga;
    GemmDone gd;
    bool arriving = false, leaving = false;
    if (int rc = gemm_arrival_of(arrival, &ga, &arriving)) return rc;
    if (int rc = gemm_done_of(departure, &gd, &leaving)) return rc;
    GemmRemoteOut ro;
    if (int rc = remote_out_of(departure, &ro)) return rc;
    LinearBwdArgs a{grad_y, x, weight, seg_offsets, act_pre, grad_x, grad_w, grad_b, n_rows, in_feat,
                    out_feat, n_expert, dtype, activation, accumulate, scratch};
    a.grad_x_colsum = grad_x_colsum;
    const bool tc = n_rows > 0 && !force_simt() && tc_backward_supported(a);
    FMOE_REQUIRE(!(leaving || ro.enabled) || (tc && (grad_x || ro.enabled) && n_expert == departure->n_expert),
                 "linear_backward: an overlapped gather was started for a product the tensor-core kernels do not take");
    if (ro.enabled) a.remote = &ro;
    // (a scatter fused into the product needs the input-gradient product to run: that one delivers the rows)
    const bool overlap = arriving && tc && n_expert == arrival->n_expert && (arrival->gather != 3 || (grad_x && n_rows > 0));
    if (arriving && !overlap) {
        if (int rc = fmoe_peer_arrival_finish(arrival, stream)) return rc;
    }
    FinishCtx ctx{arrival, stream};
    if (overlap) { a.arrival = &ga; a.after_input_grad = finish_arrival; a.after_ctx = &ctx; }
    GemmRemoteOut pin;
    GemmPushIn ps;
    if (overlap && arrival->gather == 3) {
        FMOE_REQUIRE(!ro.enabled, "linear_backward: a product cannot both deliver its input and send away its output");
        if (int rc = push_in_of(arrival, &pin, &ps)) return rc;
        a.remote = &pin;
        a.push = &ps;
    }
    if (leaving) a.done = &gd;
    return dispatch_linear_backward(a, (cudaStream_t)stream);
}
