// Smart schedule (placeholder; host planning lives here, kernels in gemm_*.cu).
#include "common.cuh"
#include "exchange.h"
using namespace fmoe;

extern "C" int fmoe_fused_compute_ptrs(const int64_t* lec, const int64_t* gec, const uint8_t* stored,
                                       int32_t rank, int32_t E, int32_t W, int64_t* local_ptr,
                                       int64_t* global_ptr, int64_t* local_global_ptr) {
    FMOE_REQUIRE(lec && gec && stored && local_ptr && global_ptr && local_global_ptr,
                 "fused_compute_ptrs: null pointer");
    FMOE_REQUIRE(E > 0 && W > 0 && rank >= 0 && rank < W, "fused_compute_ptrs: bad sizes");
    local_ptr[0] = global_ptr[0] = local_global_ptr[0] = 0;
    for (int i = 0; i < E * W; ++i) {
        local_ptr[i + 1] = local_ptr[i] + lec[i];
        local_global_ptr[i + 1] = local_global_ptr[i] + (stored[i] ? lec[i] : 0);
        const int e = i % E, w = i / E;
        global_ptr[e * W + w + 1] = stored[rank * E + e] ? 0 : gec[i];
    }
    for (int i = 0; i < E * W; ++i) global_ptr[i + 1] += global_ptr[i];
    return 0;
}

extern "C" size_t fmoe_fused_scratch_bytes(int64_t, int64_t, int64_t, int64_t, int32_t, int32_t, int32_t) {
    return 0;
}

extern "C" int fmoe_fused_forward(fmoe_comm_t, const void*, void*, void*, void*, void*,
                                  const fmoe_mlp_params_t*, const int64_t*, const int64_t*, const uint8_t*,
                                  int64_t, int64_t, int64_t, int64_t, int32_t, int32_t, int32_t, int32_t,
                                  int32_t, void*, fmoe_stream_t, fmoe_stream_t) {
    return fail(FMOE_ERR_UNSUPPORTED, "fused_forward: not built yet");
}

extern "C" int fmoe_fused_backward(fmoe_comm_t, const void*, void*, const void*, const void*, const void*,
                                   void*, void*, void*, const fmoe_mlp_params_t*, const int64_t*,
                                   const int64_t*, const uint8_t*, int64_t, int64_t, int64_t, int64_t,
                                   int32_t, int32_t, int32_t, int32_t, int32_t, void*, fmoe_stream_t,
                                   fmoe_stream_t) {
    return fail(FMOE_ERR_UNSUPPORTED, "fused_backward: not built yet");
}
