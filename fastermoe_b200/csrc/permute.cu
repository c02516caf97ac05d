// Token permutation kernels: local scatter / gather, k-way gather-sum, and the
// gate-score combine with its backward.  They replace torch.index_select,
// zeros+index_copy_/index_add_ and bmm of the reference's Python glue
// (fmoe/functions.py:72-84, fmoe/layers.py:319-322).
//
// All of them are HBM-bound row movers: one warp owns one output row (or one
// token), rows are moved with 16-byte loads/stores when the row size and the
// base pointers allow it, and every output row is written exactly once (rows
// that receive nothing are written as zeros by the same kernel, so no separate
// zero-fill pass is needed).
#include "common.cuh"

namespace fmoe {
namespace {

constexpr int kRowWarps = 8;
constexpr int kRowThreads = kRowWarps * 32;

// dst[r,:] = src[idx[r] / div,:]  or zeros when idx[r] is negative or out of range.
template <typename V>
__global__ void __launch_bounds__(kRowThreads)
rows_copy_kernel(const V* __restrict__ src, const int64_t* __restrict__ idx, V* __restrict__ dst,
                 int64_t n_dst_rows, int64_t n_src_rows, int64_t row_vecs, int div) {
    const int lane = threadIdx.x & 31;
    const int64_t r = (int64_t)blockIdx.x * kRowWarps + (threadIdx.x >> 5);
    if (r >= n_dst_rows) return;
    int64_t s = __ldg(idx + r);
    if (s >= 0 && div > 1) s /= div;
    V* d = dst + r * row_vecs;
    if (s < 0 || s >= n_src_rows) {
        V z;
        memset(&z, 0, sizeof(V));
        for (int64_t c = lane; c < row_vecs; c += 32) d[c] = z;
        return;
    }
    const V* p = src + s * row_vecs;
    int64_t c = lane;
    for (; c + 96 < row_vecs; c += 128) {
        const V v0 = __ldg(p + c), v1 = __ldg(p + c + 32), v2 = __ldg(p + c + 64), v3 = __ldg(p + c + 96);
        d[c] = v0; d[c + 32] = v1; d[c + 64] = v2; d[c + 96] = v3;
    }
    for (; c < row_vecs; c += 32) d[c] = __ldg(p + c);
}

__global__ void fill_i64_kernel(int64_t* __restrict__ p, int64_t n, int64_t v) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) p[i] = v;
}

__global__ void invert_pos_kernel(const int64_t* __restrict__ pos, int64_t n, int64_t n_out,
                                  int64_t* __restrict__ inv) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int64_t p = pos[i];
    if (p >= 0 && p < n_out) inv[p] = i;
}

template <typename V>
int launch_rows_copy(const void* src, const int64_t* idx, void* dst, int64_t n_dst_rows,
                     int64_t n_src_rows, int64_t row_bytes, int div, cudaStream_t st) {
    const unsigned blocks = (unsigned)ceil_div(n_dst_rows, kRowWarps);
    rows_copy_kernel<V><<<blocks, kRowThreads, 0, st>>>((const V*)src, idx, (V*)dst, n_dst_rows,
                                                         n_src_rows, row_bytes / (int64_t)sizeof(V), div);
    FMOE_CHECK_LAUNCH();
    return 0;
}

int rows_copy(const void* src, const int64_t* idx, void* dst, int64_t n_dst_rows, int64_t n_src_rows,
              int64_t row_bytes, int div, cudaStream_t st) {
    if (n_dst_rows == 0 || row_bytes == 0) return 0;
    const uintptr_t a = (uintptr_t)src | (uintptr_t)dst | (uintptr_t)row_bytes;
    if ((a & 15) == 0) return launch_rows_copy<uint4>(src, idx, dst, n_dst_rows, n_src_rows, row_bytes, div, st);
    if ((a & 7) == 0) return launch_rows_copy<uint2>(src, idx, dst, n_dst_rows, n_src_rows, row_bytes, div, st);
    if ((a & 3) == 0) return launch_rows_copy<uint32_t>(src, idx, dst, n_dst_rows, n_src_rows, row_bytes, div, st);
    if ((a & 1) == 0) return launch_rows_copy<uint16_t>(src, idx, dst, n_dst_rows, n_src_rows, row_bytes, div, st);
    return launch_rows_copy<uint8_t>(src, idx, dst, n_dst_rows, n_src_rows, row_bytes, div, st);
}

// ---- typed 16-byte packets -------------------------------------------------
template <typename T> struct Pack { static constexpr int N = 16 / sizeof(T); };

template <typename T>
__device__ __forceinline__ void unpack(const uint4& raw, float* f) {
    const T* p = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int i = 0; i < Pack<T>::N; ++i) f[i] = to_float<T>(p[i]);
}
template <typename T>
__device__ __forceinline__ uint4 pack(const float* f) {
    uint4 raw;
    T* p = reinterpret_cast<T*>(&raw);
#pragma unroll
    for (int i = 0; i < Pack<T>::N; ++i) p[i] = from_float<T>(f[i]);
    return raw;
}

// out[t,:] = sum_j w(t,j) * src_row(t*k+j); w = score or 1.  One warp per token.
// VEC: rows are moved as 16-byte packets (d a multiple of the packet width).
template <typename T, bool VEC, bool WEIGHTED>
__global__ void __launch_bounds__(kRowThreads)
gather_sum_kernel(const T* __restrict__ buf, const int64_t* __restrict__ inv, const T* __restrict__ score,
                  T* __restrict__ out, int64_t n_tokens, int top_k, int64_t d) {
    constexpr int N = Pack<T>::N;
    const int lane = threadIdx.x & 31;
    const int64_t t = (int64_t)blockIdx.x * kRowWarps + (threadIdx.x >> 5);
    if (t >= n_tokens) return;
    const int64_t step = VEC ? 32 * N : 32;
    for (int64_t c0 = (VEC ? lane * N : lane); c0 < d; c0 += step) {
        float acc[N];
#pragma unroll
        for (int i = 0; i < N; ++i) acc[i] = 0.f;
        for (int j = 0; j < top_k; ++j) {
            const int64_t r = t * top_k + j;
            const int64_t s = inv ? __ldg(inv + r) : r;
            if (s < 0) continue;
            const float w = WEIGHTED ? to_float<T>(score[r]) : 1.f;
            if (VEC) {
                float f[N];
                unpack<T>(__ldg(reinterpret_cast<const uint4*>(buf + s * d + c0)), f);
#pragma unroll
                for (int i = 0; i < N; ++i) acc[i] = WEIGHTED ? fmaf(w, f[i], acc[i]) : acc[i] + f[i];
            } else {
                const float f = to_float<T>(buf[s * d + c0]);
                acc[0] = WEIGHTED ? fmaf(w, f, acc[0]) : acc[0] + f;
            }
        }
        if (VEC) *reinterpret_cast<uint4*>(out + t * d + c0) = pack<T>(acc);
        else out[t * d + c0] = from_float<T>(acc[0]);
    }
}

// Same result for the common case (16-byte packets, top_k = K known at compile time):
// the K row indices and weights are read once, and each pass issues the loads of CH
// column chunks of all K source rows before it uses any of them, so that a warp keeps
// K*CH 16-byte loads per lane in flight instead of K.
template <typename T, int K, bool WEIGHTED>
__global__ void __launch_bounds__(kRowThreads)
gather_sum_fast_kernel(const T* __restrict__ buf, const int64_t* __restrict__ inv, const T* __restrict__ score,
                       T* __restrict__ out, int64_t n_tokens, int64_t d) {
    constexpr int N = Pack<T>::N, CH = 4;
    const int lane = threadIdx.x & 31;
    const int64_t t = (int64_t)blockIdx.x * kRowWarps + (threadIdx.x >> 5);
    if (t >= n_tokens) return;
    const T* rows[K];
    float w[K];
#pragma unroll
    for (int j = 0; j < K; ++j) {
        const int64_t r = t * K + j;
        const int64_t s = inv ? __ldg(inv + r) : r;
        rows[j] = s >= 0 ? buf + s * d : nullptr;
        w[j] = WEIGHTED ? to_float<T>(score[r]) : 1.f;
    }
    const int64_t step = 32 * N;
    for (int64_t c0 = lane * N; c0 < d; c0 += CH * step) {
        uint4 v[CH][K];
#pragma unroll
        for (int ch = 0; ch < CH; ++ch)
#pragma unroll
            for (int j = 0; j < K; ++j)
                v[ch][j] = (rows[j] && c0 + ch * step < d) ? __ldg(reinterpret_cast<const uint4*>(rows[j] + c0 + ch * step))
                                                           : make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int ch = 0; ch < CH; ++ch) {
            if (c0 + ch * step >= d) break;
            float acc[N];
#pragma unroll
            for (int i = 0; i < N; ++i) acc[i] = 0.f;
#pragma unroll
            for (int j = 0; j < K; ++j) {
                float f[N];
                unpack<T>(v[ch][j], f);
#pragma unroll
                for (int i = 0; i < N; ++i) acc[i] = WEIGHTED ? fmaf(w[j], f[i], acc[i]) : acc[i] + f[i];
            }
            *reinterpret_cast<uint4*>(out + t * d + c0 + ch * step) = pack<T>(acc);
        }
    }
}

// Backward of the combine, same case: grad_out's row is read once per pass for all K slots.
template <typename T, int K>
__global__ void __launch_bounds__(kRowThreads)
combine_bwd_fast_kernel(const T* __restrict__ grad_out, const T* __restrict__ buf, const int64_t* __restrict__ inv,
                        const T* __restrict__ score, T* __restrict__ grad_buf, T* __restrict__ grad_score,
                        int64_t n_tokens, int64_t d) {
    constexpr int N = Pack<T>::N, CH = 2;
    const int lane = threadIdx.x & 31;
    const int64_t t = (int64_t)blockIdx.x * kRowWarps + (threadIdx.x >> 5);
    if (t >= n_tokens) return;
    int64_t src[K];
    float w[K], dot[K];
#pragma unroll
    for (int j = 0; j < K; ++j) {
        const int64_t r = t * K + j;
        src[j] = inv ? __ldg(inv + r) : r;
        w[j] = to_float<T>(score[r]);
        dot[j] = 0.f;
    }
    const int64_t step = 32 * N;
    const T* grow = grad_out + t * d;
    for (int64_t c0 = lane * N; c0 < d; c0 += CH * step) {
        uint4 g[CH], x[CH][K];
#pragma unroll
        for (int ch = 0; ch < CH; ++ch) {
            const bool in = c0 + ch * step < d;
            g[ch] = in ? __ldg(reinterpret_cast<const uint4*>(grow + c0 + ch * step)) : make_uint4(0, 0, 0, 0);
#pragma unroll
            for (int j = 0; j < K; ++j)
                x[ch][j] = (in && grad_score && src[j] >= 0)
                               ? __ldg(reinterpret_cast<const uint4*>(buf + src[j] * d + c0 + ch * step))
                               : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int ch = 0; ch < CH; ++ch) {
            if (c0 + ch * step >= d) break;
            float gf[N];
            unpack<T>(g[ch], gf);
#pragma unroll
            for (int j = 0; j < K; ++j) {
                if (src[j] < 0) continue;
                float xf[N], o[N];
                unpack<T>(x[ch][j], xf);
#pragma unroll
                for (int i = 0; i < N; ++i) {
                    dot[j] = fmaf(gf[i], xf[i], dot[j]);
                    o[i] = w[j] * gf[i];
                }
                if (grad_buf) *reinterpret_cast<uint4*>(grad_buf + src[j] * d + c0 + ch * step) = pack<T>(o);
            }
        }
    }
    if (grad_score) {
#pragma unroll
        for (int j = 0; j < K; ++j) {
            float v = dot[j];
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
            if (lane == 0) grad_score[t * K + j] = from_float<T>(src[j] >= 0 ? v : 0.f);
        }
    }
}

// Backward of the combine.  One warp per token: reads grad_out[t,:] once, and for
// each of the k slots writes score*grad_out into the slot's buffer row and
// reduces dot(grad_out, src_row) into grad_score.
template <typename T, bool VEC>
__global__ void __launch_bounds__(kRowThreads)
combine_bwd_kernel(const T* __restrict__ grad_out, const T* __restrict__ buf, const int64_t* __restrict__ inv,
                   const T* __restrict__ score, T* __restrict__ grad_buf, T* __restrict__ grad_score,
                   int64_t n_tokens, int top_k, int64_t d) {
    constexpr int N = Pack<T>::N;
    const int lane = threadIdx.x & 31;
    const int64_t t = (int64_t)blockIdx.x * kRowWarps + (threadIdx.x >> 5);
    if (t >= n_tokens) return;
    const int64_t step = VEC ? 32 * N : 32;
    for (int j = 0; j < top_k; ++j) {
        const int64_t r = t * top_k + j;
        const int64_t s = inv ? __ldg(inv + r) : r;
        float dot = 0.f;
        if (s >= 0) {
            const float w = to_float<T>(score[r]);
            for (int64_t c0 = (VEC ? lane * N : lane); c0 < d; c0 += step) {
                if (VEC) {
                    float g[N], x[N], o[N];
                    unpack<T>(__ldg(reinterpret_cast<const uint4*>(grad_out + t * d + c0)), g);
                    if (grad_score) {
                        unpack<T>(__ldg(reinterpret_cast<const uint4*>(buf + s * d + c0)), x);
#pragma unroll
                        for (int i = 0; i < N; ++i) dot = fmaf(g[i], x[i], dot);
                    }
#pragma unroll
                    for (int i = 0; i < N; ++i) o[i] = w * g[i];
                    if (grad_buf) *reinterpret_cast<uint4*>(grad_buf + s * d + c0) = pack<T>(o);
                } else {
                    const float g = to_float<T>(grad_out[t * d + c0]);
                    if (grad_score) dot = fmaf(g, to_float<T>(buf[s * d + c0]), dot);
                    if (grad_buf) grad_buf[s * d + c0] = from_float<T>(w * g);
                }
            }
        }
        if (grad_score) {
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, off);
            if (lane == 0) grad_score[r] = from_float<T>(dot);
        }
    }
}

template <typename T>
bool vec_ok(int64_t d, std::initializer_list<const void*> ptrs) {
    if (d % Pack<T>::N) return false;
    for (const void* p : ptrs)
        if (p && ((uintptr_t)p & 15)) return false;
    return true;
}

template <typename T>
int gather_sum_t(const void* buf, const int64_t* inv, const void* score, void* out, int64_t n_tokens,
                 int top_k, int64_t d, cudaStream_t st) {
    const unsigned blocks = (unsigned)ceil_div(n_tokens, kRowWarps);
    const bool v = vec_ok<T>(d, {buf, out});
    const T *b = (const T*)buf, *s = (const T*)score;
    T* o = (T*)out;
    if (v && (top_k == 1 || top_k == 2 || top_k == 4)) {
#define FMOE_GS(K_)                                                                                                 \
        if (score) gather_sum_fast_kernel<T, K_, true><<<blocks, kRowThreads, 0, st>>>(b, inv, s, o, n_tokens, d);   \
        else gather_sum_fast_kernel<T, K_, false><<<blocks, kRowThreads, 0, st>>>(b, inv, s, o, n_tokens, d)
        if (top_k == 1) { FMOE_GS(1); } else if (top_k == 2) { FMOE_GS(2); } else { FMOE_GS(4); }
#undef FMOE_GS
        FMOE_CHECK_LAUNCH();
        return 0;
    }
    if (score) {
        if (v) gather_sum_kernel<T, true, true><<<blocks, kRowThreads, 0, st>>>(b, inv, s, o, n_tokens, top_k, d);
        else gather_sum_kernel<T, false, true><<<blocks, kRowThreads, 0, st>>>(b, inv, s, o, n_tokens, top_k, d);
    } else {
        if (v) gather_sum_kernel<T, true, false><<<blocks, kRowThreads, 0, st>>>(b, inv, s, o, n_tokens, top_k, d);
        else gather_sum_kernel<T, false, false><<<blocks, kRowThreads, 0, st>>>(b, inv, s, o, n_tokens, top_k, d);
    }
    FMOE_CHECK_LAUNCH();
    return 0;
}

template <typename T>
int combine_bwd_t(const void* grad_out, const void* buf, const int64_t* inv, const void* score,
                  void* grad_buf, void* grad_score, int64_t n_tokens, int top_k, int64_t d,
                  cudaStream_t st) {
    const unsigned blocks = (unsigned)ceil_div(n_tokens, kRowWarps);
    const bool v = vec_ok<T>(d, {grad_out, buf, grad_buf});
    if (v && (top_k == 1 || top_k == 2 || top_k == 4)) {
#define FMOE_CB(K_)                                                                                           \
        combine_bwd_fast_kernel<T, K_><<<blocks, kRowThreads, 0, st>>>((const T*)grad_out, (const T*)buf, inv,  \
            (const T*)score, (T*)grad_buf, (T*)grad_score, n_tokens, d)
        if (top_k == 1) { FMOE_CB(1); } else if (top_k == 2) { FMOE_CB(2); } else { FMOE_CB(4); }
#undef FMOE_CB
        FMOE_CHECK_LAUNCH();
        return 0;
    }
    if (v)
        combine_bwd_kernel<T, true><<<blocks, kRowThreads, 0, st>>>((const T*)grad_out, (const T*)buf, inv,
            (const T*)score, (T*)grad_buf, (T*)grad_score, n_tokens, top_k, d);
    else
        combine_bwd_kernel<T, false><<<blocks, kRowThreads, 0, st>>>((const T*)grad_out, (const T*)buf, inv,
            (const T*)score, (T*)grad_buf, (T*)grad_score, n_tokens, top_k, d);
    FMOE_CHECK_LAUNCH();
    return 0;
}

// ---- index_add_ with a fixed summation order ---------------------------------
// out[pos[i],:] += buf[i,:] over all i, rows of out that nothing maps to are zero (the
// zeros + index_add_ of fmoe/functions.py:77-81).  torch's index_add_ uses floating-point
// atomics, so its rounding depends on arrival order; here the rows that collide on one output
// row are listed first (integer atomics: the SET per output row does not depend on timing) and
// then added in ascending i.
constexpr int kListLen = 8;   // source rows listed per output row; longer collision chains are found by scanning pos

__global__ void bucket_rows_kernel(const int64_t* __restrict__ pos, int64_t n, int64_t n_out, int* __restrict__ cnt,
                                   int* __restrict__ lists) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int64_t p = pos[i];
    if (p < 0 || p >= n_out) return;
    const int slot = atomicAdd(cnt + p, 1);
    if (slot < kListLen) lists[p * kListLen + slot] = (int)i;
}

template <typename T, bool VEC>
__global__ void __launch_bounds__(kRowThreads)
rows_add_kernel(const T* __restrict__ buf, const int64_t* __restrict__ pos, const int* __restrict__ cnt,
                const int* __restrict__ lists, T* __restrict__ out, int64_t n, int64_t n_out, int64_t d) {
    constexpr int N = VEC ? Pack<T>::N : 1;
    const int lane = threadIdx.x & 31;
    const int64_t t = (int64_t)blockIdx.x * kRowWarps + (threadIdx.x >> 5);
    if (t >= n_out) return;
    const int c = cnt[t];
    // the listed source rows, sorted ascending: lane j holds the j-th smallest
    int mine = 0x7fffffff;
    if (c <= kListLen) {
        const int v = lane < c ? lists[t * kListLen + lane] : 0x7fffffff;
        int rank = 0;
        for (int j = 0; j < kListLen; ++j) {
            const int o = __shfl_sync(0xffffffffu, v, j);
            rank += (o < v) ? 1 : 0;
        }
        for (int j = 0; j < kListLen; ++j) {
            const int o = __shfl_sync(0xffffffffu, v, j), r = __shfl_sync(0xffffffffu, rank, j);
            if (r == lane && j < c) mine = o;
        }
    }
    for (int64_t cb = 0; cb < d; cb += 32 * N) {      // the same trip count on every lane: the body shuffles
        const int64_t c0 = cb + (int64_t)lane * N;
        const bool live = c0 < d;
        float acc[N];
#pragma unroll
        for (int i = 0; i < N; ++i) acc[i] = 0.f;
        auto add_row = [&](int64_t s) {
            if (!live) return;
            if (VEC) {
                float f[N];
                unpack<T>(__ldg(reinterpret_cast<const uint4*>(buf + s * d + c0)), f);
#pragma unroll
                for (int i = 0; i < N; ++i) acc[i] += f[i];
            } else {
                acc[0] += to_float<T>(buf[s * d + c0]);
            }
        };
        if (c <= kListLen) {
            for (int j = 0; j < c; ++j) add_row(__shfl_sync(0xffffffffu, mine, j));
        } else {
            for (int64_t base = 0; base < n; base += 32) {
                const bool hit = base + lane < n && pos[base + lane] == t;
                unsigned m = __ballot_sync(0xffffffffu, hit);
                while (m) {
                    const int b = __ffs(m) - 1;
                    m &= m - 1;
                    add_row(base + b);
                }
            }
        }
        if (!live) continue;
        if (VEC) *reinterpret_cast<uint4*>(out + t * d + c0) = pack<T>(acc);
        else out[t * d + c0] = from_float<T>(acc[0]);
    }
}

template <typename T>
int rows_add_t(const void* buf, const int64_t* pos, void* out, int64_t n, int64_t n_out, int64_t d, int* cnt,
               int* lists, cudaStream_t st) {
    const unsigned blocks = (unsigned)ceil_div(n_out, kRowWarps);
    if (vec_ok<T>(d, {buf, out}))
        rows_add_kernel<T, true><<<blocks, kRowThreads, 0, st>>>((const T*)buf, pos, cnt, lists, (T*)out, n, n_out, d);
    else
        rows_add_kernel<T, false><<<blocks, kRowThreads, 0, st>>>((const T*)buf, pos, cnt, lists, (T*)out, n, n_out, d);
    FMOE_CHECK_LAUNCH();
    return 0;
}

int check_typed(int64_t n_tokens, int top_k, int64_t d, int dtype) {
    FMOE_REQUIRE(n_tokens >= 0 && top_k > 0 && d > 0, "bad sizes: tokens=%lld top_k=%d d=%lld",
                 (long long)n_tokens, top_k, (long long)d);
    FMOE_REQUIRE(dtype_size(dtype) != 0, "unknown dtype %d", dtype);
    return 0;
}

}  // namespace
}  // namespace fmoe

using namespace fmoe;

extern "C" int fmoe_local_scatter(const void* inp, const int64_t* pos, void* out, int64_t n_rows,
                                  int64_t n_inp_rows, int64_t row_bytes, int32_t pos_div,
                                  fmoe_stream_t stream) {
    FMOE_REQUIRE(n_rows >= 0 && n_inp_rows >= 0 && row_bytes >= 0 && pos_div >= 1,
                 "local_scatter: bad sizes rows=%lld inp_rows=%lld row_bytes=%lld div=%d",
                 (long long)n_rows, (long long)n_inp_rows, (long long)row_bytes, pos_div);
    if (n_rows == 0) return 0;
    FMOE_REQUIRE(pos && out && (inp || n_inp_rows == 0), "local_scatter: null pointer");
    return rows_copy(inp, pos, out, n_rows, n_inp_rows, row_bytes, pos_div, (cudaStream_t)stream);
}

extern "C" int fmoe_local_gather_inv(const void* buf, const int64_t* inv, void* out, int64_t n_out_rows,
                                     int64_t row_bytes, fmoe_stream_t stream) {
    FMOE_REQUIRE(n_out_rows >= 0 && row_bytes >= 0, "local_gather: bad sizes");
    if (n_out_rows == 0) return 0;
    FMOE_REQUIRE(inv && out, "local_gather: null pointer");
    // Source rows are bounded by the number of output rows (inv is a partial permutation).
    return rows_copy(buf, inv, out, n_out_rows, n_out_rows, row_bytes, 1, (cudaStream_t)stream);
}

extern "C" int fmoe_local_gather(const void* buf, const int64_t* pos, void* out, int64_t n_rows,
                                 int64_t n_out_rows, int64_t row_bytes, int64_t* inv_scratch,
                                 fmoe_stream_t stream) {
    FMOE_REQUIRE(n_rows >= 0 && n_out_rows >= 0 && row_bytes >= 0, "local_gather: bad sizes");
    if (n_out_rows == 0) return 0;
    FMOE_REQUIRE(out && inv_scratch && (n_rows == 0 || (pos && buf)), "local_gather: null pointer");
    cudaStream_t st = (cudaStream_t)stream;
    fill_i64_kernel<<<(unsigned)ceil_div(n_out_rows, 256), 256, 0, st>>>(inv_scratch, n_out_rows, -1);
    FMOE_CHECK_LAUNCH();
    if (n_rows > 0) {
        invert_pos_kernel<<<(unsigned)ceil_div(n_rows, 256), 256, 0, st>>>(pos, n_rows, n_out_rows, inv_scratch);
        FMOE_CHECK_LAUNCH();
    }
    return rows_copy(buf, inv_scratch, out, n_out_rows, n_rows, row_bytes, 1, st);
}

extern "C" size_t fmoe_local_gather_add_scratch_bytes(int64_t n_out_rows) {
    return (size_t)(n_out_rows > 0 ? n_out_rows : 0) * (1 + kListLen) * sizeof(int) + 16;
}

extern "C" int fmoe_local_gather_add(const void* buf, const int64_t* pos, void* out, int64_t n_rows,
                                     int64_t n_out_rows, int64_t d, int32_t dtype, void* scratch,
                                     fmoe_stream_t stream) {
    if (int rc = check_typed(n_out_rows, 1, d, dtype)) return rc;
    FMOE_REQUIRE(n_rows >= 0 && n_rows < ((int64_t)1 << 31), "local_gather_add: n_rows=%lld", (long long)n_rows);
    if (n_out_rows == 0) return 0;
    FMOE_REQUIRE(out && scratch && (n_rows == 0 || (pos && buf)), "local_gather_add: null pointer");
    cudaStream_t st = (cudaStream_t)stream;
    int* cnt = (int*)scratch;
    int* lists = cnt + n_out_rows;
    FMOE_CUDA_TRY(cudaMemsetAsync(cnt, 0, (size_t)n_out_rows * sizeof(int), st));
    if (n_rows > 0) {
        bucket_rows_kernel<<<(unsigned)ceil_div(n_rows, 256), 256, 0, st>>>(pos, n_rows, n_out_rows, cnt, lists);
        FMOE_CHECK_LAUNCH();
    }
    switch (dtype) {
        case FMOE_F32: return rows_add_t<float>(buf, pos, out, n_rows, n_out_rows, d, cnt, lists, st);
        case FMOE_F16: return rows_add_t<__half>(buf, pos, out, n_rows, n_out_rows, d, cnt, lists, st);
        default: return rows_add_t<__nv_bfloat16>(buf, pos, out, n_rows, n_out_rows, d, cnt, lists, st);
    }
}

extern "C" int fmoe_local_gather_sum(const void* buf, const int64_t* inv, void* out, int64_t n_tokens,
                                     int32_t top_k, int64_t d, int32_t dtype, fmoe_stream_t stream) {
    if (int rc = check_typed(n_tokens, top_k, d, dtype)) return rc;
    if (n_tokens == 0) return 0;
    FMOE_REQUIRE(buf && out, "local_gather_sum: null pointer");
    cudaStream_t st = (cudaStream_t)stream;
    switch (dtype) {
        case FMOE_F32: return gather_sum_t<float>(buf, inv, nullptr, out, n_tokens, top_k, d, st);
        case FMOE_F16: return gather_sum_t<__half>(buf, inv, nullptr, out, n_tokens, top_k, d, st);
        default: return gather_sum_t<__nv_bfloat16>(buf, inv, nullptr, out, n_tokens, top_k, d, st);
    }
}

extern "C" int fmoe_combine_forward(const void* buf, const int64_t* inv, const void* score, void* out,
                                    int64_t n_tokens, int32_t top_k, int64_t d, int32_t dtype,
                                    fmoe_stream_t stream) {
    if (int rc = check_typed(n_tokens, top_k, d, dtype)) return rc;
    if (n_tokens == 0) return 0;
    FMOE_REQUIRE(buf && score && out, "combine_forward: null pointer");
    cudaStream_t st = (cudaStream_t)stream;
    switch (dtype) {
        case FMOE_F32: return gather_sum_t<float>(buf, inv, score, out, n_tokens, top_k, d, st);
        case FMOE_F16: return gather_sum_t<__half>(buf, inv, score, out, n_tokens, top_k, d, st);
        default: return gather_sum_t<__nv_bfloat16>(buf, inv, score, out, n_tokens, top_k, d, st);
    }
}

extern "C" int fmoe_combine_backward(const void* grad_out, const void* buf, const int64_t* inv,
                                     const void* score, void* grad_buf, void* grad_score,
                                     int64_t n_tokens, int32_t top_k, int64_t d, int32_t dtype,
                                     fmoe_stream_t stream) {
    if (int rc = check_typed(n_tokens, top_k, d, dtype)) return rc;
    if (n_tokens == 0) return 0;
    // grad_buf may be NULL (only the score gradient is wanted: the rows are produced elsewhere)
    FMOE_REQUIRE(grad_out && score && (grad_buf || grad_score), "combine_backward: null pointer");
    FMOE_REQUIRE(!grad_score || buf, "combine_backward: grad_score needs the forward buffer");
    cudaStream_t st = (cudaStream_t)stream;
    switch (dtype) {
        case FMOE_F32: return combine_bwd_t<float>(grad_out, buf, inv, score, grad_buf, grad_score, n_tokens, top_k, d, st);
        case FMOE_F16: return combine_bwd_t<__half>(grad_out, buf, inv, score, grad_buf, grad_score, n_tokens, top_k, d, st);
        default: return combine_bwd_t<__nv_bfloat16>(grad_out, buf, inv, score, grad_buf, grad_score, n_tokens, top_k, d, st);
    }
}
