// Grouped expert GEMM on the FFMA pipe (fp32 accumulate, fixed summation order).
//
// This is the path for fp32 tensors, whose parity bound (rtol 1e-5 against an
// fp32 reference) rules out TF32 tensor-core math, and for bf16/fp16 shapes the
// tcgen05 kernels do not take (feature sizes that are not multiples of their
// tiles).  It computes the three products of the reference's fmoe_linear
// (cuda/parallel_linear.cuh:55-161) for all experts in one launch each, reading
// the segment boundaries from device memory.
#include "common.cuh"
#include "gemm.h"

namespace fmoe {
namespace {

constexpr int BM = 64, BN = 64, BK = 16, TH = 256;

// Loads a BMxBK (rows x contraction) tile into sm[k][r] from a strided source.
// rows_valid / k_valid bound the tile; elements outside are zero.
template <typename T>
__device__ __forceinline__ void load_tile(const T* __restrict__ src, int64_t s_row, int64_t s_k,
                                          int rows_valid, int k_valid, float (*sm)[BM + 1]) {
    const int t = threadIdx.x;
    if (s_k == 1) {  // contraction index contiguous
        const int k = t % BK;
#pragma unroll
        for (int i = 0; i < (BM * BK) / TH; ++i) {
            const int r = t / BK + i * (TH / BK);
            float v = 0.f;
            if (r < rows_valid && k < k_valid) v = to_float<T>(src[(int64_t)r * s_row + k]);
            sm[k][r] = v;
        }
    } else {  // row index contiguous (or generic)
        const int r = t % BM;
#pragma unroll
        for (int i = 0; i < (BM * BK) / TH; ++i) {
            const int k = t / BM + i * (TH / BM);
            float v = 0.f;
            if (r < rows_valid && k < k_valid) v = to_float<T>(src[(int64_t)r * s_row + (int64_t)k * s_k]);
            sm[k][r] = v;
        }
    }
}

struct TileMap {
    int expert;
    int64_t row0;  // first row of the tile (absolute)
    int rows;      // valid rows in the tile
};

// Maps a linear m-tile index to (expert, rows) by walking the segment table (ranges are clamped
// to the buffer's n_rows rows and to run forwards, see safe_seg_range).
__device__ __forceinline__ bool find_tile(const int64_t* __restrict__ off, const HostSegs& hs, int n_expert,
                                          int64_t n_rows, int64_t tile, TileMap& tm) {
    int64_t acc = 0, prev_hi = 0;
    for (int e = 0; e < n_expert; ++e) {
        int64_t lo = hs.n ? (int64_t)hs.lo[e] : off[e], hi = hs.n ? (int64_t)hs.hi[e] : off[e + 1];
        lo = min(max(lo, prev_hi), n_rows);
        hi = min(max(hi, lo), n_rows);
        prev_hi = hi;
        const int64_t cnt = hi - lo;
        const int64_t nt = (cnt + BM - 1) / BM;
        if (tile < acc + nt) {
            const int64_t r0 = lo + (tile - acc) * BM;
            tm.expert = e;
            tm.row0 = r0;
            tm.rows = (int)min((int64_t)BM, lo + cnt - r0);
            return true;
        }
        acc += nt;
    }
    return false;
}

// MODE 0: Y[m,n]  = sum_k X[m,k] W[e][n,k] (+bias, activation)      rows ragged
// MODE 1: dX[m,k] = sum_n dY[m,n] W[e][n,k] (* saved activation derivative)  rows ragged
template <typename T, int MODE>
__global__ void __launch_bounds__(TH)
rows_gemm_kernel(const T* __restrict__ a, const T* __restrict__ w, const T* __restrict__ bias,
                 const int64_t* __restrict__ off, const __grid_constant__ HostSegs hs, T* __restrict__ c,
                 T* __restrict__ pre_out, const T* __restrict__ act_pre, int n_expert, int64_t n_rows, int64_t in_feat,
                 int64_t out_feat, int act) {
    __shared__ float As[BK][BM + 1];
    __shared__ float Bs[BK][BN + 1];
    TileMap tm;
    if (!find_tile(off, hs, n_expert, n_rows, blockIdx.x, tm)) return;
    const int64_t kdim = MODE == 0 ? in_feat : out_feat;  // contraction length
    const int64_t ndim = MODE == 0 ? out_feat : in_feat;  // output columns
    const int64_t n0 = (int64_t)blockIdx.y * BN;
    const int n_valid = (int)min((int64_t)BN, ndim - n0);
    const T* ap = a + tm.row0 * kdim;
    const T* wp = w + (int64_t)tm.expert * in_feat * out_feat;
    // B(kk, nn): MODE 0 -> W[n0+nn, kk] (stride_n = in_feat, stride_k = 1)
    //            MODE 1 -> W[kk, n0+nn] (stride_n = 1, stride_k = in_feat)
    const int64_t b_sn = MODE == 0 ? in_feat : 1, b_sk = MODE == 0 ? 1 : in_feat;
    const T* bp = wp + n0 * b_sn;
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
    float acc[4][4] = {};
    for (int64_t k0 = 0; k0 < kdim; k0 += BK) {
        const int kv = (int)min((int64_t)BK, kdim - k0);
        load_tile<T>(ap + k0, kdim, 1, tm.rows, kv, As);
        load_tile<T>(bp + k0 * b_sk, b_sn, b_sk, n_valid, kv, Bs);
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float av[4], bv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) av[i] = As[k][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) bv[j] = Bs[k][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = ty * 4 + i;
        if (r >= tm.rows) continue;
        const int64_t row = tm.row0 + r;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int cidx = tx * 4 + j;
            if (cidx >= n_valid) continue;
            const int64_t col = n0 + cidx;
            float v = acc[i][j];
            if (MODE == 0) {
                if (bias) v += to_float<T>(bias[(int64_t)tm.expert * out_feat + col]);
                if (pre_out && act == FMOE_ACT_GELU) pre_out[row * ndim + col] = from_float<T>(act_grad(v, act));
                v = apply_act(v, act);
            } else if (act_pre) {
                v *= saved_act_grad(to_float<T>(act_pre[row * ndim + col]), act);
            }
            c[row * ndim + col] = from_float<T>(v);
        }
    }
}

// dW[e][n,k] = sum_{m in seg e} dY[m,n] X[m,k]     grid (n tiles, k tiles, E)
template <typename T>
__global__ void __launch_bounds__(TH)
wgrad_kernel(const T* __restrict__ dy, const T* __restrict__ x, const int64_t* __restrict__ off,
             const __grid_constant__ HostSegs hs, T* __restrict__ dw, int64_t n_rows, int64_t in_feat, int64_t out_feat,
             int accumulate) {
    __shared__ float As[BK][BM + 1];
    __shared__ float Bs[BK][BN + 1];
    const int e = blockIdx.z;
    int64_t lo, hi;
    safe_seg_range(off, hs, e, n_rows, lo, hi);
    const int64_t n0 = (int64_t)blockIdx.x * BM, k0 = (int64_t)blockIdx.y * BN;
    const int nv = (int)min((int64_t)BM, out_feat - n0), kv = (int)min((int64_t)BN, in_feat - k0);
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
    float acc[4][4] = {};
    for (int64_t m0 = lo; m0 < hi; m0 += BK) {
        const int mv = (int)min((int64_t)BK, hi - m0);
        // A(row = n, contraction = m) = dY[m0+m, n0+n]: row stride 1, k stride out_feat
        load_tile<T>(dy + m0 * out_feat + n0, 1, out_feat, nv, mv, As);
        load_tile<T>(x + m0 * in_feat + k0, 1, in_feat, kv, mv, Bs);
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float av[4], bv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) av[i] = As[k][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) bv[j] = Bs[k][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
        __syncthreads();
    }
    T* out = dw + (int64_t)e * in_feat * out_feat;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = ty * 4 + i;
        if (r >= nv) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int cidx = tx * 4 + j;
            if (cidx >= kv) continue;
            const int64_t o = (n0 + r) * in_feat + k0 + cidx;
            float v = acc[i][j];
            if (accumulate) v += to_float<T>(out[o]);
            out[o] = from_float<T>(v);
        }
    }
}

// db[e][n] = sum_{m in seg e} dY[m,n].  Block: 32 columns x 8 row lanes.
template <typename T>
__global__ void __launch_bounds__(256)
bias_grad_kernel(const T* __restrict__ dy, const int64_t* __restrict__ off,
                 const __grid_constant__ HostSegs hs, T* __restrict__ db, int64_t n_rows, int64_t out_feat, int accumulate) {
    __shared__ float red[8][33];
    const int e = blockIdx.y;
    const int cx = threadIdx.x % 32, ry = threadIdx.x / 32;
    const int64_t col = (int64_t)blockIdx.x * 32 + cx;
    int64_t lo, hi;
    safe_seg_range(off, hs, e, n_rows, lo, hi);
    float s = 0.f;
    if (col < out_feat)
        for (int64_t m = lo + ry; m < hi; m += 8) s += to_float<T>(dy[m * out_feat + col]);
    red[ry][cx] = s;
    __syncthreads();
    if (ry == 0 && col < out_feat) {
        float t = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) t += red[i][cx];
        const int64_t o = (int64_t)e * out_feat + col;
        if (accumulate) t += to_float<T>(db[o]);
        db[o] = from_float<T>(t);
    }
}

const HostSegs kNoSegs = {};

template <typename T>
int forward_t(const LinearArgs& a, cudaStream_t st) {
    const HostSegs& hs = a.host_segs ? *a.host_segs : kNoSegs;
    const int64_t m_tiles = ceil_div(a.n_rows, BM) + a.n_expert;
    dim3 grid((unsigned)m_tiles, (unsigned)ceil_div(a.out_feat, BN));
    rows_gemm_kernel<T, 0><<<grid, TH, 0, st>>>((const T*)a.x, (const T*)a.weight, (const T*)a.bias,
                                                 a.seg_offsets, hs, (T*)a.y, (T*)a.pre_act, nullptr,
                                                 a.n_expert, a.n_rows, a.in_feat, a.out_feat, a.activation);
    FMOE_CHECK_LAUNCH();
    return 0;
}

template <typename T>
int backward_t(const LinearBwdArgs& a, cudaStream_t st) {
    const HostSegs& hs = a.host_segs ? *a.host_segs : kNoSegs;
    if (a.grad_x && a.n_rows > 0) {
        const int64_t m_tiles = ceil_div(a.n_rows, BM) + a.n_expert;
        dim3 grid((unsigned)m_tiles, (unsigned)ceil_div(a.in_feat, BN));
        rows_gemm_kernel<T, 1><<<grid, TH, 0, st>>>((const T*)a.grad_y, (const T*)a.weight, nullptr,
                                                     a.seg_offsets, hs, (T*)a.grad_x, nullptr,
                                                     (const T*)a.act_pre, a.n_expert, a.n_rows, a.in_feat,
                                                     a.out_feat, a.activation);
        FMOE_CHECK_LAUNCH();
    }
    if (a.grad_w) {
        dim3 grid((unsigned)ceil_div(a.out_feat, BM), (unsigned)ceil_div(a.in_feat, BN), (unsigned)a.n_expert);
        wgrad_kernel<T><<<grid, TH, 0, st>>>((const T*)a.grad_y, (const T*)a.x, a.seg_offsets, hs,
                                              (T*)a.grad_w, a.n_rows, a.in_feat, a.out_feat, a.accumulate);
        FMOE_CHECK_LAUNCH();
    }
    if (a.grad_b) {
        dim3 grid((unsigned)ceil_div(a.out_feat, 32), (unsigned)a.n_expert);
        bias_grad_kernel<T><<<grid, 256, 0, st>>>((const T*)a.grad_y, a.seg_offsets, hs, (T*)a.grad_b,
                                                   a.n_rows, a.out_feat, a.accumulate);
        FMOE_CHECK_LAUNCH();
    }
    return 0;
}

}  // namespace

int simt_linear_forward(const LinearArgs& a, cudaStream_t st) {
    if (a.n_rows == 0) return 0;
    switch (a.dtype) {
        case FMOE_F32: return forward_t<float>(a, st);
        case FMOE_F16: return forward_t<__half>(a, st);
        default: return forward_t<__nv_bfloat16>(a, st);
    }
}

int simt_linear_backward(const LinearBwdArgs& a, cudaStream_t st) {
    switch (a.dtype) {
        case FMOE_F32: return backward_t<float>(a, st);
        case FMOE_F16: return backward_t<__half>(a, st);
        default: return backward_t<__nv_bfloat16>(a, st);
    }
}

}  // namespace fmoe
