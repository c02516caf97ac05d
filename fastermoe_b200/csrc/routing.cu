// Routing kernels: expert histogram, stable bucketing of gate entries into
// expert segments, capacity limiting and capacity pruning.
//
// They replace the reference's atomic kernels (cuda/local_exchange.cuh:5-61,
// cuda/balancing.cuh:5-46) by a deterministic counting sort:
//   1. tile_hist:   every warp owns a contiguous tile of the flat gate array
//                   and builds the tile's histogram in its own shared-memory row
//                   (shared-memory atomics: integer sums, order does not matter);
//   2. scan_tiles:  per expert, exclusive prefix over tiles (in place, blocks of 256
//                   tiles in parallel; the block totals are scanned in step 3);
//   3. finalize:    per-expert totals -> segment starts / limits, and the
//                   in-place side effects the reference's operators have;
//   4. apply:       every warp walks its tile again in order, ranks entries by
//                   (expert, flat index) with __match_any_sync and writes positions
//                   or pruned gates.
// Gate entries are read with 16-byte loads; within an expert segment positions
// ascend with the flat index, so results are identical from run to run.
#include "common.cuh"
#include <algorithm>
#include <cooperative_groups.h>
#include <mutex>

namespace fmoe {
namespace {

constexpr int kWarps = 8;             // warps per block in the tile kernels
constexpr int kThreads = kWarps * 32;
constexpr unsigned kFull = 0xffffffffu;

enum Mode { MODE_COUNT_POS = 0, MODE_ASSIGN = 1, MODE_PRUNE = 2 };

struct Geom {
    int chunks;       // 64-entry chunks per warp tile
    int64_t n_tiles;  // number of warp tiles
    int64_t tile;     // entries per tile = chunks*64
};

Geom make_geom(int64_t n, int n_expert) {
    Geom g;
    int64_t chunks = 4;  // 256 entries per warp tile
    // Keep the per-tile histogram table under 64 MiB.
    const int64_t budget = (int64_t)64 << 20;
    while (ceil_div(n, chunks * 64) * n_expert * 4 > budget) chunks *= 2;
    g.chunks = (int)chunks;
    g.tile = chunks * 64;
    g.n_tiles = n > 0 ? ceil_div(n, g.tile) : 0;
    return g;
}

// Scratch layout (all offsets 16-byte aligned).
constexpr int kScanRows = 256;  // tiles scanned by one block of the scan kernel

struct Scratch {
    int32_t* totals;     // [E]
    int64_t* seg_start;  // [E]
    int32_t* limit;      // [E]
    int32_t* blocksum;   // [ceil(n_tiles / kScanRows)][E]: per scan block totals, then their exclusive prefix
    int32_t* hist;       // [n_tiles][E]: per tile counts, then exclusive prefix inside the scan block
};

size_t align16(size_t x) { return (x + 15) & ~(size_t)15; }

size_t scratch_bytes(int64_t n, int n_expert) {
    Geom g = make_geom(n, n_expert);
    return align16((size_t)n_expert * 4) + align16((size_t)n_expert * 8) + align16((size_t)n_expert * 4) +
           align16((size_t)ceil_div(g.n_tiles, kScanRows) * n_expert * 4) +
           align16((size_t)g.n_tiles * n_expert * 4) + 16;
}

Scratch carve(void* scratch, int64_t n, int n_expert) {
    Scratch s;
    char* p = (char*)scratch;
    s.totals = (int32_t*)p;
    p += align16((size_t)n_expert * 4);
    s.seg_start = (int64_t*)p;
    p += align16((size_t)n_expert * 8);
    s.limit = (int32_t*)p;
    p += align16((size_t)n_expert * 4);
    s.blocksum = (int32_t*)p;
    p += align16((size_t)ceil_div(make_geom(n, n_expert).n_tiles, kScanRows) * n_expert * 4);
    s.hist = (int32_t*)p;
    return s;
}

__device__ __forceinline__ int sanitize(int64_t v, int n_expert) {
    return (v >= 0 && v < (int64_t)n_expert) ? (int)v : -1;
}

// Loads the expert ids of the 64 entries [c, c+64) of the gate array so that
// lane l holds entry c+l in `ea` and entry c+32+l in `eb`.  With `vec` the
// loads are 16 bytes per lane (two consecutive int64) followed by a shuffle
// transpose; `c` is then a multiple of 2 entries from a 16-byte aligned base.
__device__ __forceinline__ void load_chunk(const int64_t* __restrict__ gate, int64_t n, int64_t c,
                                           int lane, bool vec, int n_expert, int& ea, int& eb) {
    if (vec && c + 64 <= n) {
        const longlong2 v = __ldg(reinterpret_cast<const longlong2*>(gate + c) + lane);
        const int h0 = sanitize(v.x, n_expert), h1 = sanitize(v.y, n_expert);
        const int src = lane >> 1;
        const int a0 = __shfl_sync(kFull, h0, src), a1 = __shfl_sync(kFull, h1, src);
        const int b0 = __shfl_sync(kFull, h0, 16 + src), b1 = __shfl_sync(kFull, h1, 16 + src);
        ea = (lane & 1) ? a1 : a0;
        eb = (lane & 1) ? b1 : b0;
    } else {
        const int64_t ia = c + lane, ib = c + 32 + lane;
        ea = ia < n ? sanitize(__ldg(gate + ia), n_expert) : -1;
        eb = ib < n ? sanitize(__ldg(gate + ib), n_expert) : -1;
    }
}

// The same 64 entries in whatever order the 16-byte loads deliver them (lane l: entries c+2l and c+2l+1):
// for passes that only count, the order of the entries inside a chunk does not matter, and the shuffle
// transpose of load_chunk can be left out.
__device__ __forceinline__ void load_chunk_unordered(const int64_t* __restrict__ gate, int64_t n, int64_t c,
                                                     int lane, bool vec, int n_expert, int& ea, int& eb) {
    if (vec && c + 64 <= n) {
        const longlong2 v = __ldg(reinterpret_cast<const longlong2*>(gate + c) + lane);
        ea = sanitize(v.x, n_expert);
        eb = sanitize(v.y, n_expert);
    } else {
        load_chunk(gate, n, c, lane, vec, n_expert, ea, eb);
    }
}

// Counts the 32 lanes' experts into the warp's own shared-memory row.  Native shared-memory atomics: lanes
// that name the same expert serialise on its counter (a handful per instruction on average), which costs
// far less issue time than ranking the lanes with __match_any_sync first; integer sums do not depend on
// the order, so the result is the same from run to run.  (The caller synchronises the warp before it
// reads the row.)
__device__ __forceinline__ void hist_round(int e, int /*lane*/, int32_t* my) {
    if (e >= 0) atomicAdd(my + e, 1);
}

__global__ void __launch_bounds__(kThreads)
tile_hist_kernel(const int64_t* __restrict__ gate, int64_t n, int n_expert, int chunks,
                 int64_t n_tiles, int32_t* __restrict__ hist, bool vec) {
    extern __shared__ int32_t sh[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int32_t* my = sh + (size_t)warp * n_expert;
    const int64_t tile = (int64_t)blockIdx.x * kWarps + warp;
    if (tile >= n_tiles) return;
    for (int e = lane; e < n_expert; e += 32) my[e] = 0;
    __syncwarp();
    const int64_t base = tile * (int64_t)chunks * 64;
    // four chunks (256 entries) are fetched before any is processed, so that each warp
    // keeps 2 KB of loads in flight
    for (int it = 0; it < chunks; it += 4) {
        int ea[4], eb[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int64_t c = base + (int64_t)(it + u) * 64;
            if (it + u < chunks && c < n) load_chunk_unordered(gate, n, c, lane, vec, n_expert, ea[u], eb[u]);
            else ea[u] = eb[u] = -1;
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            hist_round(ea[u], lane, my);
            hist_round(eb[u], lane, my);
        }
    }
    __syncwarp();
    int32_t* out = hist + tile * n_expert;
    for (int e = lane; e < n_expert; e += 32) out[e] = my[e];
}

// Block b scans the rows [b*kScanRows, +kScanRows) of hist[tile][e] column by column:
// each entry becomes the exclusive prefix inside the block, and blocksum[b][e] the
// block's column total.  Consecutive threads take consecutive experts of a row, so
// reads and writes are contiguous.
__global__ void __launch_bounds__(256)
scan_tiles_kernel(int32_t* __restrict__ hist, int64_t n_tiles, int n_expert, int32_t* __restrict__ blocksum) {
    __shared__ int32_t part[256];
    const int64_t row0 = (int64_t)blockIdx.x * kScanRows;
    const int rows = (int)min((int64_t)kScanRows, n_tiles - row0);
    int cw = 1;  // columns per pass: power of two, at most 256
    while (cw < n_expert && cw < 256) cw <<= 1;
    const int rl = 256 / cw;  // row lanes per column
    const int c = threadIdx.x % cw, lane_r = threadIdx.x / cw;
    const int per = (rows + rl - 1) / rl;  // rows per thread
    for (int e0 = 0; e0 < n_expert; e0 += cw) {
        const int e = e0 + c;
        const int lo = lane_r * per, hi = min(lo + per, rows);
        int32_t sum = 0;
        if (e < n_expert)
            for (int r = lo; r < hi; ++r) sum += hist[(row0 + r) * n_expert + e];
        part[threadIdx.x] = sum;
        __syncthreads();
        // exclusive prefix over the row lanes of this column (serial: at most 256 lanes)
        int32_t run = 0;
        for (int l = 0; l < lane_r; ++l) run += part[l * cw + c];
        if (e < n_expert) {
            if (lane_r == rl - 1) blocksum[(int64_t)blockIdx.x * n_expert + e] = run + sum;
            for (int r = lo; r < hi; ++r) {
                const int64_t idx = (row0 + r) * n_expert + e;
                const int32_t h = hist[idx];
                hist[idx] = run;
                run += h;
            }
        }
        __syncthreads();
    }
}

// Single block.  Turns totals into segment starts and applies the side effects
// of the operator being emulated.
__global__ void __launch_bounds__(1024)
finalize_kernel(int mode, int n_expert, int32_t* __restrict__ totals, int32_t* __restrict__ blocksum, int n_blocks,
                int64_t* __restrict__ seg_start, int32_t* __restrict__ limit,
                int64_t* __restrict__ lec64, int64_t* __restrict__ offsets,
                int32_t* __restrict__ inout /* cum_count or ec */) {
    __shared__ int64_t part[1024];
    const int t = threadIdx.x;
    // Block sums -> their exclusive prefix over scan blocks; column totals.
    for (int e = t; e < n_expert; e += 1024) {
        int32_t run = 0;
        for (int b = 0; b < n_blocks; ++b) {
            const int32_t v = blocksum[(int64_t)b * n_expert + e];
            blocksum[(int64_t)b * n_expert + e] = run;
            run += v;
        }
        totals[e] = run;
    }
    __syncthreads();
    if (mode == MODE_ASSIGN) {
        for (int e = t; e < n_expert; e += 1024) {
            const int32_t s = inout[e] - totals[e];
            seg_start[e] = s;
            inout[e] = s;
        }
        return;
    }
    if (mode == MODE_PRUNE) {
        for (int e = t; e < n_expert; e += 1024) {
            const int32_t l = inout[e];
            limit[e] = l;
            inout[e] = l - totals[e];
            seg_start[e] = 0;
        }
        return;
    }
    // MODE_COUNT_POS: exclusive prefix of totals over experts.
    const int per = (n_expert + 1023) / 1024;
    const int lo = t * per, hi = min(lo + per, n_expert);
    int64_t s = 0;
    for (int e = lo; e < hi; ++e) s += totals[e];
    part[t] = s;
    __syncthreads();
    for (int off = 1; off < 1024; off <<= 1) {
        int64_t v = t >= off ? part[t - off] : 0;
        __syncthreads();
        part[t] += v;
        __syncthreads();
    }
    int64_t run = part[t] - s;
    for (int e = lo; e < hi; ++e) {
        seg_start[e] = run;
        if (offsets) offsets[e] = run;
        if (lec64) lec64[e] = totals[e];
        run += totals[e];
    }
    if (t == 1023 && offsets) offsets[n_expert] = part[1023];
}

// Rank of this lane's entry among the lanes with the same expert, then advance
// the warp's running counters.  Returns the rank within the expert's bucket
// counted from the start of the whole array (or from seg_start).
__device__ __forceinline__ int64_t rank_round(int e, int lane, int32_t* run) {
    const unsigned m = __match_any_sync(kFull, e);
    int64_t r = -1;
    if (e >= 0) r = run[e] + __popc(m & ((1u << lane) - 1u));
    __syncwarp();
    if (e >= 0 && lane == __ffs(m) - 1) run[e] += __popc(m);
    __syncwarp();
    return r;
}

__global__ void __launch_bounds__(kThreads)
apply_kernel(int mode, const int64_t* __restrict__ gate, int64_t n, int n_expert, int chunks,
             int64_t n_tiles, const int32_t* __restrict__ base, const int32_t* __restrict__ blockbase,
             const int64_t* __restrict__ seg_start,
             const int32_t* __restrict__ limit, const int64_t* __restrict__ total_ptr,
             int64_t* __restrict__ pos, int64_t* __restrict__ inv, int64_t* __restrict__ new_gate,
             bool vec) {
    // Running position per expert and warp; positions fit 32 bits (n < 2^31 is checked on the host).
    extern __shared__ int32_t shr[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int32_t* run = shr + (size_t)warp * n_expert;
    const int64_t tile = (int64_t)blockIdx.x * kWarps + warp;
    if (tile >= n_tiles) return;
    const int32_t* b = base + tile * n_expert;
    const int32_t* bb = blockbase + (tile / kScanRows) * n_expert;
    for (int e = lane; e < n_expert; e += 32) run[e] = (int32_t)seg_start[e] + b[e] + bb[e];
    __syncwarp();
    const int64_t total = (mode == MODE_COUNT_POS && total_ptr) ? *total_ptr : n;
    const int64_t tb = tile * (int64_t)chunks * 64;
    for (int it0 = 0; it0 < chunks; it0 += 4) {
        int eas[4], ebs[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int64_t c = tb + (int64_t)(it0 + u) * 64;
            if (it0 + u < chunks && c < n) load_chunk(gate, n, c, lane, vec, n_expert, eas[u], ebs[u]);
            else eas[u] = ebs[u] = -1;
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int64_t c = tb + (int64_t)(it0 + u) * 64;
            if (it0 + u >= chunks || c >= n) break;
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int e = half ? ebs[u] : eas[u];
                const int64_t i = c + half * 32 + lane;
                const int64_t r = rank_round(e, lane, run);
                if (i < n) {
                    if (mode == MODE_PRUNE) {
                        new_gate[i] = (e >= 0 && r < (int64_t)limit[e]) ? (int64_t)e : (int64_t)-1;
                    } else {
                        if (e >= 0) pos[r] = i;
                        if (inv) inv[i] = r;  // -1 for skipped entries
                        // Slots past the number of kept entries are never a target
                        // of the scatter above; mark them empty.
                        if (mode == MODE_COUNT_POS && i >= total) pos[i] = -1;
                    }
                }
            }
        }
    }
}

// ---- one launch for small inputs ----------------------------------------------------------------
// Up to kClMaxCtas * kClWarps warp tiles of at most kClMaxChunks chunks: the four passes above run as
// ONE thread-block cluster.  The per-tile histograms never leave shared memory: a CTA scans its
// warps' rows, the CTAs read each other's totals through distributed shared memory between two
// cluster barriers, every CTA derives the segment starts for itself, and each warp then ranks its
// tile (whose entries are still in L1) exactly as apply_kernel does.  Same results, one launch
// instead of four and no scratch traffic: at the size of one layer call (tens of thousands of gate
// entries) the operators were bound by launch latency.
constexpr int kClWarps = 16, kClThreads = kClWarps * 32, kClMaxCtas = 8, kClMaxChunks = 16, kClMaxExperts = 512;

__global__ void __launch_bounds__(kClThreads)
bucket_cluster_kernel(int mode, const int64_t* __restrict__ gate, int64_t n, int n_expert, int chunks,
                      int64_t* __restrict__ lec64, int64_t* __restrict__ offsets, int32_t* __restrict__ inout,
                      int64_t* __restrict__ pos, int64_t* __restrict__ inv, int64_t* __restrict__ new_gate, bool vec) {
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    extern __shared__ int32_t shc[];
    int32_t* hist = shc;                                   // [kClWarps][E]: counts, then prefix inside the CTA, then running positions
    int32_t* ctot = hist + (size_t)kClWarps * n_expert;    // [E] this CTA's totals (read by the other CTAs)
    int32_t* cbase = ctot + n_expert;                      // [E] totals of the CTAs before this one
    int32_t* total = cbase + n_expert;                     // [E]
    int32_t* seg = total + n_expert;                       // [E] segment starts
    int32_t* lim = seg + n_expert;                         // [E] the in/out vector as it was on entry
    __shared__ int64_t s_grand;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const unsigned rank = cluster.block_rank(), n_cta = cluster.num_blocks();
    int32_t* my = hist + (size_t)warp * n_expert;
    const int64_t tb = ((int64_t)rank * kClWarps + warp) * (int64_t)chunks * 64;
    for (int e = lane; e < n_expert; e += 32) my[e] = 0;
    __syncwarp();
    for (int it = 0; it < chunks && tb < n; it += 4) {
        int ea[4], eb[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int64_t c = tb + (int64_t)(it + u) * 64;
            if (it + u < chunks && c < n) load_chunk(gate, n, c, lane, vec, n_expert, ea[u], eb[u]);
            else ea[u] = eb[u] = -1;
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            hist_round(ea[u], lane, my);
            hist_round(eb[u], lane, my);
        }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < n_expert; e += kClThreads) {
        int32_t run = 0;
        for (int w = 0; w < kClWarps; ++w) {
            const int32_t h = hist[(size_t)w * n_expert + e];
            hist[(size_t)w * n_expert + e] = run;
            run += h;
        }
        ctot[e] = run;
    }
    cluster.sync();
    for (int e = threadIdx.x; e < n_expert; e += kClThreads) {
        int32_t tot = 0, before = 0;
        for (unsigned r = 0; r < n_cta; ++r) {
            const int32_t v = cluster.map_shared_rank(ctot, r)[e];
            if (r < rank) before += v;
            tot += v;
        }
        total[e] = tot;
        cbase[e] = before;
        lim[e] = mode == MODE_COUNT_POS ? 0 : inout[e];
    }
    cluster.sync();      // nobody reads another CTA's shared memory, or the in/out vector, after this
    if (mode == MODE_COUNT_POS) {
        if (warp == 0) {
            int64_t carry = 0;
            for (int e0 = 0; e0 < n_expert; e0 += 32) {
                const int32_t v = e0 + lane < n_expert ? total[e0 + lane] : 0;
                int32_t incl = v;
#pragma unroll
                for (int off = 1; off < 32; off <<= 1) {
                    const int32_t o = __shfl_up_sync(kFull, incl, off);
                    if (lane >= off) incl += o;
                }
                if (e0 + lane < n_expert) seg[e0 + lane] = (int32_t)carry + incl - v;
                carry += __shfl_sync(kFull, incl, 31);
            }
            if (lane == 0) s_grand = carry;
        }
    } else {
        for (int e = threadIdx.x; e < n_expert; e += kClThreads) seg[e] = mode == MODE_ASSIGN ? lim[e] - total[e] : 0;
        if (threadIdx.x == 0) s_grand = n;
    }
    __syncthreads();
    if (rank == 0) {
        for (int e = threadIdx.x; e < n_expert; e += kClThreads) {
            if (mode == MODE_COUNT_POS) {
                if (lec64) lec64[e] = total[e];
                if (offsets) offsets[e] = seg[e];
            } else if (mode == MODE_ASSIGN) {
                inout[e] = seg[e];
            } else {
                inout[e] = lim[e] - total[e];
            }
        }
        if (mode == MODE_COUNT_POS && offsets && threadIdx.x == 0) offsets[n_expert] = s_grand;
    }
    if (tb >= n) return;
    for (int e = lane; e < n_expert; e += 32) my[e] += seg[e] + cbase[e];
    __syncwarp();
    const int64_t grand = (mode == MODE_COUNT_POS && offsets) ? s_grand : n;
    for (int it0 = 0; it0 < chunks; it0 += 4) {
        int eas[4], ebs[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int64_t c = tb + (int64_t)(it0 + u) * 64;
            if (it0 + u < chunks && c < n) load_chunk(gate, n, c, lane, vec, n_expert, eas[u], ebs[u]);
            else eas[u] = ebs[u] = -1;
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int64_t c = tb + (int64_t)(it0 + u) * 64;
            if (it0 + u >= chunks || c >= n) break;
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int e = half ? ebs[u] : eas[u];
                const int64_t i = c + half * 32 + lane;
                const int64_t r = rank_round(e, lane, my);
                if (i < n) {
                    if (mode == MODE_PRUNE) {
                        new_gate[i] = (e >= 0 && r < (int64_t)lim[e]) ? (int64_t)e : (int64_t)-1;
                    } else {
                        if (e >= 0) pos[r] = i;
                        if (inv) inv[i] = r;
                        if (mode == MODE_COUNT_POS && i >= grand) pos[i] = -1;
                    }
                }
            }
        }
    }
}

// Plain histogram: every warp counts into its own shared-memory row (no atomics
// between warps), rows are summed at the end, and each block issues one global
// atomic per non-empty counter.
__global__ void __launch_bounds__(kThreads)
expert_count_kernel(const int64_t* __restrict__ gate, int64_t n, int n_expert,
                    int32_t* __restrict__ expert_count, bool vec) {
    extern __shared__ int32_t sh[];
    for (int i = threadIdx.x; i < kWarps * n_expert; i += kThreads) sh[i] = 0;
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int32_t* my = sh + (size_t)warp * n_expert;
    const int64_t n_chunks = (n + 63) / 64;
    const int64_t stride = (int64_t)gridDim.x * kWarps;
    for (int64_t ch = (int64_t)blockIdx.x * kWarps + warp; ch < n_chunks; ch += 4 * stride) {
        int ea[4], eb[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int64_t c = ch + u * stride;
            if (c < n_chunks) load_chunk_unordered(gate, n, c * 64, lane, vec, n_expert, ea[u], eb[u]);
            else ea[u] = eb[u] = -1;
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            hist_round(ea[u], lane, my);
            hist_round(eb[u], lane, my);
        }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < n_expert; e += kThreads) {
        int32_t v = 0;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) v += sh[w * n_expert + e];
        if (v) atomicAdd(expert_count + e, v);
    }
}

__global__ void limit_by_capacity_kernel(const int64_t* __restrict__ ec, int32_t* __restrict__ cap,
                                         int64_t* __restrict__ eca, int n_expert, int n_worker) {
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= n_expert) return;
    int32_t left = cap[e];
    for (int w = 0; w < n_worker; ++w) {
        const int32_t proposal = (int32_t)ec[(int64_t)w * n_expert + e];
        int64_t grant;
        if (left >= proposal) grant = proposal;
        else if (left >= 0) grant = left;
        else grant = 0;
        eca[(int64_t)w * n_expert + e] = grant;
        left -= proposal;
    }
    cap[e] = left;
}

int check_routing_args(const void* gate, int64_t n, int n_expert) {
    FMOE_REQUIRE(n >= 0, "routing: negative entry count %lld", (long long)n);
    FMOE_REQUIRE(n == 0 || gate != nullptr, "routing: gate pointer is null");
    FMOE_REQUIRE(n_expert > 0 && n_expert <= FMOE_MAX_EXPERTS,
                 "routing: n_expert_total=%d outside [1,%d]", n_expert, FMOE_MAX_EXPERTS);
    FMOE_REQUIRE(n < ((int64_t)1 << 31), "routing: %lld entries exceed the int32 count range",
                 (long long)n);
    return 0;
}

int set_smem(const void* fn, size_t bytes) {
    if (bytes > 48 * 1024)
        FMOE_CUDA_TRY(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
    return 0;
}

// hist -> scan -> finalize -> apply on `stream`.
int run_bucket(int mode, const int64_t* gate, int64_t n, int n_expert, void* scratch,
               int64_t* lec64, int64_t* offsets, int32_t* inout, int64_t* pos, int64_t* inv,
               int64_t* new_gate, cudaStream_t st) {
    FMOE_REQUIRE(scratch != nullptr, "routing: scratch pointer is null");
    FMOE_REQUIRE(((uintptr_t)scratch & 15) == 0, "routing: scratch must be 16-byte aligned");
    const bool vec = ((uintptr_t)gate & 15) == 0;
    if (n > 0 && n <= (int64_t)kClMaxCtas * kClWarps * kClMaxChunks * 64 && n_expert <= kClMaxExperts) {
        // one cluster: as many CTAs as give every warp about 256 entries, at most kClMaxCtas
        const int n_cta = (int)std::min<int64_t>(kClMaxCtas, ceil_div(n, (int64_t)kClWarps * 256));
        const int chunks = (int)ceil_div(n, (int64_t)n_cta * kClWarps * 64);
        const size_t smem = ((size_t)kClWarps + 5) * n_expert * 4;
        if (int rc = set_smem((const void*)bucket_cluster_kernel, smem)) return rc;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)n_cta);
        cfg.blockDim = dim3(kClThreads);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = st;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = (unsigned)n_cta; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        FMOE_CUDA_TRY(cudaLaunchKernelEx(&cfg, bucket_cluster_kernel, mode, gate, n, n_expert, chunks, lec64, offsets, inout,
                                         pos, inv, new_gate, vec));
        return 0;
    }
    const Geom g = make_geom(n, n_expert);
    const Scratch s = carve(scratch, n, n_expert);
    const size_t sm_hist = (size_t)kWarps * n_expert * 4, sm_apply = sm_hist;
    if (int rc = set_smem((const void*)tile_hist_kernel, sm_hist)) return rc;
    if (int rc = set_smem((const void*)apply_kernel, sm_apply)) return rc;
    const unsigned blocks = (unsigned)ceil_div(g.n_tiles, kWarps);
    if (g.n_tiles > 0) {
        tile_hist_kernel<<<blocks, kThreads, sm_hist, st>>>(gate, n, n_expert, g.chunks, g.n_tiles,
                                                             s.hist, vec);
        FMOE_CHECK_LAUNCH();
    }
    const int scan_blocks = (int)ceil_div(g.n_tiles, kScanRows);
    if (scan_blocks > 0) {
        scan_tiles_kernel<<<scan_blocks, 256, 0, st>>>(s.hist, g.n_tiles, n_expert, s.blocksum);
        FMOE_CHECK_LAUNCH();
    }
    finalize_kernel<<<1, 1024, 0, st>>>(mode, n_expert, s.totals, s.blocksum, scan_blocks, s.seg_start, s.limit,
                                        lec64, offsets, inout);
    FMOE_CHECK_LAUNCH();
    if (g.n_tiles > 0) {
        apply_kernel<<<blocks, kThreads, sm_apply, st>>>(mode, gate, n, n_expert, g.chunks, g.n_tiles,
                                                          s.hist, s.blocksum, s.seg_start, s.limit,
                                                          offsets ? offsets + n_expert : nullptr, pos,
                                                          inv, new_gate, vec);
        FMOE_CHECK_LAUNCH();
    }
    return 0;
}

}  // namespace
}  // namespace fmoe

using namespace fmoe;

extern "C" size_t fmoe_routing_scratch_bytes(int64_t n, int32_t n_expert_total) {
    if (n < 0 || n_expert_total <= 0) return 0;
    return scratch_bytes(n, n_expert_total);
}

extern "C" int fmoe_expert_count(const int64_t* gate_idx, int32_t* expert_count, int64_t n,
                                 int32_t n_expert_total, fmoe_stream_t stream) {
    if (int rc = check_routing_args(gate_idx, n, n_expert_total)) return rc;
    FMOE_REQUIRE(expert_count != nullptr, "expert_count: output pointer is null");
    if (n == 0) return 0;
    const bool vec = ((uintptr_t)gate_idx & 15) == 0;
    const int64_t n_chunks = ceil_div(n, 64);
    const unsigned blocks = (unsigned)std::min<int64_t>(ceil_div(n_chunks, kWarps), (int64_t)sm_count() * 8);
    const size_t smem = (size_t)kWarps * n_expert_total * 4;
    if (int rc = set_smem((const void*)expert_count_kernel, smem)) return rc;
    expert_count_kernel<<<blocks, kThreads, smem, (cudaStream_t)stream>>>(gate_idx, n, n_expert_total,
                                                                           expert_count, vec);
    FMOE_CHECK_LAUNCH();
    return 0;
}

extern "C" int fmoe_assign_pos(int32_t* cum_count, const int64_t* gate, int64_t* pos, int64_t n,
                               int32_t n_expert_total, void* scratch, fmoe_stream_t stream) {
    if (int rc = check_routing_args(gate, n, n_expert_total)) return rc;
    FMOE_REQUIRE(cum_count != nullptr, "assign_pos: cum_count pointer is null");
    FMOE_REQUIRE(n == 0 || pos != nullptr, "assign_pos: pos pointer is null");
    return run_bucket(MODE_ASSIGN, gate, n, n_expert_total, scratch, nullptr, nullptr, cum_count, pos,
                      nullptr, nullptr, (cudaStream_t)stream);
}

extern "C" int fmoe_count_and_pos(const int64_t* gate, int64_t n, int32_t n_expert_total,
                                  int64_t* lec64, int64_t* offsets, int64_t* pos, int64_t* inv,
                                  void* scratch, fmoe_stream_t stream) {
    if (int rc = check_routing_args(gate, n, n_expert_total)) return rc;
    FMOE_REQUIRE(n == 0 || pos != nullptr, "count_and_pos: pos pointer is null");
    FMOE_REQUIRE(offsets != nullptr, "count_and_pos: offsets pointer is null");
    return run_bucket(MODE_COUNT_POS, gate, n, n_expert_total, scratch, lec64, offsets, nullptr, pos,
                      inv, nullptr, (cudaStream_t)stream);
}

extern "C" int fmoe_prune_gate_by_capacity(const int64_t* gate_idx, int64_t* new_gate_idx, int32_t* ec,
                                           int64_t n, int32_t n_expert_total, void* scratch,
                                           fmoe_stream_t stream) {
    if (int rc = check_routing_args(gate_idx, n, n_expert_total)) return rc;
    FMOE_REQUIRE(ec != nullptr, "prune_gate_by_capacity: expert_count pointer is null");
    FMOE_REQUIRE(n == 0 || new_gate_idx != nullptr, "prune_gate_by_capacity: output pointer is null");
    return run_bucket(MODE_PRUNE, gate_idx, n, n_expert_total, scratch, nullptr, nullptr, ec, nullptr,
                      nullptr, new_gate_idx, (cudaStream_t)stream);
}

extern "C" int fmoe_limit_by_capacity(const int64_t* ec, int32_t* cap, int64_t* eca, int32_t n_expert,
                                      int32_t n_worker, fmoe_stream_t stream) {
    FMOE_REQUIRE(ec && cap && eca, "limit_by_capacity: null pointer");
    FMOE_REQUIRE(n_expert > 0 && n_worker > 0, "limit_by_capacity: n_expert=%d n_worker=%d", n_expert,
                 n_worker);
    const int threads = 128;
    limit_by_capacity_kernel<<<(unsigned)ceil_div(n_expert, threads), threads, 0, (cudaStream_t)stream>>>(
        ec, cap, eca, n_expert, n_worker);
    FMOE_CHECK_LAUNCH();
    return 0;
}


// ---------------------------------------------------------------------------
// Bucketing without caller-provided scratch
// ---------------------------------------------------------------------------
//
// Some hosts of this library may not allocate device memory on the path that
// routes tokens: a serving process that handed all free HBM to its own pool at
// start-up, or a plugin host that bans the CUDA allocator from its request path
// because cudaMalloc/cudaFree serialise with the work already on the device.
// For them the per-tile histograms of the bucketing kernels live in a fixed
// array inside the library image instead of a buffer the caller supplies.
//
// The array is part of the loaded module: every GPU that loads the library
// keeps FMOE_STATIC_SCRATCH_BYTES of its memory for it until the process exits.
namespace fmoe {
namespace {

static __device__ __align__(256) unsigned char g_static_scratch[FMOE_STATIC_SCRATCH_BYTES];

// In host code `g_static_scratch` is only a handle for the runtime, not an address a
// kernel may dereference.  The device address is looked up once per device, with
// that device current, and cached.
int static_scratch_ptr(void** out) {
    static void* cache[64] = {};
    static std::mutex mtx;
    int dev = 0;
    FMOE_CUDA_TRY(cudaGetDevice(&dev));
    FMOE_REQUIRE(dev >= 0 && dev < 64, "static scratch: device index %d not supported", dev);
    std::lock_guard<std::mutex> lk(mtx);
    if (!cache[dev]) {
        void* p = nullptr;
        FMOE_CUDA_TRY(cudaGetSymbolAddress(&p, g_static_scratch));
        FMOE_REQUIRE(p != nullptr, "static scratch: symbol has no device address");
        cache[dev] = p;
    }
    *out = cache[dev];
    return 0;
}

}  // namespace
}  // namespace fmoe

extern "C" size_t fmoe_static_scratch_capacity(void) { return FMOE_STATIC_SCRATCH_BYTES; }

extern "C" int fmoe_count_and_pos_static(const int64_t* gate, int64_t n, int32_t n_expert_total,
                                         int64_t* lec64, int64_t* offsets, int64_t* pos, int64_t* inv,
                                         fmoe_stream_t stream) {
    if (int rc = check_routing_args(gate, n, n_expert_total)) return rc;
    FMOE_REQUIRE(n == 0 || pos != nullptr, "count_and_pos_static: pos pointer is null");
    FMOE_REQUIRE(offsets != nullptr, "count_and_pos_static: offsets pointer is null");
    const size_t need = scratch_bytes(n, n_expert_total);
    if (need > (size_t)FMOE_STATIC_SCRATCH_BYTES)
        return fail(FMOE_ERR_UNSUPPORTED,
                    "count_and_pos_static: %lld entries x %d experts need %zu bytes of scratch, the built-in "
                    "array holds %zu; use fmoe_count_and_pos with caller-provided scratch",
                    (long long)n, n_expert_total, need, (size_t)FMOE_STATIC_SCRATCH_BYTES);
    void* scratch = nullptr;
    if (int rc = static_scratch_ptr(&scratch)) return rc;
    // Nothing in the array has to start at zero: the histogram rows, the totals and the
    // segment starts are each written in full by an earlier kernel of this call before
    // a later one reads them, so whatever the previous call left behind is never read.
    return run_bucket(MODE_COUNT_POS, gate, n, n_expert_total, scratch, lec64, offsets, nullptr, pos, inv, nullptr,
                      (cudaStream_t)stream);
}
