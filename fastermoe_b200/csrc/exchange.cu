// Expert-parallel exchange over NCCL: count exchange, token all-to-all-v,
// shadow-parameter broadcast and shadow-gradient reduce.
//
// Replaces cuda/global_exchange.{cu,cuh} of the reference.  Differences by
// design: the communicator is created from a unique id that the host program
// distributes (no dependency on c10d internals); each exchange is ONE NCCL
// group on the caller's stream (the reference opens one group per local
// expert and blocks the host afterwards); rows that stay on this GPU move with
// a device-to-device copy instead of a self send/recv.
//
// NCCL is bound at run time from the copy already loaded into the process (the
// one PyTorch ships), so that the process never holds two NCCL instances.
#include "common.cuh"
#include "exchange.h"
#include <dlfcn.h>
#include <mutex>
#include <vector>
#include <cstring>

namespace fmoe {

NcclApi g_nccl;
static std::once_flag g_nccl_once;
static int g_nccl_rc = FMOE_ERR_NCCL;
static char g_nccl_msg[256] = "NCCL not loaded";

static void load_nccl() {
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!h) {
        snprintf(g_nccl_msg, sizeof(g_nccl_msg), "cannot load libnccl.so.2: %s", dlerror());
        return;
    }
#define BIND(name)                                                                   \
    g_nccl.name = (decltype(g_nccl.name))dlsym(h, "nccl" #name);                     \
    if (!g_nccl.name) {                                                              \
        snprintf(g_nccl_msg, sizeof(g_nccl_msg), "libnccl lacks symbol nccl" #name); \
        return;                                                                      \
    }
    BIND(GetUniqueId) BIND(CommInitRank) BIND(CommDestroy) BIND(CommUserRank) BIND(CommCount)
    BIND(AllGather) BIND(Send) BIND(Recv) BIND(GroupStart) BIND(GroupEnd) BIND(Broadcast)
    BIND(Reduce) BIND(GetErrorString)
#undef BIND
    g_nccl_rc = 0;
}

int ensure_nccl_loaded() {
    std::call_once(g_nccl_once, load_nccl);
    if (g_nccl_rc) return fail(FMOE_ERR_NCCL, "%s", g_nccl_msg);
    return 0;
}

static_assert(sizeof(ncclUniqueId) == 128, "unique id is 128 bytes");

namespace {

// aec[src][dst][e] -> agec[dst][src][e]; gec = agec[rank].
__global__ void transpose_counts_kernel(const int64_t* __restrict__ aec, int64_t* __restrict__ agec,
                                        int64_t* __restrict__ gec, int n_expert, int n_workers, int rank) {
    const int64_t total = (int64_t)n_workers * n_workers * n_expert;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int e = (int)(i % n_expert);
        const int src = (int)((i / n_expert) % n_workers);
        const int dst = (int)(i / ((int64_t)n_expert * n_workers));
        const int64_t v = aec[((int64_t)src * n_workers + dst) * n_expert + e];
        agec[i] = v;
        if (dst == rank) gec[(int64_t)src * n_expert + e] = v;
    }
}

__global__ void cached_count_kernel(const int64_t* __restrict__ lec, const int64_t* __restrict__ gec,
                                    const uint8_t* __restrict__ stored, int64_t* __restrict__ out,
                                    int rank, int n_expert, int n_workers) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_expert * n_workers) return;
    const int w = i / n_expert, e = i % n_expert;
    int64_t v = stored[i] ? lec[i] : 0;
    if (w == rank && !stored[rank * n_expert + e]) {
        int64_t s = 0;
        for (int j = 0; j < n_workers; ++j) s += gec[j * n_expert + e];
        v += s;
    }
    out[i] = v;
}

int check_counts(const int64_t* lec, const int64_t* gec, const uint8_t* stored, int n_expert,
                 int n_workers) {
    FMOE_REQUIRE(lec && gec && stored, "exchange: null count pointer");
    FMOE_REQUIRE(n_expert > 0 && n_workers > 0, "exchange: n_expert=%d n_workers=%d", n_expert, n_workers);
    for (int i = 0; i < n_expert * n_workers; ++i)
        FMOE_REQUIRE(lec[i] >= 0 && gec[i] >= 0, "exchange: negative count at %d", i);
    return 0;
}

}  // namespace

int plan_scatter(const int64_t* lec, const int64_t* gec, const uint8_t* stored, int rank, int E, int W,
                 std::vector<fmoe_move_t>& moves, int64_t* recv_rows, int64_t* send_rows) {
    if (int rc = check_counts(lec, gec, stored, E, W)) return rc;
    FMOE_REQUIRE(rank >= 0 && rank < W, "exchange: rank %d outside [0,%d)", rank, W);
    std::vector<int64_t> eptr((size_t)E * W + 1, 0);
    for (int i = 0; i < E * W; ++i) eptr[i + 1] = eptr[i] + lec[i];
    int64_t rp = 0;
    auto local_block = [&](int j) {
        for (int i = 0; i < E; ++i) {
            const int idx = i + j * E;
            if (stored[idx] && lec[idx] > 0)
                moves.push_back({rank, 0, eptr[idx], rp, lec[idx], 1, 0});
            if (stored[idx]) rp += lec[idx];
        }
    };
    for (int j = 0; j < rank; ++j) local_block(j);
    for (int i = 0; i < E; ++i) {
        for (int j = 0; j < W; ++j) {
            const int idx = i + j * E;
            const bool do_send = lec[idx] > 0 && (!stored[idx] || j == rank);
            const bool do_recv = gec[idx] > 0 && (!stored[rank * E + i] || j == rank);
            if (j == rank) {
                if (do_send != do_recv || (do_send && lec[idx] != gec[idx]))
                    return fail(FMOE_ERR_MISMATCH,
                                "exchange: rank %d keeps %lld rows for its expert %d but expects %lld",
                                rank, (long long)lec[idx], i, (long long)gec[idx]);
                if (do_send) moves.push_back({rank, 0, eptr[idx], rp, lec[idx], 1, 0});
            } else {
                if (do_send) moves.push_back({j, 1, eptr[idx], 0, lec[idx], 0, 0});
                if (do_recv) moves.push_back({j, 0, 0, rp, gec[idx], 0, 0});
            }
            if (do_recv) rp += gec[idx];
        }
    }
    for (int j = rank + 1; j < W; ++j) local_block(j);
    *recv_rows = rp;
    if (send_rows) *send_rows = eptr[(size_t)E * W];
    return 0;
}

namespace {

int run_exchange(Comm* c, const void* src, void* dst, const std::vector<fmoe_move_t>& moves, bool reverse,
                 int64_t row_bytes, cudaStream_t st) {
    const char* s = (const char*)src;
    char* d = (char*)dst;
    bool any_remote = false;
    for (const auto& m : moves) any_remote |= !m.local;
    if (any_remote) {
        FMOE_NCCL_TRY(g_nccl.GroupStart());
        for (const auto& m : moves) {
            if (m.local) continue;
            const size_t bytes = (size_t)m.rows * row_bytes;
            // Forward: sends read `src` at src_row, receives write `dst` at dst_row.
            // Reverse (gather): the roles and the buffers swap.
            const bool send = reverse ? !m.is_send : m.is_send;
            ncclResult_t r;
            if (send) r = g_nccl.Send(s + (reverse ? m.dst_row : m.src_row) * row_bytes, bytes, ncclChar, m.peer, c->comm, st);
            else r = g_nccl.Recv(d + (reverse ? m.src_row : m.dst_row) * row_bytes, bytes, ncclChar, m.peer, c->comm, st);
            if (r != ncclSuccess) {
                g_nccl.GroupEnd();
                return fail(FMOE_ERR_NCCL, "ncclSend/Recv failed: %s", g_nccl.GetErrorString(r));
            }
        }
        FMOE_NCCL_TRY(g_nccl.GroupEnd());
    }
    for (const auto& m : moves) {
        if (!m.local || m.rows == 0) continue;
        const int64_t from = reverse ? m.dst_row : m.src_row, to = reverse ? m.src_row : m.dst_row;
        FMOE_CUDA_TRY(cudaMemcpyAsync(d + to * row_bytes, s + from * row_bytes, (size_t)m.rows * row_bytes,
                                      cudaMemcpyDeviceToDevice, st));
    }
    return 0;
}

// ---- merged exchange ---------------------------------------------------------------
// With a staging buffer the exchange uses ONE send and ONE receive per peer: the rows a
// rank sends to a peer are contiguous on the token side (all experts of that peer), and
// the rows it receives from a peer land contiguously in the staging buffer; one copy
// kernel then moves them (and the rows that never leave the GPU) to the expert-major
// layout.  Large messages keep NVLink busy where many expert-sized ones do not.
constexpr int kSegMax = 160;
struct SegTable {
    int n;
    int prefix[kSegMax + 1];  // rows before segment k
    int src_row[kSegMax], dst_row[kSegMax];
    unsigned char src_sel[kSegMax], dst_sel[kSegMax];
};

__global__ void __launch_bounds__(256)
segment_copy_kernel(const __grid_constant__ SegTable t, const uint4* __restrict__ src0, const uint4* __restrict__ src1,
                    uint4* __restrict__ dst0, uint4* __restrict__ dst1, int64_t row_vecs) {
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (row >= t.prefix[t.n]) return;
    int lo = 0, hi = t.n - 1;  // last segment whose prefix <= row
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (t.prefix[mid] <= row) lo = mid; else hi = mid - 1;
    }
    const int k = lo, off = row - t.prefix[k];
    const uint4* s = (t.src_sel[k] ? src1 : src0) + (int64_t)(t.src_row[k] + off) * row_vecs;
    uint4* d = (t.dst_sel[k] ? dst1 : dst0) + (int64_t)(t.dst_row[k] + off) * row_vecs;
    int64_t c = lane;
    for (; c + 96 < row_vecs; c += 128) {
        const uint4 v0 = __ldg(s + c), v1 = __ldg(s + c + 32), v2 = __ldg(s + c + 64), v3 = __ldg(s + c + 96);
        d[c] = v0; d[c + 32] = v1; d[c + 64] = v2; d[c + 96] = v3;
    }
    for (; c < row_vecs; c += 32) d[c] = __ldg(s + c);
}

struct P2P { int peer; int64_t row, rows; };

}  // namespace

int launch_segment_copies(const std::vector<SegCopy>& copies, const void* src0, const void* src1, void* dst0,
                          void* dst1, int64_t row_bytes, cudaStream_t st) {
    SegTable t;
    size_t i = 0;
    while (i < copies.size()) {
        t.n = 0;
        t.prefix[0] = 0;
        for (; i < copies.size() && t.n < kSegMax; ++i) {
            const SegCopy& c = copies[i];
            if (c.rows == 0) continue;
            t.src_sel[t.n] = (unsigned char)c.src_sel; t.dst_sel[t.n] = (unsigned char)c.dst_sel;
            t.src_row[t.n] = (int)c.src_row; t.dst_row[t.n] = (int)c.dst_row;
            t.prefix[t.n + 1] = t.prefix[t.n] + (int)c.rows;
            ++t.n;
        }
        if (t.n == 0) break;
        const unsigned blocks = (unsigned)ceil_div(t.prefix[t.n], 8);
        segment_copy_kernel<<<blocks, 256, 0, st>>>(t, (const uint4*)src0, (const uint4*)src1, (uint4*)dst0, (uint4*)dst1,
                                                    row_bytes / 16);
        FMOE_CHECK_LAUNCH();
    }
    return 0;
}

namespace {

// token: token-side buffer, expert: expert-side buffer, staging: >= rows received from
// peers.  forward = global_scatter, otherwise global_gather.
int run_exchange_merged(Comm* c, const void* token_c, const void* expert_c, void* staging, bool forward,
                        const int64_t* lec, const int64_t* gec, const uint8_t* stored, int E, int W,
                        int64_t row_bytes, cudaStream_t st) {
    const int rank = c->rank;
    char* token = (char*)token_c;
    char* expert = (char*)expert_c;
    std::vector<int64_t> eptr((size_t)E * W + 1, 0);
    for (int i = 0; i < E * W; ++i) eptr[i + 1] = eptr[i] + lec[i];
    std::vector<P2P> tok_runs, stg_runs;   // token-side runs (per peer) and staging runs (per peer)
    std::vector<SegCopy> copies;            // sel 0: staging, sel 1: token buffer (source side, forward)
    // token-side runs: experts of peer j that are not shadowed here, in maximal consecutive ranges
    for (int j = 0; j < W; ++j) {
        if (j == rank) continue;
        int i = 0;
        while (i < E) {
            if (stored[j * E + i]) { ++i; continue; }
            int i1 = i;
            while (i1 < E && !stored[j * E + i1]) ++i1;
            const int64_t rows = eptr[j * E + i1] - eptr[j * E + i];
            if (rows) tok_runs.push_back({j, eptr[j * E + i], rows});
            i = i1;
        }
    }
    // expert-side layout, walked exactly as plan_scatter does
    std::vector<int64_t> stg_off((size_t)E * W, -1);  // staging row of segment (i, j)
    int64_t stg = 0;
    for (int j = 0; j < W; ++j) {
        if (j == rank) continue;
        int i = 0;
        while (i < E) {
            if (stored[rank * E + i]) { ++i; continue; }
            int i1 = i;
            int64_t rows = 0;
            while (i1 < E && !stored[rank * E + i1]) {
                stg_off[i1 + j * E] = stg + rows;
                rows += gec[i1 + j * E];
                ++i1;
            }
            if (rows) stg_runs.push_back({j, stg, rows});
            stg += rows;
            i = i1;
        }
    }
    int64_t rp = 0;
    auto local_block = [&](int j) {
        for (int i = 0; i < E; ++i) {
            const int idx = i + j * E;
            if (stored[idx]) {
                copies.push_back({1, 0, eptr[idx], rp, lec[idx]});
                rp += lec[idx];
            }
        }
    };
    for (int j = 0; j < rank; ++j) local_block(j);
    for (int i = 0; i < E; ++i)
        for (int j = 0; j < W; ++j) {
            const int idx = i + j * E;
            const bool do_recv = gec[idx] > 0 && (!stored[rank * E + i] || j == rank);
            if (!do_recv) continue;
            if (j == rank) copies.push_back({1, 0, eptr[idx], rp, gec[idx]});
            else copies.push_back({0, 0, stg_off[idx], rp, gec[idx]});
            rp += gec[idx];
        }
    for (int j = rank + 1; j < W; ++j) local_block(j);

    auto group = [&](const std::vector<P2P>& sends, const char* sbuf, const std::vector<P2P>& recvs, char* rbuf) -> int {
        if (sends.empty() && recvs.empty()) return 0;
        FMOE_NCCL_TRY(g_nccl.GroupStart());
        for (const auto& r : sends) {
            ncclResult_t e = g_nccl.Send(sbuf + r.row * row_bytes, (size_t)r.rows * row_bytes, ncclChar, r.peer, c->comm, st);
            if (e != ncclSuccess) { g_nccl.GroupEnd(); return fail(FMOE_ERR_NCCL, "ncclSend failed: %s", g_nccl.GetErrorString(e)); }
        }
        for (const auto& r : recvs) {
            ncclResult_t e = g_nccl.Recv(rbuf + r.row * row_bytes, (size_t)r.rows * row_bytes, ncclChar, r.peer, c->comm, st);
            if (e != ncclSuccess) { g_nccl.GroupEnd(); return fail(FMOE_ERR_NCCL, "ncclRecv failed: %s", g_nccl.GetErrorString(e)); }
        }
        FMOE_NCCL_TRY(g_nccl.GroupEnd());
        return 0;
    };
    if (forward) {
        if (int rc = group(tok_runs, token, stg_runs, (char*)staging)) return rc;
        return launch_segment_copies(copies, staging, token, expert, nullptr, row_bytes, st);
    }
    // gather: expert-side rows go back: into the staging runs (remote) or straight to the token side (local)
    std::vector<SegCopy> back;
    back.reserve(copies.size());
    for (const auto& cp : copies) back.push_back({0, cp.src_sel, cp.dst_row, cp.src_row, cp.rows});
    if (int rc = launch_segment_copies(back, expert, nullptr, staging, token, row_bytes, st)) return rc;
    return group(stg_runs, (const char*)staging, tok_runs, token);
}

}  // namespace
}  // namespace fmoe

using namespace fmoe;

extern "C" int fmoe_comm_unique_id(void* id128_host) {
    FMOE_REQUIRE(id128_host, "comm_unique_id: null pointer");
    if (int rc = ensure_nccl_loaded()) return rc;
    ncclUniqueId id;
    FMOE_NCCL_TRY(g_nccl.GetUniqueId(&id));
    memcpy(id128_host, &id, 128);
    return 0;
}

extern "C" int fmoe_comm_init(const void* id128_host, int32_t rank, int32_t world_size, int32_t device,
                              fmoe_comm_t* comm_out) {
    FMOE_REQUIRE(id128_host && comm_out, "comm_init: null pointer");
    FMOE_REQUIRE(world_size > 0 && rank >= 0 && rank < world_size, "comm_init: rank %d of %d", rank, world_size);
    if (int rc = ensure_nccl_loaded()) return rc;
    FMOE_CUDA_TRY(cudaSetDevice(device));
    ncclUniqueId id;
    memcpy(&id, id128_host, 128);
    Comm* c = new Comm();
    c->rank = rank;
    c->world = world_size;
    c->device = device;
    ncclResult_t r = g_nccl.CommInitRank(&c->comm, world_size, id, rank);
    if (r != ncclSuccess) {
        delete c;
        return fail(FMOE_ERR_NCCL, "ncclCommInitRank failed: %s", g_nccl.GetErrorString(r));
    }
    *comm_out = c;
    return 0;
}

extern "C" int fmoe_comm_destroy(fmoe_comm_t comm) {
    if (!comm) return 0;
    Comm* c = (Comm*)comm;
    peer_release(c);
    if (c->comm) g_nccl.CommDestroy(c->comm);
    for (auto& ev : c->events) cudaEventDestroy(ev);
    delete c;
    return 0;
}

extern "C" int fmoe_comm_rank(fmoe_comm_t comm, int32_t* rank_out, int32_t* world_out) {
    FMOE_REQUIRE(comm, "comm_rank: null communicator");
    Comm* c = (Comm*)comm;
    if (rank_out) *rank_out = c->rank;
    if (world_out) *world_out = c->world;
    return 0;
}

extern "C" int fmoe_expert_exchange(fmoe_comm_t comm, const int64_t* lec, int64_t* aec, int64_t* agec,
                                    int64_t* gec, int32_t n_expert, int32_t n_workers,
                                    fmoe_stream_t stream) {
    FMOE_REQUIRE(comm && lec && aec && agec && gec, "expert_exchange: null pointer");
    Comm* c = (Comm*)comm;
    FMOE_REQUIRE(n_workers == c->world, "expert_exchange: n_workers=%d but communicator has %d ranks",
                 n_workers, c->world);
    FMOE_REQUIRE(n_expert > 0, "expert_exchange: n_expert=%d", n_expert);
    cudaStream_t st = (cudaStream_t)stream;
    const size_t bytes = (size_t)n_workers * n_expert * sizeof(int64_t);
    FMOE_NCCL_TRY(g_nccl.AllGather(lec, aec, bytes, ncclChar, c->comm, st));
    const int64_t total = (int64_t)n_workers * n_workers * n_expert;
    transpose_counts_kernel<<<(unsigned)std::min<int64_t>(ceil_div(total, 256), 1024), 256, 0, st>>>(
        aec, agec, gec, n_expert, n_workers, c->rank);
    FMOE_CHECK_LAUNCH();
    return 0;
}

extern "C" int fmoe_plan_global_scatter(const int64_t* lec_host, const int64_t* gec_host,
                                        const uint8_t* stored_models_host, int32_t rank, int32_t n_expert,
                                        int32_t n_workers, fmoe_move_t* moves, int32_t max_moves,
                                        int32_t* n_moves, int64_t* recv_rows) {
    FMOE_REQUIRE(n_moves && recv_rows, "plan_global_scatter: null output pointer");
    std::vector<fmoe_move_t> v;
    if (int rc = plan_scatter(lec_host, gec_host, stored_models_host, rank, n_expert, n_workers, v, recv_rows, nullptr))
        return rc;
    *n_moves = (int32_t)v.size();
    if (moves) {
        FMOE_REQUIRE((int32_t)v.size() <= max_moves, "plan_global_scatter: %zu moves exceed max_moves=%d",
                     v.size(), max_moves);
        memcpy(moves, v.data(), v.size() * sizeof(fmoe_move_t));
    }
    return 0;
}

static int global_move(fmoe_comm_t comm, const void* in, void* out, const int64_t* lec, const int64_t* gec,
                       const uint8_t* stored, int64_t in_rows, int64_t out_rows, int64_t row_bytes,
                       int n_expert, int n_workers, bool reverse, void* staging, cudaStream_t st) {
    FMOE_REQUIRE(comm, "global exchange: null communicator");
    Comm* c = (Comm*)comm;
    FMOE_REQUIRE(n_workers == c->world, "global exchange: n_workers=%d but communicator has %d ranks",
                 n_workers, c->world);
    FMOE_REQUIRE(row_bytes > 0, "global exchange: row_bytes=%lld", (long long)row_bytes);
    std::vector<fmoe_move_t> moves;
    int64_t recv_rows = 0, send_rows = 0;
    if (int rc = plan_scatter(lec, gec, stored, c->rank, n_expert, n_workers, moves, &recv_rows, &send_rows))
        return rc;
    const int64_t local_rows = reverse ? out_rows : in_rows, global_rows = reverse ? in_rows : out_rows;
    if (global_rows != recv_rows)
        return fail(FMOE_ERR_MISMATCH, "global exchange: expert-side buffer has %lld rows, counts say %lld",
                    (long long)global_rows, (long long)recv_rows);
    if (local_rows < send_rows)
        return fail(FMOE_ERR_MISMATCH, "global exchange: token-side buffer has %lld rows, counts say %lld",
                    (long long)local_rows, (long long)send_rows);
    FMOE_REQUIRE((in || in_rows == 0) && (out || out_rows == 0), "global exchange: null buffer");
    if (reverse && out_rows > send_rows)
        FMOE_CUDA_TRY(cudaMemsetAsync((char*)out + send_rows * row_bytes, 0,
                                      (size_t)(out_rows - send_rows) * row_bytes, st));
    // The choice must be the same on every rank: it may only depend on arguments that are.
    const bool can_merge = staging && row_bytes % 16 == 0;
    if (can_merge) {
        FMOE_REQUIRE((((uintptr_t)in | (uintptr_t)out | (uintptr_t)staging) & 15) == 0,
                     "global exchange: buffers must be 16-byte aligned when a staging buffer is given");
        FMOE_REQUIRE(recv_rows < ((int64_t)1 << 31) && send_rows < ((int64_t)1 << 31),
                     "global exchange: row counts exceed the 32-bit range of the staged form");
    }
    if (can_merge)
        return run_exchange_merged(c, reverse ? out : in, reverse ? in : out, staging, !reverse, lec, gec, stored,
                                   n_expert, n_workers, row_bytes, st);
    return run_exchange(c, in, out, moves, reverse, row_bytes, st);
}

extern "C" int fmoe_global_scatter(fmoe_comm_t comm, const void* local_in, void* global_out,
                                   const int64_t* lec_host, const int64_t* gec_host,
                                   const uint8_t* stored_models_host, int64_t in_rows, int64_t out_rows,
                                   int64_t row_bytes, int32_t n_expert, int32_t n_workers, void* staging,
                                   fmoe_stream_t stream) {
    return global_move(comm, local_in, global_out, lec_host, gec_host, stored_models_host, in_rows, out_rows,
                       row_bytes, n_expert, n_workers, false, staging, (cudaStream_t)stream);
}

extern "C" int fmoe_global_gather(fmoe_comm_t comm, const void* global_in, void* local_out,
                                  const int64_t* lec_host, const int64_t* gec_host,
                                  const uint8_t* stored_models_host, int64_t in_rows, int64_t out_rows,
                                  int64_t row_bytes, int32_t n_expert, int32_t n_workers, void* staging,
                                  fmoe_stream_t stream) {
    return global_move(comm, global_in, local_out, lec_host, gec_host, stored_models_host, in_rows, out_rows,
                       row_bytes, n_expert, n_workers, true, staging, (cudaStream_t)stream);
}

extern "C" int fmoe_exchange_cache_info(fmoe_comm_t comm, const uint8_t* sent_models, uint8_t* stored_models,
                                        int32_t n_expert, int32_t n_workers, fmoe_stream_t stream) {
    FMOE_REQUIRE(comm && sent_models && stored_models, "exchange_cache_info: null pointer");
    Comm* c = (Comm*)comm;
    FMOE_REQUIRE(n_workers == c->world && n_expert > 0, "exchange_cache_info: bad sizes");
    FMOE_NCCL_TRY(g_nccl.AllGather(sent_models, stored_models, (size_t)n_expert, ncclChar, c->comm,
                                   (cudaStream_t)stream));
    return 0;
}

extern "C" int fmoe_model_broadcast(fmoe_comm_t comm, void* buf, int64_t bytes, int32_t root,
                                    fmoe_stream_t stream) {
    FMOE_REQUIRE(comm && buf && bytes >= 0, "model_broadcast: bad argument");
    Comm* c = (Comm*)comm;
    FMOE_REQUIRE(root >= 0 && root < c->world, "model_broadcast: root %d of %d", root, c->world);
    if (bytes == 0) return 0;
    FMOE_NCCL_TRY(g_nccl.Broadcast(buf, buf, (size_t)bytes, ncclChar, root, c->comm, (cudaStream_t)stream));
    return 0;
}

extern "C" int fmoe_gradient_reduce(fmoe_comm_t comm, void* buf, int64_t count, int32_t dtype, int32_t root,
                                    fmoe_stream_t stream) {
    FMOE_REQUIRE(comm && buf && count >= 0, "gradient_reduce: bad argument");
    Comm* c = (Comm*)comm;
    FMOE_REQUIRE(root >= 0 && root < c->world, "gradient_reduce: root %d of %d", root, c->world);
    ncclDataType_t t;
    switch (dtype) {
        case FMOE_F32: t = ncclFloat; break;
        case FMOE_F16: t = ncclHalf; break;
        case FMOE_BF16: t = ncclBfloat16; break;
        default: return fail(FMOE_ERR_INVALID, "gradient_reduce: unknown dtype %d", dtype);
    }
    if (count == 0) return 0;
    FMOE_NCCL_TRY(g_nccl.Reduce(buf, buf, (size_t)count, t, ncclSum, root, c->comm, (cudaStream_t)stream));
    return 0;
}

extern "C" int fmoe_generate_cached_count(const int64_t* lec, const int64_t* gec, const uint8_t* stored_models,
                                          int64_t* out, int32_t rank, int32_t n_expert, int32_t n_workers,
                                          fmoe_stream_t stream) {
    FMOE_REQUIRE(lec && gec && stored_models && out, "generate_cached_count: null pointer");
    FMOE_REQUIRE(n_expert > 0 && n_workers > 0 && rank >= 0 && rank < n_workers,
                 "generate_cached_count: bad sizes");
    const int n = n_expert * n_workers;
    cached_count_kernel<<<(unsigned)ceil_div(n, 128), 128, 0, (cudaStream_t)stream>>>(
        lec, gec, stored_models, out, rank, n_expert, n_workers);
    FMOE_CHECK_LAUNCH();
    return 0;
}
