// Smart schedule: the all-to-all-v of token rows is cut into steps (groups of
// peers); the expert MLP of a step starts as soon as that step's rows have
// arrived and its results travel back while later steps compute.
//
// Replaces cuda/fused_compute.{cu,cuh} of the reference.  Same schedule (ring
// offset between groups of `gran` peers, three phases send / compute / return
// ordered with events on two streams), but: one NCCL group per step instead of
// one per expert, the expert MLP runs on the grouped tensor-core GEMMs with the
// activation (and optional bias) fused into their epilogues, buffers come from
// the caller, nothing blocks the host, and rows of shadowed experts are staged
// into the tail of the expert-side buffers so that one kernel family serves both.
#include "common.cuh"
#include "exchange.h"
#include "gemm.h"
#include <vector>

namespace fmoe {
namespace {

struct Geometry {
    int n_steps, gran, group_rank, rank, E, W;
    int64_t B, S;
    std::vector<int64_t> local_ptr, global_ptr, lg_ptr;  // E*W+1 each
};

void compute_ptrs(const int64_t* lec, const int64_t* gec, const uint8_t* stored, int rank, int E, int W,
                  int64_t* local_ptr, int64_t* global_ptr, int64_t* lg_ptr) {
    local_ptr[0] = global_ptr[0] = lg_ptr[0] = 0;
    for (int i = 0; i < E * W; ++i) {
        local_ptr[i + 1] = local_ptr[i] + lec[i];
        lg_ptr[i + 1] = lg_ptr[i] + (stored[i] ? lec[i] : 0);
        const int e = i % E, w = i / E;
        global_ptr[e * W + w + 1] = stored[rank * E + e] ? 0 : gec[i];
    }
    for (int i = 0; i < E * W; ++i) global_ptr[i + 1] += global_ptr[i];
}

int make_geometry(const int64_t* lec, const int64_t* gec, const uint8_t* stored, int rank, int E, int W,
                  int gran, Geometry& g) {
    FMOE_REQUIRE(lec && gec && stored, "smart schedule: null count pointer");
    FMOE_REQUIRE(E > 0 && W > 0 && rank >= 0 && rank < W, "smart schedule: bad sizes E=%d W=%d rank=%d", E, W, rank);
    for (int i = 0; i < E * W; ++i)
        FMOE_REQUIRE(lec[i] >= 0 && gec[i] >= 0, "smart schedule: negative count at %d", i);
    if (gran < 1) gran = 1;
    if (gran > W) gran = W;
    while (W % gran) --gran;
    g.gran = gran;
    g.n_steps = W / gran;
    g.group_rank = rank / gran;
    g.rank = rank; g.E = E; g.W = W;
    g.local_ptr.assign((size_t)E * W + 1, 0);
    g.global_ptr.assign((size_t)E * W + 1, 0);
    g.lg_ptr.assign((size_t)E * W + 1, 0);
    compute_ptrs(lec, gec, stored, rank, E, W, g.local_ptr.data(), g.global_ptr.data(), g.lg_ptr.data());
    g.B = g.global_ptr[(size_t)E * W];
    g.S = g.lg_ptr[(size_t)E * W];
    FMOE_REQUIRE(g.B + g.S < ((int64_t)1 << 31), "smart schedule: %lld rows exceed the 32-bit row range",
                 (long long)(g.B + g.S));
    return 0;
}

struct Events {
    std::vector<cudaEvent_t> ev;
    ~Events() {
        for (auto e : ev) cudaEventDestroy(e);
    }
    int make(int n) {
        for (int i = 0; i < n; ++i) {
            cudaEvent_t e;
            FMOE_CUDA_TRY(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
            ev.push_back(e);
        }
        return 0;
    }
};

// One step of the exchange (cuda/fused_compute.cuh:289-306 and 332-349).
// forward_dir: token-side rows travel to the experts' owners; this rank sends to
// the peers of group (g + step) and receives from those of group (g - step).
// Otherwise the results travel back along the same pairs.  All transfers of the
// step form one NCCL group; rows that stay on this GPU are copied.
int exchange_step(Comm* c, const Geometry& g, int step, bool forward_dir, const void* src, void* dst,
                  const int64_t* lec, const int64_t* gec, const uint8_t* stored, int64_t row_bytes,
                  cudaStream_t st) {
    const int to_base = (g.group_rank + step) % g.n_steps * g.gran;
    const int from_base = (g.group_rank + g.n_steps - step) % g.n_steps * g.gran;
    const char* s = (const char*)src;
    char* d = (char*)dst;
    bool grouped = false;
    auto begin_group = [&]() -> int {
        if (!grouped) {
            FMOE_NCCL_TRY(g_nccl.GroupStart());
            grouped = true;
        }
        return 0;
    };
    struct Copy { int64_t from, to, rows; };
    std::vector<Copy> copies;
    for (int ei = 0; ei < g.E; ++ei) {
        const bool own_shadowed = stored[ei + g.rank * g.E] != 0;
        for (int j = 0; j < g.gran; ++j) {
            const int tok_peer = j + to_base;    // peer whose expert ei holds rows of ours
            const int exp_peer = j + from_base;  // peer whose rows our expert ei holds
            const int idx_tok = ei + tok_peer * g.E;
            const int64_t tok_rows = stored[idx_tok] ? 0 : lec[idx_tok];           // ours, on tok_peer
            const int64_t exp_rows = own_shadowed ? 0 : gec[ei + exp_peer * g.E];  // theirs, on us
            const int64_t tok_off = g.local_ptr[idx_tok];
            const int64_t exp_off = g.global_ptr[ei * g.W + exp_peer];
            // forward: token rows out, expert rows in.  return: expert rows out, token rows in.
            const int send_to = forward_dir ? tok_peer : exp_peer, recv_from = forward_dir ? exp_peer : tok_peer;
            const int64_t send_rows = forward_dir ? tok_rows : exp_rows, recv_rows = forward_dir ? exp_rows : tok_rows;
            const int64_t send_off = forward_dir ? tok_off : exp_off, recv_off = forward_dir ? exp_off : tok_off;
            if (send_to == g.rank) {
                // tok_peer == exp_peer == rank (step 0): both sides of the pair are this GPU.
                if (send_rows) copies.push_back({send_off, recv_off, send_rows});
                continue;
            }
            if (send_rows) {
                if (int rc = begin_group()) return rc;
                FMOE_NCCL_TRY(g_nccl.Send(s + send_off * row_bytes, (size_t)send_rows * row_bytes, ncclChar, send_to,
                                          c->comm, st));
            }
            if (recv_rows) {
                if (int rc = begin_group()) return rc;
                FMOE_NCCL_TRY(g_nccl.Recv(d + recv_off * row_bytes, (size_t)recv_rows * row_bytes, ncclChar, recv_from,
                                          c->comm, st));
            }
        }
    }
    if (grouped) FMOE_NCCL_TRY(g_nccl.GroupEnd());
    for (const auto& cp : copies)
        FMOE_CUDA_TRY(cudaMemcpyAsync(d + cp.to * row_bytes, s + cp.from * row_bytes, (size_t)cp.rows * row_bytes,
                                      cudaMemcpyDeviceToDevice, st));
    return 0;
}

// Shadow flags that are all-or-none per worker (what the layer produces): the rows a
// rank sends to a peer are then one contiguous token-side range.
bool flags_uniform(const uint8_t* stored, int E, int W) {
    for (int j = 0; j < W; ++j)
        for (int i = 1; i < E; ++i)
            if ((stored[j * E + i] != 0) != (stored[j * E] != 0)) return false;
    return true;
}

// Same step with ONE send and ONE receive per peer: rows from a peer land contiguously in
// `staging` (at a per-peer offset that is the same in every step) and one copy kernel moves
// them to their expert-major positions; on the way back a copy kernel packs them first.
int exchange_step_merged(Comm* c, const Geometry& g, int step, bool forward_dir, const void* token_c,
                         const void* expert_c, void* staging, const int64_t* lec, const int64_t* gec,
                         const uint8_t* stored, int64_t row_bytes, cudaStream_t st) {
    const int to_base = (g.group_rank + step) % g.n_steps * g.gran;
    const int from_base = (g.group_rank + g.n_steps - step) % g.n_steps * g.gran;
    char* token = (char*)token_c;
    char* expert = (char*)expert_c;
    char* stg = (char*)staging;
    const bool own_shadowed = stored[g.rank * g.E] != 0;
    auto rows_from = [&](int q) -> int64_t {  // rows peer q routed to this rank's experts
        if (own_shadowed) return 0;
        int64_t r = 0;
        for (int i = 0; i < g.E; ++i) r += gec[i + q * g.E];
        return r;
    };
    auto staging_off = [&](int q) -> int64_t {
        int64_t off = 0;
        for (int q2 = 0; q2 < q; ++q2)
            if (q2 != g.rank) off += rows_from(q2);
        return off;
    };
    struct Xfer { int peer; int64_t off, rows; };
    std::vector<Xfer> tok, exp;  // token-side ranges (per tok_peer), staging ranges (per exp_peer)
    std::vector<SegCopy> copies;
    for (int j = 0; j < g.gran; ++j) {
        const int tp = j + to_base, ep = j + from_base;
        if (tp == g.rank) {
            // both sides of the pair are this GPU (step 0): token rows <-> expert rows directly
            if (!own_shadowed)
                for (int i = 0; i < g.E; ++i) {
                    const int64_t n = lec[i + g.rank * g.E];
                    if (!n) continue;
                    if (forward_dir) copies.push_back({1, 0, g.local_ptr[i + g.rank * g.E], g.global_ptr[i * g.W + g.rank], n});
                    else copies.push_back({0, 1, g.global_ptr[i * g.W + g.rank], g.local_ptr[i + g.rank * g.E], n});
                }
            continue;
        }
        if (!stored[tp * g.E]) {
            const int64_t n = g.local_ptr[(tp + 1) * g.E] - g.local_ptr[tp * g.E];
            if (n) tok.push_back({tp, g.local_ptr[tp * g.E], n});
        }
        const int64_t r = rows_from(ep);
        if (r) {
            const int64_t s0 = staging_off(ep);
            exp.push_back({ep, s0, r});
            int64_t pre = 0;
            for (int i = 0; i < g.E; ++i) {
                const int64_t n = gec[i + ep * g.E];
                if (n) {
                    if (forward_dir) copies.push_back({0, 0, s0 + pre, g.global_ptr[i * g.W + ep], n});
                    else copies.push_back({0, 0, g.global_ptr[i * g.W + ep], s0 + pre, n});
                }
                pre += n;
            }
        }
    }
    auto group = [&](const std::vector<Xfer>& sends, const char* sbuf, const std::vector<Xfer>& recvs, char* rbuf) -> int {
        if (sends.empty() && recvs.empty()) return 0;
        FMOE_NCCL_TRY(g_nccl.GroupStart());
        for (const auto& x : sends) {
            ncclResult_t e = g_nccl.Send(sbuf + x.off * row_bytes, (size_t)x.rows * row_bytes, ncclChar, x.peer, c->comm, st);
            if (e != ncclSuccess) { g_nccl.GroupEnd(); return fail(FMOE_ERR_NCCL, "ncclSend failed: %s", g_nccl.GetErrorString(e)); }
        }
        for (const auto& x : recvs) {
            ncclResult_t e = g_nccl.Recv(rbuf + x.off * row_bytes, (size_t)x.rows * row_bytes, ncclChar, x.peer, c->comm, st);
            if (e != ncclSuccess) { g_nccl.GroupEnd(); return fail(FMOE_ERR_NCCL, "ncclRecv failed: %s", g_nccl.GetErrorString(e)); }
        }
        FMOE_NCCL_TRY(g_nccl.GroupEnd());
        return 0;
    };
    if (forward_dir) {
        if (int rc = group(tok, token, exp, stg)) return rc;
        // sources: 0 = staging, 1 = token buffer; destination 0 = expert buffer
        return launch_segment_copies(copies, stg, token, expert, nullptr, row_bytes, st);
    }
    // sources: 0 = expert buffer; destinations: 0 = staging, 1 = token buffer
    if (int rc = launch_segment_copies(copies, expert, nullptr, stg, token, row_bytes, st)) return rc;
    return group(exp, stg, tok, token);
}

// Picks the merged form when a staging buffer is given and the layout allows it.
int do_exchange_step(Comm* c, const Geometry& g, int step, bool forward_dir, const void* token, const void* expert,
                     void* staging, const int64_t* lec, const int64_t* gec, const uint8_t* stored, int64_t row_bytes,
                     cudaStream_t st) {
    // The choice must come out the same on every rank (the two forms pair sends and receives
    // differently), so it depends only on arguments that are identical everywhere.
    const bool merged = staging && g.E > 1 && row_bytes % 16 == 0 && flags_uniform(stored, g.E, g.W);
    if (merged)
        FMOE_REQUIRE(((((uintptr_t)token) | ((uintptr_t)expert) | ((uintptr_t)staging)) & 15) == 0,
                     "smart schedule: buffers must be 16-byte aligned when a staging buffer is given");
    if (merged) return exchange_step_merged(c, g, step, forward_dir, token, expert, staging, lec, gec, stored, row_bytes, st);
    if (forward_dir) return exchange_step(c, g, step, true, token, (void*)expert, lec, gec, stored, row_bytes, st);
    return exchange_step(c, g, step, false, expert, (void*)token, lec, gec, stored, row_bytes, st);
}

// Row ranges of one pipeline step, per local expert, in expert-side coordinates.
void step_segments(const Geometry& g, int step, HostSegs& hs) {
    const int from_base = (g.group_rank + g.n_steps - step) % g.n_steps * g.gran;
    hs.n = g.E;
    for (int ei = 0; ei < g.E; ++ei) {
        hs.lo[ei] = (int)g.global_ptr[ei * g.W + from_base];
        hs.hi[ei] = (int)g.global_ptr[ei * g.W + from_base + g.gran];
    }
}

// Row ranges of shadowed worker j's experts in the tail of the expert-side buffers.
void shadow_segments(const Geometry& g, int j, HostSegs& hs) {
    hs.n = g.E;
    for (int i = 0; i < g.E; ++i) {
        hs.lo[i] = (int)(g.B + g.lg_ptr[j * g.E + i]);
        hs.hi[i] = (int)(g.B + g.lg_ptr[j * g.E + i + 1]);
    }
}

bool worker_shadowed(const uint8_t* stored, int j, int E) {
    for (int i = 0; i < E; ++i)
        if (stored[j * E + i]) return true;
    return false;
}

int mlp_forward(const fmoe_mlp_params_t& pr, const HostSegs& hs, const void* x, void* mid, void* pre, void* out,
                int64_t rows, int64_t d, int64_t h, int E, int dtype, int act, cudaStream_t st) {
    LinearArgs a1{x, pr.w1, pr.b1, nullptr, mid, pre, rows, d, h, E, dtype, act, &hs};
    if (int rc = dispatch_linear_forward(a1, st)) return rc;
    LinearArgs a2{mid, pr.w2, pr.b2, nullptr, out, nullptr, rows, h, d, E, dtype, FMOE_ACT_NONE, &hs};
    return dispatch_linear_forward(a2, st);
}

int mlp_backward(const fmoe_mlp_params_t& pr, const HostSegs& hs, const void* x, const void* mid, const void* pre,
                 const void* gout, void* gmid, void* gin, int64_t rows, int64_t d, int64_t h, int E, int dtype,
                 int act, int accumulate, cudaStream_t st) {
    const void* act_pre = act == FMOE_ACT_RELU ? mid : (act == FMOE_ACT_GELU ? pre : nullptr);
    LinearBwdArgs b2{gout, mid, pr.w2, nullptr, act_pre, gmid, pr.gw2, pr.b2 ? pr.gb2 : nullptr,
                     rows, h, d, E, dtype, act, accumulate, nullptr, &hs};
    if (int rc = dispatch_linear_backward(b2, st)) return rc;
    LinearBwdArgs b1{gmid, x, pr.w1, nullptr, nullptr, gin, pr.gw1, pr.b1 ? pr.gb1 : nullptr,
                     rows, d, h, E, dtype, FMOE_ACT_NONE, accumulate, nullptr, &hs};
    return dispatch_linear_backward(b1, st);
}

int check_common(fmoe_comm_t comm, const fmoe_mlp_params_t* params, int n_workers, int n_expert, int dtype,
                 int act, int64_t d, int64_t h, Comm** c_out, int* rank_out) {
    FMOE_REQUIRE(params, "smart schedule: null parameter table");
    FMOE_REQUIRE(n_expert > 0 && n_expert <= kMaxHostSegs, "smart schedule: %d experts per worker (limit %d)",
                 n_expert, kMaxHostSegs);
    FMOE_REQUIRE(dtype_size(dtype) != 0, "smart schedule: unknown dtype %d", dtype);
    FMOE_REQUIRE(act >= FMOE_ACT_NONE && act <= FMOE_ACT_GELU, "smart schedule: unknown activation %d", act);
    FMOE_REQUIRE(d > 0 && h > 0, "smart schedule: bad widths");
    Comm* c = (Comm*)comm;
    if (n_workers > 1) {
        FMOE_REQUIRE(c, "smart schedule: null communicator with %d workers", n_workers);
        FMOE_REQUIRE(c->world == n_workers, "smart schedule: n_workers=%d but communicator has %d ranks",
                     n_workers, c->world);
    }
    *c_out = c;
    *rank_out = c ? c->rank : 0;
    return 0;
}

}  // namespace
}  // namespace fmoe

using namespace fmoe;

extern "C" int fmoe_fused_compute_ptrs(const int64_t* lec, const int64_t* gec, const uint8_t* stored,
                                       int32_t rank, int32_t E, int32_t W, int64_t* local_ptr,
                                       int64_t* global_ptr, int64_t* local_global_ptr) {
    FMOE_REQUIRE(lec && gec && stored && local_ptr && global_ptr && local_global_ptr,
                 "fused_compute_ptrs: null pointer");
    FMOE_REQUIRE(E > 0 && W > 0 && rank >= 0 && rank < W, "fused_compute_ptrs: bad sizes");
    compute_ptrs(lec, gec, stored, rank, E, W, local_ptr, global_ptr, local_global_ptr);
    return 0;
}

extern "C" int fmoe_fused_geometry(const int64_t* lec, const int64_t* gec, const uint8_t* stored, int32_t rank,
                                   int32_t E, int32_t W, int32_t pipeline_gran, fmoe_fused_geometry_t* out) {
    FMOE_REQUIRE(out, "fused_geometry: null output");
    Geometry g;
    if (int rc = make_geometry(lec, gec, stored, rank, E, W, pipeline_gran, g)) return rc;
    out->n_steps = g.n_steps;
    out->gran = g.gran;
    out->global_rows = g.B;
    out->shadow_rows = g.S;
    return 0;
}

extern "C" int fmoe_fused_forward(fmoe_comm_t comm, const void* local_in, void* local_out, void* global_in,
                                  void* middle, void* middle_pre, void* global_out,
                                  const fmoe_mlp_params_t* params, const int64_t* lec, const int64_t* gec,
                                  const uint8_t* stored, int64_t local_rows, int64_t d, int64_t h, int32_t E,
                                  int32_t W, int32_t dtype, int32_t act, int32_t gran, void* staging,
                                  fmoe_stream_t stream, fmoe_stream_t comm_stream) {
    Comm* c;
    int rank;
    if (int rc = check_common(comm, params, W, E, dtype, act, d, h, &c, &rank)) return rc;
    Geometry g;
    if (int rc = make_geometry(lec, gec, stored, rank, E, W, gran, g)) return rc;
    FMOE_REQUIRE(local_rows >= g.local_ptr[(size_t)E * W], "fused_forward: token-side buffer has %lld rows, counts say %lld",
                 (long long)local_rows, (long long)g.local_ptr[(size_t)E * W]);
    FMOE_REQUIRE(act != FMOE_ACT_GELU || middle_pre || g.B + g.S == 0, "fused_forward: GELU needs middle_pre");
    const int64_t rows = g.B + g.S;
    if (local_rows == 0 && rows == 0 && W == 1) return 0;
    FMOE_REQUIRE((local_in && local_out) || local_rows == 0, "fused_forward: null token-side buffer");
    FMOE_REQUIRE((global_in && middle && global_out) || rows == 0, "fused_forward: null expert-side buffer");
    cudaStream_t cs = (cudaStream_t)stream, ms = (cudaStream_t)comm_stream;
    const int64_t row_bytes = d * dtype_size(dtype);
    Events evs;
    if (int rc = evs.make(2 * g.n_steps + 2)) return rc;
    cudaEvent_t* in_ready = evs.ev.data();
    cudaEvent_t* out_ready = evs.ev.data() + g.n_steps;
    cudaEvent_t start = evs.ev[2 * g.n_steps], done = evs.ev[2 * g.n_steps + 1];

    // The token-side rows were produced on `stream`.
    FMOE_CUDA_TRY(cudaEventRecord(start, cs));
    FMOE_CUDA_TRY(cudaStreamWaitEvent(ms, start, 0));
    for (int step = 0; step < g.n_steps; ++step) {
        if (int rc = do_exchange_step(c, g, step, true, local_in, global_in, staging, lec, gec, stored, row_bytes, ms)) return rc;
        FMOE_CUDA_TRY(cudaEventRecord(in_ready[step], ms));
    }
    // Rows of shadowed experts stay here: stage them behind the received rows.
    for (int j = 0; j < W; ++j) {
        if (!worker_shadowed(stored, j, E)) continue;  // includes this rank when its own experts are shadowed
        const int64_t n = g.lg_ptr[(j + 1) * E] - g.lg_ptr[j * E];
        if (n)
            FMOE_CUDA_TRY(cudaMemcpyAsync((char*)global_in + (g.B + g.lg_ptr[j * E]) * row_bytes,
                                          (const char*)local_in + g.local_ptr[j * E] * row_bytes,
                                          (size_t)n * row_bytes, cudaMemcpyDeviceToDevice, cs));
    }
    for (int step = 0; step < g.n_steps; ++step) {
        FMOE_CUDA_TRY(cudaStreamWaitEvent(cs, in_ready[step], 0));
        HostSegs hs;
        step_segments(g, step, hs);
        if (int rc = mlp_forward(params[rank], hs, global_in, middle, middle_pre, global_out, rows, d, h, E, dtype, act, cs))
            return rc;
        FMOE_CUDA_TRY(cudaEventRecord(out_ready[step], cs));
    }
    for (int step = 0; step < g.n_steps; ++step) {
        FMOE_CUDA_TRY(cudaStreamWaitEvent(ms, out_ready[step], 0));
        if (int rc = do_exchange_step(c, g, step, false, local_out, global_out, staging, lec, gec, stored, row_bytes, ms)) return rc;
    }
    // Shadowed experts: compute locally with the fetched parameters while results travel.
    for (int j = 0; j < W; ++j) {
        if (!worker_shadowed(stored, j, E)) continue;  // includes this rank when its own experts are shadowed
        const int64_t n = g.lg_ptr[(j + 1) * E] - g.lg_ptr[j * E];
        if (!n) continue;
        HostSegs hs;
        shadow_segments(g, j, hs);
        if (int rc = mlp_forward(params[j], hs, global_in, middle, middle_pre, global_out, rows, d, h, E, dtype, act, cs))
            return rc;
        FMOE_CUDA_TRY(cudaMemcpyAsync((char*)local_out + g.local_ptr[j * E] * row_bytes,
                                      (const char*)global_out + (g.B + g.lg_ptr[j * E]) * row_bytes,
                                      (size_t)n * row_bytes, cudaMemcpyDeviceToDevice, cs));
    }
    FMOE_CUDA_TRY(cudaEventRecord(done, ms));
    FMOE_CUDA_TRY(cudaStreamWaitEvent(cs, done, 0));
    return 0;
}

extern "C" int fmoe_fused_backward(fmoe_comm_t comm, const void* grad_out_local, void* grad_in_local,
                                   const void* global_in, const void* middle, const void* middle_pre,
                                   void* global_grad_out, void* grad_middle, void* global_grad_in,
                                   const fmoe_mlp_params_t* params, const int64_t* lec, const int64_t* gec,
                                   const uint8_t* stored, int64_t local_rows, int64_t d, int64_t h, int32_t E,
                                   int32_t W, int32_t dtype, int32_t act, int32_t gran, void* staging,
                                   fmoe_stream_t stream, fmoe_stream_t comm_stream) {
    Comm* c;
    int rank;
    if (int rc = check_common(comm, params, W, E, dtype, act, d, h, &c, &rank)) return rc;
    Geometry g;
    if (int rc = make_geometry(lec, gec, stored, rank, E, W, gran, g)) return rc;
    FMOE_REQUIRE(local_rows >= g.local_ptr[(size_t)E * W], "fused_backward: token-side buffer has %lld rows, counts say %lld",
                 (long long)local_rows, (long long)g.local_ptr[(size_t)E * W]);
    const int64_t rows = g.B + g.S;
    FMOE_REQUIRE(act != FMOE_ACT_GELU || middle_pre || rows == 0, "fused_backward: GELU needs middle_pre");
    FMOE_REQUIRE((grad_out_local && grad_in_local) || local_rows == 0, "fused_backward: null token-side buffer");
    FMOE_REQUIRE((global_in && middle && global_grad_out && grad_middle && global_grad_in) || rows == 0,
                 "fused_backward: null expert-side buffer");
    FMOE_REQUIRE(params[rank].gw1 && params[rank].gw2, "fused_backward: null weight-gradient buffer");
    cudaStream_t cs = (cudaStream_t)stream, ms = (cudaStream_t)comm_stream;
    const int64_t row_bytes = d * dtype_size(dtype);
    Events evs;
    if (int rc = evs.make(2 * g.n_steps + 2)) return rc;
    cudaEvent_t* in_ready = evs.ev.data();
    cudaEvent_t* out_ready = evs.ev.data() + g.n_steps;
    cudaEvent_t start = evs.ev[2 * g.n_steps], done = evs.ev[2 * g.n_steps + 1];

    FMOE_CUDA_TRY(cudaEventRecord(start, cs));
    FMOE_CUDA_TRY(cudaStreamWaitEvent(ms, start, 0));
    for (int step = 0; step < g.n_steps; ++step) {
        if (int rc = do_exchange_step(c, g, step, true, grad_out_local, global_grad_out, staging, lec, gec, stored, row_bytes, ms))
            return rc;
        FMOE_CUDA_TRY(cudaEventRecord(in_ready[step], ms));
    }
    for (int j = 0; j < W; ++j) {
        if (!worker_shadowed(stored, j, E)) continue;  // includes this rank when its own experts are shadowed
        const int64_t n = g.lg_ptr[(j + 1) * E] - g.lg_ptr[j * E];
        if (n)
            FMOE_CUDA_TRY(cudaMemcpyAsync((char*)global_grad_out + (g.B + g.lg_ptr[j * E]) * row_bytes,
                                          (const char*)grad_out_local + g.local_ptr[j * E] * row_bytes,
                                          (size_t)n * row_bytes, cudaMemcpyDeviceToDevice, cs));
    }
    for (int step = 0; step < g.n_steps; ++step) {
        FMOE_CUDA_TRY(cudaStreamWaitEvent(cs, in_ready[step], 0));
        HostSegs hs;
        step_segments(g, step, hs);
        // The first step overwrites the own experts' weight gradients, later steps add
        // (cuda/fused_compute.cuh:120, 470).
        if (int rc = mlp_backward(params[rank], hs, global_in, middle, middle_pre, global_grad_out, grad_middle,
                                  global_grad_in, rows, d, h, E, dtype, act, step == 0 ? 0 : 1, cs))
            return rc;
        FMOE_CUDA_TRY(cudaEventRecord(out_ready[step], cs));
    }
    for (int step = 0; step < g.n_steps; ++step) {
        FMOE_CUDA_TRY(cudaStreamWaitEvent(ms, out_ready[step], 0));
        if (int rc = do_exchange_step(c, g, step, false, grad_in_local, global_grad_in, staging, lec, gec, stored, row_bytes, ms))
            return rc;
    }
    for (int j = 0; j < W; ++j) {
        if (!worker_shadowed(stored, j, E)) continue;  // includes this rank when its own experts are shadowed
        const int64_t n = g.lg_ptr[(j + 1) * E] - g.lg_ptr[j * E];
        if (!n) continue;
        FMOE_REQUIRE(params[j].gw1 && params[j].gw2, "fused_backward: null gradient buffer for shadowed worker %d", j);
        HostSegs hs;
        shadow_segments(g, j, hs);
        if (int rc = mlp_backward(params[j], hs, global_in, middle, middle_pre, global_grad_out, grad_middle,
                                  global_grad_in, rows, d, h, E, dtype, act, 1, cs))
            return rc;
        FMOE_CUDA_TRY(cudaMemcpyAsync((char*)grad_in_local + g.local_ptr[j * E] * row_bytes,
                                      (const char*)global_grad_in + (g.B + g.lg_ptr[j * E]) * row_bytes,
                                      (size_t)n * row_bytes, cudaMemcpyDeviceToDevice, cs));
    }
    FMOE_CUDA_TRY(cudaEventRecord(done, ms));
    FMOE_CUDA_TRY(cudaStreamWaitEvent(cs, done, 0));
    return 0;
}
