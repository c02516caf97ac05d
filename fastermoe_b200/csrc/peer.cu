// Token all-to-all-v over NVLink peer memory: the rows of global_scatter /
// global_gather are stored straight into the destination GPU's memory by a copy
// kernel, with no NCCL send/receive pairs and no staging pass on the sender.
//
// Same data movement as cuda/global_exchange.cuh:75-124 of the reference (which
// issues one ncclSend/ncclRecv per expert and peer and needs the counts on the host);
// the row layout on both sides is the reference's (expert-major, then source worker,
// bracketed by the rows kept local for shadowed workers).
//
// Every rank owns an allocation that its peers map through CUDA IPC:
//
//     [ header 4 MiB | slot 0 | slot 1 | receive pool ]
//
// The header holds flags, the count tables the ranks write into each other, and the
// exchange epochs.  Nothing of the protocol lives on the host: epochs are device words
// that the kernels advance themselves, and the row plan of an exchange is built ON THE
// DEVICE from the count table (peer_plan_kernel), so a layer's forward never has to read
// the counts back.
//
// Count exchange + plan (one block): every rank writes its local expert counts (and the
// row capacity of its expert-side buffers) into every peer's header, waits for the
// peers' tables, and derives from the full [W][W][E] table every rank's token-side
// offsets and expert-side layout, the row segments it has to push in either direction,
// and the offsets of its own experts' rows (what the grouped GEMM reads).  If any rank
// would receive more rows than it announced room for, every rank sees it (same table,
// same capacities): all plans become empty and bit 64 of the status word is raised.
//
// One exchange, numbered by an epoch that advances in step on all ranks (parity = epoch & 1):
//   1. push kernel: its first block ANNOUNCES where this rank wants its incoming rows (a byte
//      offset into its allocation, dest[parity][rank], then ann[parity][rank] = epoch, in every
//      peer's header); every block then waits for the announcements of all peers, stores this
//      rank's outgoing rows at the announced places at their final row offsets (rows that stay
//      on this GPU go straight to the output), and the last block to finish publishes
//      arrived[parity][rank] = epoch in every peer's header;
//   2. consume kernel: waits for arrived == epoch from every peer; nothing else when the
//      announced place was the output buffer itself, else it copies the rows that came from
//      peers out of the slot into the output.  Its last block advances the epoch word.
// The output buffer can be announced directly when it lies in the receive pool: the Python
// layer allocates exchange outputs there through a torch memory pool whose allocator is
// fmoe_pool_alloc/fmoe_pool_free below, so tensor lifetimes stay with torch's caching
// allocator.  Otherwise rows land in slot `parity` and are copied once more.  An announcement
// is made by a kernel that is stream-ordered after every earlier use of the announced memory
// on its GPU, and entry `parity` is rewritten two epochs later, after the peers have arrived
// for the epoch in between, so neither the memory nor the entry is overwritten while in use.
// A receiver whose landing place is too small announces a refusal instead: senders drop the
// rows for it and raise bit 64.
//
// All waits are bounded (wall-clock limit, FMOE_B200_PEER_TIMEOUT_MS, default
// 20000): when one expires the kernel raises bit 16 (no announcement / no count table) or
// 32 (rows not arrived) in the device status word and carries on, so that the stream
// drains; rows for a peer that never announced are dropped, not stored anywhere.
//
// The kernels of one communicator must be issued in one total order (one stream, or
// streams ordered by events): the epoch words are per communicator.
#include "common.cuh"
#include "exchange.h"
#include "gemm.h"
#include <cstdlib>
#include <cstring>
#include <iterator>
#include <map>
#include <mutex>
#include <vector>

namespace fmoe {
void pool_register(int device, char* base, size_t size);
void* pool_take(int device, size_t bytes);
void pool_give(int device, void* ptr, size_t bytes);
namespace {

// ---- header layout (byte offsets) ----------------------------------------------------------
constexpr int64_t kHeaderBytes = 4 << 20;
constexpr int kArrivedOff = 0;        // u64 [2][kMaxPeers]   rows of epoch e from rank p have landed
constexpr int kAnnOff = 1024;         // u64 [2][kMaxPeers]   rank p announced its landing place for epoch e
constexpr int kDestOff = 2048;        // u64 [2][kMaxPeers]   that place (byte offset in p's allocation)
constexpr int kCntFlagOff = 3072;     // u64 [2][kMaxPeers]   rank p's counts of count-exchange c are here
constexpr int kSeqOff = 4096;         // u64 [2]              own words: exchange epoch, count-exchange epoch
constexpr int kCapsOff = 5120;        // i64 [2][kMaxPeers]   expert-side row capacity of rank p
constexpr int kTableOff = 8192;       // i64 [2][kTableMax]   count tables [W][W*E]
constexpr int64_t kTableMax = ((1 << 20) - kTableOff) / 16;   // entries (W*W*E) per parity
constexpr int64_t kExpArrOff = 1 << 20;   // u64 [2][kMaxPeers][kArrivalExperts]: rows of (source p, this GPU's expert i) landed
static_assert(2 * kMaxPeers * kArrivalExperts * 8 <= (1 << 20), "arrival flags fit their MiB");
constexpr int64_t kCompatOff = 2 << 20;   // 2 MiB: uploaded table + flags + plan of the host-table entry points
constexpr int64_t kProbeBytes = 128 << 10;    // tail of that area: the empty plan of fmoe_peer_wait_probe
constexpr int64_t kCompatBytes = (2 << 20) - kProbeBytes;
static_assert(kArrivedOff + 2 * kMaxPeers * 8 <= kAnnOff && kCapsOff + 2 * kMaxPeers * 8 <= kTableOff, "flag arrays overlap");
constexpr unsigned long long kRefused = ~0ull;   // announcement of a receiver that has no room

constexpr int kLocal = 255;                 // destination of rows that stay on this GPU
enum { LIST_PUSH_FWD = 0, LIST_PULL_FWD = 1, LIST_PUSH_BWD = 2, LIST_PULL_BWD = 3 };

// ---- the plan as it lies in device memory -------------------------------------------------------
// Built by peer_plan_kernel, read by the exchange kernels (and, through own_offsets, by the
// grouped GEMM).  S = (2W-1)*E segment slots per list: (W-1)*E for rows kept local because their
// expert is shadowed here, then E groups of W slots, group i = local expert index i: first the rows
// of this rank's own expert i (they stay here), then the rows exchanged with the peers rank+1,
// rank+2, ... for their / this rank's expert i.  Expert-major order lets a consumer start on expert 0
// while later experts are still on their way; the ring order of the peers lets ranks that work in
// step store into different GPUs.  Slots without rows stay in the lists with rows = 0.
struct PlanHead {
    int32_t n_expert, n_workers, rank, n_slots;
    int32_t overflow, pad0;
    int64_t expert_rows, token_rows;      // rows of this rank's expert-side / token-side buffers
    int64_t max_expert_rows, max_token_rows;  // the largest of those over all ranks
};
struct PlanDims {
    int E, W, S;
    int64_t WE, T;        // W*E, W*W*E
    size_t own_off, table_off, stored_off, caps_off, eptr_off, lay_off, total_off, lists_off, segdone_off, done_off, back_off, bytes;
};
__host__ __device__ inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }
__host__ __device__ inline PlanDims plan_dims(int E, int W) {
    PlanDims d;
    d.E = E; d.W = W; d.S = (2 * W - 1) * E;
    d.WE = (int64_t)W * E; d.T = d.WE * W;
    size_t o = align_up(sizeof(PlanHead), 64);
    d.own_off = o;    o = align_up(o + (size_t)(E + 1) * 8, 64);          // i64 own_offsets[E+1]
    d.table_off = o;  o = align_up(o + (size_t)d.T * 8, 64);              // i64 table[W][W*E]
    d.stored_off = o; o = align_up(o + (size_t)d.WE, 64);                 // u8 stored[W*E]
    d.caps_off = o;   o = align_up(o + (size_t)W * 8, 64);                // i64 caps[W]
    d.eptr_off = o;   o = align_up(o + (size_t)W * (d.WE + 1) * 4, 64);   // i32 eptr[W][W*E+1]
    d.lay_off = o;    o = align_up(o + (size_t)W * (d.S + 1) * 4, 64);    // i32 lay[W][S+1]: expert-side scan of every rank
    d.total_off = o;  o = align_up(o + (size_t)W * 8, 64);
    d.lists_off = o;  o = align_up(o + (size_t)4 * (4 * (size_t)d.S + 1) * 4, 64);  // 4 x {prefix[S+1], sel[S], src[S], dst[S]}
    d.segdone_off = o; o = align_up(o + (size_t)d.S * 4, 64);             // i32 rows of each push segment stored so far (overlapped push)
    d.done_off = o;   o = align_up(o + (size_t)(4 * E + 16) * 4, 64);     // i32 done[2][E], expected[2][E], ready[2]: see GemmDone
    d.back_off = o;   o = align_up(o + (size_t)E * W * 4, 64);            // i32 [E][W]: token-side row, on rank j, of the rows it sent to this rank's expert i
    d.bytes = o;
    return d;
}
struct ListView { int* prefix; int* sel; int* src; int* dst; };
__host__ __device__ inline ListView list_view(char* plan, const PlanDims& d, int which) {
    int* base = (int*)(plan + d.lists_off) + (size_t)which * (4 * (size_t)d.S + 1);
    return ListView{base, base + d.S + 1, base + 2 * d.S + 1, base + 3 * d.S + 1};
}

// Position m of rank p's expert-side buffer order (the reference's layout, cuda/global_exchange.cuh:82-140):
//   m in [0, p*E):              rows p keeps for shadowed expert (j, i), j = m / E < p
//   m in [p*E, p*E + E*W):      rows from source j for p's expert i, (i, j) = divmod(m - p*E, W)
//   m in [p*E + E*W, (2W-1)*E): rows p keeps for shadowed expert (j, i), j > p
// Returns the row count of that position.
__device__ __forceinline__ int64_t lay_count(const int64_t* table, const unsigned char* stored, int p, int E, int W, int m) {
    const int64_t WE = (int64_t)W * E;
    if (m < p * E) return stored[m] ? table[p * WE + m] : 0;
    const int q = m - p * E;
    if (q < E * W) {
        const int i = q / W, j = q % W;
        if (stored[p * E + i] && j != p) return 0;
        return table[j * WE + p * E + i];
    }
    const int idx = (p + 1) * E + (q - E * W);
    return stored[idx] ? table[p * WE + idx] : 0;
}
__device__ __forceinline__ int lay_pos_recv(int p, int E, int W, int i, int j) { return p * E + i * W + j; }
__device__ __forceinline__ int lay_pos_shadow(int p, int E, int W, int idx) {      // idx = j*E + i, j != p
    return idx < p * E ? idx : idx - E + E * W;
}

__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(unsigned long long* p, unsigned long long v) {
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long now_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Waits until *flag >= want; gives up after timeout_ns (or 2^28 polls).
__device__ bool wait_flag(const unsigned long long* flag, unsigned long long want, unsigned long long timeout_ns) {
    if (ld_acquire_sys(flag) >= want) return true;
    const unsigned long long t0 = now_ns();
    for (unsigned it = 0; it < (1u << 28); ++it) {
        if (ld_acquire_sys(flag) >= want) return true;
        if (now_ns() - t0 > timeout_ns) return false;
        __nanosleep(256);
    }
    return false;
}

struct PeerBases { char* base[kMaxPeers]; };

// Exclusive scan by one warp over n values given by a functor; out[m] = sum of value(0..m-1),
// out[n] = total.  Returns the total (same on every lane).
template <typename F>
__device__ __forceinline__ int64_t warp_scan_store(int n, F value, int* out, int lane) {
    int64_t run = 0;
    for (int base = 0; base < n; base += 32) {
        const int m = base + lane;
        const int64_t v = m < n ? value(m) : 0;
        int64_t inc = v;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            const int64_t o = __shfl_up_sync(0xffffffffu, inc, off);
            if (lane >= off) inc += o;
        }
        if (m < n) out[m] = (int)(run + inc - v);
        run += __shfl_sync(0xffffffffu, inc, 31);
    }
    if (lane == 0) out[n] = (int)run;
    return run;
}

struct PlanArgs {
    int rank, world, n_expert;
    int exchange;                          // 1: swap counts through the peers' headers; 0: the table is given
    const int64_t* lec;                    // exchange: this rank's counts [W*E]
    const int64_t* table_in;               // else: the full table [W][W*E]
    const unsigned char* stored_in;        // [W*E] or null (nothing shadowed)
    const int64_t* caps_in;                // given table: capacities [W] or null (unlimited)
    int64_t cap_rows;                      // exchange: this rank's capacity (< 0: unlimited)
    unsigned long long timeout_ns;
    int* status;
    char* plan;
};

__global__ void __launch_bounds__(256)
peer_plan_kernel(const __grid_constant__ PeerBases b, const __grid_constant__ PlanArgs a) {
    const int E = a.n_expert, W = a.world, r = a.rank;
    const PlanDims d = plan_dims(E, W);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, n_warps = blockDim.x >> 5;
    PlanHead* head = (PlanHead*)a.plan;
    int64_t* own = (int64_t*)(a.plan + d.own_off);
    int64_t* table = (int64_t*)(a.plan + d.table_off);
    unsigned char* stored = (unsigned char*)(a.plan + d.stored_off);
    int64_t* caps = (int64_t*)(a.plan + d.caps_off);
    int* eptr = (int*)(a.plan + d.eptr_off);
    int* lay = (int*)(a.plan + d.lay_off);
    int64_t* total = (int64_t*)(a.plan + d.total_off);
    __shared__ int s_bad;
    if (tid == 0) s_bad = 0;

    // ---- 1. the full count table -----------------------------------------------------------
    if (a.exchange) {
        unsigned long long* hdr = (unsigned long long*)b.base[r];
        const unsigned long long c = __ldcg(hdr + kSeqOff / 8 + 1) + 1;
        const int par = (int)(c & 1);
        for (int64_t t = tid; t < (int64_t)W * d.WE; t += blockDim.x) {     // (peer, idx): my counts into everyone's table
            const int p = (int)(t / d.WE);
            const int64_t idx = t % d.WE;
            int64_t* dst = (int64_t*)(b.base[p] + kTableOff) + (int64_t)par * kTableMax + (int64_t)r * d.WE + idx;
            *dst = a.lec[idx];
        }
        if (tid < W) ((int64_t*)(b.base[tid] + kCapsOff))[par * kMaxPeers + r] = a.cap_rows;
        __threadfence_system();
        __syncthreads();
        if (tid < W && tid != r)
            st_release_sys((unsigned long long*)(b.base[tid] + kCntFlagOff) + par * kMaxPeers + r, c);
        if (tid < W && tid != r) {
            if (!wait_flag(hdr + kCntFlagOff / 8 + par * kMaxPeers + tid, c, a.timeout_ns)) {
                atomicOr(a.status, 16);
                s_bad = 1;
            }
        }
        __syncthreads();
        const int64_t* src = (const int64_t*)(b.base[r] + kTableOff) + (int64_t)par * kTableMax;
        for (int64_t t = tid; t < d.T; t += blockDim.x) table[t] = __ldcg(src + t);
        if (tid < W) caps[tid] = __ldcg((const int64_t*)(b.base[r] + kCapsOff) + par * kMaxPeers + tid);
        if (tid == 0) hdr[kSeqOff / 8 + 1] = c;
    } else {
        for (int64_t t = tid; t < d.T; t += blockDim.x) table[t] = a.table_in[t];
        if (tid < W) caps[tid] = a.caps_in ? a.caps_in[tid] : -1;
    }
    for (int64_t t = tid; t < d.WE; t += blockDim.x) stored[t] = a.stored_in ? a.stored_in[t] : 0;
    __syncthreads();
    // counts must be sane before they become row offsets
    for (int64_t t = tid; t < d.T; t += blockDim.x)
        if (table[t] < 0 || table[t] >= ((int64_t)1 << 31)) s_bad = 1;
    __syncthreads();

    // ---- 2. token-side offsets and expert-side layout of every rank (one warp per rank) -------
    for (int p = warp; p < W; p += n_warps) {
        const int64_t* row = table + (int64_t)p * d.WE;
        const int64_t tok = warp_scan_store((int)d.WE, [&](int m) { return row[m]; }, eptr + (size_t)p * (d.WE + 1), lane);
        const int64_t ex = warp_scan_store(d.S, [&](int m) { return lay_count(table, stored, p, E, W, m); },
                                           lay + (size_t)p * (d.S + 1), lane);
        if (lane == 0) {
            total[p] = ex;
            if (tok >= ((int64_t)1 << 31) || ex >= ((int64_t)1 << 31)) s_bad = 1;
            if (caps[p] >= 0 && ex > caps[p]) { s_bad = 1; atomicOr(a.status, 64); }
        }
    }
    __syncthreads();
    const bool bad = s_bad != 0;

    // ---- 3. this rank's segments --------------------------------------------------------------
    const int64_t* mine = table + (int64_t)r * d.WE;
    const int* my_eptr = eptr + (size_t)r * (d.WE + 1);
    const int* my_lay = lay + (size_t)r * (d.S + 1);
    ListView L[4];
    for (int w = 0; w < 4; ++w) L[w] = list_view(a.plan, d, w);
    // the row counts are staged in the prefix arrays first and scanned in place afterwards
    for (int s = tid; s < d.S; s += blockDim.x) {
        int sel = kLocal, tok = 0, ex = 0;
        int64_t rows_pf = 0, rows_lf = 0, rows_pb = 0, rows_lb = 0;   // push fwd, pull fwd, push bwd, pull bwd
        int src_pb = 0, dst_pb = 0, src_lf = 0, src_lb = 0;
        if (s < (W - 1) * E) {                      // rows kept here for a shadowed expert of another rank
            const int idx = s < r * E ? s : s + E;
            tok = my_eptr[idx];
            ex = my_lay[lay_pos_shadow(r, E, W, idx)];
            rows_pf = rows_pb = stored[idx] ? mine[idx] : 0;
            src_pb = ex; dst_pb = tok;
        } else if ((s - (W - 1) * E) % W == 0) {    // rows for this rank's own expert i
            const int i = (s - (W - 1) * E) / W, idx = r * E + i;
            tok = my_eptr[idx];
            ex = my_lay[lay_pos_recv(r, E, W, i, r)];
            rows_pf = rows_pb = mine[idx];
            src_pb = ex; dst_pb = tok;
        } else {                                    // rows exchanged with peer p for expert i (of p outbound, of r inbound)
            const int q = s - (W - 1) * E, i = q / W, dlt = q % W, p = (r + dlt) % W;
            sel = p;
            const int out_idx = p * E + i;          // my rows for expert i of rank p
            const int64_t out_rows = stored[out_idx] ? 0 : mine[out_idx];
            const int64_t in_rows = stored[r * E + i] ? 0 : table[(int64_t)p * d.WE + r * E + i];
            tok = my_eptr[out_idx];
            ex = (lay + (size_t)p * (d.S + 1))[lay_pos_recv(p, E, W, i, r)];      // where they sit in p's expert-side buffer
            rows_pf = out_rows;                                                   // forward push: tok (mine) -> ex (p's)
            rows_lb = out_rows;                                                   // backward pull: they come back to tok
            const int my_ex = my_lay[lay_pos_recv(r, E, W, i, p)];                // p's rows in my expert-side buffer
            const int p_tok = (eptr + (size_t)p * (d.WE + 1))[r * E + i];         // and in p's token-side buffer
            rows_lf = in_rows;                                                    // forward pull: slot[my_ex] -> out[my_ex]
            rows_pb = in_rows;                                                    // backward push: my_ex (mine) -> p_tok (p's)
            src_pb = my_ex; dst_pb = p_tok;
            src_lf = my_ex; src_lb = tok;
        }
        L[LIST_PUSH_FWD].sel[s] = sel; L[LIST_PUSH_FWD].src[s] = tok;    L[LIST_PUSH_FWD].dst[s] = ex;
        L[LIST_PUSH_BWD].sel[s] = sel; L[LIST_PUSH_BWD].src[s] = src_pb; L[LIST_PUSH_BWD].dst[s] = dst_pb;
        L[LIST_PULL_FWD].sel[s] = kLocal; L[LIST_PULL_FWD].src[s] = src_lf; L[LIST_PULL_FWD].dst[s] = src_lf;
        L[LIST_PULL_BWD].sel[s] = kLocal; L[LIST_PULL_BWD].src[s] = src_lb; L[LIST_PULL_BWD].dst[s] = src_lb;
        if (bad) rows_pf = rows_lf = rows_pb = rows_lb = 0;
        L[LIST_PUSH_FWD].prefix[s] = (int)rows_pf; L[LIST_PULL_FWD].prefix[s] = (int)rows_lf;
        L[LIST_PUSH_BWD].prefix[s] = (int)rows_pb; L[LIST_PULL_BWD].prefix[s] = (int)rows_lb;
    }
    __syncthreads();
    // in-place exclusive scans: one warp per list (each lane reads its count before it writes its prefix)
    for (int w = warp; w < 4; w += n_warps) {
        int* pre = L[w].prefix;
        int64_t run = 0;
        for (int base = 0; base < d.S; base += 32) {
            const int m = base + lane;
            const int64_t v = m < d.S ? pre[m] : 0;
            int64_t inc = v;
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
                const int64_t o = __shfl_up_sync(0xffffffffu, inc, off);
                if (lane >= off) inc += o;
            }
            __syncwarp();
            if (m < d.S) pre[m] = (int)(run + inc - v);
            run += __shfl_sync(0xffffffffu, inc, 31);
        }
        if (lane == 0) pre[d.S] = (int)run;
    }
    for (int s = tid; s < d.S; s += blockDim.x) ((int*)(a.plan + d.segdone_off))[s] = 0;
    for (int s = tid; s < 4 * E + 16; s += blockDim.x) ((int*)(a.plan + d.done_off))[s] = 0;
    for (int s = tid; s < E * W; s += blockDim.x) {
        const int i = s / W, j = s % W;
        ((int*)(a.plan + d.back_off))[s] = (eptr + (size_t)j * (d.WE + 1))[r * E + i];
    }
    // ---- 4. what the GEMM and the host read ----------------------------------------------------
    for (int i = tid; i <= E; i += blockDim.x)
        own[i] = bad ? 0 : (int64_t)my_lay[i < E ? lay_pos_recv(r, E, W, i, 0) : r * E + E * W];
    if (tid == 0) {
        head->n_expert = E; head->n_workers = W; head->rank = r; head->n_slots = d.S;
        head->overflow = bad ? 1 : 0; head->pad0 = 0;
        head->expert_rows = bad ? 0 : total[r];
        head->token_rows = bad ? 0 : (int64_t)my_eptr[d.WE];
        int64_t me = 0, mt = 0;
        for (int p = 0; p < W; ++p) {
            me = max(me, total[p]);
            mt = max(mt, (int64_t)(eptr + (size_t)p * (d.WE + 1))[d.WE]);
        }
        head->max_expert_rows = me; head->max_token_rows = mt;
    }
}

struct MoveArgs {
    int rank, world, dir;                  // dir 0: global_scatter (token -> expert side), 1: global_gather
    int direct;                            // rows land in the output buffer itself (it lies in the receive pool)
    int probe;                             // waits for an epoch nobody will publish; touches no state
    unsigned long long my_dest;            // push: byte offset of the landing place in this rank's allocation (direct)
    int64_t slot_bytes, row_bytes;
    int64_t in_rows, out_rows;             // rows of the buffers given to this call
    unsigned long long timeout_ns;
    unsigned int* counter;
    int* status;
    const char* plan;
    const int64_t* row_of;                 // push of rows that are not stored anywhere yet: token-side row i is
    const void* row_scale;                 //   row_scale[row_of[i]] * src[row_of[i] / row_div] (no scale: a plain copy)
    int row_div, row_dtype;
    int64_t src_rows;
    int* done;                             // overlapped gather: per-expert completion counters of the producing GEMM,
    int* expected;                         //   the counts at which an expert is complete,
    int* ready;                            //   and the word that says those counts are valid
};

// Row `row` of a list -> its segment, by bisection of the prefix array in shared memory.
__device__ __forceinline__ int find_seg(const int* prefix, int n, int row) {
    int lo = 0, hi = n - 1;        // last segment whose prefix <= row
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (prefix[mid] <= row) lo = mid; else hi = mid - 1;
    }
    return lo;
}

__device__ __forceinline__ void copy_row(const uint4* __restrict__ s, uint4* __restrict__ d, int64_t row_vecs, int lane) {
    // Rows in a slot were written by other GPUs while this kernel may already have been running:
    // read through L2 (ld.cg), never through the non-coherent path.
    int64_t c = lane;
    for (; c + 96 < row_vecs; c += 128) {
        const uint4 v0 = __ldcg(s + c), v1 = __ldcg(s + c + 32), v2 = __ldcg(s + c + 64), v3 = __ldcg(s + c + 96);
        d[c] = v0; d[c + 32] = v1; d[c + 64] = v2; d[c + 96] = v3;
    }
    for (; c < row_vecs; c += 32) d[c] = __ldcg(s + c);
}

// d[...] = w * s[...] in the rows' own type: one rounding per element, as a kernel that stored the
// scaled rows first would have produced them.
template <typename T>
__device__ __forceinline__ void copy_row_scaled_t(const uint4* __restrict__ s, uint4* __restrict__ d, int64_t row_vecs, int lane, float w) {
    constexpr int N = 16 / sizeof(T);
    for (int64_t c = lane; c < row_vecs; c += 32) {
        uint4 v = __ldcg(s + c);
        T* e = reinterpret_cast<T*>(&v);
#pragma unroll
        for (int i = 0; i < N; ++i) e[i] = from_float<T>(w * to_float<T>(e[i]));
        d[c] = v;
    }
}

__device__ __forceinline__ float scale_at(const void* scale, int dtype, int64_t i) {
    if (dtype == FMOE_F32) return ((const float*)scale)[i];
    if (dtype == FMOE_F16) return __half2float(((const __half*)scale)[i]);
    return __bfloat162float(((const __nv_bfloat16*)scale)[i]);
}

__device__ __forceinline__ void copy_row_scaled(const uint4* __restrict__ s, uint4* __restrict__ d, int64_t row_vecs, int lane, float w, int dtype) {
    if (dtype == FMOE_F32) copy_row_scaled_t<float>(s, d, row_vecs, lane, w);
    else if (dtype == FMOE_F16) copy_row_scaled_t<__half>(s, d, row_vecs, lane, w);
    else copy_row_scaled_t<__nv_bfloat16>(s, d, row_vecs, lane, w);
}

constexpr int kMoveThreads = 256, kMoveWarps = kMoveThreads / 32;

template <bool kPush>
__global__ void __launch_bounds__(kMoveThreads)
peer_move_kernel(const __grid_constant__ PeerBases b, const __grid_constant__ MoveArgs a, const uint4* __restrict__ src,
                 uint4* __restrict__ out) {
    extern __shared__ int s_prefix[];                // [S + 1]
    __shared__ int s_last;
    __shared__ unsigned long long s_dest[kMaxPeers];
    __shared__ unsigned long long s_dead;            // peers that get no rows: never announced, or refused
    const PlanHead* head = (const PlanHead*)a.plan;
    const PlanDims d = plan_dims(head->n_expert, head->n_workers);
    const ListView L = list_view(const_cast<char*>(a.plan), d, (kPush ? LIST_PUSH_FWD : LIST_PULL_FWD) + 2 * a.dir);
    unsigned long long* hdr = (unsigned long long*)b.base[a.rank];
    const unsigned long long epoch = __ldcg(hdr + kSeqOff / 8) + 1 + (a.probe ? (1ull << 40) : 0ull);
    const int parity = (int)(epoch & 1);
    const int64_t row_vecs = a.row_bytes / 16;
    // what this rank receives in this exchange and whether the place it was given can hold it
    const int64_t recv_rows = a.dir == 0 ? head->expert_rows : head->token_rows;
    const int64_t send_rows = a.dir == 0 ? head->token_rows : head->expert_rows;
    const bool room = recv_rows <= a.out_rows && send_rows <= a.in_rows &&
                      (a.direct || recv_rows * a.row_bytes <= a.slot_bytes);
    for (int i = threadIdx.x; i <= d.S; i += kMoveThreads) s_prefix[i] = L.prefix[i];
    if (threadIdx.x == 0) s_dead = 0ull;
    __syncthreads();
    {
        const int p = threadIdx.x;
        if (p < a.world && p != a.rank) {
            if (kPush) {
                if (blockIdx.x == 0 && !a.probe) {
                    unsigned long long* peer_hdr = (unsigned long long*)b.base[p];
                    const unsigned long long place = !room ? kRefused
                        : a.direct ? a.my_dest : (unsigned long long)(kHeaderBytes + (int64_t)parity * a.slot_bytes);
                    peer_hdr[kDestOff / 8 + parity * kMaxPeers + a.rank] = place;
                    st_release_sys(peer_hdr + kAnnOff / 8 + parity * kMaxPeers + a.rank, epoch);
                }
                // Where peer p wants its rows.  Without an announcement of this epoch the word holds
                // an older epoch's address (or nothing), so rows for that peer are dropped, not stored.
                const bool announced = wait_flag(hdr + kAnnOff / 8 + parity * kMaxPeers + p, epoch, a.timeout_ns);
                const unsigned long long dest = __ldcg(hdr + kDestOff / 8 + parity * kMaxPeers + p);
                s_dest[p] = dest;
                if (!announced) { atomicOr(a.status, 16); atomicOr(&s_dead, 1ull << p); }
                else if (dest == kRefused || dest < (unsigned long long)kHeaderBytes) { atomicOr(a.status, 64); atomicOr(&s_dead, 1ull << p); }
            } else {           // everyone's rows of this epoch must have landed
                if (!wait_flag(hdr + kArrivedOff / 8 + parity * kMaxPeers + p, epoch, a.timeout_ns)) atomicOr(a.status, 32);
            }
        }
        if (kPush && threadIdx.x == 0 && blockIdx.x == 0 && !room) atomicOr(a.status, 64);
        __syncthreads();
    }
    const int lane = threadIdx.x & 31;
    // without room nothing moves, not even the local rows; rows that landed in the output itself need no copy
    const int total = (!room || (!kPush && a.direct)) ? 0 : s_prefix[d.S];
    const uint4* slot = (const uint4*)(b.base[a.rank] + kHeaderBytes + (int64_t)parity * a.slot_bytes);
    for (int row = blockIdx.x * kMoveWarps + (threadIdx.x >> 5); row < total; row += gridDim.x * kMoveWarps) {
        const int k = find_seg(s_prefix, d.S, row), off = row - s_prefix[k];
        const uint4* s;
        uint4* dptr;
        if (kPush) {
            const int sel = L.sel[k];
            if (sel != kLocal && ((s_dead >> sel) & 1ull)) continue;
            dptr = (sel == kLocal ? out : (uint4*)(b.base[sel] + s_dest[sel])) + (int64_t)(L.dst[k] + off) * row_vecs;
            if (a.row_of) {
                // the token-side row is produced here: a row of src picked by index, scaled or not
                const int64_t at = __ldg(a.row_of + L.src[k] + off), from = at / a.row_div;
                if (at < 0 || from >= a.src_rows) { if (lane == 0) atomicOr(a.status, 8); continue; }
                s = src + from * row_vecs;
                if (a.row_scale) {
                    copy_row_scaled(s, dptr, row_vecs, lane, scale_at(a.row_scale, a.row_dtype, at), a.row_dtype);
                    continue;
                }
            } else {
                s = src + (int64_t)(L.src[k] + off) * row_vecs;
            }
        } else {
            s = slot + (int64_t)(L.src[k] + off) * row_vecs;
            dptr = out + (int64_t)(L.dst[k] + off) * row_vecs;
        }
        copy_row(s, dptr, row_vecs, lane);
    }
    if (!kPush && a.dir == 1 && !a.probe) {
        // global_gather's contract: token-side rows past the ones the counts describe are zero
        const int64_t first = room ? head->token_rows : 0;
        for (int64_t row = first + blockIdx.x * kMoveWarps + (threadIdx.x >> 5); row < a.out_rows; row += (int64_t)gridDim.x * kMoveWarps)
            for (int64_t c = lane; c < row_vecs; c += 32) out[row * row_vecs + c] = make_uint4(0, 0, 0, 0);
    }
    if (a.probe) return;
    // The last block to finish publishes (push: the rows have landed; consume: the epoch is over).
    // All of a block's stores are ordered before thread 0's fence by the barrier, and the fence is
    // cumulative: one fence per block publishes them.
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();
        s_last = atomicAdd(a.counter + (kPush ? 0 : 1), 1u) == gridDim.x - 1;
    }
    __syncthreads();
    if (s_last) {
        __threadfence_system();
        if (kPush) {
            const int p = threadIdx.x;
            if (p < a.world && p != a.rank)
                st_release_sys((unsigned long long*)b.base[p] + kArrivedOff / 8 + parity * kMaxPeers + a.rank, epoch);
        } else if (threadIdx.x == 0) {
            hdr[kSeqOff / 8] = epoch;
        }
        if (threadIdx.x == 0) a.counter[kPush ? 0 : 1] = 0;
    }
}

// ---- push that runs beside the consumer of its rows ---------------------------------------------
// The same protocol as peer_move_kernel<true> for global_scatter, shaped to run on a few SMs while a
// grouped GEMM occupies the others and starts on an expert's rows as soon as they are complete:
//   * a warp moves units of kUnitRows consecutive rows of the push list (expert-major order);
//   * every segment = rows of one (destination, expert); when its last row has been stored, the warp
//     that stored it publishes flag[parity][this rank][expert] = epoch in the destination's landing
//     area (this GPU's own for rows that stay); segments without rows are published at once;
//   * the last block publishes the whole-exchange `arrived` flags as the plain push does, so the
//     consume step that closes the epoch is unchanged.
constexpr int kUnitRows = 32, kPushThreads = 1024, kPushWarps = kPushThreads / 32;

// n consecutive rows of a contiguous block.  The block is moved in pieces of 512 bytes per warp
// (one 16-byte load per lane) and eight pieces are in flight per lane before the first store is
// issued -- a warp is latency-bound otherwise, all the more while a GEMM on the other SMs keeps
// the memory system busy.  (Rows of a segment are contiguous on both sides, so the block is too.)
__device__ __forceinline__ void copy_rows(const uint4* __restrict__ s, uint4* __restrict__ d, int n, int64_t row_vecs, int lane) {
    const int64_t vecs = (int64_t)n * row_vecs;
    int64_t c = lane;
    for (; c + 7 * 32 < vecs; c += 8 * 32) {
        uint4 v[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = __ldcg(s + c + 32 * i);
#pragma unroll
        for (int i = 0; i < 8; ++i) d[c + 32 * i] = v[i];
    }
    for (; c < vecs; c += 32) d[c] = __ldcg(s + c);
}

__device__ __forceinline__ void publish_segment(const PeerBases& b, const MoveArgs& a, int W, int E, int s, int parity,
                                                unsigned long long epoch) {
    if (s < (W - 1) * E) return;                                  // rows kept for shadowed experts: not used in this mode
    const int q = s - (W - 1) * E, i = q / W, p = (a.rank + q % W) % W;
    if (i >= kArrivalExperts) return;
    unsigned long long* flag = (unsigned long long*)(b.base[p] + kExpArrOff) + ((size_t)parity * kMaxPeers + a.rank) * kArrivalExperts + i;
    st_release_sys(flag, epoch);
}

__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// Bounded wait until the GEMM that produces this GPU's expert-side rows has stored all rows of expert i.
__device__ bool wait_expert_done(const MoveArgs& a, int i) {
    const unsigned long long t0 = now_ns();
    for (unsigned it = 0; it < (1u << 28); ++it) {
        if (ld_acquire_gpu(a.ready) != 0 && ld_acquire_gpu(a.done + i) >= ld_acquire_gpu(a.expected + i)) return true;
        if (now_ns() - t0 > a.timeout_ns) return false;
        __nanosleep(200);
    }
    return false;
}

// kGather = false: global_scatter whose rows a GEMM on this GPU's peers consumes as they land (see above).
// kGather = true:  global_gather whose rows a GEMM on THIS GPU is still producing: a unit of rows is
//   moved once the expert it belongs to is complete (per-expert counters that the GEMM's epilogue
//   advances, GemmDone); the receivers wait for the whole exchange as usual.
template <bool kGather>
__global__ void __launch_bounds__(kPushThreads, 1)
peer_push_overlap_kernel(const __grid_constant__ PeerBases b, const __grid_constant__ MoveArgs a, const uint4* __restrict__ src,
                         uint4* __restrict__ out) {
    extern __shared__ int s_prefix[];                // [S + 1]
    __shared__ int s_last;
    __shared__ unsigned long long s_dest[kMaxPeers];
    __shared__ unsigned long long s_dead;
    const PlanHead* head = (const PlanHead*)a.plan;
    const int E = head->n_expert, W = head->n_workers;
    const PlanDims d = plan_dims(E, W);
    const ListView L = list_view(const_cast<char*>(a.plan), d, kGather ? LIST_PUSH_BWD : LIST_PUSH_FWD);
    int* seg_done = (int*)(const_cast<char*>(a.plan) + d.segdone_off);
    unsigned long long* hdr = (unsigned long long*)b.base[a.rank];
    const unsigned long long epoch = __ldcg(hdr + kSeqOff / 8) + 1;
    const int parity = (int)(epoch & 1);
    const int64_t row_vecs = a.row_bytes / 16;
    // (the output lies in the receive pool: no slot is involved)
    const bool room = kGather ? (head->token_rows <= a.out_rows && head->expert_rows <= a.in_rows)
                              : (head->expert_rows <= a.out_rows && head->token_rows <= a.in_rows);
    for (int i = threadIdx.x; i <= d.S; i += kPushThreads) s_prefix[i] = L.prefix[i];
    if (threadIdx.x == 0) s_dead = 0ull;
    __syncthreads();
    {
        const int p = threadIdx.x;
        if (p < W && p != a.rank) {
            if (blockIdx.x == 0) {
                unsigned long long* peer_hdr = (unsigned long long*)b.base[p];
                peer_hdr[kDestOff / 8 + parity * kMaxPeers + a.rank] = room ? a.my_dest : kRefused;
                st_release_sys(peer_hdr + kAnnOff / 8 + parity * kMaxPeers + a.rank, epoch);
            }
            const bool announced = wait_flag(hdr + kAnnOff / 8 + parity * kMaxPeers + p, epoch, a.timeout_ns);
            const unsigned long long dest = __ldcg(hdr + kDestOff / 8 + parity * kMaxPeers + p);
            s_dest[p] = dest;
            if (!announced) { atomicOr(a.status, 16); atomicOr(&s_dead, 1ull << p); }
            else if (dest == kRefused || dest < (unsigned long long)kHeaderBytes) { atomicOr(a.status, 64); atomicOr(&s_dead, 1ull << p); }
        }
        if (threadIdx.x == 0 && blockIdx.x == 0 && !room) atomicOr(a.status, 64);
        __syncthreads();
    }
    const int total = room ? s_prefix[d.S] : 0;
    if (!kGather && room && blockIdx.x == 0)          // nothing will ever be stored for these: their consumers need not wait
        for (int s = (W - 1) * E + threadIdx.x; s < d.S; s += kPushThreads)
            if (s_prefix[s + 1] == s_prefix[s]) publish_segment(b, a, W, E, s, parity, epoch);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    // Units of rows are dealt to the moving warps round-robin, so at any time all of them work on one
    // stretch of the list; a stretch should be about one expert's rows, so that experts complete one
    // after the other.
    //   gather:  all 32 warps of a block move rows; nothing is published per segment.
    //   scatter: warps 0..30 move rows and never wait for their stores; warp 31 publishes.  A mover that
    //     has issued the stores of its unit of round r bumps the round's counter in shared memory.  The
    //     publisher takes all rounds that every mover has finished, issues ONE system fence for them --
    //     their stores are ordered before it through the counters, and the fence is cumulative --
    //     books their rows per segment and raises the flags of the segments that are complete.  The
    //     fence waits for the stores in flight (10+ microseconds on a busy link), but only the
    //     publisher waits: the movers may run kRing rounds ahead of what it has taken.
    constexpr int kMovers = kGather ? kPushWarps : kPushWarps - 1;
    constexpr int kRing = 16;
    __shared__ int s_issued[kRing];                   // movers that have finished round r (slot r % kRing)
    __shared__ int s_taken;                           // rounds the publisher has taken
    if (threadIdx.x < kRing) s_issued[threadIdx.x] = 0;
    if (threadIdx.x == 0) s_taken = 0;
    __syncthreads();
    const int movers_total = (int)gridDim.x * kMovers;
    const int unit_rows = max(4, min(kUnitRows, total / max(1, E * movers_total)));
    const int n_units = (total + unit_rows - 1) / unit_rows;
    const int n_rounds = (n_units + movers_total - 1) / movers_total;
    if (kGather || warp < kMovers) {
        int done_expert = -1;                             // kGather: the expert this warp saw complete last
        bool gave_up = false;
        for (int r = 0; r < n_rounds; ++r) {
            if (!kGather && r >= kRing) {                 // the ring slot of round r must have been taken
                if (lane == 0) {
                    unsigned spins = 0;
                    while (*(volatile int*)&s_taken + kRing <= r) {
                        __nanosleep(100);
                        if (++spins > (1u << 24)) { atomicOr(a.status, 32); break; }    // never seen: do not hang
                    }
                }
                __syncwarp();
            }
            const int u = r * movers_total + (int)blockIdx.x * kMovers + warp;
            int row = u * unit_rows;
            const int row_end = u < n_units ? min(row + unit_rows, total) : row;
            int k = row < row_end ? find_seg(s_prefix, d.S, row) : 0;
            while (row < row_end) {
                const int n = min(row_end, s_prefix[k + 1]) - row;
                const int sel = L.sel[k];
                bool dead = sel != kLocal && ((s_dead >> sel) & 1ull);
                if (kGather && k >= (W - 1) * E) {
                    const int i = (k - (W - 1) * E) / W;
                    if (i != done_expert && !gave_up) {
                        int ok = 1;
                        if (lane == 0) ok = wait_expert_done(a, i) ? 1 : 0;
                        ok = __shfl_sync(0xffffffffu, ok, 0);
                        if (ok) done_expert = i;
                        else { gave_up = true; if (lane == 0) atomicOr(a.status, 32); }
                    }
                    dead = dead || gave_up;               // rows that were never produced are not forwarded
                }
                if (!dead) {
                    const uint4* sp = src + (int64_t)(L.src[k] + (row - s_prefix[k])) * row_vecs;
                    uint4* dptr = (sel == kLocal ? out : (uint4*)(b.base[sel] + s_dest[sel])) + (int64_t)(L.dst[k] + (row - s_prefix[k])) * row_vecs;
                    copy_rows(sp, dptr, n, row_vecs, lane);
                }
                row += n;
                ++k;
                while (k < d.S && s_prefix[k + 1] == s_prefix[k]) ++k;
            }
            if (!kGather) {
                __syncwarp();
                if (lane == 0) { __threadfence_block(); atomicAdd(&s_issued[r % kRing], 1); }
            }
        }
    } else {
        int next = 0;
        unsigned idle = 0;
        while (next < n_rounds) {
            if (idle > (1u << 24)) { if (lane == 0) atomicOr(a.status, 32); break; }            // never seen: do not hang
            // rounds [next, hi) have been finished by every mover (rounds complete in order per mover, so a
            // full counter of round r implies nothing about r+1: check them one by one)
            int hi = next;
            if (lane == 0) {
                while (hi < n_rounds && hi < next + kRing && *(volatile int*)&s_issued[hi % kRing] == kMovers) ++hi;
                if (hi == next) __nanosleep(200);
            }
            hi = __shfl_sync(0xffffffffu, hi, 0);
            if (hi == next) { ++idle; continue; }
            idle = 0;
            __threadfence_block();
            __threadfence_system();
            // lanes book the units of the taken rounds
            for (int idx = lane; idx < (hi - next) * kMovers; idx += 32) {
                const int r = next + idx / kMovers, w = idx % kMovers;
                const int u = r * movers_total + (int)blockIdx.x * kMovers + w;
                if (u >= n_units) continue;
                int row = u * unit_rows;
                const int row_end = min(row + unit_rows, total);
                int k = find_seg(s_prefix, d.S, row);
                while (row < row_end) {
                    const int n = min(row_end, s_prefix[k + 1]) - row;
                    const int sel = L.sel[k];
                    const bool dead = sel != kLocal && ((s_dead >> sel) & 1ull);
                    const int before = atomicAdd(seg_done + k, n);
                    if (before + n == s_prefix[k + 1] - s_prefix[k] && !dead) {
                        __threadfence_system();       // the other blocks' shares of the segment were fenced before they were booked
                        publish_segment(b, a, W, E, k, parity, epoch);
                    }
                    row += n;
                    ++k;
                    while (k < d.S && s_prefix[k + 1] == s_prefix[k]) ++k;
                }
            }
            __syncwarp();
            if (lane == 0) {
                for (int r = next; r < hi; ++r) s_issued[r % kRing] = 0;
                __threadfence_block();
                *(volatile int*)&s_taken = hi;
            }
            __syncwarp();
            next = hi;
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();
        s_last = atomicAdd(a.counter, 1u) == gridDim.x - 1;
    }
    __syncthreads();
    if (s_last) {
        __threadfence_system();
        const int p = threadIdx.x;
        if (p < W && p != a.rank)
            st_release_sys((unsigned long long*)b.base[p] + kArrivedOff / 8 + parity * kMaxPeers + a.rank, epoch);
        // the plan may serve another exchange
        if (!kGather) for (int s = threadIdx.x; s < d.S; s += kPushThreads) seg_done[s] = 0;
        if (kGather) {
            for (int i = threadIdx.x; i < E; i += kPushThreads) a.done[i] = 0;
            if (threadIdx.x == 0) *a.ready = 0;
        }
        if (threadIdx.x == 0) a.counter[0] = 0;
    }
}

int launch_plan(Comm* c, int rank, int W, int E, bool exchange, const int64_t* lec, const int64_t* table,
                const uint8_t* stored, const int64_t* caps, int64_t cap_rows, void* plan, cudaStream_t st) {
    FMOE_REQUIRE(E > 0 && W > 0 && W <= kMaxPeers && rank >= 0 && rank < W, "peer plan: bad E=%d W=%d rank=%d", E, W, rank);
    FMOE_REQUIRE((int64_t)W * W * E <= kTableMax, "peer plan: W*W*E = %lld exceeds %lld", (long long)W * W * E, (long long)kTableMax);
    FMOE_REQUIRE(plan && ((uintptr_t)plan & 63) == 0, "peer plan: plan buffer must be 64-byte aligned");
    PeerBases b;
    memset(&b, 0, sizeof(b));
    PlanArgs a;
    memset(&a, 0, sizeof(a));
    a.rank = rank; a.world = W; a.n_expert = E; a.exchange = exchange ? 1 : 0;
    a.lec = lec; a.table_in = table; a.stored_in = stored; a.caps_in = caps; a.cap_rows = cap_rows;
    a.plan = (char*)plan;
    a.status = device_status_ptr();
    FMOE_REQUIRE(a.status, "peer plan: no device status word");
    if (exchange) {
        FMOE_REQUIRE(c && c->peer.slot_bytes > 0, "peer plan: the peer-memory exchange is off");
        for (int p = 0; p < kMaxPeers; ++p) b.base[p] = c->peer.base[p];
        a.timeout_ns = c->peer.timeout_ns;
    }
    peer_plan_kernel<<<1, 256, 0, st>>>(b, a);
    FMOE_CHECK_LAUNCH();
    return 0;
}

// Rows of a push that exist nowhere yet: see MoveArgs::row_of.
struct RowSource {
    const int64_t* row_of;
    int div;
    const void* scale;
    int dtype;
    int64_t src_rows;
};

int launch_move(Comm* c, const void* in, void* out, const void* plan, int E, int64_t in_rows, int64_t out_rows,
                int64_t row_bytes, bool reverse, cudaStream_t st, int phases = 3, int overlap_sms = 0, int done_use = 0,
                const RowSource* rows = nullptr);

bool lies_in_pool(Comm* c, const void* out, int64_t bytes) {
    char* pool = c->peer.base[c->rank] + kHeaderBytes + 2 * c->peer.slot_bytes;
    return c->peer.pool_bytes > 0 && (char*)out >= pool && (char*)out + bytes <= pool + c->peer.pool_bytes;
}

// phases: bit 0 = push, bit 1 = consume.  overlap_sms > 0 (push of a scatter into a pool buffer only):
// the few-SM push that publishes per-expert arrival flags.
int launch_move(Comm* c, const void* in, void* out, const void* plan, int E, int64_t in_rows, int64_t out_rows,
                int64_t row_bytes, bool reverse, cudaStream_t st, int phases, int overlap_sms, int done_use,
                const RowSource* rows) {
    FMOE_REQUIRE(row_bytes > 0 && row_bytes % 16 == 0, "peer exchange: row_bytes=%lld (a positive multiple of 16)", (long long)row_bytes);
    FMOE_REQUIRE(in_rows >= 0 && out_rows >= 0 && in_rows < ((int64_t)1 << 31) && out_rows < ((int64_t)1 << 31),
                 "peer exchange: rows in=%lld out=%lld", (long long)in_rows, (long long)out_rows);
    FMOE_REQUIRE((in || in_rows == 0 || !(phases & 1)) && (out || out_rows == 0) && plan, "peer exchange: null buffer");
    FMOE_REQUIRE((((uintptr_t)in | (uintptr_t)out) & 15) == 0, "peer exchange: buffers must be 16-byte aligned");
    PeerBases b;
    for (int p = 0; p < kMaxPeers; ++p) b.base[p] = c->peer.base[p];
    // Rows can land in the output itself when it lies in this rank's receive pool.
    char* pool = c->peer.base[c->rank] + kHeaderBytes + 2 * c->peer.slot_bytes;
    const int64_t recv_bytes = out_rows * row_bytes;
    const bool direct = c->peer.pool_bytes > 0 && (char*)out >= pool && (char*)out + recv_bytes <= pool + c->peer.pool_bytes;
    MoveArgs a;
    memset(&a, 0, sizeof(a));
    a.rank = c->rank; a.world = c->world; a.dir = reverse ? 1 : 0; a.direct = direct ? 1 : 0;
    a.my_dest = direct ? (unsigned long long)((char*)out - c->peer.base[c->rank]) : 0;
    a.slot_bytes = c->peer.slot_bytes; a.row_bytes = row_bytes; a.in_rows = in_rows; a.out_rows = out_rows;
    a.timeout_ns = c->peer.timeout_ns; a.counter = c->peer.counter; a.plan = (const char*)plan;
    a.status = device_status_ptr();
    FMOE_REQUIRE(a.status, "peer exchange: no device status word");
    if (rows) {
        FMOE_REQUIRE(!reverse && overlap_sms == 0 && rows->row_of && rows->div > 0 && rows->src_rows >= 0,
                     "peer exchange: indexed rows are for the plain scatter");
        a.row_of = rows->row_of; a.row_div = rows->div; a.row_scale = rows->scale; a.row_dtype = rows->dtype;
        a.src_rows = rows->src_rows;
    }
    const PlanDims d = plan_dims(E, c->world);
    const size_t smem = (size_t)(d.S + 1) * sizeof(int);
    FMOE_REQUIRE(smem <= 40 * 1024, "peer exchange: %d segment slots do not fit the kernels' shared memory", d.S);
    const int cap_blocks = sm_count() * 8;
    if ((phases & 1) && overlap_sms > 0) {
        FMOE_REQUIRE(direct, "peer exchange: the overlapped push needs an output in the receive pool");
        // clusters of two blocks: the push then occupies whole SM pairs and leaves the others to the
        // CTA pairs of the GEMM that runs beside it
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)((overlap_sms + 1) / 2 * 2));
        cfg.blockDim = dim3(kPushThreads);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = st;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        if (reverse) {
            const PlanDims pd = plan_dims(E, c->world);
            int* words = (int*)((char*)const_cast<void*>(plan) + pd.done_off);
            a.done = words + (size_t)done_use * E; a.expected = words + (size_t)(2 + done_use) * E; a.ready = words + 4 * (size_t)E + done_use;
            FMOE_CUDA_TRY(cudaLaunchKernelEx(&cfg, peer_push_overlap_kernel<true>, b, a, (const uint4*)in, (uint4*)out));
        } else {
            FMOE_CUDA_TRY(cudaLaunchKernelEx(&cfg, peer_push_overlap_kernel<false>, b, a, (const uint4*)in, (uint4*)out));
        }
    } else if (phases & 1) {
        const unsigned push_blocks = (unsigned)std::max<int64_t>(1, std::min<int64_t>(ceil_div(in_rows, kMoveWarps), cap_blocks));
        peer_move_kernel<true><<<push_blocks, kMoveThreads, smem, st>>>(b, a, (const uint4*)in, (uint4*)out);
        FMOE_CHECK_LAUNCH();
    }
    if (!(phases & 2)) return 0;
    // consume: one block when nothing has to be copied or cleared
    const bool work = !direct || reverse;
    // (direct + gather: only the usually empty tail of the token-side buffer may need clearing)
    const unsigned pull_blocks = !work ? 1u : direct ? 16u
        : (unsigned)std::max<int64_t>(1, std::min<int64_t>(ceil_div(out_rows, kMoveWarps), cap_blocks));
    peer_move_kernel<false><<<pull_blocks, kMoveThreads, smem, st>>>(b, a, nullptr, (uint4*)out);
    FMOE_CHECK_LAUNCH();
    return 0;
}

}  // namespace

// ---- receive pool: first-fit free list over one region per device ------------------------
namespace {
struct Pool {
    char* base = nullptr;
    size_t size = 0;
    std::map<size_t, size_t> free_;   // offset -> length, coalesced
};
Pool g_pool[64];
std::mutex g_pool_mtx;
constexpr size_t kPoolAlign = 512;
}  // namespace

void pool_register(int device, char* base, size_t size) {
    if (device < 0 || device >= 64) return;
    std::lock_guard<std::mutex> lk(g_pool_mtx);
    Pool& p = g_pool[device];
    p.base = base;
    p.size = size;
    p.free_.clear();
    if (base && size) p.free_[0] = size;
}

void* pool_take(int device, size_t bytes) {
    if (device < 0 || device >= 64) return nullptr;
    bytes = (bytes + kPoolAlign - 1) & ~(kPoolAlign - 1);
    std::lock_guard<std::mutex> lk(g_pool_mtx);
    Pool& p = g_pool[device];
    for (auto it = p.free_.begin(); it != p.free_.end(); ++it) {
        if (it->second < bytes) continue;
        const size_t off = it->first, len = it->second;
        p.free_.erase(it);
        if (len > bytes) p.free_[off + bytes] = len - bytes;
        return p.base + off;
    }
    return nullptr;
}

void pool_give(int device, void* ptr, size_t bytes) {
    if (device < 0 || device >= 64 || !ptr) return;
    bytes = (bytes + kPoolAlign - 1) & ~(kPoolAlign - 1);
    std::lock_guard<std::mutex> lk(g_pool_mtx);
    Pool& p = g_pool[device];
    if (!p.base || (char*)ptr < p.base || (char*)ptr + bytes > p.base + p.size) return;   // region already gone
    size_t off = (size_t)((char*)ptr - p.base), len = bytes;
    auto next = p.free_.lower_bound(off);
    if (next != p.free_.begin()) {
        auto prev = std::prev(next);
        if (prev->first + prev->second == off) { off = prev->first; len += prev->second; p.free_.erase(prev); }
    }
    if (next != p.free_.end() && off + len == next->first) { len += next->second; p.free_.erase(next); }
    p.free_[off] = len;
}

void peer_forget(Comm* c);

void peer_release(Comm* c) {
    PeerState& ps = c->peer;
    peer_forget(c);
    if (ps.slot_bytes == 0) return;
    cudaDeviceSynchronize();
    if (ps.pool_bytes) pool_register(c->device, nullptr, 0);
    ps.pool_bytes = 0;
    for (int p = 0; p < c->world && p < kMaxPeers; ++p) {
        if (!ps.base[p]) continue;
        if (p == c->rank) cudaFree(ps.base[p]);
        else cudaIpcCloseMemHandle(ps.base[p]);
        ps.base[p] = nullptr;
    }
    if (ps.counter) cudaFree(ps.counter);
    ps.counter = nullptr;
    if (ps.side) cudaStreamDestroy(ps.side);
    if (ps.fork) cudaEventDestroy(ps.fork);
    if (ps.join) cudaEventDestroy(ps.join);
    ps.side = nullptr; ps.fork = ps.join = nullptr;
    ps.slot_bytes = 0;
    (void)cudaGetLastError();
}

// ---- host mirror of the plan (no GPU): what the device builds, for inspection and tests -------
namespace {
struct Seg { int sel; int64_t src_row, dst_row, rows; };
struct Layout {
    std::vector<int64_t> off;     // [i + j * E]
    std::vector<int64_t> shadow;  // [j * E + i]: row of the block of rank p's own rows for shadowed expert (j, i)
    int64_t total = 0;
};

void expert_layout(const int64_t* table, const uint8_t* stored, int p, int E, int W, Layout& L) {
    const int64_t* lec = table + (int64_t)p * W * E;
    L.off.assign((size_t)E * W, -1);
    L.shadow.assign((size_t)E * W, -1);
    int64_t rp = 0;
    auto local_block = [&](int j) {
        for (int i = 0; i < E; ++i) {
            const int idx = i + j * E;
            if (stored[idx]) { L.shadow[idx] = rp; rp += lec[idx]; }
        }
    };
    for (int j = 0; j < p; ++j) local_block(j);
    for (int i = 0; i < E; ++i)
        for (int j = 0; j < W; ++j) {
            const int64_t g = table[((int64_t)j * W + p) * E + i];
            if (g > 0 && (!stored[p * E + i] || j == p)) { L.off[i + j * E] = rp; rp += g; }
        }
    for (int j = p + 1; j < W; ++j) local_block(j);
    L.total = rp;
}

struct Plan {
    std::vector<Seg> push, pull;
    int64_t slot_rows = 0, expert_rows = 0, token_rows = 0, max_rows = 0;
};

int plan_peer(const int64_t* table, const uint8_t* stored, int r, int E, int W, bool reverse, Plan& plan) {
    FMOE_REQUIRE(table && stored && E > 0 && W > 0 && r >= 0 && r < W, "peer exchange: bad argument");
    const size_t n = (size_t)W * E;
    for (size_t i = 0; i < n * W; ++i) FMOE_REQUIRE(table[i] >= 0, "peer exchange: negative count at %zu", i);
    std::vector<std::vector<int64_t>> eptr(W, std::vector<int64_t>(n + 1, 0));
    std::vector<Layout> lay(W);
    int64_t max_token = 0, max_expert = 0;
    for (int p = 0; p < W; ++p) {
        for (size_t i = 0; i < n; ++i) eptr[p][i + 1] = eptr[p][i] + table[(size_t)p * n + i];
        expert_layout(table, stored, p, E, W, lay[p]);
        max_token = std::max(max_token, eptr[p][n]);
        max_expert = std::max(max_expert, lay[p].total);
    }
    plan.slot_rows = reverse ? max_token : max_expert;
    plan.max_rows = std::max(max_token, max_expert);
    plan.expert_rows = lay[r].total;
    plan.token_rows = eptr[r][n];
    std::vector<Seg>& push = plan.push;
    std::vector<Seg>& pull = plan.pull;
    const int64_t* mine = table + (size_t)r * n;
    // rows that stay here: own rows of shadowed experts, and rows for this rank's own experts
    for (size_t idx = 0; idx < n; ++idx)
        if ((int)(idx / E) != r && stored[idx] && mine[idx] > 0) {
            const int64_t tok = eptr[r][idx], ex = lay[r].shadow[idx];
            push.push_back(reverse ? Seg{kLocal, ex, tok, mine[idx]} : Seg{kLocal, tok, ex, mine[idx]});
        }
    // Expert-major: the rows of this rank's own expert i, then the peers in the order r+1, r+2, ...:
    // ranks that work in step store into different GPUs at any moment, and every receiver's
    // experts fill up in ascending order.
    for (int i = 0; i < E; ++i) {
        const int64_t own_ex = lay[r].off[i + r * E];
        if (own_ex >= 0) {
            const int64_t tok = eptr[r][r * E + i], rows = mine[r * E + i];
            push.push_back(reverse ? Seg{kLocal, own_ex, tok, rows} : Seg{kLocal, tok, own_ex, rows});
        }
        for (int dlt = 1; dlt < W; ++dlt) {
            const int p = (r + dlt) % W;
            // rows this rank routes to expert i of rank p
            const int64_t out_rows_pi = mine[p * E + i];
            if (out_rows_pi > 0 && !stored[p * E + i]) {
                const int64_t tok = eptr[r][p * E + i], ex = lay[p].off[i + r * E];
                if (!reverse) push.push_back({p, tok, ex, out_rows_pi});   // to p's expert-side layout
                else pull.push_back({kLocal, tok, tok, out_rows_pi});      // back, into this rank's token-side layout
            }
            // rows rank p routes to expert i of this rank
            const int64_t in_rows_pi = table[((size_t)p * W + r) * E + i];
            if (in_rows_pi > 0 && !stored[r * E + i]) {
                const int64_t ex = lay[r].off[i + p * E], tok = eptr[p][r * E + i];
                if (!reverse) pull.push_back({kLocal, ex, ex, in_rows_pi});
                else push.push_back({p, ex, tok, in_rows_pi});             // to p's token-side layout
            }
        }
    }
    return 0;
}

// The host-table entry points keep their uploaded table, flags and plan in the compat area of the
// header; a call whose table and flags equal the previous call's reuses the plan that is there.
struct CompatCache {
    std::vector<int64_t> table;
    std::vector<uint8_t> stored;
    int E = 0;
    bool valid = false;
};
std::map<Comm*, CompatCache> g_compat;
std::mutex g_compat_mtx;

int peer_move_host_table(fmoe_comm_t comm, const void* in, void* out, const int64_t* table, const uint8_t* stored,
                         int64_t in_rows, int64_t out_rows, int64_t row_bytes, int E, int W, bool reverse, cudaStream_t st) {
    FMOE_REQUIRE(comm, "peer exchange: null communicator");
    Comm* c = (Comm*)comm;
    FMOE_REQUIRE(W == c->world, "peer exchange: n_workers=%d but communicator has %d ranks", W, c->world);
    FMOE_REQUIRE(row_bytes > 0, "peer exchange: row_bytes=%lld", (long long)row_bytes);
    if (c->peer.slot_bytes == 0 || row_bytes % 16 != 0) return FMOE_PEER_UNAVAILABLE;
    const PlanDims d = plan_dims(E, W);
    const size_t up_bytes = align_up((size_t)d.T * 8 + (size_t)d.WE, 64);
    if ((int64_t)W * W * E > kTableMax || up_bytes + d.bytes > (size_t)kCompatBytes || (size_t)(d.S + 1) * 4 > 40 * 1024)
        return FMOE_PEER_UNAVAILABLE;      // the same on every rank: it depends on E and W only
    Plan plan;
    if (int rc = plan_peer(table, stored, c->rank, E, W, reverse, plan)) return rc;
    // Whether the rows fit must be decided identically on every rank, so only what the shared table
    // says may enter: the largest buffer any rank receives fits a landing slot, or (when outputs are
    // taken from the receive pools) a quarter of a pool, so that a pool can hold the four exchange
    // outputs of a layer step.  A rank whose output then turns out to lie outside its pool AND to
    // exceed its slot refuses the rows on the device (status bit 64) instead of hanging its peers.
    const int64_t need = plan.slot_rows * row_bytes;
    if (plan.max_rows >= ((int64_t)1 << 31) || (need > c->peer.slot_bytes && need * 4 > c->peer.pool_bytes))
        return FMOE_PEER_UNAVAILABLE;
    const int64_t token_rows = reverse ? out_rows : in_rows, expert_rows = reverse ? in_rows : out_rows;
    if (expert_rows != plan.expert_rows)
        return fail(FMOE_ERR_MISMATCH, "peer exchange: expert-side buffer has %lld rows, counts say %lld",
                    (long long)expert_rows, (long long)plan.expert_rows);
    if (token_rows < plan.token_rows)
        return fail(FMOE_ERR_MISMATCH, "peer exchange: token-side buffer has %lld rows, counts say %lld",
                    (long long)token_rows, (long long)plan.token_rows);
    char* area = c->peer.base[c->rank] + kCompatOff;
    char* dev_plan = area + up_bytes;
    {
        std::lock_guard<std::mutex> lk(g_compat_mtx);
        CompatCache& cc = g_compat[c];
        const bool same = cc.valid && cc.E == E && cc.table.size() == (size_t)d.T &&
                          memcmp(cc.table.data(), table, (size_t)d.T * 8) == 0 && memcmp(cc.stored.data(), stored, (size_t)d.WE) == 0;
        if (!same) {
            cc.valid = false;
            FMOE_CUDA_TRY(cudaMemcpyAsync(area, table, (size_t)d.T * 8, cudaMemcpyHostToDevice, st));
            FMOE_CUDA_TRY(cudaMemcpyAsync(area + (size_t)d.T * 8, stored, (size_t)d.WE, cudaMemcpyHostToDevice, st));
            if (int rc = launch_plan(c, c->rank, W, E, false, nullptr, (const int64_t*)area, (const uint8_t*)(area + (size_t)d.T * 8),
                                     nullptr, -1, dev_plan, st))
                return rc;
            cc.table.assign(table, table + d.T);
            cc.stored.assign(stored, stored + d.WE);
            cc.E = E;
            cc.valid = true;
        }
    }
    return launch_move(c, in, out, dev_plan, E, in_rows, out_rows, row_bytes, reverse, st);
}

}  // namespace

void peer_forget(Comm* c) {
    std::lock_guard<std::mutex> lk(g_compat_mtx);
    g_compat.erase(c);
}

}  // namespace fmoe

using namespace fmoe;

extern "C" int fmoe_peer_enable(fmoe_comm_t comm, int64_t slot_bytes, int64_t pool_bytes, fmoe_stream_t stream) {
    FMOE_REQUIRE(comm, "peer_enable: null communicator");
    Comm* c = (Comm*)comm;
    FMOE_REQUIRE(slot_bytes >= 0 && pool_bytes >= 0, "peer_enable: slot_bytes=%lld pool_bytes=%lld", (long long)slot_bytes,
                 (long long)pool_bytes);
    pool_bytes = (pool_bytes + 511) & ~(int64_t)511;
    if (c->peer.slot_bytes) return 0;          // already on
    if (c->world < 2 || c->world > kMaxPeers || slot_bytes == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    const int W = c->world;
    slot_bytes = (slot_bytes + 255) & ~(int64_t)255;

    // Every step below is taken by all ranks, whatever happened before, so that the
    // collectives match: every allocation is made before the first agreement and a failure
    // only lowers `ok`, this rank's verdict; the final verdict is the AND over all ranks.
    int ok = 1;
    char* own = nullptr;
    char* dev_buf = nullptr;
    unsigned int* counter = nullptr;
    cudaIpcMemHandle_t handle;
    memset(&handle, 0, sizeof(handle));
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle is 64 bytes");
    const size_t rec = sizeof(cudaIpcMemHandle_t) + 8;     // handle + verdict
    if (cudaMalloc((void**)&own, (size_t)kHeaderBytes + 2 * (size_t)slot_bytes + (size_t)pool_bytes) != cudaSuccess) { ok = 0; own = nullptr; }
    if (ok && (cudaMemset(own, 0, kHeaderBytes) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess)) ok = 0;
    if (ok && cudaIpcGetMemHandle(&handle, own) != cudaSuccess) ok = 0;
    if (cudaMalloc((void**)&counter, 4 * sizeof(unsigned int)) != cudaSuccess) { ok = 0; counter = nullptr; }
    if (counter && cudaMemset(counter, 0, 4 * sizeof(unsigned int)) != cudaSuccess) ok = 0;
    (void)cudaGetLastError();
    char* base[kMaxPeers] = {};
    auto release_all = [&]() {
        for (int p = 0; p < W; ++p)
            if (base[p] && p != c->rank) cudaIpcCloseMemHandle(base[p]);
        if (own) cudaFree(own);
        if (counter) cudaFree(counter);
        if (dev_buf) cudaFree(dev_buf);
        (void)cudaGetLastError();
    };
    // The gather buffer is the one allocation without which no agreement can be reached at all:
    // its failure is an error of this call (the peers then fail in the collective, not silently).
    if (cudaMalloc((void**)&dev_buf, rec * (W + 1)) != cudaSuccess) {
        dev_buf = nullptr;
        release_all();
        return fail(FMOE_ERR_CUDA, "peer_enable: cannot allocate %zu bytes for the handle exchange", rec * (W + 1));
    }
    std::vector<char> host(rec * (W + 1), 0);
    auto gather = [&](int verdict) -> int {
        memcpy(host.data(), &handle, sizeof(handle));
        memcpy(host.data() + sizeof(handle), &verdict, sizeof(int));
        FMOE_CUDA_TRY(cudaMemcpyAsync(dev_buf, host.data(), rec, cudaMemcpyHostToDevice, st));
        FMOE_NCCL_TRY(g_nccl.AllGather(dev_buf, dev_buf + rec, rec, ncclChar, c->comm, st));
        FMOE_CUDA_TRY(cudaMemcpyAsync(host.data() + rec, dev_buf + rec, rec * W, cudaMemcpyDeviceToHost, st));
        FMOE_CUDA_TRY(cudaStreamSynchronize(st));
        return 0;
    };
    auto verdict_of = [&](int p) { int v; memcpy(&v, host.data() + rec * (p + 1) + sizeof(handle), sizeof(int)); return v; };
    if (int rc = gather(ok)) { release_all(); return rc; }
    for (int p = 0; p < W; ++p) ok &= verdict_of(p);

    if (ok) {
        base[c->rank] = own;
        for (int p = 0; p < W; ++p) {
            if (p == c->rank) continue;
            cudaIpcMemHandle_t h;
            memcpy(&h, host.data() + rec * (p + 1), sizeof(h));
            void* mapped = nullptr;
            if (cudaIpcOpenMemHandle(&mapped, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) { ok = 0; break; }
            base[p] = (char*)mapped;
        }
        (void)cudaGetLastError();
    }
    // second agreement: everybody mapped everybody
    if (int rc = gather(ok)) { release_all(); return rc; }
    int all = 1;
    for (int p = 0; p < W; ++p) all &= verdict_of(p);
    if (!all) {
        release_all();
        return 0;                                // stays off, on every rank
    }
    cudaFree(dev_buf);
    dev_buf = nullptr;
    {
        int lo = 0, hi = 0;
        cudaDeviceGetStreamPriorityRange(&lo, &hi);
        if (cudaStreamCreateWithPriority(&c->peer.side, cudaStreamNonBlocking, hi) != cudaSuccess) c->peer.side = nullptr;
        if (cudaEventCreateWithFlags(&c->peer.fork, cudaEventDisableTiming) != cudaSuccess) c->peer.fork = nullptr;
        if (cudaEventCreateWithFlags(&c->peer.join, cudaEventDisableTiming) != cudaSuccess) c->peer.join = nullptr;
        (void)cudaGetLastError();
    }
    for (int p = 0; p < W; ++p) c->peer.base[p] = base[p];
    c->peer.counter = counter;
    const char* env = getenv("FMOE_B200_PEER_TIMEOUT_MS");
    long ms = env ? atol(env) : 20000;
    if (ms < 1) ms = 1;
    c->peer.timeout_ns = (unsigned long long)ms * 1000000ull;
    c->peer.slot_bytes = slot_bytes;
    c->peer.pool_bytes = pool_bytes;
    if (pool_bytes > 0) pool_register(c->device, own + kHeaderBytes + 2 * slot_bytes, (size_t)pool_bytes);
    return 0;
}

extern "C" int64_t fmoe_peer_pool_bytes(fmoe_comm_t comm) { return comm ? ((Comm*)comm)->peer.pool_bytes : 0; }

// Allocator functions for torch.cuda.memory.CUDAPluggableAllocator: sub-allocate this device's
// receive pool.  A NULL result makes torch report an out-of-memory condition for the request.
extern "C" void* fmoe_pool_alloc(ptrdiff_t size, int device, void*) { return pool_take(device, size > 0 ? (size_t)size : 1); }
extern "C" void fmoe_pool_free(void* ptr, ptrdiff_t size, int device, void*) { pool_give(device, ptr, size > 0 ? (size_t)size : 1); }

extern "C" size_t fmoe_peer_plan_bytes(int32_t n_expert, int32_t n_workers) {
    if (n_expert <= 0 || n_workers <= 0) return 0;
    return plan_dims(n_expert, n_workers).bytes;
}

extern "C" int64_t fmoe_peer_plan_offsets_at(int32_t n_expert, int32_t n_workers) {
    if (n_expert <= 0 || n_workers <= 0) return -1;
    return (int64_t)plan_dims(n_expert, n_workers).own_off;
}

extern "C" int64_t fmoe_peer_plan_table_at(int32_t n_expert, int32_t n_workers) {
    if (n_expert <= 0 || n_workers <= 0) return -1;
    return (int64_t)plan_dims(n_expert, n_workers).table_off;
}

extern "C" int fmoe_peer_plan_exchange(fmoe_comm_t comm, const int64_t* lec, const uint8_t* stored_models, int64_t cap_rows,
                                       void* plan, int32_t n_expert, fmoe_stream_t stream) {
    FMOE_REQUIRE(comm && lec, "peer_plan_exchange: null pointer");
    Comm* c = (Comm*)comm;
    if (c->peer.slot_bytes == 0) return FMOE_PEER_UNAVAILABLE;
    return launch_plan(c, c->rank, c->world, n_expert, true, lec, nullptr, stored_models, nullptr, cap_rows, plan,
                       (cudaStream_t)stream);
}

extern "C" int fmoe_peer_plan_from_table(const int64_t* all_expert_count, const uint8_t* stored_models, const int64_t* caps,
                                         int32_t rank, int32_t n_expert, int32_t n_workers, void* plan, fmoe_stream_t stream) {
    FMOE_REQUIRE(all_expert_count, "peer_plan_from_table: null table");
    return launch_plan(nullptr, rank, n_workers, n_expert, false, nullptr, all_expert_count, stored_models, caps, -1, plan,
                       (cudaStream_t)stream);
}

extern "C" int fmoe_peer_plan_read(const void* plan_host, int32_t n_expert, int32_t n_workers, int32_t list, fmoe_peer_seg_t* segs,
                                   int32_t max_segs, int32_t* n_segs, int64_t* expert_rows, int64_t* token_rows, int32_t* overflow) {
    FMOE_REQUIRE(plan_host && n_segs && list >= 0 && list < 4, "peer_plan_read: bad argument");
    const PlanDims d = plan_dims(n_expert, n_workers);
    const PlanHead* head = (const PlanHead*)plan_host;
    FMOE_REQUIRE(head->n_expert == n_expert && head->n_workers == n_workers && head->n_slots == d.S,
                 "peer_plan_read: the buffer does not hold a plan for E=%d W=%d", n_expert, n_workers);
    const ListView L = list_view((char*)const_cast<void*>(plan_host), d, list);
    int k = 0;
    for (int s = 0; s < d.S; ++s) {
        const int rows = L.prefix[s + 1] - L.prefix[s];
        if (rows == 0) continue;
        if (segs) {
            FMOE_REQUIRE(k < max_segs, "peer_plan_read: more than max_segs=%d segments", max_segs);
            segs[k] = {L.sel[s] == kLocal ? n_workers : L.sel[s], 0, L.src[s], L.dst[s], rows};
        }
        ++k;
    }
    *n_segs = k;
    if (expert_rows) *expert_rows = head->expert_rows;
    if (token_rows) *token_rows = head->token_rows;
    if (overflow) *overflow = head->overflow;
    return 0;
}

extern "C" int fmoe_peer_scatter_planned(fmoe_comm_t comm, const void* local_in, void* global_out, const void* plan,
                                         int64_t in_rows, int64_t out_rows, int64_t row_bytes, int32_t n_expert,
                                         fmoe_stream_t stream) {
    FMOE_REQUIRE(comm, "peer exchange: null communicator");
    Comm* c = (Comm*)comm;
    if (c->peer.slot_bytes == 0) return FMOE_PEER_UNAVAILABLE;
    return launch_move(c, local_in, global_out, plan, n_expert, in_rows, out_rows, row_bytes, false, (cudaStream_t)stream);
}

extern "C" int fmoe_peer_scatter_planned_rows(fmoe_comm_t comm, const void* src, int64_t src_rows, const int64_t* row_of,
                                              int32_t row_div, const void* scale, int32_t dtype, void* global_out,
                                              const void* plan, int64_t in_rows, int64_t out_rows, int64_t row_bytes,
                                              int32_t n_expert, fmoe_stream_t stream) {
    FMOE_REQUIRE(comm && row_of && row_div > 0, "peer exchange: null pointer");
    FMOE_REQUIRE(dtype == FMOE_F32 || dtype == FMOE_F16 || dtype == FMOE_BF16, "peer exchange: dtype %d", dtype);
    Comm* c = (Comm*)comm;
    if (c->peer.slot_bytes == 0) return FMOE_PEER_UNAVAILABLE;
    const RowSource rows{row_of, row_div, scale, dtype, src_rows};
    return launch_move(c, src, global_out, plan, n_expert, in_rows, out_rows, row_bytes, false, (cudaStream_t)stream, 3, 0, 0, &rows);
}

extern "C" int fmoe_peer_gather_planned(fmoe_comm_t comm, const void* global_in, void* local_out, const void* plan,
                                        int64_t in_rows, int64_t out_rows, int64_t row_bytes, int32_t n_expert,
                                        fmoe_stream_t stream) {
    FMOE_REQUIRE(comm, "peer exchange: null communicator");
    Comm* c = (Comm*)comm;
    if (c->peer.slot_bytes == 0) return FMOE_PEER_UNAVAILABLE;
    return launch_move(c, global_in, local_out, plan, n_expert, in_rows, out_rows, row_bytes, true, (cudaStream_t)stream);
}

namespace fmoe {
// Fills what a grouped GEMM needs to wait for the rows of the exchange that was queued last.
int arrival_wait_of(const fmoe_arrival_t* arrival, ArrivalWait* w) {
    *w = ArrivalWait{};
    if (!arrival || !arrival->comm) return 0;
    Comm* c = (Comm*)arrival->comm;
    FMOE_REQUIRE(c->peer.slot_bytes > 0 && arrival->plan, "arrival: stale handle");
    const int E = arrival->n_expert, W = c->world;
    const PlanDims d = plan_dims(E, W);
    w->flags = (const unsigned long long*)(c->peer.base[c->rank] + kExpArrOff);
    w->seq = (const unsigned long long*)(c->peer.base[c->rank] + kSeqOff);
    w->src_off = (const int*)((const char*)arrival->plan + d.lay_off) + (size_t)c->rank * (d.S + 1) + (size_t)c->rank * E;
    w->world = W;
    w->n_expert = E;
    w->reserve_sms = arrival->overlap_sms;
    return 0;
}
}  // namespace fmoe

extern "C" int fmoe_peer_scatter_planned_async(fmoe_comm_t comm, const void* local_in, void* global_out, const void* plan,
                                               int64_t in_rows, int64_t out_rows, int64_t row_bytes, int32_t n_expert,
                                               int32_t overlap_sms, fmoe_stream_t stream, fmoe_arrival_t* arrival) {
    FMOE_REQUIRE(comm && arrival, "peer exchange: null pointer");
    Comm* c = (Comm*)comm;
    memset(arrival, 0, sizeof(*arrival));
    if (c->peer.slot_bytes == 0) return FMOE_PEER_UNAVAILABLE;
    cudaStream_t st = (cudaStream_t)stream;
    const bool can = overlap_sms > 0 && c->peer.side && c->peer.fork && c->peer.join && c->world <= 32 &&
                     n_expert <= kArrivalExperts && lies_in_pool(c, global_out, out_rows * row_bytes) && overlap_sms < sm_count();
    if (!can)      // the plain exchange on the caller's stream; nothing left to finish
        return launch_move(c, local_in, global_out, plan, n_expert, in_rows, out_rows, row_bytes, false, st);
    FMOE_CUDA_TRY(cudaEventRecord(c->peer.fork, st));
    FMOE_CUDA_TRY(cudaStreamWaitEvent(c->peer.side, c->peer.fork, 0));
    if (int rc = launch_move(c, local_in, global_out, plan, n_expert, in_rows, out_rows, row_bytes, false, c->peer.side, 1, overlap_sms))
        return rc;
    FMOE_CUDA_TRY(cudaEventRecord(c->peer.join, c->peer.side));
    arrival->comm = comm; arrival->plan = plan; arrival->out = global_out;
    arrival->in_rows = in_rows; arrival->out_rows = out_rows; arrival->row_bytes = row_bytes;
    arrival->n_expert = n_expert; arrival->overlap_sms = overlap_sms;
    return 0;
}

extern "C" int fmoe_peer_arrival_finish(const fmoe_arrival_t* arrival, fmoe_stream_t stream) {
    FMOE_REQUIRE(arrival, "arrival_finish: null pointer");
    if (!arrival->comm) return 0;                 // the exchange was queued whole
    Comm* c = (Comm*)arrival->comm;
    cudaStream_t st = (cudaStream_t)stream;
    if (arrival->gather == 3) {
        // the scatter a product was to perform itself: if none did, the whole exchange runs here
        const RowSource rows{arrival->row_of, arrival->row_div > 0 ? arrival->row_div : 1, arrival->scale, arrival->dtype, arrival->src_rows};
        return launch_move(c, arrival->src, arrival->out, arrival->plan, arrival->n_expert, arrival->in_rows, arrival->out_rows,
                           arrival->row_bytes, false, st, arrival->use ? 2 : 3, 0, 0, arrival->row_of && !arrival->use ? &rows : nullptr);
    }
    // (a fused gather has no input buffer of its own: its rows came out of a GEMM's epilogue)
    const int64_t in_rows = arrival->gather == 2 ? ((int64_t)1 << 31) - 1 : arrival->in_rows;
    if (arrival->gather != 2) FMOE_CUDA_TRY(cudaStreamWaitEvent(st, c->peer.join, 0));
    return launch_move(c, nullptr, arrival->out, arrival->plan, arrival->n_expert, in_rows, arrival->out_rows,
                       arrival->row_bytes, arrival->gather != 0, st, 2, 0);
}

namespace fmoe {
int done_words_of(const fmoe_arrival_t* departure, int** done, int** expected, int** ready, int* reserve_sms) {
    *done = *expected = *ready = nullptr;
    *reserve_sms = 0;
    if (!departure || !departure->comm || departure->gather >= 2) return 0;
    Comm* c = (Comm*)departure->comm;
    FMOE_REQUIRE(departure->gather && departure->plan, "departure: not the handle of an overlapped gather");
    const int E = departure->n_expert;
    const PlanDims d = plan_dims(E, c->world);
    int* words = (int*)((char*)const_cast<void*>(departure->plan) + d.done_off);
    const int use = departure->use;
    *done = words + (size_t)use * E; *expected = words + (size_t)(2 + use) * E; *ready = words + 4 * (size_t)E + use;
    *reserve_sms = departure->overlap_sms;
    return 0;
}
}  // namespace fmoe

namespace fmoe {
namespace {
// Tells every peer where this rank receives the rows of the coming exchange (or that it has no room);
// what the first block of a push kernel does, for exchanges whose rows are stored by another kernel.
__global__ void peer_announce_kernel(const __grid_constant__ PeerBases b, int rank, int world, unsigned long long my_dest,
                                     int64_t out_rows, const char* plan, int* status, int scatter) {
    const PlanHead* head = (const PlanHead*)plan;
    const unsigned long long epoch = __ldcg((const unsigned long long*)(b.base[rank] + kSeqOff)) + 1;
    const int parity = (int)(epoch & 1);
    const bool room = (scatter ? head->expert_rows : head->token_rows) <= out_rows;
    const int p = threadIdx.x;
    if (p < world && p != rank) {
        unsigned long long* peer_hdr = (unsigned long long*)b.base[p];
        peer_hdr[kDestOff / 8 + parity * kMaxPeers + rank] = room ? my_dest : kRefused;
        st_release_sys(peer_hdr + kAnnOff / 8 + parity * kMaxPeers + rank, epoch);
    }
    if (p == 0 && !room) atomicOr(status, 64);
}
}  // namespace

// What a grouped GEMM needs to deliver its own input rows (the handle of fmoe_peer_scatter_fused_begin).
int push_in_of(const fmoe_arrival_t* h, GemmRemoteOut* ro, GemmPushIn* ps) {
    memset(ps, 0, sizeof(*ps));
    memset(ro, 0, sizeof(*ro));
    if (!h || !h->comm || h->gather != 3) return 0;
    fmoe_arrival_t as_out = *h;
    as_out.gather = 2;                             // the peer context is the same as for a fused gather
    if (int rc = remote_out_of(&as_out, ro)) return rc;
    ro->enabled = 2;
    Comm* c = (Comm*)h->comm;
    const int E = h->n_expert, W = c->world;
    const PlanDims d = plan_dims(E, W);
    char* plan = (char*)const_cast<void*>(h->plan);
    const ListView L = list_view(plan, d, LIST_PUSH_FWD);
    const PlanHead* head = (const PlanHead*)plan;
    ps->src = h->src; ps->row_of = h->row_of; ps->scale = h->scale; ps->src_rows = h->src_rows; ps->row_div = h->row_div > 0 ? h->row_div : 1;
    ps->prefix = L.prefix; ps->seg_sel = L.sel; ps->seg_src = L.src; ps->seg_dst = L.dst;
    ps->seg_done = (int*)(plan + d.segdone_off);
    ps->expert_rows = &head->expert_rows; ps->token_rows = &head->token_rows;
    ps->in_rows = h->in_rows; ps->out_rows = h->out_rows; ps->row_vecs = h->row_bytes / 16;
    ps->n_slots = d.S; ps->n_expert = E; ps->local_sel = kLocal;
    ps->flags_at = (int)kExpArrOff; ps->flag_sources = kMaxPeers; ps->flag_experts = kArrivalExperts;
    return 0;
}

// What a grouped GEMM needs to store its output rows straight into their owners' memory.
int remote_out_of(const fmoe_arrival_t* h, GemmRemoteOut* ro) {
    memset(ro, 0, sizeof(*ro));
    if (!h || !h->comm || h->gather != 2) return 0;
    Comm* c = (Comm*)h->comm;
    FMOE_REQUIRE(c->peer.slot_bytes > 0 && h->plan && c->world <= kRemoteMaxWorld, "remote output: stale handle");
    const int E = h->n_expert, W = c->world;
    const PlanDims d = plan_dims(E, W);
    for (int p = 0; p < W; ++p) ro->base[p] = c->peer.base[p];
    ro->header = (const unsigned long long*)c->peer.base[c->rank];
    ro->seq = (const unsigned long long*)(c->peer.base[c->rank] + kSeqOff);
    ro->src_off = (const int*)((const char*)h->plan + d.lay_off) + (size_t)c->rank * (d.S + 1) + (size_t)c->rank * E;
    ro->dst_off = (const int*)((const char*)h->plan + d.back_off);
    ro->counter = c->peer.counter + 3;
    ro->my_dest = (unsigned long long)((char*)h->out - c->peer.base[c->rank]);
    ro->min_dest = (unsigned long long)kHeaderBytes;
    ro->timeout_cycles = c->peer.timeout_ns * 2ull;
    ro->arrived_at = kArrivedOff; ro->ann_at = kAnnOff; ro->dest_at = kDestOff; ro->stride = kMaxPeers;
    ro->world = W; ro->rank = c->rank; ro->enabled = 1;
    return 0;
}
}  // namespace fmoe

extern "C" int fmoe_peer_scatter_fused_begin(fmoe_comm_t comm, const void* src, int64_t src_rows, const int64_t* row_of,
                                             int32_t row_div, const void* scale, int32_t dtype, void* global_out,
                                             const void* plan, int64_t in_rows, int64_t out_rows, int64_t row_bytes,
                                             int32_t n_expert, fmoe_stream_t stream, fmoe_arrival_t* arrival) {
    FMOE_REQUIRE(comm && arrival && plan && src, "peer exchange: null pointer");
    Comm* c = (Comm*)comm;
    memset(arrival, 0, sizeof(*arrival));
    if (c->peer.slot_bytes == 0) return FMOE_PEER_UNAVAILABLE;
    const bool can = c->world <= kRemoteMaxWorld && n_expert <= kArrivalExperts && row_bytes > 0 && row_bytes % 16 == 0 &&
                     (dtype == FMOE_F16 || dtype == FMOE_BF16) && (row_of || !scale) && (!row_of || row_div > 0) &&
                     (((uintptr_t)src | (uintptr_t)global_out) & 15) == 0 && in_rows < ((int64_t)1 << 31) &&
                     out_rows < ((int64_t)1 << 31) && lies_in_pool(c, global_out, out_rows * row_bytes);
    if (!can) return 0;                       // nothing queued: the caller runs the exchange as a call of its own
    PeerBases b;
    for (int p = 0; p < kMaxPeers; ++p) b.base[p] = c->peer.base[p];
    int* status = device_status_ptr();
    FMOE_REQUIRE(status, "peer exchange: no device status word");
    peer_announce_kernel<<<1, 64, 0, (cudaStream_t)stream>>>(b, c->rank, c->world, (unsigned long long)((char*)global_out - c->peer.base[c->rank]),
                                                            out_rows, (const char*)plan, status, 1);
    FMOE_CHECK_LAUNCH();
    arrival->comm = comm; arrival->plan = plan; arrival->out = global_out;
    arrival->in_rows = in_rows; arrival->out_rows = out_rows; arrival->row_bytes = row_bytes;
    arrival->n_expert = n_expert; arrival->gather = 3; arrival->use = 0;
    arrival->src = src; arrival->row_of = row_of; arrival->scale = scale; arrival->src_rows = src_rows;
    arrival->row_div = row_div; arrival->dtype = dtype;
    return 0;
}

extern "C" int fmoe_peer_gather_fused_begin(fmoe_comm_t comm, void* local_out, const void* plan, int64_t out_rows,
                                            int64_t row_bytes, int32_t n_expert, fmoe_stream_t stream, fmoe_arrival_t* departure) {
    FMOE_REQUIRE(comm && departure && plan, "peer exchange: null pointer");
    Comm* c = (Comm*)comm;
    memset(departure, 0, sizeof(*departure));
    if (c->peer.slot_bytes == 0) return FMOE_PEER_UNAVAILABLE;
    if (c->world > kRemoteMaxWorld || row_bytes <= 0 || row_bytes % 16 != 0 || !lies_in_pool(c, local_out, out_rows * row_bytes))
        return 0;     // nothing queued: the caller stores the rows locally and gathers them afterwards
    PeerBases b;
    for (int p = 0; p < kMaxPeers; ++p) b.base[p] = c->peer.base[p];
    int* status = device_status_ptr();
    FMOE_REQUIRE(status, "peer exchange: no device status word");
    peer_announce_kernel<<<1, 64, 0, (cudaStream_t)stream>>>(b, c->rank, c->world, (unsigned long long)((char*)local_out - c->peer.base[c->rank]),
                                                            out_rows, (const char*)plan, status, 0);
    FMOE_CHECK_LAUNCH();
    departure->comm = comm; departure->plan = plan; departure->out = local_out;
    departure->in_rows = 0; departure->out_rows = out_rows; departure->row_bytes = row_bytes;
    departure->n_expert = n_expert; departure->gather = 2;
    return 0;
}

extern "C" int fmoe_peer_gather_planned_async(fmoe_comm_t comm, const void* global_in, void* local_out, const void* plan,
                                              int64_t in_rows, int64_t out_rows, int64_t row_bytes, int32_t n_expert,
                                              int32_t overlap_sms, int32_t use, fmoe_stream_t stream, fmoe_arrival_t* departure) {
    FMOE_REQUIRE(comm && departure && (use == 0 || use == 1), "peer exchange: bad argument");
    Comm* c = (Comm*)comm;
    memset(departure, 0, sizeof(*departure));
    if (c->peer.slot_bytes == 0) return FMOE_PEER_UNAVAILABLE;
    cudaStream_t st = (cudaStream_t)stream;
    const bool can = overlap_sms > 0 && c->peer.side && c->peer.fork && c->peer.join && c->world <= 32 &&
                     lies_in_pool(c, local_out, out_rows * row_bytes) && overlap_sms < sm_count();
    if (!can) return 0;     // nothing queued: the caller runs the plain gather after the product (departure->comm == NULL)
    FMOE_CUDA_TRY(cudaEventRecord(c->peer.fork, st));
    FMOE_CUDA_TRY(cudaStreamWaitEvent(c->peer.side, c->peer.fork, 0));
    if (int rc = launch_move(c, global_in, local_out, plan, n_expert, in_rows, out_rows, row_bytes, true, c->peer.side, 1, overlap_sms, use))
        return rc;
    FMOE_CUDA_TRY(cudaEventRecord(c->peer.join, c->peer.side));
    departure->comm = comm; departure->plan = plan; departure->out = local_out;
    departure->in_rows = in_rows; departure->out_rows = out_rows; departure->row_bytes = row_bytes;
    departure->n_expert = n_expert; departure->overlap_sms = overlap_sms; departure->gather = 1; departure->use = use;
    return 0;
}

extern "C" int fmoe_peer_wait_probe(fmoe_comm_t comm, int32_t timeout_ms, int32_t push, fmoe_stream_t stream) {
    FMOE_REQUIRE(comm, "peer_wait_probe: null communicator");
    Comm* c = (Comm*)comm;
    FMOE_REQUIRE(c->peer.slot_bytes > 0, "peer_wait_probe: the peer-memory exchange is off");
    FMOE_REQUIRE(timeout_ms >= 1 && timeout_ms <= 10000, "peer_wait_probe: timeout_ms=%d (1..10000)", timeout_ms);
    // One block of the push (or consume) kernel that waits for an epoch no peer will ever publish:
    // it announces nothing, moves nothing, and leaves the epoch words alone.  The plan it reads is a
    // zeroed one (no rows) in the compat area's tail.
    PeerBases b;
    for (int p = 0; p < kMaxPeers; ++p) b.base[p] = c->peer.base[p];
    char* plan = c->peer.base[c->rank] + kCompatOff + kCompatBytes;
    const PlanDims pd = plan_dims(1, c->world);
    FMOE_REQUIRE(pd.bytes <= (size_t)kProbeBytes, "peer_wait_probe: plan of %zu bytes", pd.bytes);
    FMOE_CUDA_TRY(cudaMemsetAsync(plan, 0, pd.bytes, (cudaStream_t)stream));
    PlanHead head;
    memset(&head, 0, sizeof(head));
    head.n_expert = 1; head.n_workers = c->world; head.rank = c->rank; head.n_slots = pd.S;
    FMOE_CUDA_TRY(cudaMemcpyAsync(plan, &head, sizeof(head), cudaMemcpyHostToDevice, (cudaStream_t)stream));
    MoveArgs a;
    memset(&a, 0, sizeof(a));
    a.rank = c->rank; a.world = c->world; a.probe = 1; a.direct = 1;
    a.slot_bytes = c->peer.slot_bytes; a.row_bytes = 16;
    a.timeout_ns = (unsigned long long)timeout_ms * 1000000ull;
    a.counter = c->peer.counter + 2;
    a.plan = plan;
    a.status = device_status_ptr();
    FMOE_REQUIRE(a.status, "peer_wait_probe: no device status word");
    const size_t smem = (size_t)(pd.S + 1) * sizeof(int);
    if (push) peer_move_kernel<true><<<1, kMoveThreads, smem, (cudaStream_t)stream>>>(b, a, nullptr, nullptr);
    else peer_move_kernel<false><<<1, kMoveThreads, smem, (cudaStream_t)stream>>>(b, a, nullptr, nullptr);
    FMOE_CHECK_LAUNCH();
    return 0;
}

extern "C" int fmoe_peer_set_timeout_ms(fmoe_comm_t comm, int32_t timeout_ms) {
    FMOE_REQUIRE(comm && timeout_ms >= 1, "peer_set_timeout_ms: bad argument");
    ((Comm*)comm)->peer.timeout_ns = (unsigned long long)timeout_ms * 1000000ull;
    return 0;
}

extern "C" int64_t fmoe_peer_slot_bytes(fmoe_comm_t comm) {
    return comm ? ((Comm*)comm)->peer.slot_bytes : 0;
}

extern "C" int fmoe_peer_global_scatter(fmoe_comm_t comm, const void* local_in, void* global_out,
                                        const int64_t* all_expert_count_host, const uint8_t* stored_models_host,
                                        int64_t in_rows, int64_t out_rows, int64_t row_bytes, int32_t n_expert,
                                        int32_t n_workers, fmoe_stream_t stream) {
    return peer_move_host_table(comm, local_in, global_out, all_expert_count_host, stored_models_host, in_rows, out_rows,
                                row_bytes, n_expert, n_workers, false, (cudaStream_t)stream);
}

extern "C" int fmoe_peer_global_gather(fmoe_comm_t comm, const void* global_in, void* local_out,
                                       const int64_t* all_expert_count_host, const uint8_t* stored_models_host,
                                       int64_t in_rows, int64_t out_rows, int64_t row_bytes, int32_t n_expert,
                                       int32_t n_workers, fmoe_stream_t stream) {
    return peer_move_host_table(comm, global_in, local_out, all_expert_count_host, stored_models_host, in_rows, out_rows,
                                row_bytes, n_expert, n_workers, true, (cudaStream_t)stream);
}

extern "C" int fmoe_peer_plan(const int64_t* all_expert_count_host, const uint8_t* stored_models_host, int32_t rank,
                              int32_t n_expert, int32_t n_workers, int32_t reverse, fmoe_peer_seg_t* push,
                              int32_t* n_push, fmoe_peer_seg_t* pull, int32_t* n_pull, int32_t max_segs,
                              int64_t* slot_rows) {
    FMOE_REQUIRE(n_push && n_pull && slot_rows, "peer_plan: null output pointer");
    Plan plan;
    if (int rc = plan_peer(all_expert_count_host, stored_models_host, rank, n_expert, n_workers, reverse != 0, plan))
        return rc;
    auto emit = [&](const std::vector<Seg>& v, fmoe_peer_seg_t* out, int32_t* n) -> int {
        int k = 0;
        for (const Seg& sg : v) {
            if (sg.rows == 0) continue;
            if (out) {
                FMOE_REQUIRE(k < max_segs, "peer_plan: more than max_segs=%d segments", max_segs);
                out[k] = {sg.sel == kLocal ? n_workers : sg.sel, 0, sg.src_row, sg.dst_row, sg.rows};
            }
            ++k;
        }
        *n = k;
        return 0;
    };
    if (int rc = emit(plan.push, push, n_push)) return rc;
    if (int rc = emit(plan.pull, pull, n_pull)) return rc;
    *slot_rows = plan.slot_rows;
    return 0;
}
