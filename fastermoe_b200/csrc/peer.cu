// Token all-to-all-v over NVLink peer memory: the rows of global_scatter /
// global_gather are stored straight into the destination GPU's memory by a copy
// kernel, with no NCCL send/receive pairs and no staging pass on the sender.
//
// Same data movement as cuda/global_exchange.cuh:75-124 of the reference (which
// issues one ncclSend/ncclRecv per expert and peer); the row layout on both sides
// is the one plan_scatter describes.
//
// Every rank owns an allocation that its peers map through CUDA IPC:
//
//     [ header 4 KiB | slot 0 | slot 1 | receive pool ]
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
//      peers out of the slot into the output.
// The output buffer can be announced directly when it lies in the receive pool: the Python
// layer allocates exchange outputs there through a torch memory pool whose allocator is
// fmoe_pool_alloc/fmoe_pool_free below, so tensor lifetimes stay with torch's caching
// allocator.  Otherwise rows land in slot `parity` and are copied once more.  An announcement
// is made by a kernel that is stream-ordered after every earlier use of the announced memory
// on its GPU, and entry `parity` is rewritten two epochs later, after the peers have arrived
// for the epoch in between, so neither the memory nor the entry is overwritten while in use.
//
// All waits are bounded (wall-clock limit, FMOE_B200_PEER_TIMEOUT_MS, default
// 20000): when one expires the kernel raises bit 16 (no announcement) or 32 (rows
// not arrived) in the device status word and carries on, so that the stream drains.
//
// Whether an exchange goes over peer memory must be decided identically on all
// ranks; the entry points therefore take the all-gathered count table, from which
// every rank derives every other rank's layout and the largest slot any rank needs.
#include "common.cuh"
#include "exchange.h"
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

constexpr int kHeaderBytes = 4096;
// header words (u64): arrived[2][kMaxPeers] at byte 0, ann[2][kMaxPeers] at 1024, dest[2][kMaxPeers] at 2048
constexpr int kAnnWord = 1024 / 8, kDestWord = 2048 / 8;
constexpr int kPeerSegMax = 128;
constexpr int kLocal = 255;                 // dst_sel of rows that stay on this GPU
static_assert(3 * 2 * kMaxPeers * 8 <= kHeaderBytes, "flags fit the header");

struct PeerSegs {
    int n;
    int prefix[kPeerSegMax + 1];            // rows before segment k
    int src_row[kPeerSegMax], dst_row[kPeerSegMax];
    unsigned char dst_sel[kPeerSegMax];     // destination rank, or kLocal
};
struct PeerBases { char* base[kMaxPeers]; };

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

// Waits until *flag + slack >= want; gives up after timeout_ns (or 2^28 polls).
__device__ bool wait_flag(const unsigned long long* flag, unsigned long long want, unsigned long long slack,
                          unsigned long long timeout_ns) {
    if (ld_acquire_sys(flag) + slack >= want) return true;
    const unsigned long long t0 = now_ns();
    for (unsigned it = 0; it < (1u << 28); ++it) {
        if (ld_acquire_sys(flag) + slack >= want) return true;
        if (now_ns() - t0 > timeout_ns) return false;
        __nanosleep(256);
    }
    return false;
}

struct PeerLaunch {
    int rank, world, parity;
    int announce, signal_last;              // this launch opens / closes the push phase
    unsigned long long epoch, timeout_ns;
    unsigned long long my_dest;             // push: byte offset in this rank's allocation where its rows shall land
    int64_t row_vecs, slot_off;             // 16-byte units per row; consume: byte offset of the slot
    unsigned int* counter;
    int* status;
};

template <bool kPush>
__global__ void __launch_bounds__(256)
peer_rows_kernel(const __grid_constant__ PeerSegs t, const __grid_constant__ PeerBases b,
                 const __grid_constant__ PeerLaunch a, const uint4* __restrict__ src, uint4* __restrict__ out) {
    __shared__ int s_last;
    __shared__ unsigned long long s_dest[kMaxPeers];
    __shared__ unsigned long long s_dead;   // peers whose announcement never came: nothing is stored there
    unsigned long long* hdr = (unsigned long long*)b.base[a.rank];
    {
        const int p = threadIdx.x;
        if (p == 0) s_dead = 0ull;
        __syncthreads();
        if (p < a.world && p != a.rank) {
            if (kPush) {
                if (a.announce && blockIdx.x == 0) {
                    unsigned long long* peer_hdr = (unsigned long long*)b.base[p];
                    peer_hdr[kDestWord + a.parity * kMaxPeers + a.rank] = a.my_dest;
                    st_release_sys(peer_hdr + kAnnWord + a.parity * kMaxPeers + a.rank, a.epoch);
                }
                // Where peer p wants its rows.  Without an announcement of this epoch the word holds
                // an older epoch's address (or nothing), so rows for that peer are dropped, not stored.
                const bool announced = wait_flag(hdr + kAnnWord + a.parity * kMaxPeers + p, a.epoch, 0, a.timeout_ns);
                const unsigned long long dest = hdr[kDestWord + a.parity * kMaxPeers + p];
                s_dest[p] = dest;
                if (!announced || dest < (unsigned long long)kHeaderBytes) {
                    atomicOr(a.status, 16);
                    atomicOr(&s_dead, 1ull << p);
                }
            } else {           // everyone's rows of this epoch must have landed
                if (!wait_flag(hdr + a.parity * kMaxPeers + p, a.epoch, 0, a.timeout_ns)) atomicOr(a.status, 32);
            }
        }
        __syncthreads();
    }
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
    bool live = row < t.prefix[t.n];
    int k = 0;
    if (live) {
        int lo = 0, hi = t.n - 1;  // last segment whose prefix <= row
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (t.prefix[mid] <= row) lo = mid; else hi = mid - 1;
        }
        k = lo;
        if (kPush && t.dst_sel[k] != kLocal && ((s_dead >> t.dst_sel[k]) & 1ull)) live = false;
    }
    if (live) {
        const int off = row - t.prefix[k];
        const uint4* s;
        uint4* d;
        if (kPush) {
            s = src + (int64_t)(t.src_row[k] + off) * a.row_vecs;
            const int sel = t.dst_sel[k];
            d = (sel == kLocal ? out : (uint4*)(b.base[sel] + s_dest[sel])) + (int64_t)(t.dst_row[k] + off) * a.row_vecs;
        } else {
            s = (const uint4*)(b.base[a.rank] + a.slot_off) + (int64_t)(t.src_row[k] + off) * a.row_vecs;
            d = out + (int64_t)(t.dst_row[k] + off) * a.row_vecs;
        }
        // Rows in the slot were written by other GPUs while this kernel may already have
        // been running: read them through L2 (ld.cg), never through the non-coherent path.
        int64_t c = lane;
        for (; c + 96 < a.row_vecs; c += 128) {
            const uint4 v0 = __ldcg(s + c), v1 = __ldcg(s + c + 32), v2 = __ldcg(s + c + 64), v3 = __ldcg(s + c + 96);
            d[c] = v0; d[c + 32] = v1; d[c + 64] = v2; d[c + 96] = v3;
        }
        for (; c < a.row_vecs; c += 32) d[c] = __ldcg(s + c);
    }
    if (kPush && a.signal_last) {
        // All of this block's stores are ordered before thread 0's fence by the barrier,
        // and the fence is cumulative: one fence per block publishes them.
        __syncthreads();
        if (threadIdx.x == 0) {
            __threadfence_system();
            s_last = atomicAdd(a.counter, 1u) == gridDim.x - 1;
        }
        __syncthreads();
        if (s_last) {
            __threadfence_system();
            const int p = threadIdx.x;
            if (p < a.world && p != a.rank) {
                unsigned long long* peer_hdr = (unsigned long long*)b.base[p];
                st_release_sys(peer_hdr + a.parity * kMaxPeers + a.rank, a.epoch);
            }
            if (threadIdx.x == 0) *a.counter = 0;
        }
    }
}

struct Seg { int sel; int64_t src_row, dst_row, rows; };

template <bool kPush>
int launch_phase(Comm* c, const std::vector<Seg>& segs, const void* src, void* out, int64_t row_bytes, int parity,
                 unsigned long long my_dest, cudaStream_t st) {
    PeerBases b;
    for (int p = 0; p < kMaxPeers; ++p) b.base[p] = c->peer.base[p];
    PeerLaunch a;
    a.rank = c->rank; a.world = c->world; a.parity = parity;
    a.epoch = c->peer.epoch; a.timeout_ns = c->peer.timeout_ns;
    a.my_dest = my_dest;
    a.row_vecs = row_bytes / 16;
    a.slot_off = kHeaderBytes + (int64_t)parity * c->peer.slot_bytes;
    a.counter = c->peer.counter;
    a.status = device_status_ptr();
    FMOE_REQUIRE(a.status, "peer exchange: no device status word");
    PeerSegs t;
    size_t i = 0;
    bool first = true;
    do {
        t.n = 0;
        t.prefix[0] = 0;
        for (; i < segs.size() && t.n < kPeerSegMax; ++i) {
            const Seg& s = segs[i];
            if (s.rows == 0) continue;
            t.dst_sel[t.n] = (unsigned char)s.sel;
            t.src_row[t.n] = (int)s.src_row; t.dst_row[t.n] = (int)s.dst_row;
            t.prefix[t.n + 1] = t.prefix[t.n] + (int)s.rows;
            ++t.n;
        }
        if (t.n == 0) t.prefix[1] = 0;
        a.announce = first;
        a.signal_last = i >= segs.size();
        const unsigned blocks = (unsigned)std::max<int64_t>(1, ceil_div(t.n ? t.prefix[t.n] : 0, 8));
        peer_rows_kernel<kPush><<<blocks, 256, 0, st>>>(t, b, a, (const uint4*)src, (uint4*)out);
        FMOE_CHECK_LAUNCH();
        first = false;
    } while (i < segs.size());
    return 0;
}

// Expert-side row of segment (expert i of rank p, source rank j), as plan_scatter lays
// rank p's buffer out; -1 for segments that are not exchanged.  table is [W][W][E]:
// rows that rank `src` routes to expert e of rank `dst`.
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

// Row segments of one exchange for rank r: `push` = what its push kernel stores (sel = kLocal:
// the rows stay on this GPU and go straight to the output), `pull` = what its consume kernel
// copies out of its own landing slot.  slot_rows = rows of the largest slot any rank needs (the
// same on every rank, because it depends on the shared table only).
struct Plan {
    std::vector<Seg> push, pull;
    int64_t slot_rows = 0, expert_rows = 0, token_rows = 0, max_rows = 0;
};

int plan_peer(const int64_t* table, const uint8_t* stored, int r, int E, int W, bool reverse, Plan& plan) {
    FMOE_REQUIRE(table && stored && E > 0 && W > 0 && r >= 0 && r < W, "peer exchange: bad argument");
    const size_t n = (size_t)W * E;
    for (size_t i = 0; i < n * W; ++i) FMOE_REQUIRE(table[i] >= 0, "peer exchange: negative count at %zu", i);
    // token-side offsets of every rank, expert-side layout of every rank
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
    for (int i = 0; i < E; ++i) {
        const int64_t ex = lay[r].off[i + r * E];
        if (ex < 0) continue;
        const int64_t tok = eptr[r][r * E + i], rows = mine[r * E + i];
        push.push_back(reverse ? Seg{kLocal, ex, tok, rows} : Seg{kLocal, tok, ex, rows});
    }
    // Peers are visited in the order r+1, r+2, ...: at any moment every rank stores into a
    // different peer, so no GPU's NVLink ingress is shared by several senders.
    for (int dlt = 1; dlt < W; ++dlt) {
        const int p = (r + dlt) % W;
        for (int i = 0; i < E; ++i) {
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

int peer_move(fmoe_comm_t comm, const void* in, void* out, const int64_t* table, const uint8_t* stored,
              int64_t in_rows, int64_t out_rows, int64_t row_bytes, int E, int W, bool reverse, cudaStream_t st) {
    FMOE_REQUIRE(comm, "peer exchange: null communicator");
    Comm* c = (Comm*)comm;
    FMOE_REQUIRE(W == c->world, "peer exchange: n_workers=%d but communicator has %d ranks", W, c->world);
    FMOE_REQUIRE(row_bytes > 0, "peer exchange: row_bytes=%lld", (long long)row_bytes);
    if (c->peer.slot_bytes == 0 || row_bytes % 16 != 0) return FMOE_PEER_UNAVAILABLE;
    Plan plan;
    if (int rc = plan_peer(table, stored, c->rank, E, W, reverse, plan)) return rc;
    if (plan.slot_rows * row_bytes > c->peer.slot_bytes || plan.max_rows >= ((int64_t)1 << 31))
        return FMOE_PEER_UNAVAILABLE;     // same verdict on every rank: it depends on the shared table only

    const int64_t token_rows = reverse ? out_rows : in_rows, expert_rows = reverse ? in_rows : out_rows;
    if (expert_rows != plan.expert_rows)
        return fail(FMOE_ERR_MISMATCH, "peer exchange: expert-side buffer has %lld rows, counts say %lld",
                    (long long)expert_rows, (long long)plan.expert_rows);
    if (token_rows < plan.token_rows)
        return fail(FMOE_ERR_MISMATCH, "peer exchange: token-side buffer has %lld rows, counts say %lld",
                    (long long)token_rows, (long long)plan.token_rows);
    FMOE_REQUIRE((in || in_rows == 0) && (out || out_rows == 0), "peer exchange: null buffer");
    FMOE_REQUIRE((((uintptr_t)in | (uintptr_t)out) & 15) == 0, "peer exchange: buffers must be 16-byte aligned");
    if (reverse && out_rows > plan.token_rows)
        FMOE_CUDA_TRY(cudaMemsetAsync((char*)out + plan.token_rows * row_bytes, 0,
                                      (size_t)(out_rows - plan.token_rows) * row_bytes, st));
    c->peer.epoch += 1;
    const int parity = (int)(c->peer.epoch & 1);
    // Rows can land in the output itself when it lies in this rank's receive pool.
    char* pool = c->peer.base[c->rank] + kHeaderBytes + 2 * c->peer.slot_bytes;
    const int64_t recv_bytes = (reverse ? out_rows : plan.expert_rows) * row_bytes;
    const bool direct = c->peer.pool_bytes > 0 && (char*)out >= pool && (char*)out + recv_bytes <= pool + c->peer.pool_bytes;
    const unsigned long long my_dest = direct ? (unsigned long long)((char*)out - c->peer.base[c->rank])
                                              : (unsigned long long)(kHeaderBytes + (int64_t)parity * c->peer.slot_bytes);
    if (int rc = launch_phase<true>(c, plan.push, in, out, row_bytes, parity, my_dest, st)) return rc;
    static const std::vector<Seg> nothing;
    return launch_phase<false>(c, direct ? nothing : plan.pull, nullptr, out, row_bytes, parity, 0, st);
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

void peer_release(Comm* c) {
    PeerState& ps = c->peer;
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
    ps.slot_bytes = 0;
    (void)cudaGetLastError();
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
    if (cudaMalloc((void**)&counter, 2 * sizeof(unsigned int)) != cudaSuccess) { ok = 0; counter = nullptr; }
    if (counter && cudaMemset(counter, 0, 2 * sizeof(unsigned int)) != cudaSuccess) ok = 0;
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
    for (int p = 0; p < W; ++p) c->peer.base[p] = base[p];
    c->peer.counter = counter;
    c->peer.epoch = 0;
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

extern "C" int fmoe_peer_wait_probe(fmoe_comm_t comm, int32_t timeout_ms, fmoe_stream_t stream) {
    FMOE_REQUIRE(comm, "peer_wait_probe: null communicator");
    Comm* c = (Comm*)comm;
    FMOE_REQUIRE(c->peer.slot_bytes > 0, "peer_wait_probe: the peer-memory exchange is off");
    FMOE_REQUIRE(timeout_ms >= 1 && timeout_ms <= 10000, "peer_wait_probe: timeout_ms=%d (1..10000)", timeout_ms);
    // A consume phase without rows that waits for an epoch no peer will ever publish.
    const unsigned long long epoch = c->peer.epoch, limit = c->peer.timeout_ns;
    c->peer.epoch = epoch + (1ull << 40);
    c->peer.timeout_ns = (unsigned long long)timeout_ms * 1000000ull;
    PeerBases b;
    for (int p = 0; p < kMaxPeers; ++p) b.base[p] = c->peer.base[p];
    PeerSegs t;
    t.n = 0; t.prefix[0] = 0; t.prefix[1] = 0;
    PeerLaunch a;
    a.rank = c->rank; a.world = c->world; a.parity = 0;
    a.announce = 0; a.signal_last = 0; a.my_dest = 0;
    a.epoch = c->peer.epoch; a.timeout_ns = c->peer.timeout_ns;
    a.row_vecs = 1; a.slot_off = kHeaderBytes;
    a.counter = c->peer.counter;
    a.status = device_status_ptr();
    c->peer.epoch = epoch;
    c->peer.timeout_ns = limit;
    FMOE_REQUIRE(a.status, "peer_wait_probe: no device status word");
    peer_rows_kernel<false><<<1, 256, 0, (cudaStream_t)stream>>>(t, b, a, nullptr, nullptr);
    FMOE_CHECK_LAUNCH();
    return 0;
}

extern "C" int64_t fmoe_peer_slot_bytes(fmoe_comm_t comm) {
    return comm ? ((Comm*)comm)->peer.slot_bytes : 0;
}

extern "C" int fmoe_peer_global_scatter(fmoe_comm_t comm, const void* local_in, void* global_out,
                                        const int64_t* all_expert_count_host, const uint8_t* stored_models_host,
                                        int64_t in_rows, int64_t out_rows, int64_t row_bytes, int32_t n_expert,
                                        int32_t n_workers, fmoe_stream_t stream) {
    return peer_move(comm, local_in, global_out, all_expert_count_host, stored_models_host, in_rows, out_rows,
                     row_bytes, n_expert, n_workers, false, (cudaStream_t)stream);
}

extern "C" int fmoe_peer_global_gather(fmoe_comm_t comm, const void* global_in, void* local_out,
                                       const int64_t* all_expert_count_host, const uint8_t* stored_models_host,
                                       int64_t in_rows, int64_t out_rows, int64_t row_bytes, int32_t n_expert,
                                       int32_t n_workers, fmoe_stream_t stream) {
    return peer_move(comm, global_in, local_out, all_expert_count_host, stored_models_host, in_rows, out_rows,
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
