// Communicator state and the run-time NCCL binding shared by the exchange and
// smart-schedule code.
#pragma once
#include <nccl.h>
#include <cuda_runtime.h>
#include <vector>
#include "../../include/fmoe_b200.h"

namespace fmoe {

struct NcclApi {
    ncclResult_t (*GetUniqueId)(ncclUniqueId*);
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int);
    ncclResult_t (*CommDestroy)(ncclComm_t);
    ncclResult_t (*CommUserRank)(const ncclComm_t, int*);
    ncclResult_t (*CommCount)(const ncclComm_t, int*);
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t);
    ncclResult_t (*Send)(const void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t);
    ncclResult_t (*Recv)(void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t);
    ncclResult_t (*GroupStart)();
    ncclResult_t (*GroupEnd)();
    ncclResult_t (*Broadcast)(const void*, void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t);
    ncclResult_t (*Reduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, int, ncclComm_t, cudaStream_t);
    const char* (*GetErrorString)(ncclResult_t);
};

extern NcclApi g_nccl;
int ensure_nccl_loaded();

// Peer-memory exchange state (see peer.cu).  `base[p]` is rank p's landing allocation
// as mapped into this process (own allocation at p == rank); slot_bytes == 0: off.
constexpr int kMaxPeers = 64;
struct PeerState {
    int64_t slot_bytes = 0;
    int64_t pool_bytes = 0;            // receive pool behind the two slots (0: none)
    char* base[kMaxPeers] = {};
    unsigned int* counter = nullptr;   // device words for last-block detection
    cudaStream_t side = nullptr;       // the overlapped push runs here, beside the GEMM on the caller's stream
    cudaEvent_t fork = nullptr, join = nullptr;
    unsigned long long timeout_ns = 0;
};

struct Comm {
    ncclComm_t comm = nullptr;
    int rank = 0, world = 1, device = 0;
    std::vector<cudaEvent_t> events;  // pool reused by the smart schedule
    PeerState peer;
};

// What a grouped GEMM needs to start on rows while they are still arriving (see fmoe_arrival_t).
struct ArrivalWait {
    const unsigned long long* flags = nullptr;   // [2][kMaxPeers][kArrivalExperts] in this GPU's landing area
    const unsigned long long* seq = nullptr;     // this GPU's exchange epoch word
    const int* src_off = nullptr;                // [E*W + 1]: first row of (expert i, source j) at [i*W + j]
    int world = 0, n_expert = 0;
    int reserve_sms = 0;                         // SMs to leave to the push kernel
};
constexpr int kArrivalExperts = 256;

int arrival_wait_of(const fmoe_arrival_t* arrival, ArrivalWait* w);
// The completion counters (GemmDone in gemm.h) of an overlapped gather's handle; nulls when it is not pending.
int done_words_of(const fmoe_arrival_t* departure, int** done, int** expected, int** ready, int* reserve_sms);
// Fills the remote-output description of a fused gather's handle (gather == 2); enabled = 0 otherwise.
struct GemmRemoteOut;
struct GemmPushIn;
int remote_out_of(const fmoe_arrival_t* departure, GemmRemoteOut* ro);
// The same for the handle of a scatter that the consuming product performs itself (gather == 3).
int push_in_of(const fmoe_arrival_t* arrival, GemmRemoteOut* ro, GemmPushIn* ps);

// Device address of the status word that bounded waits raise (per device).
int* device_status_ptr();
void peer_release(Comm* c);

#define FMOE_NCCL_TRY(expr)                                                              \
    do {                                                                                 \
        ncclResult_t r__ = (expr);                                                       \
        if (r__ != ncclSuccess)                                                          \
            return ::fmoe::fail(FMOE_ERR_NCCL, "%s failed: %s", #expr,                   \
                                ::fmoe::g_nccl.GetErrorString(r__));                     \
    } while (0)

// Row-range copies between up to two source and two destination buffers in one
// kernel launch per ~160 ranges (used to turn per-peer staging into the
// expert-major layout and back).  sel picks buffer 0 or 1.
struct SegCopy { int src_sel, dst_sel; int64_t src_row, dst_row, rows; };
int launch_segment_copies(const std::vector<SegCopy>& copies, const void* src0, const void* src1, void* dst0,
                          void* dst1, int64_t row_bytes, cudaStream_t st);

// Row moves of global_scatter for this rank (see fmoe_plan_global_scatter).
int plan_scatter(const int64_t* lec, const int64_t* gec, const uint8_t* stored, int rank, int E, int W,
                 std::vector<fmoe_move_t>& moves, int64_t* recv_rows, int64_t* send_rows);

}  // namespace fmoe
