/*
 * fmoe_b200.h -- C ABI of libfmoe_b200.so, the sm_100a implementation of the
 * FasterMoE mixture-of-experts layer hot path.
 *
 * Every entry point below replaces one operator that the reference registers
 * in its pybind11 module `fmoe_cuda` (cuda/fmoe_cuda.cpp:105-130) or one torch
 * index op that the reference's Python glue issues between those operators.
 * The citation on each declaration names the reference interface it stands for.
 *
 * Conventions
 *   - plain pointers and sizes only; no torch types.
 *   - pointers are DEVICE pointers unless the parameter name ends in `_host`.
 *   - nothing here allocates device memory or synchronises the host with the
 *     device unless the comment says so; all work is queued on `stream`.
 *   - return value: 0 on success, a negative FMOE_ERR_* code on failure; the
 *     text of the last failure on the calling thread is returned by
 *     fmoe_last_error_string().  Nothing in the library calls exit().
 *   - count vectors use the reference's index convention
 *     idx = expert + worker * n_expert   (cuda/global_exchange.cuh:84,101).
 */
#ifndef FMOE_B200_H
#define FMOE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* fmoe_stream_t; /* a cudaStream_t */
typedef void* fmoe_comm_t;   /* opaque communicator created by fmoe_comm_init */

enum {
    FMOE_OK = 0,
    FMOE_ERR_INVALID = -1,     /* bad argument (null pointer, size, alignment, dtype) */
    FMOE_ERR_CUDA = -2,        /* a CUDA runtime/driver call failed */
    FMOE_ERR_NCCL = -3,        /* an NCCL call failed or NCCL could not be loaded */
    FMOE_ERR_UNSUPPORTED = -4, /* shape outside what the kernels handle */
    FMOE_ERR_MISMATCH = -5     /* count vectors inconsistent with buffer sizes */
};

enum { FMOE_F32 = 0, FMOE_F16 = 1, FMOE_BF16 = 2 };
enum { FMOE_ACT_NONE = 0, FMOE_ACT_RELU = 1, FMOE_ACT_GELU = 2 };

const char* fmoe_last_error_string(void);
/* Library version, and the compute capability it was built for (100). */
int fmoe_version(void);
/* sizeof() of a struct of this header as the library was built ("fmoe_move_t", "fmoe_peer_seg_t", "fmoe_arrival_t",
 * "fmoe_mlp_params_t", "fmoe_fused_geometry_t"; 0 for an unknown name): lets a binding check its own declarations. */
size_t fmoe_abi_sizeof(const char* struct_name);
int fmoe_built_for_sm(void);
/* Reads the status word that the tensor-core kernels raise when one of their
 * bounded waits expires (0 = none; 1..4 = which wait; 7 = misaligned shared memory;
 * 8 = segment offsets that overshot the buffer or ran backwards were clamped; bits 16
 * and 32: waits of the peer-memory exchange).  Copies from the device,
 * so it waits for the work queued before it.  No counterpart in the reference. */
int fmoe_device_status(int32_t* status_out);
/* Sets the status word back to 0 (after the caller has dealt with an expired wait). */
int fmoe_device_status_clear(void);
/* Which kernels fmoe_linear_forward / fmoe_linear_backward use for 16-bit tensors whose shapes
 * the tensor-core kernels take: AUTO picks CTA pairs (256-row tiles) or single CTAs by size,
 * PAIR / SINGLE force one of them, SIMT forces the FFMA kernels.  Process-wide; the initial
 * value comes from the environment (FMOE_B200_GEMM=pair|tc1|simt), read once.  Tests use it to
 * cross-check the forms.  The reference has one form (cuBLAS, cuda/parallel_linear.cuh:73-145). */
enum { FMOE_GEMM_AUTO = 0, FMOE_GEMM_PAIR = 1, FMOE_GEMM_SINGLE = 2, FMOE_GEMM_SIMT = 3 };
int fmoe_gemm_set_form(int32_t form);
/* Upper bound on the SMs the persistent tensor-core GEMM grids occupy (0: all), so that kernels
 * on other streams (the token exchange) find free SMs beside them.  Process-wide; initial value
 * from FMOE_B200_GEMM_SMS, read once.  No counterpart in the reference. */
int fmoe_gemm_set_sm_limit(int32_t n_sms);

/* ------------------------------------------------------------------------
 * Gate top-k                                         (selection: bit-exact)
 * ---------------------------------------------------------------------- */

/* The torch.topk(gate, k, largest=True, sorted=False) call of the reference's
 * gates (fmoe/gates/naive_gate.py:31-34) and its backward.
 *   logits  [n_tokens, n_expert_total] of dtype (FMOE_F32/F16/BF16), device
 *   values  [n_tokens, k] same dtype: the k largest logits of each token, copied
 *   indices [n_tokens, k] int64: their expert indices
 * Order inside a token: descending value; equal values by ascending index; NaN
 * ranks above every number (as torch.topk does).  1 <= k <= 8.
 * Backward: grad_logits [n_tokens, n_expert_total] = zeros with grad_values
 * scattered to the selected columns (every element is written). */
int fmoe_gate_topk(const void* logits, int64_t n_tokens, int32_t n_expert_total, int32_t k,
                   int32_t dtype, void* values, int64_t* indices, fmoe_stream_t stream);
int fmoe_gate_topk_backward(const void* grad_values, const int64_t* indices, int64_t n_tokens,
                            int32_t n_expert_total, int32_t k, int32_t dtype, void* grad_logits,
                            fmoe_stream_t stream);

/* ------------------------------------------------------------------------
 * Routing: counting, bucketing, capacity            (integer work, bit-exact)
 * ---------------------------------------------------------------------- */

/* Upper bound on n_expert_total accepted by the routing kernels. */
#define FMOE_MAX_EXPERTS 4096

/* Bytes of scratch that the bucketing kernels below need for `n` gate entries
 * and `n_expert_total` experts (per-tile histograms). */
size_t fmoe_routing_scratch_bytes(int64_t n, int32_t n_expert_total);

/* expert_count(gate_idx, expert_count): cuda/fmoe_cuda.cpp:52-54,
 * cuda/local_exchange.cu:22-32.  Adds, for every entry of gate_idx[0..n) that
 * is not -1, one to expert_count[gate_idx[i]].  expert_count is int32 and is
 * accumulated into (the caller zero-fills it, as fmoe/functions.py:21-24). */
int fmoe_expert_count(const int64_t* gate_idx, int32_t* expert_count,
                      int64_t n, int32_t n_expert_total, fmoe_stream_t stream);

/* assign_pos(cum_count, gate, pos): cuda/fmoe_cuda.cpp:48-51,
 * cuda/local_exchange.cu:5-20.  cum_count is the inclusive prefix sum of the
 * expert counts; segment e of pos, [cum[e]-cnt[e], cum[e]), receives the flat
 * indices i with gate[i]==e.  Inside a segment the reference's order is the
 * arrival order of atomics; this library always writes ascending i, which is
 * one of the orders the reference can produce.  Like the reference, cum_count
 * is consumed: on return it holds cum[e]-cnt[e].
 * scratch: fmoe_routing_scratch_bytes(n, n_expert_total) bytes. */
int fmoe_assign_pos(int32_t* cum_count, const int64_t* gate, int64_t* pos,
                    int64_t n, int32_t n_expert_total, void* scratch,
                    fmoe_stream_t stream);

/* Fused replacement of the sequence in count_by_gate (fmoe/functions.py:19-41):
 * expert_count -> .long() -> cumsum -> assign_pos, without the host read of
 * the total.  Outputs (any may be NULL except pos):
 *   lec64[E_tot]      counts as int64
 *   offsets[E_tot+1]  exclusive prefix sum as int64 (offsets[E_tot] = #kept)
 *   pos[n]            bucketed flat indices; entries past offsets[E_tot] are -1
 *   inv[n]            inverse: inv[i] = row of flat index i in pos, -1 if gate[i]==-1
 */
int fmoe_count_and_pos(const int64_t* gate, int64_t n, int32_t n_expert_total,
                       int64_t* lec64, int64_t* offsets, int64_t* pos, int64_t* inv,
                       void* scratch, fmoe_stream_t stream);

/* Same result as fmoe_count_and_pos, for callers that may not allocate device
 * memory on this path and therefore have no scratch buffer to pass (a server
 * whose memory pool owns all free HBM, a plugin host that keeps cudaMalloc off
 * its request path).  Has no counterpart in the reference.  The scratch is a
 * fixed array of FMOE_STATIC_SCRATCH_BYTES inside the library, resident on every
 * GPU that loads the library until the process exits; the call allocates nothing.
 *   - Limit: fmoe_routing_scratch_bytes(n, n_expert_total) must not exceed
 *     fmoe_static_scratch_capacity() (e.g. 1 Mi entries x 256 experts, or
 *     16 Mi entries x 16 experts); larger requests return FMOE_ERR_UNSUPPORTED.
 *   - The first call on a device looks up the array's device address
 *     (cudaGetSymbolAddress, with that device current); make that first call
 *     before starting any stream capture.
 *   - All calls on a device share the one array: two calls whose kernels can
 *     overlap on the GPU (different streams, no ordering) race on it.  Calls
 *     ordered on one stream are safe; nothing needs clearing between them. */
#define FMOE_STATIC_SCRATCH_BYTES (4u * 1024u * 1024u + 64u * 1024u)
size_t fmoe_static_scratch_capacity(void);
int fmoe_count_and_pos_static(const int64_t* gate, int64_t n, int32_t n_expert_total,
                              int64_t* lec64, int64_t* offsets, int64_t* pos, int64_t* inv,
                              fmoe_stream_t stream);

/* limit_by_capacity(expert_count, capacity, n_expert, n_worker):
 * cuda/fmoe_cuda.cpp:72-74, cuda/balancing.cu:7-20.  For each local expert e,
 * sources w are served in ascending order: eca[w*E+e] = min(ec[w*E+e], what is
 * left of cap[e]).  cap[e] is decremented by the sum of all requests, as the
 * reference's atomicSub does. */
int fmoe_limit_by_capacity(const int64_t* ec, int32_t* cap, int64_t* eca,
                           int32_t n_expert, int32_t n_worker, fmoe_stream_t stream);

/* prune_gate_by_capacity(gate_idx, expert_count, n_expert, n_worker):
 * cuda/fmoe_cuda.cpp:75-77, cuda/balancing.cu:22-37.  The first ec[e] entries
 * (lowest flat index) routed to expert e keep their value, the others become
 * -1; ec[e] is decremented by the number of entries routed to e.  Entries that
 * are already -1 stay -1 and are not counted (the reference leaves that case
 * undefined). */
int fmoe_prune_gate_by_capacity(const int64_t* gate_idx, int64_t* new_gate_idx,
                                int32_t* ec, int64_t n, int32_t n_expert_total,
                                void* scratch, fmoe_stream_t stream);

/* ------------------------------------------------------------------------
 * Token permutation                                  (byte copies, bit-exact)
 * ---------------------------------------------------------------------- */

/* _local_scatter: fmoe/functions.py:72-74 (torch.index_select).
 * out[i,:] = inp[pos[i] / pos_div, :] for i in [0,n_rows).  The reference's
 * callers pass pos//top_k (fmoe/layers.py:136); pos_div performs that division
 * inside the kernel.  row_bytes = d_model * element size. */
int fmoe_local_scatter(const void* inp, const int64_t* pos, void* out,
                       int64_t n_rows, int64_t n_inp_rows, int64_t row_bytes,
                       int32_t pos_div, fmoe_stream_t stream);

/* _local_gather with maybe_overlap=False: fmoe/functions.py:77-84
 * (zeros + index_copy_).  out has n_out_rows rows; out[pos[i],:] = buf[i,:],
 * every other row is zero.  inv_scratch: n_out_rows int64 (inverse map built
 * here) so that each output row is written exactly once. */
int fmoe_local_gather(const void* buf, const int64_t* pos, void* out,
                      int64_t n_rows, int64_t n_out_rows, int64_t row_bytes,
                      int64_t* inv_scratch, fmoe_stream_t stream);

/* Same as fmoe_local_gather when the caller already holds the inverse map
 * (inv[r] = source row or -1), e.g. from fmoe_count_and_pos. */
int fmoe_local_gather_inv(const void* buf, const int64_t* inv, void* out,
                          int64_t n_out_rows, int64_t row_bytes, fmoe_stream_t stream);

/* _local_gather with maybe_overlap=True as used by MOEScatter.backward:
 * fmoe/functions.py:77-84,232-248 (zeros + index_add_ at pos//top_k).
 * out[t,:] = sum_j buf[inv[t*top_k+j],:] over the j with inv >= 0, added in
 * ascending j in fp32 (the reference adds with atomics in arbitrary order). */
int fmoe_local_gather_sum(const void* buf, const int64_t* inv, void* out,
                          int64_t n_tokens, int32_t top_k, int64_t d, int32_t dtype,
                          fmoe_stream_t stream);

/* _local_gather with maybe_overlap=True for an arbitrary index vector: fmoe/functions.py:77-81
 * (zeros + index_add_).  out has n_out_rows rows of d elements; out[pos[i],:] += buf[i,:] over
 * i in [0,n_rows), rows that nothing maps to are zero, entries of pos outside [0,n_out_rows)
 * are skipped.  Rows that collide on one output row are added in ascending i in fp32 (torch
 * adds with floating-point atomics in arrival order).  scratch:
 * fmoe_local_gather_add_scratch_bytes(n_out_rows) bytes, 16-byte aligned. */
size_t fmoe_local_gather_add_scratch_bytes(int64_t n_out_rows);
int fmoe_local_gather_add(const void* buf, const int64_t* pos, void* out, int64_t n_rows,
                          int64_t n_out_rows, int64_t d, int32_t dtype, void* scratch,
                          fmoe_stream_t stream);

/* Weighted combine: fmoe/layers.py:319-322 (bmm of score[T,1,k] with x[T,k,d]),
 * optionally fused with the preceding local gather (inv != NULL):
 *   out[t,:] = sum_j score[t,j] * src_row(t*k+j),
 *   src_row(r) = inv ? (inv[r] >= 0 ? buf[inv[r]] : 0) : buf[r].
 * score has the dtype of buf. */
int fmoe_combine_forward(const void* buf, const int64_t* inv, const void* score,
                         void* out, int64_t n_tokens, int32_t top_k, int64_t d,
                         int32_t dtype, fmoe_stream_t stream);

/* Backward of fmoe_combine_forward:
 *   grad_buf[inv[r],:] = score[r] * grad_out[r / k,:]   (rows of grad_buf are
 *       indexed through inv when inv != NULL, else grad_buf[r,:]),
 *   grad_score[t,j]    = dot(grad_out[t,:], src_row(t*k+j))   (may be NULL). */
int fmoe_combine_backward(const void* grad_out, const void* buf, const int64_t* inv,
                          const void* score, void* grad_buf, void* grad_score,
                          int64_t n_tokens, int32_t top_k, int64_t d, int32_t dtype,
                          fmoe_stream_t stream);

/* ------------------------------------------------------------------------
 * Grouped expert GEMM (fmoe_linear)
 * ---------------------------------------------------------------------- */

/* Bytes of scratch that fmoe_linear_backward_colsum needs (fp32 partial column sums of the
 * input gradient, one row per 32-row block); fmoe_linear_backward accepts the same buffer
 * or NULL. */
size_t fmoe_linear_scratch_bytes(int64_t n_rows, int64_t in_feat, int64_t out_feat,
                                 int32_t n_expert, int32_t dtype);

/* linear_forward(input, expert_count, weight, bias): cuda/fmoe_cuda.cpp:57-62,
 * cuda/parallel_linear.cu:5-49.  For each expert e with rows
 * [seg_offsets[e], seg_offsets[e+1]):  Y = X * W_e^T (+ b_e), then the optional
 * activation (the reference applies its activation as a separate torch call,
 * fmoe/transformer.py:28).  X [n_rows,in_feat], W [E,out_feat,in_feat],
 * bias [E,out_feat] or NULL, Y [n_rows,out_feat], all row-major, dtype as given;
 * accumulation is fp32.  seg_offsets: DEVICE int64[E+1], exclusive prefix sum
 * of the reference's expert_count.  pre_act (may be NULL; used with GELU):
 * receives activation'(z) of the value z before the activation, in the tensor
 * dtype -- the factor the backward of the activation multiplies by, computed
 * here where z is still in registers. */
int fmoe_linear_forward(const void* x, const void* weight, const void* bias,
                        const int64_t* seg_offsets, void* y, void* pre_act,
                        int64_t n_rows, int64_t in_feat, int64_t out_feat,
                        int32_t n_expert, int32_t dtype, int32_t activation,
                        fmoe_stream_t stream);

/* linear_backward(grad_out, input, expert_count, weight, bias):
 * cuda/fmoe_cuda.cpp:63-69, cuda/parallel_linear.cu:52-94.
 *   dX[seg_e] = dY[seg_e] * W_e           [n_rows,in_feat]
 *   dW_e      = dY[seg_e]^T * X[seg_e]    [E,out_feat,in_feat]  (zero if empty)
 *   db_e      = column sums of dY[seg_e]  [E,out_feat]          (NULL to skip)
 * Any of grad_x, grad_w, grad_b may be NULL to skip that product.
 * When act_pre [n_rows,in_feat] != NULL, dX is multiplied element-wise by the
 * derivative of the activation that produced x before it is stored (the
 * reference runs this as a separate kernel, cuda/fused_compute.cuh:155, or
 * leaves it to autograd).  For FMOE_ACT_RELU act_pre is the activation OUTPUT
 * (the factor is 1 where it is > 0); for FMOE_ACT_GELU it is the derivative
 * buffer that fmoe_linear_forward wrote through pre_act.
 * accumulate != 0 adds into dW/db instead of overwriting them (what the smart
 * schedule's later pipeline steps do, cuda/fused_compute.cuh:120). */
int fmoe_linear_backward(const void* grad_y, const void* x, const void* weight,
                         const int64_t* seg_offsets, const void* act_pre,
                         void* grad_x, void* grad_w, void* grad_b,
                         int64_t n_rows, int64_t in_feat, int64_t out_feat,
                         int32_t n_expert, int32_t dtype, int32_t activation,
                         int32_t accumulate, void* scratch, fmoe_stream_t stream);

/* fmoe_linear_backward that also returns the per-expert column sums of grad_x
 * (grad_x_colsum [n_expert, in_feat], same dtype; needs grad_x): when x is the output of
 * another expert layer, that is that layer's bias gradient, and the tensor-core
 * input-gradient kernel produces it from the output blocks it stages anyway (fp32 partial
 * sums per 32-row block in `scratch`, added in block order: deterministic), which saves
 * the separate pass over grad_x that the reference makes (cuda/parallel_linear.cuh:
 * column_reduce).  No counterpart in the reference. */
int fmoe_linear_backward_colsum(const void* grad_y, const void* x, const void* weight,
                                const int64_t* seg_offsets, const void* act_pre, void* grad_x,
                                void* grad_w, void* grad_b, void* grad_x_colsum, int64_t n_rows,
                                int64_t in_feat, int64_t out_feat, int32_t n_expert, int32_t dtype,
                                int32_t activation, int32_t accumulate, void* scratch,
                                fmoe_stream_t stream);

/* ------------------------------------------------------------------------
 * Expert-parallel exchange over NCCL
 * ---------------------------------------------------------------------- */

/* Replaces ensure_nccl (cuda/fmoe_cuda.cpp:44, cuda/global_exchange.cu:84-119):
 * rank 0 obtains a 128-byte id, the host program broadcasts it (any channel),
 * and every rank calls fmoe_comm_init with the CUDA device it computes on. */
int fmoe_comm_unique_id(void* id128_host);
int fmoe_comm_init(const void* id128_host, int32_t rank, int32_t world_size,
                   int32_t device, fmoe_comm_t* comm_out);
int fmoe_comm_destroy(fmoe_comm_t comm);
int fmoe_comm_rank(fmoe_comm_t comm, int32_t* rank_out, int32_t* world_out);

/* expert_exchange(local_expert_count, n_expert, n_workers):
 * cuda/fmoe_cuda.cpp:8-10, cuda/global_exchange.cu:8-24.
 * aec[src][dst][e] = all-gather of lec; agec[dst][src][e] = its transpose;
 * gec = agec[rank].  All int64 on the device. */
int fmoe_expert_exchange(fmoe_comm_t comm, const int64_t* lec, int64_t* aec,
                         int64_t* agec, int64_t* gec, int32_t n_expert,
                         int32_t n_workers, fmoe_stream_t stream);

/* One entry of an exchange plan: `rows` rows move from row offset src_row of
 * the source buffer to row offset dst_row of the destination buffer.
 * peer == rank means a copy inside this GPU. */
typedef struct {
    int32_t peer;
    int32_t is_send;  /* 1: this rank sends src rows to peer; 0: receives into dst */
    int64_t src_row;  /* valid when is_send or local */
    int64_t dst_row;  /* valid when !is_send or local */
    int64_t rows;
    int32_t local;    /* 1: device-to-device copy on this GPU */
    int32_t step;     /* smart-schedule pipeline step the move belongs to (0 if unused) */
} fmoe_move_t;

/* Host-only planning of global_scatter (cuda/global_exchange.cuh:60-144): which
 * row ranges go where, including the rows kept local for shadowed experts.
 * Writes at most max_moves entries and returns the count in *n_moves, the
 * number of rows of the receive buffer in *recv_rows.  The plan of
 * global_gather (cuda/global_exchange.cuh:146-230) is the same list with
 * source and destination swapped.  Touches no GPU. */
int fmoe_plan_global_scatter(const int64_t* lec_host, const int64_t* gec_host,
                             const uint8_t* stored_models_host, int32_t rank,
                             int32_t n_expert, int32_t n_workers,
                             fmoe_move_t* moves, int32_t max_moves,
                             int32_t* n_moves, int64_t* recv_rows);

/* global_scatter / global_gather: cuda/fmoe_cuda.cpp:11-22,
 * cuda/global_exchange.cu:26-80.  Counts and flags are HOST pointers, as in the
 * reference.  The whole exchange is one NCCL group.  out_rows is checked
 * against the plan (FMOE_ERR_MISMATCH) before anything is queued.
 * global_gather zero-fills local_out rows that receive nothing.
 * staging (may be NULL): a device buffer of the expert-side size (out_rows rows
 * for scatter, in_rows rows for gather).  With it each peer is served by one
 * send and one receive (rows to a peer are contiguous on the token side; rows
 * from a peer land contiguously in staging) and one copy kernel produces the
 * expert-major layout; without it every (expert, peer) segment is its own
 * send/receive, as in the reference.  All ranks must make the same choice
 * (pass a buffer, of at least one row, on every rank or on none). */
int fmoe_global_scatter(fmoe_comm_t comm, const void* local_in, void* global_out,
                        const int64_t* lec_host, const int64_t* gec_host,
                        const uint8_t* stored_models_host, int64_t in_rows,
                        int64_t out_rows, int64_t row_bytes, int32_t n_expert,
                        int32_t n_workers, void* staging, fmoe_stream_t stream);
int fmoe_global_gather(fmoe_comm_t comm, const void* global_in, void* local_out,
                       const int64_t* lec_host, const int64_t* gec_host,
                       const uint8_t* stored_models_host, int64_t in_rows,
                       int64_t out_rows, int64_t row_bytes, int32_t n_expert,
                       int32_t n_workers, void* staging, fmoe_stream_t stream);

/* Peer-memory form of the two exchanges above (no counterpart in the reference,
 * which always goes through ncclSend/ncclRecv, cuda/global_exchange.cuh:75-124, and needs the
 * counts on the host): rows are stored straight into the destination GPU's memory over NVLink
 * by a copy kernel and published with flags; no NCCL call is made, and the row plan is built on
 * the device, so the host never has to read the counts.
 *
 * fmoe_peer_enable is collective over the communicator: every rank allocates a landing area
 * (4 MiB of flags, count tables and scratch; 2 slots of slot_bytes; an optional receive pool of
 * pool_bytes), the ranks swap CUDA IPC handles and map each other's areas.  If any rank cannot
 * (no peer access, IPC closed to the process), the form stays off on every rank and FMOE_OK is
 * returned; fmoe_peer_slot_bytes then reports 0.  This call allocates device memory and
 * synchronises; nothing else in this section does.
 *
 * The kernels of one communicator keep their epochs in device memory and must be queued in one
 * total order (one stream, or streams ordered by events), the same order on every rank.  Waits
 * on other ranks are bounded (FMOE_B200_PEER_TIMEOUT_MS, default 20000): an expired wait
 * raises bit 16 or 32 of fmoe_device_status, rows for a peer that never announced are dropped;
 * bit 64: a rank had no room for the rows routed to it (nothing was stored out of bounds). */
#define FMOE_PEER_UNAVAILABLE 1
typedef struct {
    int32_t dst_rank, reserved;
    int64_t src_row, dst_row, rows;
} fmoe_peer_seg_t;
int fmoe_peer_enable(fmoe_comm_t comm, int64_t slot_bytes, int64_t pool_bytes, fmoe_stream_t stream);
int64_t fmoe_peer_slot_bytes(fmoe_comm_t comm);
/* Receive pool (pool_bytes > 0 above): a region of the same peer-mapped allocation out of which a
 * host can allocate the OUTPUT buffers of the exchanges; rows then land in the output directly
 * instead of in a slot from which they are copied once more.  fmoe_pool_alloc / fmoe_pool_free have
 * the signature torch.cuda.memory.CUDAPluggableAllocator expects (first-fit sub-allocation of the
 * region, NULL when it is exhausted); fmoe_peer_pool_bytes: its size. */
int64_t fmoe_peer_pool_bytes(fmoe_comm_t comm);
void* fmoe_pool_alloc(ptrdiff_t size, int device, void* stream);
void fmoe_pool_free(void* ptr, ptrdiff_t size, int device, void* stream);

/* The plan of a layer call's exchanges, built on the device.  It stands for the five host copies
 * and the host-side pointer arithmetic of prepare_forward + global_scatter / global_gather
 * (fmoe/functions.py:45-69, cuda/global_exchange.cuh:60-230).
 *   plan: device buffer of fmoe_peer_plan_bytes(n_expert, n_workers) bytes, 64-byte aligned; it
 *     must stay alive until the last exchange that uses it (forward and backward) has run.
 *   fmoe_peer_plan_exchange: collective.  lec = this rank's local expert counts [W*E] (device);
 *     the ranks write them into each other's landing areas (no NCCL), so afterwards every rank
 *     holds the full table [W][W][E].  stored_models (device, may be NULL = none) = shadowed
 *     experts [W*E], identical on all ranks.  cap_rows = rows of this rank's expert-side buffers
 *     (< 0: unchecked); if any rank would receive more, every rank's plan comes out empty and bit
 *     64 is raised on all of them.  Returns FMOE_PEER_UNAVAILABLE when the form is off.
 *   fmoe_peer_plan_from_table: the same plan for `rank` from a full table already on the device
 *     (e.g. the one fmoe_expert_exchange gathered); caps (device, [W], may be NULL).  Not
 *     collective, needs no communicator.
 * At byte fmoe_peer_plan_offsets_at() of the plan: int64 [n_expert+1], the row offsets of this
 * rank's experts in its expert-side buffer (the seg_offsets of fmoe_linear_*; valid when none of
 * this rank's own experts is shadowed).  At fmoe_peer_plan_table_at(): the table, int64 [W][W][E].
 * fmoe_peer_plan_read decodes one list of a plan that was copied to the host (list 0: rows the
 * push kernel of global_scatter moves, 1: rows its consume kernel copies out of a slot, 2 and 3:
 * the same for global_gather); dst_rank == n_workers means "stays on this GPU". */
size_t fmoe_peer_plan_bytes(int32_t n_expert, int32_t n_workers);
int64_t fmoe_peer_plan_offsets_at(int32_t n_expert, int32_t n_workers);
int64_t fmoe_peer_plan_table_at(int32_t n_expert, int32_t n_workers);
int fmoe_peer_plan_exchange(fmoe_comm_t comm, const int64_t* lec, const uint8_t* stored_models,
                            int64_t cap_rows, void* plan, int32_t n_expert, fmoe_stream_t stream);
int fmoe_peer_plan_from_table(const int64_t* all_expert_count, const uint8_t* stored_models,
                              const int64_t* caps, int32_t rank, int32_t n_expert, int32_t n_workers,
                              void* plan, fmoe_stream_t stream);
int fmoe_peer_plan_read(const void* plan_host, int32_t n_expert, int32_t n_workers, int32_t list,
                        fmoe_peer_seg_t* segs, int32_t max_segs, int32_t* n_segs, int64_t* expert_rows,
                        int64_t* token_rows, int32_t* overflow);
/* global_scatter / global_gather (cuda/global_exchange.cu:26-80) driven by such a plan.  in_rows /
 * out_rows are the rows of the buffers as allocated: they may exceed what the counts describe
 * (buffers sized for the worst case); a buffer that is too small makes this rank refuse the rows
 * (bit 64).  The gather clears token-side rows past the ones the counts describe.  Returns
 * FMOE_PEER_UNAVAILABLE when the form is off. */
int fmoe_peer_scatter_planned(fmoe_comm_t comm, const void* local_in, void* global_out, const void* plan,
                              int64_t in_rows, int64_t out_rows, int64_t row_bytes, int32_t n_expert,
                              fmoe_stream_t stream);
/* fmoe_peer_scatter_planned whose token-side rows are produced on the way instead of being read from a
 * buffer: row i (i < in_rows entries of row_of) is  src[row_of[i] / row_div]  (scale NULL: the local
 * scatter of fmoe/functions.py:72-74 with the division by top_k folded in), or that row times
 * scale[row_of[i]] rounded once to `dtype` (the gradient rows of the gate-score combine,
 * fmoe/layers.py:319-322 backward).  src has src_rows rows; an index outside it drops the row and raises
 * status bit 8.  scale has the rows' dtype.  One pass over the data where local scatter + exchange make two. */
int fmoe_peer_scatter_planned_rows(fmoe_comm_t comm, const void* src, int64_t src_rows, const int64_t* row_of,
                                   int32_t row_div, const void* scale, int32_t dtype, void* global_out,
                                   const void* plan, int64_t in_rows, int64_t out_rows, int64_t row_bytes,
                                   int32_t n_expert, fmoe_stream_t stream);
int fmoe_peer_gather_planned(fmoe_comm_t comm, const void* global_in, void* local_out, const void* plan,
                             int64_t in_rows, int64_t out_rows, int64_t row_bytes, int32_t n_expert,
                             fmoe_stream_t stream);
/* global_scatter overlapped with the grouped GEMM that consumes its rows (the smart schedule's aim,
 * cuda/fused_compute.cuh:289-349, without splitting the GEMM into per-step launches).  The push runs
 * on a stream of the communicator's own, on overlap_sms SMs, and publishes per (source rank, expert)
 * when that expert's rows from that source are complete; fmoe_linear_forward_overlapped /
 * fmoe_linear_backward_overlapped, queued on `stream` right after this call and given the handle,
 * leave overlap_sms SMs free and let each tile wait (bounded; status code 5 on expiry) only for the
 * sources whose rows it reads.  fmoe_peer_arrival_finish, queued on `stream` after that GEMM, joins
 * the push and closes the exchange; no other exchange of the communicator may be queued in between.
 * Falls back, on every rank alike only if every rank passes the same overlap_sms, to the plain
 * exchange queued whole on `stream` (arrival->comm == NULL: nothing to wait for or to finish) when
 * global_out does not lie in the receive pool or overlap_sms is 0. */
typedef struct {
    fmoe_comm_t comm;      /* NULL: the exchange was queued whole, nothing is pending */
    const void* plan;
    void* out;
    int64_t in_rows, out_rows, row_bytes;
    int32_t n_expert, overlap_sms;
    int32_t gather, use;   /* gather: 0 scatter pushed by a kernel of its own; 1 fmoe_peer_gather_planned_async (use: which of
                              the plan's two counter sets); 2 fmoe_peer_gather_fused_begin; 3 fmoe_peer_scatter_fused_begin
                              (use 1: the rows have been pushed by the product the handle was given to) */
    /* gather == 3: where the token-side rows come from (as in fmoe_peer_scatter_planned_rows) */
    const void* src;
    const int64_t* row_of;
    const void* scale;
    int64_t src_rows;
    int32_t row_div, dtype;
} fmoe_arrival_t;
int fmoe_peer_scatter_planned_async(fmoe_comm_t comm, const void* local_in, void* global_out, const void* plan,
                                    int64_t in_rows, int64_t out_rows, int64_t row_bytes, int32_t n_expert,
                                    int32_t overlap_sms, fmoe_stream_t stream, fmoe_arrival_t* arrival);
int fmoe_peer_arrival_finish(const fmoe_arrival_t* arrival, fmoe_stream_t stream);
/* global_gather overlapped with the grouped GEMM that PRODUCES its rows.  Queue it on `stream` right
 * BEFORE that GEMM (fmoe_linear_forward_overlapped / fmoe_linear_backward_overlapped with the handle
 * as `departure`): the push starts on the communicator's own stream, on overlap_sms SMs, and forwards
 * an expert's rows as soon as the GEMM's epilogue reports that expert complete (counters inside the
 * plan; `use` 0 or 1 picks one of its two sets, so that the forward and the backward pass of a layer
 * call do not share one).  fmoe_peer_arrival_finish with the handle, queued after the GEMM, joins the
 * push and closes the exchange.  When it cannot overlap (local_out outside the receive pool,
 * overlap_sms 0) it queues NOTHING and leaves departure->comm NULL: the caller then runs
 * fmoe_peer_gather_planned after the GEMM. */
int fmoe_peer_gather_planned_async(fmoe_comm_t comm, const void* global_in, void* local_out, const void* plan,
                                   int64_t in_rows, int64_t out_rows, int64_t row_bytes, int32_t n_expert,
                                   int32_t overlap_sms, int32_t use, fmoe_stream_t stream, fmoe_arrival_t* departure);
/* global_scatter FUSED into the grouped GEMM that consumes its rows: the product queued next with the handle
 * as `arrival` (fmoe_linear_forward_overlapped, or fmoe_linear_backward_overlapped, whose input-gradient
 * product takes it) moves this GPU's token-side rows to the experts' owners with the two spare warps of each
 * of its CTAs while its tensor-core warps already work on the experts whose rows are complete (per
 * (source, expert) arrival flags, bounded waits), and closes the exchange.  The rows are given as in
 * fmoe_peer_scatter_planned_rows (row_of NULL: src holds the token-side rows themselves).  This call only
 * tells the peers where global_out is; global_out must lie in the receive pool.  Replaces
 * cuda/global_exchange.h:60-113 (global_scatter) + the wait for it before the experts' first product.  When
 * it cannot take this form (output outside the pool, more than 32 ranks or 256 experts, rows that are not
 * 16-bit) it queues NOTHING and leaves arrival->comm NULL.  A handle that no product took is closed by
 * fmoe_peer_arrival_finish, which then runs the exchange as fmoe_peer_scatter_planned_rows does. */
int fmoe_peer_scatter_fused_begin(fmoe_comm_t comm, const void* src, int64_t src_rows, const int64_t* row_of,
                                  int32_t row_div, const void* scale, int32_t dtype, void* global_out, const void* plan,
                                  int64_t in_rows, int64_t out_rows, int64_t row_bytes, int32_t n_expert,
                                  fmoe_stream_t stream, fmoe_arrival_t* arrival);
/* global_gather FUSED into the grouped GEMM that produces its rows: the product queued next with the
 * handle as `departure` (fmoe_linear_forward_overlapped, or fmoe_linear_backward_overlapped for the input
 * gradient) stores every output row straight into the token-side buffer of the rank that owns it --
 * local_out [out_rows, row_bytes] on each rank, which must lie in the receive pool -- and writes no
 * expert-side output (the y / grad_x argument of that call may be NULL).  This call only tells the peers
 * where local_out is (one tiny kernel); fmoe_peer_arrival_finish after the product waits, bounded, for the
 * peers' rows and clears what no row covers.  Replaces cuda/global_exchange.h:115-174 (global_gather) plus
 * the store of the expert outputs of cuda/parallel_linear.cuh.  Needs bf16/fp16 rows, at most 32 ranks and
 * a product of `n_expert` groups with n_rows > 0; when local_out is not in the pool it queues NOTHING and
 * leaves departure->comm NULL (departure->gather is 2 otherwise). */
int fmoe_peer_gather_fused_begin(fmoe_comm_t comm, void* local_out, const void* plan, int64_t out_rows,
                                 int64_t row_bytes, int32_t n_expert, fmoe_stream_t stream, fmoe_arrival_t* departure);
/* fmoe_linear_forward / fmoe_linear_backward_colsum (arguments as there) beside an exchange:
 *   arrival (may be NULL): the scatter that is still delivering x (forward) or grad_y (backward).  The
 *     call consumes the handle: the forward closes the exchange after its product, the backward
 *     between the input-gradient product (which waits tile by tile) and the weight- and bias-gradient
 *     products (which need every row).  Shapes the tensor-core kernels do not take close the exchange
 *     first and run as usual.
 *   departure (may be NULL): the gather that forwards y (forward) or grad_x (backward) while the
 *     product runs; the caller closes it with fmoe_peer_arrival_finish afterwards.  All products of the
 *     call leave departure->overlap_sms SMs to the push. */
int fmoe_linear_forward_overlapped(const void* x, const void* weight, const void* bias,
                                   const int64_t* seg_offsets, void* y, void* pre_act, int64_t n_rows,
                                   int64_t in_feat, int64_t out_feat, int32_t n_expert, int32_t dtype,
                                   int32_t activation, const fmoe_arrival_t* arrival,
                                   const fmoe_arrival_t* departure, fmoe_stream_t stream);
int fmoe_linear_backward_overlapped(const void* grad_y, const void* x, const void* weight,
                                    const int64_t* seg_offsets, const void* act_pre, void* grad_x,
                                    void* grad_w, void* grad_b, void* grad_x_colsum, int64_t n_rows,
                                    int64_t in_feat, int64_t out_feat, int32_t n_expert, int32_t dtype,
                                    int32_t activation, int32_t accumulate, void* scratch,
                                    const fmoe_arrival_t* arrival, const fmoe_arrival_t* departure,
                                    fmoe_stream_t stream);
/* The same exchanges with the reference's argument style: all_expert_count_host[W][W][E] (rows that
 * rank s routes to expert e of rank d at [s][d][e]; the table fmoe_expert_exchange gathers) and the
 * flags on the HOST.  The table is uploaded and planned on the device (a call with the same table
 * and flags as the previous one reuses its plan).  They return FMOE_PEER_UNAVAILABLE, having
 * queued nothing, when the form is off, row_bytes is not a multiple of 16, or the largest buffer
 * any rank receives fits neither a landing slot nor a quarter of a receive pool -- a verdict that
 * depends on the shared table only, so it is the same on every rank; the caller then uses
 * fmoe_global_scatter / _gather.  Buffers and row counts mean what they mean there. */
int fmoe_peer_global_scatter(fmoe_comm_t comm, const void* local_in, void* global_out,
                             const int64_t* all_expert_count_host,
                             const uint8_t* stored_models_host, int64_t in_rows,
                             int64_t out_rows, int64_t row_bytes, int32_t n_expert,
                             int32_t n_workers, fmoe_stream_t stream);
int fmoe_peer_global_gather(fmoe_comm_t comm, const void* global_in, void* local_out,
                            const int64_t* all_expert_count_host,
                            const uint8_t* stored_models_host, int64_t in_rows,
                            int64_t out_rows, int64_t row_bytes, int32_t n_expert,
                            int32_t n_workers, fmoe_stream_t stream);
/* Host mirror of the plan (no GPU; for inspection and tests): the row segments of one exchange
 * for `rank`.  push: rows its push kernel stores, dst_rank == n_workers meaning "stays on this
 * GPU, written to the output buffer", else rows src_row.. of its input go to rows dst_row.. of
 * dst_rank's landing place.  pull: rows its consume kernel copies from its own slot (src_row) to
 * its output (dst_row).  reverse = 0: global_scatter, 1: global_gather.  slot_rows: rows of the
 * largest buffer any rank receives.  Pass push = pull = NULL to get the counts only. */
int fmoe_peer_plan(const int64_t* all_expert_count_host, const uint8_t* stored_models_host,
                   int32_t rank, int32_t n_expert, int32_t n_workers, int32_t reverse,
                   fmoe_peer_seg_t* push, int32_t* n_push, fmoe_peer_seg_t* pull, int32_t* n_pull,
                   int32_t max_segs, int64_t* slot_rows);
/* Queues one block of the exchange's push (push != 0) or consume step that waits, for at most
 * timeout_ms, for an epoch that no peer will ever publish: when the wait expires the kernel raises
 * bit 16 (push) or 32 (consume) of fmoe_device_status and returns; it announces nothing, stores
 * nothing and leaves the exchange state untouched.  Lets a host check that its handling of an
 * expired wait works without a peer having to fail. */
int fmoe_peer_wait_probe(fmoe_comm_t comm, int32_t timeout_ms, int32_t push, fmoe_stream_t stream);
/* Limit of the waits on other ranks in the kernels queued from now on (initially
 * FMOE_B200_PEER_TIMEOUT_MS or 20000). */
int fmoe_peer_set_timeout_ms(fmoe_comm_t comm, int32_t timeout_ms);

/* exchange_cache_info(sent_models, num_expert, world_size):
 * cuda/fmoe_cuda.cpp:24-27, cuda/global_exchange.cuh:232-249.  All-gather of
 * n_expert flag bytes per rank. */
int fmoe_exchange_cache_info(fmoe_comm_t comm, const uint8_t* sent_models,
                             uint8_t* stored_models, int32_t n_expert,
                             int32_t n_workers, fmoe_stream_t stream);

/* model_exchange: cuda/fmoe_cuda.cpp:28-32, cuda/global_exchange.cuh:251-282.
 * One broadcast of `bytes` bytes rooted at `root`; buf is the owner's flat
 * parameter buffer on the root and the shadow buffer elsewhere. */
int fmoe_model_broadcast(fmoe_comm_t comm, void* buf, int64_t bytes, int32_t root,
                         fmoe_stream_t stream);

/* gradient_exchange: cuda/fmoe_cuda.cpp:38-42, cuda/global_exchange.cuh:285-348.
 * In-place sum-reduce of `count` elements to `root`. */
int fmoe_gradient_reduce(fmoe_comm_t comm, void* buf, int64_t count, int32_t dtype,
                         int32_t root, fmoe_stream_t stream);

/* generate_cached_count: cuda/fmoe_cuda.cpp:33-37, cuda/global_exchange.cu:175-196.
 * out[w*E+e] = lec[w*E+e]*stored[w*E+e]; out[rank*E+e] += sum_w gec[w*E+e] when
 * stored[rank*E+e] is false.  All device pointers; int64 counts, byte flags. */
int fmoe_generate_cached_count(const int64_t* lec, const int64_t* gec,
                               const uint8_t* stored_models, int64_t* out,
                               int32_t rank, int32_t n_expert, int32_t n_workers,
                               fmoe_stream_t stream);

/* ------------------------------------------------------------------------
 * Smart schedule: pipelined exchange + two-layer expert MLP
 * ---------------------------------------------------------------------- */

typedef struct {
    const void* w1;  /* [E, d_hidden, d_model] */
    const void* w2;  /* [E, d_model, d_hidden] */
    const void* b1;  /* [E, d_hidden] or NULL  */
    const void* b2;  /* [E, d_model]  or NULL  */
    void* gw1;       /* gradients, same shapes; used by fused_backward only */
    void* gw2;
    void* gb1;
    void* gb2;
} fmoe_mlp_params_t;

/* Row offsets that the smart schedule uses (cuda/fused_compute.cuh:216-248):
 * local_ptr[i] = exclusive prefix of lec; global_ptr[e*W+w] = exclusive prefix,
 * expert-major then source, of the rows this rank still receives;
 * local_global_ptr[i] = exclusive prefix of the rows kept local for shadowed
 * experts.  Each output has E*W+1 entries.  Host-only. */
int fmoe_fused_compute_ptrs(const int64_t* lec_host, const int64_t* gec_host,
                            const uint8_t* stored_models_host, int32_t rank,
                            int32_t n_expert, int32_t n_workers,
                            int64_t* local_ptr, int64_t* global_ptr,
                            int64_t* local_global_ptr);

/* Geometry of one smart-schedule call, computed on the host from the counts. */
typedef struct {
    int32_t n_steps;      /* pipeline steps = n_workers / gran */
    int32_t gran;         /* peers exchanged per step: the largest divisor of n_workers
                             that is <= the requested pipeline_gran (the reference silently
                             drops ranks when n_workers is not a multiple,
                             cuda/fused_compute.cuh:276-279) */
    int64_t global_rows;  /* B: rows this rank receives for its own experts */
    int64_t shadow_rows;  /* S: rows kept on this rank for shadowed experts */
} fmoe_fused_geometry_t;

int fmoe_fused_geometry(const int64_t* lec_host, const int64_t* gec_host,
                        const uint8_t* stored_models_host, int32_t rank, int32_t n_expert,
                        int32_t n_workers, int32_t pipeline_gran, fmoe_fused_geometry_t* out);

/* fused_forward: cuda/fmoe_cuda.cpp:80-87, cuda/fused_compute.cu:12-62,
 * cuda/fused_compute.cuh:250-388.  params_host[w] is the parameter set of
 * worker w's experts (own experts at index rank; shadows where stored_models
 * says so; other entries are ignored).  Buffers are allocated by the caller:
 *   local_in, local_out [A, d_model]      token-side rows, ordered by (worker, expert)
 *   global_in, global_out [B+S, d_model]  expert-side rows: [0,B) received, expert-major
 *                                         then source; [B,B+S) rows of shadowed experts
 *   middle [B+S, d_hidden]                activation output; middle_pre: derivative of the
 *                                         activation (written and needed for GELU, else NULL)
 * with B, S from fmoe_fused_geometry.  The exchange with the peers of step s is
 * queued on comm_stream, the expert GEMMs of step s on `stream` once its rows have
 * arrived, and the results travel back as each step finishes.  On return all work
 * is queued and `stream` waits for comm_stream.  staging (may be NULL): B rows of
 * d_model; with it and more than one expert per worker every peer is served by one
 * send and one receive per step plus a copy kernel, instead of one per expert
 * (pass it on every rank or on none, also on a rank with B = 0).
 * Unlike the reference (ReLU only,
 * no bias) the activation is selectable and biases are applied when non-NULL.
 * comm may be NULL when n_workers == 1. */
int fmoe_fused_forward(fmoe_comm_t comm, const void* local_in, void* local_out,
                       void* global_in, void* middle, void* middle_pre, void* global_out,
                       const fmoe_mlp_params_t* params_host,
                       const int64_t* lec_host, const int64_t* gec_host,
                       const uint8_t* stored_models_host, int64_t local_rows,
                       int64_t d_model, int64_t d_hidden, int32_t n_expert,
                       int32_t n_workers, int32_t dtype, int32_t activation,
                       int32_t pipeline_gran, void* staging, fmoe_stream_t stream,
                       fmoe_stream_t comm_stream);

/* fused_backward: cuda/fmoe_cuda.cpp:88-100, cuda/fused_compute.cu:64-131,
 * cuda/fused_compute.cuh:391-542.  global_in, middle, middle_pre are the buffers
 * the forward filled; global_grad_out [B+S,d], grad_middle [B+S,h] and
 * global_grad_in [B+S,d] are work buffers.  Weight (and bias) gradients go to
 * params_host[w].g*: the own experts' are overwritten by the first pipeline step
 * and accumulated by the later ones; shadowed experts' are accumulated into
 * (the caller zero-fills them), as in the reference. */
int fmoe_fused_backward(fmoe_comm_t comm, const void* grad_out_local, void* grad_in_local,
                        const void* global_in, const void* middle, const void* middle_pre,
                        void* global_grad_out, void* grad_middle, void* global_grad_in,
                        const fmoe_mlp_params_t* params_host,
                        const int64_t* lec_host, const int64_t* gec_host,
                        const uint8_t* stored_models_host, int64_t local_rows,
                        int64_t d_model, int64_t d_hidden, int32_t n_expert,
                        int32_t n_workers, int32_t dtype, int32_t activation,
                        int32_t pipeline_gran, void* staging, fmoe_stream_t stream,
                        fmoe_stream_t comm_stream);

#ifdef __cplusplus
}
#endif
#endif /* FMOE_B200_H */
