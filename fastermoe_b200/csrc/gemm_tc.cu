// Grouped expert GEMM on the 5th-generation tensor cores (tcgen05 + TMEM + TMA).
//
// One persistent, warp-specialised kernel per product of the reference's
// fmoe_linear (cuda/parallel_linear.cuh:55-161, where each is a loop of cuBLAS
// calls, one per expert):
//
//   FWD    Y[m,n]     = sum_k X[m,k]  W_e[n,k]   (+bias, activation)   m ragged per expert
//   DGRAD  dX[m,k]    = sum_n dY[m,n] W_e[n,k]   (* saved act. derivative) m ragged per expert
//   WGRAD  dW_e[n,k]  = sum_m dY[m,n] X[m,k]                           contraction ragged
//
// CTA = 18 warps: warp 0 issues TMA loads (one lane), warp 1 issues tcgen05.mma
// (one lane; the whole warp helps to zero ragged tails for WGRAD), warps 2-17
// drain the accumulator from TMEM (tcgen05.ld; four warps per 32-lane quarter,
// each taking 64 of the 256 columns), apply the epilogue and store through a
// per-warp staging buffer so that rows are written in contiguous 64-byte pieces.
// Tile 128 x 256 x 64 (bf16/fp16 in, fp32 accumulate), 4 shared-memory stages of
// 48 KB, two 256-column TMEM accumulators so that the epilogue of a tile overlaps
// the main loop of the next one.  Operands are staged with the 128-byte swizzle;
// K-major operands use one 64x(128|256) box, MN-major operands (the transposed
// reads of DGRAD/WGRAD) are fetched as 64x64 boxes laid 8 KB apart, which is the
// canonical MN-major layout of the UMMA shared-memory descriptor.
//
// The work list is derived on the device from the expert segment offsets, so
// the host never reads the counts.  Every mbarrier wait is bounded: on expiry
// the kernel raises a status word, drains and exits (see fmoe_device_status).
#include "common.cuh"
#include "gemm.h"
#include <cuda.h>
#include <algorithm>
#include <atomic>
#include <cstdlib>
#include <mutex>

namespace fmoe {
namespace {

constexpr int BM = 128, BN = 256, BK = 64;
constexpr int A_BYTES = BM * BK * 2;    // 16 KB: the CTA's 128 rows of A
constexpr int SUB_BYTES = 64 * BK * 2;  // one 64x64 box: 8 KB
constexpr int RING_BYTES = 192 * 1024;  // operand ring of one CTA
constexpr int MAX_STAGES = 6;

// One CTA per tile (128 x 256), or a pair of CTAs per tile (256 x 256, cta_group::2):
// in a pair each CTA holds its own 128 rows of A and 128 of the 256 B columns, so
// the bytes a CTA pulls from L2 per flop drop by a third.
template <bool CTA2> struct Cfg {
    static constexpr int B_COLS = CTA2 ? 128 : 256;          // B columns (tile N) staged by this CTA
    static constexpr int B_BYTES = B_COLS * BK * 2;          // 16 or 32 KB
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;    // 32 or 48 KB
    static constexpr int STAGES = RING_BYTES / STAGE_BYTES;  // 6 or 4
    static constexpr int TILE_M = CTA2 ? 256 : 128;          // tile rows across the CTA group
};
constexpr int MAX_EXPERTS_TC = 128;
// Warp roles.  Warps 0..3: 0 = TMA producer, 1 = MMA issuer, 2-3 idle (they keep the
// epilogue warps aligned to the TMEM lane quarters); warps 4..19 drain the accumulators.
// The epilogues are bound by instruction issue (a warp issues at most every other cycle
// on dependent code), so there are four epilogue warps per scheduler, each handling 32
// columns at a time so that 640 threads x 96 registers fit the register file without spills.
constexpr int EPI_WARPS = 16;                // EPI_WARPS/4 per TMEM lane quarter, splitting the 256 columns
constexpr int FIRST_EPI_WARP = 4;
constexpr int CW = 32;                       // columns handled per epilogue iteration (32 or 64)
constexpr int STAGING_BYTES = 32 * CW * 2;  // per epilogue warp: 32 rows x CW columns of 16-bit values
constexpr int COLS_PER_WARP = BN / (EPI_WARPS / 4);
constexpr int THREADS = (FIRST_EPI_WARP + EPI_WARPS) * 32;
constexpr int TMEM_COLS = 512;
constexpr unsigned long long WAIT_LIMIT_CYCLES = 4000000000ull;  // ~2 s at 1.9 GHz

enum { MODE_FWD = 0, MODE_DGRAD = 1, MODE_WGRAD = 2 };

struct Params {
    const int64_t* seg;  // [n_expert + 1]
    int n_expert;
    int n_out;    // output columns (FWD: out_feat, DGRAD: in_feat, WGRAD: in_feat)
    int n_contr;  // contraction length for FWD/DGRAD (WGRAD: ragged, from seg)
    int w_rows;   // rows of one expert's weight matrix (out_feat): B row offset per expert
    int out_rows_per_expert;  // WGRAD: out_feat
    void* out;
    void* pre_out;        // FWD only
    const void* bias;     // FWD only
    const void* act_pre;  // DGRAD only
    int act;
    int accumulate;  // WGRAD only
    int is_bf16;
    float* colsum;  // DGRAD: fp32 partial column sums of the output, one row per 32-row block, or null
    int tma_store;  // outputs have tensor maps: full 32-row blocks leave through TMA stores
    int* status;  // device status word
    int64_t n_rows;  // rows of the ragged-side buffers (FWD/DGRAD: A and the output; WGRAD: both operands)
    // FWD/DGRAD whose A rows are still arriving from other GPUs (null: they are all there)
    const unsigned long long* arr_flags;
    const unsigned long long* arr_seq;
    const int* arr_src_off;
    int arr_world;
    // FWD/DGRAD whose output rows are forwarded while the product runs (null: nobody is waiting)
    int* done;
    int* done_expected;
    int* done_ready;
};

struct Shared {
    // full: the operands of a stage have landed (TMA; in a pair, both CTAs' operands, counted on
    // the leader's barrier).  empty: the MMAs reading the stage have completed.
    unsigned long long full[MAX_STAGES], empty[MAX_STAGES], tmem_full[2], tmem_empty[2];
    uint32_t tmem_base;
    int abort;
    int cum_tiles[MAX_EXPERTS_TC + 1];
    int blk_base[MAX_EXPERTS_TC + 1];  // DGRAD with column sums: 32-row blocks before each expert
    int seg_lo[MAX_EXPERTS_TC], seg_hi[MAX_EXPERTS_TC];
    unsigned long long rem_dest[kRemoteMaxWorld];   // remote output: where each rank receives (0: it never announced)
};

__device__ int g_status = 0;

// Tensor maps of the outputs (box: 32 rows x 32 columns, 64-byte swizzle = the layout of the
// epilogue's staging buffers): `out`, and the forward's second output (saved derivative).
struct OutMaps { CUtensorMap out, out2; };

// ---- PTX wrappers ------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(unsigned long long* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(unsigned long long* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned long long* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(unsigned long long* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false (and raises the status word) when the barrier did
// not complete within the limit or another role has already given up.
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, uint32_t parity, Shared* sh, int* status, int code) {
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = clock64();
    while (true) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*(volatile int*)&sh->abort) return false;
        if (clock64() - t0 > WAIT_LIMIT_CYCLES) {
            *(volatile int*)&sh->abort = 1;
            atomicCAS(status, 0, code);
            return false;
        }
    }
}
// Bounded wait for rows that another GPU delivers: flag >= epoch.  Raises status code 5 on expiry.
__device__ __forceinline__ bool arrival_wait(const unsigned long long* flag, unsigned long long epoch, Shared* sh, int* status) {
    unsigned long long v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(flag) : "memory");
    if (v >= epoch) return true;
    const unsigned long long t0 = clock64();
    while (true) {
        asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(flag) : "memory");
        if (v >= epoch) return true;
        if (*(volatile int*)&sh->abort) return false;
        if (clock64() - t0 > WAIT_LIMIT_CYCLES) {
            *(volatile int*)&sh->abort = 1;
            atomicCAS(status, 0, 5);
            return false;
        }
        __nanosleep(100);
    }
}
// --- cluster (CTA pair) helpers ---
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Address of the same shared-memory object in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_cta(const void* p, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_u32(p)), "r"(rank));
    return r;
}
__device__ __forceinline__ void st_cluster_zero16(uint32_t cluster_addr) {
    asm volatile("st.shared::cluster.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(cluster_addr), "r"(0) : "memory");
}
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(unsigned long long* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait on a barrier that CTAs of the cluster arrive on.
__device__ __forceinline__ bool mbar_wait_cluster(unsigned long long* bar, uint32_t parity, Shared* sh, int* status, int code) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    const unsigned long long t0 = clock64();
    while (true) {
        if (mbar_try_wait_cluster(bar, parity)) return true;
        if (*(volatile int*)&sh->abort) return false;
        if (clock64() - t0 > WAIT_LIMIT_CYCLES) {
            *(volatile int*)&sh->abort = 1;
            atomicCAS(status, 0, code);
            return false;
        }
    }
}
// Completion of all MMAs issued so far by this thread -> arrive on the barrier at the
// same shared-memory offset in both CTAs of the pair.
__device__ __forceinline__ void tc_commit_pair(unsigned long long* bar) {
    asm volatile(
        "{\n\t.reg .b16 m;\n\tmov.b16 m, 3;\n\t"
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], m;\n\t}"
        ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_mma_pair(uint32_t tmem_c, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_c), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ void tma_load_2d(const CUtensorMap* map, unsigned long long* bar, void* dst, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}
// Pair form: the bytes land in this CTA's shared memory, the completion is counted on a
// barrier that may live in the other CTA of the pair (bar_cluster: shared::cluster address).
__device__ __forceinline__ void tma_load_2d_pair(const CUtensorMap* map, uint32_t bar_cluster, void* dst, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(bar_cluster), "r"(x), "r"(y)
        : "memory");
}
// Bulk store of one staging buffer (smem, written by this warp) to the tile of `map` at (x, y).
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* src, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(map), "r"(smem_u32(src)), "r"(x), "r"(y) : "memory");
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
// The bulk stores issued by this thread have finished READING shared memory.
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(unsigned long long* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_mma(uint32_t tmem_c, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_c), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t* v) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
          "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
          "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor for tcgen05.mma (128-byte swizzle).
//   bits [0,14)  start address >> 4      bits [16,30) leading byte offset >> 4
//   bits [32,46) stride byte offset >> 4 bits [46,48) version = 1
//   bits [61,64) layout type, 2 = SWIZZLE_128B
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr >> 4) & 0x3FFF);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// Instruction descriptor, kind::f16: fp32 accumulate, A/B both bf16 or both fp16.
//   [4,6) C format (1 = f32)  [7,10) A format  [10,13) B format (0 = f16, 1 = bf16)
//   [15] A major (1 = MN)  [16] B major (1 = MN)  [17,23) N >> 3  [24,29) M >> 4
__host__ __device__ constexpr uint32_t make_idesc(bool bf16, bool a_mn, bool b_mn, int m) {
    return (1u << 4) | ((bf16 ? 1u : 0u) << 7) | ((bf16 ? 1u : 0u) << 10) | ((a_mn ? 1u : 0u) << 15) |
           ((b_mn ? 1u : 0u) << 16) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// ---- packed fp32 arithmetic ----------------------------------------------------
// sm_100 executes add/mul/fma on two fp32 values held in one 64-bit register pair
// (fma.rn.f32x2 ...).  The epilogues are bound by instruction issue (two epilogue warps
// per scheduler), so they do their per-element math on column pairs.
typedef unsigned long long f32x2;
__device__ __forceinline__ f32x2 pk(float lo, float hi) {
    f32x2 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ f32x2 pk1(float c) { return pk(c, c); }
__device__ __forceinline__ void unpk(f32x2 v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) {
    f32x2 d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b) {
    f32x2 d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ f32x2 add2(f32x2 a, f32x2 b) {
    f32x2 d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ float rcp_approx(float d) {
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(d));
    return r;
}
__device__ __forceinline__ float ex2_approx(float d) {
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(d));
    return r;
}

// GELU (exact, erf form) and its derivative for the 16-bit epilogues, on a column pair.
//   Phi(x)  = 1/2 + sign(x) (1/2 - T(|x|)),   T(a) = erfc(a / sqrt 2) / 2
//   T(a)    = (b1 t + ... + b5 t^5) exp(-a^2 / 2),   t = 1 / (1 + p a / sqrt 2)
// is Abramowitz-Stegun 7.1.26 (|error| of erf <= 1.5e-7) with the halving folded into
// the coefficients.  The exponential is the one the density needs, so value and
// derivative  gelu'(x) = Phi(x) + x exp(-x^2/2) / sqrt(2 pi)  share everything:
// two special-function instructions and ~10 packed operations per pair.  Absolute
// error 5e-7 (value), 3e-7 (derivative): far below bf16/fp16 resolution.
template <bool GRAD>
__device__ __forceinline__ void gelu_pair(f32x2 x, f32x2& val, f32x2& grad) {
    const f32x2 ax = x & 0x7fffffff7fffffffull;
    float d0, d1, u0, u1;
    unpk(fma2(ax, pk1(0.23164189f), pk1(1.f)), d0, d1);
    const f32x2 t = pk(rcp_approx(d0), rcp_approx(d1));
    unpk(mul2(mul2(x, pk1(-0.72134752f)), x), u0, u1);          // -x^2/2 in base 2
    const f32x2 e = pk(ex2_approx(u0), ex2_approx(u1));
    f32x2 q = fma2(pk1(0.5307027145f), t, pk1(-0.7265760135f));
    q = fma2(q, t, pk1(0.7107068705f));
    q = fma2(q, t, pk1(-0.142248368f));
    q = fma2(q, t, pk1(0.127414796f));
    const f32x2 tail = mul2(mul2(q, t), e);
    const f32x2 inner = fma2(tail, pk1(-1.f), pk1(0.5f));         // 1/2 - T >= 0
    const f32x2 cdf = add2(inner | (x & 0x8000000080000000ull), pk1(0.5f));
    val = mul2(x, cdf);
    if (GRAD) grad = fma2(mul2(x, pk1(0.39894228f)), e, cdf);
}
__device__ __forceinline__ float gelu_fast(float x) {
    f32x2 v, g;
    gelu_pair<false>(pk(x, x), v, g);
    float lo, hi;
    unpk(v, lo, hi);
    return lo;
}
__device__ __forceinline__ float act_fast(float v, int act) {
    if (act == FMOE_ACT_RELU) return v > 0.f ? v : 0.f;
    if (act == FMOE_ACT_GELU) return gelu_fast(v);
    return v;
}
// Two 16-bit values of one 32-bit word as a packed fp32 pair.
template <bool BF16> __device__ __forceinline__ f32x2 cvt_in2(uint32_t w) {
    if (BF16) return pk(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
    const __half2 h = *reinterpret_cast<const __half2*>(&w);
    const float2 f = __half22float2(h);
    return pk(f.x, f.y);
}
template <bool BF16> __device__ __forceinline__ float cvt_in(uint16_t raw) {
    if (BF16) return __uint_as_float((uint32_t)raw << 16);
    return __half2float(__ushort_as_half(raw));
}
template <bool BF16> __device__ __forceinline__ uint32_t cvt_pack(float lo, float hi) {
    if (BF16) {
        __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<uint32_t*>(&v);
    }
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// ---- epilogue staging ----------------------------------------------------------
// A warp's staging buffer holds 32 rows of CW 16-bit values (NCH = CW/8 chunks of 16
// bytes).  Chunk j of row r sits at slot j ^ f(r), f chosen so that both access
// patterns are free of bank conflicts: lane = row (register side) and NCH lanes per
// row (global-memory side, CW*2 contiguous bytes per row).
constexpr int NCH = CW / 8;
__device__ __forceinline__ int stage_slot(int row, int j) {
    return row * NCH + (NCH == 8 ? (j ^ (row & 7)) : (j ^ ((row >> 1) & 3)));
}

template <bool BF16>
__device__ __forceinline__ void stage_put(uint4* stage, int lane, const float* v) {
#pragma unroll
    for (int q = 0; q < NCH; ++q)
        stage[stage_slot(lane, q)] =
            make_uint4(cvt_pack<BF16>(v[q * 8], v[q * 8 + 1]), cvt_pack<BF16>(v[q * 8 + 2], v[q * 8 + 3]),
                       cvt_pack<BF16>(v[q * 8 + 4], v[q * 8 + 5]), cvt_pack<BF16>(v[q * 8 + 6], v[q * 8 + 7]));
    __syncwarp();
}
// staging -> global: rows [0, rows) of the block, CW columns starting at dst.
__device__ __forceinline__ void stage_store(const uint4* stage, int lane, uint16_t* dst, size_t ld, int rows) {
    constexpr int RPI = 32 / NCH;  // rows per instruction
    const int j = lane % NCH;
#pragma unroll
    for (int it = 0; it < 32 / RPI; ++it) {
        const int row = it * RPI + lane / NCH;
        if (row < rows) *reinterpret_cast<uint4*>(dst + (size_t)row * ld + j * 8) = stage[stage_slot(row, j)];
    }
    __syncwarp();
}
// CW values of this lane's own row (contiguous), or zeros when the row is absent.
__device__ __forceinline__ void row_load(uint4* q, const uint16_t* src, bool valid) {
#pragma unroll
    for (int i = 0; i < NCH; ++i) q[i] = valid ? __ldg(reinterpret_cast<const uint4*>(src) + i) : make_uint4(0, 0, 0, 0);
}

// ---- the spare warps' job when the product delivers its own input rows (GemmPushIn) ------------------
// Segment k of the push list that holds token-side row `row` (last k with prefix[k] <= row).
__device__ __forceinline__ int push_find_seg(const int* __restrict__ prefix, int n, int row) {
    int lo = 0, hi = n - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (__ldg(prefix + mid) <= row) lo = mid; else hi = mid - 1;
    }
    return lo;
}

template <bool BF16>
__device__ __forceinline__ uint4 push_scale(uint4 v, float w) {
    uint32_t* q = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float lo = w * cvt_in<BF16>((uint16_t)(q[i] & 0xffffu)), hi = w * cvt_in<BF16>((uint16_t)(q[i] >> 16));
        q[i] = cvt_pack<BF16>(lo, hi);
    }
    return v;
}

// Mover `mover` of `movers` (two per CTA, all CTAs of the grid): units of consecutive rows of the push
// list are dealt round-robin, so that at any time all movers work on one stretch of the list and
// experts complete one after the other.  After the stores of a unit the warp fences once, books the rows
// per segment and raises the arrival flag of a (destination, expert) segment that is complete.  Nothing
// here waits for another GPU: a peer that never announced its buffer (rem_dest 0) gets no rows.
template <bool BF16>
__device__ void push_rows(const GemmPushIn& ps, const GemmRemoteOut& ro, const unsigned long long* rem_dest, int mover,
                          int movers, int lane, unsigned long long epoch, int* status) {
    const int S = ps.n_slots, W = ro.world, E = ps.n_expert;
    const bool room = __ldcg(ps.expert_rows) <= ps.out_rows && __ldcg(ps.token_rows) <= ps.in_rows;
    const int total = room ? __ldg(ps.prefix + S) : 0;
    const int par = (int)(epoch & 1);
    const int first_group = (W - 1) * E;              // slots before it hold rows kept for shadowed experts
    auto flag_of = [&](int k) -> unsigned long long* {
        const int q = k - first_group, i = q / W, dst = (ro.rank + q % W) % W;
        if (k < first_group || i >= ps.flag_experts) return nullptr;
        if (dst != ro.rank && rem_dest[dst] == 0ull) return nullptr;
        return (unsigned long long*)(ro.base[dst] + ps.flags_at) + ((size_t)par * ps.flag_sources + ro.rank) * ps.flag_experts + i;
    };
    if (room && mover == 0) {
        // segments without rows: their consumers need not wait
        for (int k = first_group + lane; k < S; k += 32)
            if (__ldg(ps.prefix + k + 1) == __ldg(ps.prefix + k)) {
                unsigned long long* f = flag_of(k);
                if (f) asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(f), "l"(epoch) : "memory");
            }
    }
    // The first round moves small units, so that the first expert's rows are complete (and the tensor-core
    // warps start) early; later rounds move up to 32 rows per unit: a unit ends with a system fence, which
    // waits for the stores in flight (10+ microseconds on a busy link), so there should be few of them.
    const int first_rows = max(4, min(8, total / max(1, movers)));
    const int later_rows = max(8, min(32, (total - first_rows * movers) / max(1, 3 * movers)));
    const int first_span = first_rows * movers;
    bool bad_index = false;
    for (int round = 0;; ++round) {
        const int row_lo = round == 0 ? mover * first_rows : first_span + ((round - 1) * movers + mover) * later_rows;
        if (row_lo >= total) break;
        const int row_hi = min(row_lo + (round == 0 ? first_rows : later_rows), total);
        const int k_lo = push_find_seg(ps.prefix, S, row_lo);
        int row = row_lo, k = k_lo;
        while (row < row_hi && k < S) {
            const int k_beg = __ldg(ps.prefix + k), k_end = __ldg(ps.prefix + k + 1), n = min(row_hi, k_end) - row;
            if (n > 0) {
                const int sel = __ldg(ps.seg_sel + k), dst = sel == ps.local_sel ? ro.rank : sel;
                const unsigned long long dest = rem_dest[dst];
                if (dest) {
                    const int off = row - k_beg;
                    uint4* d = (uint4*)(ro.base[dst] + dest) + (int64_t)(__ldg(ps.seg_dst + k) + off) * ps.row_vecs;
                    const int i0 = __ldg(ps.seg_src + k) + off;
                    // lane l looks up where row l of the piece comes from (n <= 32), once for the whole piece
                    int64_t from_l = -1;
                    float w_l = 1.f;
                    if (lane < n) {
                        const int64_t at = ps.row_of ? __ldg(ps.row_of + i0 + lane) : (int64_t)(i0 + lane);
                        from_l = ps.row_of ? at / ps.row_div : at;
                        if (at < 0 || (ps.row_of && from_l >= ps.src_rows)) { from_l = -1; bad_index = true; }
                        else if (ps.scale) w_l = cvt_in<BF16>(__ldg((const uint16_t*)ps.scale + at));
                    }
                    // two rows at a time, four 16-byte pieces of each per lane in flight
                    for (int r = 0; r < n; r += 2) {
                        const int64_t f0 = __shfl_sync(0xffffffffu, from_l, r), f1 = __shfl_sync(0xffffffffu, from_l, min(r + 1, 31));
                        const float w0 = __shfl_sync(0xffffffffu, w_l, r), w1 = __shfl_sync(0xffffffffu, w_l, min(r + 1, 31));
                        const bool ok0 = f0 >= 0, ok1 = r + 1 < n && f1 >= 0;
                        const uint4* s0 = (const uint4*)ps.src + (ok0 ? f0 : 0) * ps.row_vecs;
                        const uint4* s1 = (const uint4*)ps.src + (ok1 ? f1 : 0) * ps.row_vecs;
                        uint4* d0 = d + (int64_t)r * ps.row_vecs;
                        uint4* d1 = d0 + ps.row_vecs;
                        for (int64_t c = lane; c < ps.row_vecs; c += 128) {
                            uint4 v0[4], v1[4];
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                const bool in = c + 32 * j < ps.row_vecs;
                                v0[j] = in && ok0 ? __ldcg(s0 + c + 32 * j) : make_uint4(0, 0, 0, 0);
                                v1[j] = in && ok1 ? __ldcg(s1 + c + 32 * j) : make_uint4(0, 0, 0, 0);
                            }
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                if (c + 32 * j >= ps.row_vecs) break;
                                if (ok0) d0[c + 32 * j] = ps.scale ? push_scale<BF16>(v0[j], w0) : v0[j];
                                if (ok1) d1[c + 32 * j] = ps.scale ? push_scale<BF16>(v1[j], w1) : v1[j];
                            }
                        }
                    }
                }
                row += n;
            }
            ++k;
        }
        // this unit's stores are ordered before lane 0's fence by the warp barrier; the fence is cumulative
        __syncwarp();
        if (lane == 0) {
            __threadfence_system();
            int row2 = row_lo, k2 = k_lo;
            while (row2 < row_hi && k2 < S) {
                const int k_beg = __ldg(ps.prefix + k2), k_end = __ldg(ps.prefix + k2 + 1), n = min(row_hi, k_end) - row2;
                if (n > 0) {
                    const int before = atomicAdd(ps.seg_done + k2, n);
                    if (before + n == k_end - k_beg) {
                        unsigned long long* f = flag_of(k2);
                        __threadfence_system();   // the other movers' shares were fenced before they were booked
                        if (f) asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(f), "l"(epoch) : "memory");
                    }
                    row2 += n;
                }
                ++k2;
            }
        }
        __syncwarp();
    }
    bad_index = __any_sync(0xffffffffu, bad_index);
    if (bad_index && lane == 0) atomicOr(status, 8);
    if (!room && mover == 0 && lane == 0) atomicOr(status, 64);
}

struct Tile {
    int e, row0, rows, col0, chunks;  // rows/row0: output rows of the tile (FWD/DGRAD: tokens; WGRAD: weight rows)
    int m_lo, m_hi;                   // WGRAD: contraction range
};

// Tile of the CTA group; row0/rows span TILE_M rows (a CTA of a pair takes 128 of them).
template <int MODE, int TILE_M>
__device__ __forceinline__ void locate(const Shared* sh, const Params& p, int tile, int& e_cursor, Tile& t) {
    while (tile >= sh->cum_tiles[e_cursor + 1]) ++e_cursor;
    const int local = tile - sh->cum_tiles[e_cursor];
    const int nt = (p.n_out + BN - 1) / BN;
    t.e = e_cursor;
    const int lo = sh->seg_lo[e_cursor], hi = sh->seg_hi[e_cursor];
    if (MODE == MODE_WGRAD) {
        t.row0 = (local / nt) * TILE_M;
        t.rows = min(TILE_M, p.out_rows_per_expert - t.row0);
        t.col0 = (local % nt) * BN;
        t.m_lo = lo;
        t.m_hi = hi;
        t.chunks = (hi - lo + BK - 1) / BK;
    } else {
        t.row0 = lo + (local / nt) * TILE_M;
        t.rows = min(TILE_M, hi - t.row0);
        t.col0 = (local % nt) * BN;
        t.chunks = (p.n_contr + BK - 1) / BK;
        t.m_lo = t.m_hi = 0;
    }
}

template <int MODE, bool BF16, bool CTA2>
__global__ void __launch_bounds__(THREADS, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const __grid_constant__ HostSegs hs, const __grid_constant__ OutMaps om,
                    const __grid_constant__ GemmRemoteOut ro, const __grid_constant__ GemmPushIn ps, const Params p) {
    using C = Cfg<CTA2>;
    constexpr int STAGES = C::STAGES, STAGE_BYTES = C::STAGE_BYTES, TILE_M = C::TILE_M, B_COLS = C::B_COLS;
    // Pairs: TMA completions of both CTAs go straight to the leader's barriers, so the MMA
    // issuer waits on one barrier and no warp of the second CTA sits in the critical path.
    // (The weight gradient's ragged contraction tail is then patched by the leader in both
    // CTAs' shared memory, see below.)
    constexpr bool DIRECT = CTA2;
    // The operand ring needs 1024-byte alignment (128-byte swizzle atoms).  The dynamic shared
    // memory of a kernel without static shared memory starts on such a boundary; no slack is
    // spent on it, the address is checked below.
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* tiles = smem_raw;
    Shared* sh = (Shared*)(tiles + RING_BYTES + EPI_WARPS * STAGING_BYTES);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // In a pair, CTA 0 (the leader) issues the MMAs for both; each CTA loads its own
    // operands and drains its own 128 accumulator rows.
    const int cta = CTA2 ? (int)cluster_ctarank() : 0;
    const int first_tile = CTA2 ? blockIdx.x / 2 : blockIdx.x;
    const int tile_step = CTA2 ? gridDim.x / 2 : gridDim.x;

    // ---- set-up ---------------------------------------------------------------
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&sh->full[s], 1);
            mbar_init(&sh->empty[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&sh->tmem_full[a], 1);
            mbar_init(&sh->tmem_empty[a], CTA2 ? 2 * EPI_WARPS : EPI_WARPS);
        }
        sh->abort = 0;
        if (smem_u32(smem_raw) & 1023u) {   // never seen; every wait below then ends at once
            sh->abort = 1;
            atomicCAS(p.status, 0, 7);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (threadIdx.x == 0) {
        // Segment offsets come from device memory that no host code has looked at: ranges are made
        // to run forwards and to end inside the buffers (code 8 in the status word when that
        // changed anything), so tile counts, scratch indices and stores stay in bounds.
        const int nt = (p.n_out + BN - 1) / BN;
        int acc = 0, blk = 0;
        int64_t prev_hi = 0;
        bool clamped = false;
        sh->cum_tiles[0] = 0;
        sh->blk_base[0] = 0;
        for (int e = 0; e < p.n_expert; ++e) {
            const int64_t raw_lo = hs.n ? (int64_t)hs.lo[e] : p.seg[e], raw_hi = hs.n ? (int64_t)hs.hi[e] : p.seg[e + 1];
            int64_t lo = raw_lo < prev_hi ? prev_hi : raw_lo;
            if (lo > p.n_rows) lo = p.n_rows;
            int64_t hi = raw_hi < lo ? lo : raw_hi;
            if (hi > p.n_rows) hi = p.n_rows;
            clamped |= lo != raw_lo || hi != raw_hi;
            prev_hi = hi;
            sh->seg_lo[e] = (int)lo;
            sh->seg_hi[e] = (int)hi;
            int mt;
            if (MODE == MODE_WGRAD) mt = (p.out_rows_per_expert + TILE_M - 1) / TILE_M;
            else mt = ((int)(hi - lo) + TILE_M - 1) / TILE_M;
            acc += mt * nt;
            sh->cum_tiles[e + 1] = acc;
            blk += ((int)(hi - lo) + 31) >> 5;
            sh->blk_base[e + 1] = blk;
        }
        if (clamped && blockIdx.x == 0) atomicCAS(p.status, 0, 8);
        if (MODE != MODE_WGRAD && p.done && blockIdx.x == 0) {
            // completions per expert: every epilogue warp of every CTA of the group, once per tile
            for (int e = 0; e < p.n_expert; ++e)
                p.done_expected[e] = (sh->cum_tiles[e + 1] - sh->cum_tiles[e]) * EPI_WARPS * (CTA2 ? 2 : 1);
            __threadfence();
            *(volatile int*)p.done_ready = 1;
        }
    }
    // ro.enabled: 1 = the output rows go to their owners (epilogue), 2 = the input rows are delivered by
    // the spare warps of this kernel on every GPU (ps); both exchange through the peers' announcements.
    const bool peer = MODE != MODE_WGRAD && ro.enabled != 0;
    const bool remote = peer && ro.enabled == 1;
    unsigned long long rem_epoch = 0;
    if (peer) {
        // where every rank wants the rows of this exchange (bounded wait for its announcement)
        rem_epoch = __ldcg(ro.seq) + 1;
        const int par = (int)(rem_epoch & 1);
        const int q = threadIdx.x;
        if (q < ro.world) {
            unsigned long long dest = ro.my_dest;
            if (q != ro.rank) {
                const unsigned long long* flag = ro.header + ro.ann_at / 8 + par * ro.stride + q;
                const unsigned long long t0 = clock64();
                bool there = false;
                while (!there) {
                    unsigned long long v;
                    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(flag) : "memory");
                    there = v >= rem_epoch;
                    if (!there && clock64() - t0 > ro.timeout_cycles) break;
                    if (!there) __nanosleep(100);
                }
                dest = there ? __ldcg(ro.header + ro.dest_at / 8 + par * ro.stride + q) : 0ull;
                if (!there) atomicOr(p.status, 16);
                else if (dest == ~0ull || dest < ro.min_dest) { dest = 0ull; atomicOr(p.status, 64); }   // no room (or a bad offset): its rows are dropped
            }
            sh->rem_dest[q] = dest;
        }
    }
    if (warp == 0) {
        if (CTA2) {
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sh->tmem_base)), "r"(TMEM_COLS) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sh->tmem_base)), "r"(TMEM_COLS) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
    }
    tc_fence_before();
    __syncthreads();
    if (CTA2) cluster_sync_all();  // both CTAs' barriers exist before anything arrives on them
    tc_fence_after();
    const uint32_t tmem_base = sh->tmem_base;
    const int total_tiles = sh->cum_tiles[p.n_expert];

    if (warp == 0) {
        // ---- TMA producer -----------------------------------------------------
        // Lane 0 issues the copies.  When the rows of A are still arriving from other GPUs, the lanes
        // first wait, one source rank each, for the sources whose rows this CTA's part of the tile reads.
        {
            int s = 0, e_cur = 0;
            uint32_t ph = 0;
            bool ok = true;
            const int my_row = cta * BM;      // this CTA's rows inside the tile
            const int my_col = cta * B_COLS;  // this CTA's share of the tile's B columns (pairs)
            const bool arriving = MODE != MODE_WGRAD && p.arr_flags != nullptr;
            unsigned long long epoch = 0;
            int seen_e = -1, next_e = -1;
            bool seen = false;                // this lane's source has delivered its rows of expert seen_e
            unsigned long long next_val = 0;  // its flag for expert next_e, read ahead of need
            if (arriving) epoch = __ldcg(p.arr_seq) + 1;
            for (int tile = first_tile; tile < total_tiles && ok; tile += tile_step) {
                Tile t;
                locate<MODE, TILE_M>(sh, p, tile, e_cur, t);
                if (arriving && t.chunks > 0) {
                    const unsigned long long* my_flags = p.arr_flags + ((size_t)(epoch & 1) * 64 + lane) * 256;
                    // the flag of the expert that comes next was read while the previous tile was being loaded
                    if (t.e != seen_e) { seen = next_e == t.e && next_val >= epoch; seen_e = t.e; }
                    const int r_lo = t.row0 + my_row, r_hi = min(t.row0 + t.rows, r_lo + BM);
                    bool good = true;
                    if (lane < p.arr_world && !seen && r_hi > r_lo) {
                        const int b0 = p.arr_src_off[t.e * p.arr_world + lane], b1 = p.arr_src_off[t.e * p.arr_world + lane + 1];
                        if (b1 > b0 && b0 < r_hi && b1 > r_lo) {
                            good = arrival_wait(my_flags + t.e, epoch, sh, p.status);
                            seen = good;
                        }
                    }
                    good = __all_sync(0xffffffffu, good);
                    if (!good) { ok = false; break; }
                    asm volatile("fence.proxy.async.global;" ::: "memory");   // rows written through the generic proxy, read by TMA
                    if (lane < p.arr_world && t.e + 1 < p.n_expert) {
                        asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(next_val) : "l"(my_flags + t.e + 1) : "memory");
                        next_e = t.e + 1;
                    }
                }
                if (lane == 0)
                for (int ch = 0; ch < t.chunks; ++ch) {
                    if (!(ok = mbar_wait(&sh->empty[s], ph ^ 1, sh, p.status, 1))) break;
                    uint8_t* a_dst = tiles + s * STAGE_BYTES;
                    uint8_t* b_dst = a_dst + A_BYTES;
                    if (DIRECT) {
                        // Both CTAs' bytes are counted on the leader's barrier, which the MMA
                        // issuer waits on: no relay through the other CTA's warps.
                        const uint32_t bar = map_to_cta(&sh->full[s], 0);
                        if (cta == 0) mbar_expect_tx(&sh->full[s], 2 * STAGE_BYTES);
                        if (MODE == MODE_FWD) {
                            tma_load_2d_pair(&map_a, bar, a_dst, ch * BK, t.row0 + my_row);
                            tma_load_2d_pair(&map_b, bar, b_dst, ch * BK, t.e * p.w_rows + t.col0 + my_col);
                        } else if (MODE == MODE_DGRAD) {
                            tma_load_2d_pair(&map_a, bar, a_dst, ch * BK, t.row0 + my_row);
#pragma unroll
                            for (int j = 0; j < B_COLS / 64; ++j)
                                tma_load_2d_pair(&map_b, bar, b_dst + j * SUB_BYTES, t.col0 + my_col + j * 64,
                                                 t.e * p.w_rows + ch * BK);
                        } else {
                            const int m0 = t.m_lo + ch * BK;
#pragma unroll
                            for (int j = 0; j < BM / 64; ++j)
                                tma_load_2d_pair(&map_a, bar, a_dst + j * SUB_BYTES, t.row0 + my_row + j * 64, m0);
#pragma unroll
                            for (int j = 0; j < B_COLS / 64; ++j)
                                tma_load_2d_pair(&map_b, bar, b_dst + j * SUB_BYTES, t.col0 + my_col + j * 64, m0);
                        }
                        if (++s == STAGES) { s = 0; ph ^= 1; }
                        continue;
                    }
                    mbar_expect_tx(&sh->full[s], STAGE_BYTES);
                    if (MODE == MODE_FWD) {
                        tma_load_2d(&map_a, &sh->full[s], a_dst, ch * BK, t.row0 + my_row);
                        tma_load_2d(&map_b, &sh->full[s], b_dst, ch * BK, t.e * p.w_rows + t.col0 + my_col);
                    } else if (MODE == MODE_DGRAD) {
                        tma_load_2d(&map_a, &sh->full[s], a_dst, ch * BK, t.row0 + my_row);
#pragma unroll
                        for (int j = 0; j < B_COLS / 64; ++j)
                            tma_load_2d(&map_b, &sh->full[s], b_dst + j * SUB_BYTES, t.col0 + my_col + j * 64,
                                        t.e * p.w_rows + ch * BK);
                    } else {
                        const int m0 = t.m_lo + ch * BK;
#pragma unroll
                        for (int j = 0; j < BM / 64; ++j)
                            tma_load_2d(&map_a, &sh->full[s], a_dst + j * SUB_BYTES, t.row0 + my_row + j * 64, m0);
#pragma unroll
                        for (int j = 0; j < B_COLS / 64; ++j)
                            tma_load_2d(&map_b, &sh->full[s], b_dst + j * SUB_BYTES, t.col0 + my_col + j * 64, m0);
                    }
                    if (++s == STAGES) { s = 0; ph ^= 1; }
                }
                ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer -------------------------------------------------------
        constexpr bool A_MN = MODE == MODE_WGRAD, B_MN = MODE != MODE_FWD;
        constexpr uint32_t idesc = make_idesc(BF16, A_MN, B_MN, TILE_M);
        // K-major: 8-row groups 1024 B apart, K advance 32 B per UMMA_K=16.
        // MN-major: 64-element column blocks 8 KB apart (leading), 8-row K groups 1024 B apart (stride),
        //           K advance 16 rows x 128 B = 2048 B.
        constexpr uint32_t A_LBO = A_MN ? SUB_BYTES : 16, A_ADV = A_MN ? 2048 : 32;
        constexpr uint32_t B_LBO = B_MN ? SUB_BYTES : 16, B_ADV = B_MN ? 2048 : 32;
        int s = 0, e_cur = 0, acc = 0;
        uint32_t ph = 0, acc_ph = 0;
        bool ok = true;
        const bool leader = cta == 0;
        for (int tile = first_tile; tile < total_tiles && ok; tile += tile_step) {
            Tile t;
            locate<MODE, TILE_M>(sh, p, tile, e_cur, t);
            if (t.chunks == 0) continue;
            if (DIRECT && !leader) continue;
            if (leader) {
                if (!(ok = mbar_wait_cluster(&sh->tmem_empty[acc], acc_ph ^ 1, sh, p.status, 2))) break;
                tc_fence_after();
            }
            const uint32_t tmem_c = tmem_base + acc * BN;
            for (int ch = 0; ch < t.chunks; ++ch) {
                if (!(ok = mbar_wait(&sh->full[s], ph, sh, p.status, 3))) break;
                tc_fence_after();
                uint8_t* a_src = tiles + s * STAGE_BYTES;
                uint8_t* b_src = a_src + A_BYTES;
                int k_steps = BK / 16;  // UMMA_K = 16 rows of the chunk per instruction
                if (MODE == MODE_WGRAD) {
                    // Rows of the chunk past the end of the expert's segment belong to the next
                    // expert (or are uninitialised).  K steps that lie entirely past the end are
                    // not issued; in the one step that straddles it the rows past the end are
                    // cleared in both operands (a row is one 128-byte line per 64-column block,
                    // whatever the swizzle).
                    const int valid = t.m_hi - (t.m_lo + ch * BK);
                    if (valid < BK) {
                        k_steps = (valid + 15) >> 4;
                        const int row_end = k_steps << 4;
                        constexpr int BLOCKS = (BM + B_COLS) / 64;  // blocks of A then B are contiguous
                        for (int blk = 0; blk < BLOCKS; ++blk)
                            for (int r = valid + (lane >> 3); r < row_end; r += 4) {
                                uint8_t* dst = a_src + blk * SUB_BYTES + r * 128 + (lane & 7) * 16;
                                *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
                                // pairs: the same rows of the other CTA's operands, through distributed shared memory
                                if (CTA2) st_cluster_zero16(map_to_cta(dst, 1));
                            }
                        if (CTA2) asm volatile("fence.proxy.async;" ::: "memory");
                        else asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                        __syncwarp();
                    }
                }
                if (lane == 0) {
                    const uint64_t adesc = make_desc(smem_u32(a_src), A_LBO, 1024);
                    const uint64_t bdesc = make_desc(smem_u32(b_src), B_LBO, 1024);
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k) {
                        if (k >= k_steps) break;
                        const uint64_t ad = adesc + (uint64_t)((k * A_ADV) >> 4), bd = bdesc + (uint64_t)((k * B_ADV) >> 4);
                        const uint32_t accum = (ch > 0 || k > 0) ? 1u : 0u;
                        if (CTA2) tc_mma_pair(tmem_c, ad, bd, idesc, accum);
                        else tc_mma(tmem_c, ad, bd, idesc, accum);
                    }
                    if (CTA2) tc_commit_pair(&sh->empty[s]);
                    else tc_commit(&sh->empty[s]);
                }
                __syncwarp();
                if (++s == STAGES) { s = 0; ph ^= 1; }
            }
            if (!ok) break;
            if (leader) {
                if (lane == 0) {
                    if (CTA2) tc_commit_pair(&sh->tmem_full[acc]);
                    else tc_commit(&sh->tmem_full[acc]);
                }
                __syncwarp();
            }
            if (++acc == 2) { acc = 0; acc_ph ^= 1; }
        }
    } else if (warp < FIRST_EPI_WARP) {
        // ---- spare warps: the scatter that delivers this product's input rows -------------------
        if (peer && ro.enabled == 2)
            push_rows<BF16>(ps, ro, sh->rem_dest, (int)blockIdx.x * 2 + (warp - 2), (int)gridDim.x * 2, lane, rem_epoch, p.status);
    } else if (warp >= FIRST_EPI_WARP) {
        // ---- epilogue ----------------------------------------------------------
        const int quarter = warp & 3;    // TMEM lanes [32*quarter, +32) are readable by this warp
        const int cgrp = (warp - FIRST_EPI_WARP) >> 2;  // which COLS_PER_WARP of the tile's 256 columns
        const int r = quarter * 32 + lane;
        uint4* stage = reinterpret_cast<uint4*>(tiles + STAGES * STAGE_BYTES) + (warp - FIRST_EPI_WARP) * (STAGING_BYTES / 16);
        int e_cur = 0, acc = 0;
        uint32_t acc_ph = 0;
        bool ok = true;
        const uint32_t tmem_empty_addr[2] = {CTA2 ? map_to_cta(&sh->tmem_empty[0], 0) : 0u,
                                             CTA2 ? map_to_cta(&sh->tmem_empty[1], 0) : 0u};
        for (int tile = first_tile; tile < total_tiles && ok; tile += tile_step) {
            Tile t;
            locate<MODE, TILE_M>(sh, p, tile, e_cur, t);
            // this CTA's 128 rows of the tile
            t.row0 += cta * BM;
            t.rows = min(BM, t.rows - cta * BM);
            const size_t ld = (size_t)p.n_out;
            const int col_lo = t.col0 + cgrp * COLS_PER_WARP;  // this warp's first column
            if (t.chunks == 0) {
                // WGRAD of an expert without rows: the gradient is zero.
                if (!p.accumulate && r < t.rows && col_lo < p.n_out) {
                    uint16_t* zrow = (uint16_t*)p.out + ((size_t)t.e * p.out_rows_per_expert + t.row0 + r) * ld + col_lo;
#pragma unroll
                    for (int c = 0; c < COLS_PER_WARP; c += 8)
                        if (col_lo + c < p.n_out) *reinterpret_cast<uint4*>(zrow + c) = make_uint4(0, 0, 0, 0);
                }
                continue;
            }
            // Rows of this warp: tile rows [32*quarter, +32).  Stores go through the warp's
            // staging buffer so that 4 lanes write 64 contiguous bytes of a row.
            const int rows_here = min(32, t.rows - quarter * 32);  // <= 0: nothing to store
            const bool active = rows_here > 0 && col_lo < p.n_out;
            // Full 32-row blocks leave through TMA stores; ragged ones (the end of an expert's
            // segment: the rows below belong to the next expert) through per-row stores.
            const bool bulk = p.tma_store && rows_here == 32 && !remote;
            // remote output: where this lane's row (tile row 32*quarter + lane) goes
            unsigned long long my_rowptr = 0ull;
            if (remote && active && lane < rows_here) {
                const int r_abs = t.row0 + quarter * 32 + lane;
                const int* so = ro.src_off + t.e * ro.world;
                int j_lo = 0, j_hi = ro.world - 1;              // the block (expert, source j) that holds r_abs
                while (j_lo < j_hi) {
                    const int mid = (j_lo + j_hi) >> 1;
                    if (so[mid + 1] > r_abs) j_hi = mid; else j_lo = mid + 1;
                }
                const unsigned long long dest = sh->rem_dest[j_lo];
                if (dest)
                    my_rowptr = (unsigned long long)(ro.base[j_lo] + dest) +
                                ((unsigned long long)(ro.dst_off[t.e * ro.world + j_lo] + (r_abs - so[j_lo])) * ld) * 2ull;
            }
            const bool row_ok = r < t.rows;
            const size_t row_off = (MODE == MODE_WGRAD ? (size_t)t.e * p.out_rows_per_expert : 0) + t.row0;
            uint16_t* out_blk = (uint16_t*)p.out + (row_off + quarter * 32) * ld + col_lo;  // block origin
            // Operands of the epilogue that do not depend on the accumulator are fetched
            // before waiting for it: bias (FWD), pre-activation (DGRAD), old gradient (WGRAD).
            const uint16_t* aux_src = nullptr;
            bool aux_row = false;
            if (MODE == MODE_FWD && p.bias) { aux_src = (const uint16_t*)p.bias + (size_t)t.e * ld + col_lo; aux_row = true; }
            if (MODE == MODE_DGRAD && p.act_pre) { aux_src = (const uint16_t*)p.act_pre + (row_off + r) * ld + col_lo; aux_row = row_ok; }
            if (MODE == MODE_WGRAD && p.accumulate) { aux_src = (const uint16_t*)p.out + (row_off + r) * ld + col_lo; aux_row = row_ok; }
            uint4 aux[NCH];
            if (aux_src && active) row_load(aux, aux_src, aux_row);
            if (!(ok = mbar_wait(&sh->tmem_full[acc], acc_ph, sh, p.status, 4))) break;
            tc_fence_after();
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BN + cgrp * COLS_PER_WARP;
            if (active) {
                for (int c = 0; c < COLS_PER_WARP / CW; ++c) {
                    if (col_lo + c * CW >= p.n_out) break;
                    uint32_t raw[CW];
                    tc_ld32(taddr + c * CW, raw);
                    if (CW == 64) tc_ld32(taddr + c * CW + 32, raw + 32);
                    if (c > 0 && aux_src) row_load(aux, aux_src + c * CW, aux_row);
                    tc_wait_ld();
                    float* v = reinterpret_cast<float*>(raw);
                    const uint4* aq = aux;
                    if (MODE == MODE_FWD) {
                        if (p.bias) {
#pragma unroll
                            for (int q = 0; q < NCH; ++q) {
                                const uint32_t w[4] = {aq[q].x, aq[q].y, aq[q].z, aq[q].w};
#pragma unroll
                                for (int i = 0; i < 4; ++i) {
                                    const f32x2 sum = add2(pk(v[q * 8 + 2 * i], v[q * 8 + 2 * i + 1]), cvt_in2<BF16>(w[i]));
                                    unpk(sum, v[q * 8 + 2 * i], v[q * 8 + 2 * i + 1]);
                                }
                            }
                        }
                        if (p.pre_out && p.act == FMOE_ACT_GELU) {
                            // keep the derivative for the backward, then continue with the value
                            if (p.tma_store) {   // an earlier bulk store may still be reading the buffer
                                if (lane == 0) tma_store_wait_read();
                                __syncwarp();
                            }
#pragma unroll
                            for (int q = 0; q < NCH; ++q) {
                                float g[8];
#pragma unroll
                                for (int i = 0; i < 4; ++i) {
                                    f32x2 val, grad;
                                    gelu_pair<true>(pk(v[q * 8 + 2 * i], v[q * 8 + 2 * i + 1]), val, grad);
                                    unpk(val, v[q * 8 + 2 * i], v[q * 8 + 2 * i + 1]);
                                    unpk(grad, g[2 * i], g[2 * i + 1]);
                                }
                                stage[stage_slot(lane, q)] =
                                    make_uint4(cvt_pack<BF16>(g[0], g[1]), cvt_pack<BF16>(g[2], g[3]),
                                               cvt_pack<BF16>(g[4], g[5]), cvt_pack<BF16>(g[6], g[7]));
                            }
                            __syncwarp();
                            if (bulk) {
                                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                                __syncwarp();
                                if (lane == 0) {
                                    tma_store_2d(&om.out2, stage, col_lo + c * CW, (int)row_off + quarter * 32);
                                    tma_store_wait_read();      // the staging buffer is reused right away
                                }
                                __syncwarp();
                            } else {
                                stage_store(stage, lane, (uint16_t*)p.pre_out + (row_off + quarter * 32) * ld + col_lo + c * CW, ld, rows_here);
                            }
                        } else if (p.act == FMOE_ACT_GELU) {
#pragma unroll
                            for (int i = 0; i < CW / 2; ++i) {
                                f32x2 val, grad;
                                gelu_pair<false>(pk(v[2 * i], v[2 * i + 1]), val, grad);
                                unpk(val, v[2 * i], v[2 * i + 1]);
                            }
                        } else if (p.act != FMOE_ACT_NONE) {
#pragma unroll
                            for (int i = 0; i < CW; ++i) v[i] = act_fast(v[i], p.act);
                        }
                    } else if (MODE == MODE_DGRAD) {
                        if (p.act_pre && p.act == FMOE_ACT_GELU) {
                            // the forward saved gelu'(pre-activation)
#pragma unroll
                            for (int q = 0; q < NCH; ++q) {
                                const uint32_t w[4] = {aq[q].x, aq[q].y, aq[q].z, aq[q].w};
#pragma unroll
                                for (int i = 0; i < 4; ++i) {
                                    const f32x2 prod = mul2(pk(v[q * 8 + 2 * i], v[q * 8 + 2 * i + 1]), cvt_in2<BF16>(w[i]));
                                    unpk(prod, v[q * 8 + 2 * i], v[q * 8 + 2 * i + 1]);
                                }
                            }
                        } else if (p.act_pre) {
#pragma unroll
                            for (int q = 0; q < NCH; ++q) {
                                const uint32_t w[4] = {aq[q].x, aq[q].y, aq[q].z, aq[q].w};
#pragma unroll
                                for (int i = 0; i < 4; ++i) {
                                    v[q * 8 + 2 * i] *= saved_act_grad(cvt_in<BF16>((uint16_t)(w[i] & 0xffff)), p.act);
                                    v[q * 8 + 2 * i + 1] *= saved_act_grad(cvt_in<BF16>((uint16_t)(w[i] >> 16)), p.act);
                                }
                            }
                        }
                    } else if (p.accumulate) {
#pragma unroll
                        for (int q = 0; q < NCH; ++q) {
                            const uint32_t w[4] = {aq[q].x, aq[q].y, aq[q].z, aq[q].w};
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const f32x2 sum = add2(pk(v[q * 8 + 2 * i], v[q * 8 + 2 * i + 1]), cvt_in2<BF16>(w[i]));
                                unpk(sum, v[q * 8 + 2 * i], v[q * 8 + 2 * i + 1]);
                            }
                        }
                    }
                    {
                        if (p.tma_store) {   // an earlier bulk store may still be reading the buffer
                            if (lane == 0) tma_store_wait_read();
                            __syncwarp();
                        }
                        stage_put<BF16>(stage, lane, v);
                        if (MODE == MODE_DGRAD && p.colsum) {
                            // Column sums of this 32x32 block of the (rounded) output, read back from
                            // the staging buffer: lane = (row parity, column pair), 16 rows each.
                            const uint32_t* st32 = reinterpret_cast<const uint32_t*>(stage);
                            const int half = lane >> 4, cp = lane & 15;
                            f32x2 sum = 0ull;
#pragma unroll
                            for (int i = 0; i < 16; ++i) {
                                const int row = 2 * i + half;
                                const uint32_t w = st32[row * 16 + (((cp >> 2) ^ (i & 3)) << 2) + (cp & 3)];
                                if (row < rows_here) sum = add2(sum, cvt_in2<BF16>(w));
                            }
                            float lo, hi;
                            unpk(sum, lo, hi);
                            lo += __shfl_xor_sync(0xffffffffu, lo, 16);
                            hi += __shfl_xor_sync(0xffffffffu, hi, 16);
                            const int blk = sh->blk_base[t.e] + ((t.row0 - sh->seg_lo[t.e]) >> 5) + quarter;
                            if (lane < 16)
                                *reinterpret_cast<float2*>(p.colsum + (size_t)blk * ld + col_lo + c * CW + cp * 2) = make_float2(lo, hi);
                        }
                        if (remote) {
                            // rows leave for their owners: 16-byte pieces, 4 lanes per row, 8 rows per instruction
                            constexpr int RPI = 32 / NCH;
                            const int j = lane % NCH;
#pragma unroll
                            for (int it = 0; it < 32 / RPI; ++it) {
                                const int row = it * RPI + lane / NCH;
                                const unsigned long long rp = __shfl_sync(0xffffffffu, my_rowptr, row);
                                if (row < rows_here && rp)
                                    *reinterpret_cast<uint4*>(rp + (unsigned long long)(col_lo + c * CW + j * 8) * 2ull) = stage[stage_slot(row, j)];
                            }
                            __syncwarp();
                        } else if (bulk) {
                            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                            __syncwarp();
                            if (lane == 0) tma_store_2d(&om.out, stage, col_lo + c * CW, (int)row_off + quarter * 32);
                        } else {
                            stage_store(stage, lane, out_blk + c * CW, ld, rows_here);
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                if (CTA2) mbar_arrive_remote(tmem_empty_addr[acc]);  // the leader's barrier (also from the leader)
                else mbar_arrive(&sh->tmem_empty[acc]);
            }
            if (++acc == 2) { acc = 0; acc_ph ^= 1; }
            if (MODE != MODE_WGRAD && p.done) {
                // this warp's part of the tile is in memory: bulk stores complete, plain stores of the
                // other lanes ordered before the fence by the barrier above
                if (lane == 0) {
                    if (p.tma_store) tma_store_wait_all();
                    asm volatile("fence.proxy.async.global;" ::: "memory");
                    __threadfence();
                    atomicAdd(p.done + t.e, 1);
                }
            }
        }
        if (p.tma_store && lane == 0) tma_store_wait_all();
    }

    // ---- teardown -------------------------------------------------------------
    if (*(volatile int*)&sh->abort) {
        // Give copies that may still be in flight time to land before the CTA's
        // shared memory is released.
        const unsigned long long t0 = clock64();
        while (clock64() - t0 < 2000000ull) { }
    }
    tc_fence_before();
    __syncthreads();
    if (peer && threadIdx.x == 0) {
        // every store of this CTA is ordered before the fence by the barrier; the last CTA tells the
        // peers that this GPU's rows of the epoch have landed (arrived[parity][this rank] = epoch)
        __threadfence_system();
        if (atomicAdd(ro.counter, 1u) == gridDim.x - 1) {
            __threadfence_system();
            const int par = (int)(rem_epoch & 1);
            for (int q = 0; q < ro.world; ++q) {
                if (q == ro.rank) continue;
                unsigned long long* flag = (unsigned long long*)ro.base[q] + ro.arrived_at / 8 + par * ro.stride + ro.rank;
                asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(flag), "l"(rem_epoch) : "memory");
            }
            if (ro.enabled == 2)        // the plan may serve another exchange
                for (int k = 0; k < ps.n_slots; ++k) ps.seg_done[k] = 0;
            *ro.counter = 0;
        }
    }
    if (CTA2) cluster_sync_all();  // the peer may still arrive on this CTA's barriers until here
    if (warp == 0) {
        if (CTA2) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
        else asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// ---- host side ---------------------------------------------------------------
typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                             const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                             CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn get_encode() {
    static EncodeFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeFn)p;
    });
    return fn;
}

// 2-D row-major tensor [rows, cols] of 16-bit elements, box [box_rows, 64 cols], 128-byte swizzle.
int make_map(CUtensorMap* map, const void* base, int64_t rows, int64_t cols, int box_rows, bool bf16) {
    EncodeFn enc = get_encode();
    if (!enc) return fail(FMOE_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                     const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(FMOE_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d) for a [%lld, %lld] tensor", (int)r,
                    (long long)rows, (long long)cols);
    return 0;
}

// Output tensor [rows, cols] of 16-bit elements, box 32 x 32, 64-byte swizzle.
int make_out_map(CUtensorMap* map, const void* base, int64_t rows, int64_t cols, bool bf16) {
    EncodeFn enc = get_encode();
    if (!enc) return fail(FMOE_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    cuuint32_t box[2] = {(cuuint32_t)CW, 32u};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                     const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(FMOE_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d) for a [%lld, %lld] output", (int)r,
                    (long long)rows, (long long)cols);
    return 0;
}

constexpr size_t SMEM_BYTES = (size_t)RING_BYTES + (size_t)EPI_WARPS * STAGING_BYTES + sizeof(Shared);
static_assert(SMEM_BYTES <= 232448, "shared memory budget of one CTA exceeded");

// Device address of the status word on the current device (cached per device).
int* status_ptr() {
    static int* cache[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
    if (!cache[dev]) {
        int* p = nullptr;
        if (cudaGetSymbolAddress((void**)&p, g_status) == cudaSuccess) cache[dev] = p;
    }
    return cache[dev];
}

const HostSegs kNoSegs = {};

// One CTA per 128x256 tile, or a pair of CTAs (cta_group::2) per 256x256 tile.  A pair
// pulls a third fewer operand bytes per flop through each SM's L2 port, which is what
// bounds the one-CTA kernel once the epilogue's stores share that port; on the other hand
// its 256-row tiles waste more rows at the ragged end of each expert's segment.  The
// weight gradient (MN-major operands, long contraction, small epilogue) does not gain
// from pairs: measured 1.16 vs 1.36 PFLOP/s on dense input.  Default: pairs for the
// forward and input-gradient products when segments are long and there is work for every
// pair; FMOE_B200_GEMM=pair / tc1 forces one form for all products.
// The environment gives the initial values (read once); fmoe_gemm_set_form / fmoe_gemm_set_sm_limit
// change them at run time.
std::atomic<int> g_form{-1}, g_sm_limit{-1};
int forced_form() {
    int f = g_form.load(std::memory_order_relaxed);
    if (f < 0) {
        const char* p = getenv("FMOE_B200_GEMM");
        f = FMOE_GEMM_AUTO;
        if (p && p[0] == 'p') f = FMOE_GEMM_PAIR;
        else if (p && p[0] == 't') f = FMOE_GEMM_SINGLE;
        else if (p && p[0] == 's') f = FMOE_GEMM_SIMT;
        g_form.store(f, std::memory_order_relaxed);
    }
    return f;
}
bool use_pairs(int mode, int64_t n_rows, int n_expert, int64_t n_out) {
    const int form = forced_form();
    if (form == FMOE_GEMM_PAIR) return n_rows >= 2048;
    if (form == FMOE_GEMM_SINGLE || mode == MODE_WGRAD) return false;
    const int64_t pair_tiles = ceil_div(n_rows, 256) * ceil_div(n_out, BN);
    return n_rows >= (int64_t)512 * n_expert && pair_tiles >= 2 * (sm_count() / 2);
}

// CTAs the persistent GEMM grids may use: all SMs, or fewer (FMOE_B200_GEMM_SMS=n, or
// fmoe_gemm_set_sm_limit) to leave SMs to kernels that run beside them on other streams.
int cta_cap() {
    int lim = g_sm_limit.load(std::memory_order_relaxed);
    if (lim < 0) {
        const char* e = getenv("FMOE_B200_GEMM_SMS");
        lim = e ? std::max(atoi(e), 0) : 0;
        g_sm_limit.store(lim, std::memory_order_relaxed);
    }
    int cap = sm_count();
    if (lim > 0) cap = std::min(cap, lim);
    return std::max(cap, 2);
}

const GemmRemoteOut kNoRemote = {};
const GemmPushIn kNoPush = {};

template <int MODE, bool CTA2>
int launch(const CUtensorMap& ma, const CUtensorMap& mb, const HostSegs* hsp, const Params& p_in, int64_t max_tiles,
           int64_t out_rows, cudaStream_t st, int reserve_sms = 0, const GemmRemoteOut* rop = nullptr,
           const GemmPushIn* psp = nullptr) {
    const GemmRemoteOut& ro = rop ? *rop : kNoRemote;
    const GemmPushIn& ps = psp ? *psp : kNoPush;
    reserve_sms = (reserve_sms + 1) / 2 * 2;      // the kernel beside this one occupies whole SM pairs
    const HostSegs& hs = hsp ? *hsp : kNoSegs;
    Params p = p_in;
    static_assert(CW == 32, "the output tensor maps assume 32-column staging buffers");
    OutMaps om;
    memset(&om, 0, sizeof(om));
    p.tma_store = 0;
    if (out_rows > 0 && p.out && ro.enabled != 1) {
        if (int rc = make_out_map(&om.out, p.out, out_rows, p.n_out, p.is_bf16 != 0)) return rc;
        if (p.pre_out) {
            if (int rc = make_out_map(&om.out2, p.pre_out, out_rows, p.n_out, p.is_bf16 != 0)) return rc;
        }
        p.tma_store = 1;
    }
    auto kern = p.is_bf16 ? grouped_gemm_kernel<MODE, true, CTA2> : grouped_gemm_kernel<MODE, false, CTA2>;
    FMOE_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES));
    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = SMEM_BYTES;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    if (CTA2) {
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        // one pair per two SMs, as many pairs as can be resident at once
        static int max_pairs[64] = {};
        int dev = 0;
        FMOE_CUDA_TRY(cudaGetDevice(&dev));
        if (dev < 0 || dev >= 64) dev = 0;
        if (!max_pairs[dev]) {
            cfg.gridDim = dim3((unsigned)(sm_count() / 2 * 2));
            int n = 0;
            FMOE_CUDA_TRY(cudaOccupancyMaxActiveClusters(&n, kern, &cfg));
            max_pairs[dev] = n > 0 ? n : 1;
        }
        const int cap = std::max(2, std::min(cta_cap(), sm_count() - reserve_sms));
        const int64_t pairs = std::max<int64_t>(1, std::min<int64_t>(max_tiles, std::min(max_pairs[dev], cap / 2)));
        cfg.gridDim = dim3((unsigned)(2 * pairs));
    } else {
        const int cap = std::max(1, std::min(cta_cap(), sm_count() - reserve_sms));
        cfg.gridDim = dim3((unsigned)std::max<int64_t>(1, std::min<int64_t>(max_tiles, cap)));
    }
    FMOE_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, ma, mb, hs, om, ro, ps, p));
    return 0;
}

bool aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }

bool shape_ok(int64_t n_rows, int64_t in_feat, int64_t out_feat, int n_expert, int dtype) {
    return (dtype == FMOE_BF16 || dtype == FMOE_F16) && n_expert <= MAX_EXPERTS_TC && in_feat % 64 == 0 &&
           out_feat % 64 == 0 && in_feat >= 256 && out_feat >= 256 && n_rows > 0 && n_rows < ((int64_t)1 << 31) &&
           (int64_t)n_expert * out_feat < ((int64_t)1 << 31);
}

// Column sums of dY per expert segment (bias gradient), fp32 accumulate.
// Block = CL column lanes (8 columns each, one 16-byte load) x 256/CL row lanes;
// every thread keeps four independent row loads in flight.  CL = 16 (128 columns per
// block) for wide outputs, 8 (64 columns) when that gives too few blocks.
template <bool BF16, int CL>
__global__ void __launch_bounds__(256)
bias_grad_tc_kernel(const uint16_t* __restrict__ dy, const int64_t* __restrict__ seg,
                    const __grid_constant__ HostSegs hs, uint16_t* __restrict__ db, int64_t n_rows, int out_feat, int accumulate) {
    constexpr int RL = 256 / CL, COLS = CL * 8;
    __shared__ float red[RL][COLS + 1];
    const int e = blockIdx.y;
    const int cl = threadIdx.x % CL, ry = threadIdx.x / CL;
    const int col = blockIdx.x * COLS + cl * 8;
    int64_t lo, hi;
    safe_seg_range(seg, hs, e, n_rows, lo, hi);
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (col < out_feat) {
        const uint16_t* base = dy + col;
        int64_t m = lo + ry;
        for (; m + 3 * RL < hi; m += 4 * RL) {
            uint4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) v[u] = __ldg(reinterpret_cast<const uint4*>(base + (m + RL * u) * out_feat));
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const uint32_t w[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    acc[2 * i] += cvt_in<BF16>((uint16_t)(w[i] & 0xffff));
                    acc[2 * i + 1] += cvt_in<BF16>((uint16_t)(w[i] >> 16));
                }
            }
        }
        for (; m < hi; m += RL) {
            const uint4 v = __ldg(reinterpret_cast<const uint4*>(base + m * out_feat));
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                acc[2 * i] += cvt_in<BF16>((uint16_t)(w[i] & 0xffff));
                acc[2 * i + 1] += cvt_in<BF16>((uint16_t)(w[i] >> 16));
            }
        }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) red[ry][cl * 8 + i] = acc[i];
    __syncthreads();
    if (threadIdx.x < COLS) {
        const int c = blockIdx.x * COLS + threadIdx.x;
        if (c < out_feat) {
            float t = 0.f;
#pragma unroll
            for (int i = 0; i < RL; ++i) t += red[i][threadIdx.x];
            uint16_t* o = db + (size_t)e * out_feat + c;
            if (accumulate) t += cvt_in<BF16>(*o);
            const uint32_t packed = cvt_pack<BF16>(t, 0.f);
            *o = (uint16_t)(packed & 0xffff);
        }
    }
}

// Adds up the per-block partial column sums that the input-gradient kernel left in the
// scratch buffer: out[e, col] = sum over the 32-row blocks of expert e.  Four thread rows
// take a quarter of the blocks each (in block order) and the quarters are added in order,
// so the result does not depend on timing.
template <bool BF16>
__global__ void __launch_bounds__(512)
colsum_finish_kernel(const float* __restrict__ partial, const int64_t* __restrict__ seg, const __grid_constant__ HostSegs hs,
                     uint16_t* __restrict__ out, int64_t n_rows, int n_cols, int accumulate) {
    __shared__ float2 part[4][128];
    const int e = blockIdx.y, q = threadIdx.y;
    const int col = (blockIdx.x * 128 + threadIdx.x) * 2;
    // the same (clamped) ranges and 32-row block numbering as the kernel that wrote the partial sums
    int base = 0;
    int64_t lo = 0, hi = 0, prev_hi = 0;
    for (int j = 0; j <= e; ++j) {
        if (j) base += (int)((hi - lo + 31) >> 5);
        lo = hs.n ? (int64_t)hs.lo[j] : seg[j];
        hi = hs.n ? (int64_t)hs.hi[j] : seg[j + 1];
        lo = min(max(lo, prev_hi), n_rows);
        hi = min(max(hi, lo), n_rows);
        prev_hi = hi;
    }
    const int nb = (int)((hi - lo + 31) >> 5);
    const int per = (nb + 3) >> 2;
    const int b0 = min(nb, q * per), b1 = min(nb, b0 + per);
    float t0 = 0.f, t1 = 0.f;
    if (col < n_cols) {
        const float* src = partial + (size_t)base * n_cols + col;
        int b = b0;
        for (; b + 3 < b1; b += 4) {
            const float2 v0 = *reinterpret_cast<const float2*>(src + (size_t)b * n_cols);
            const float2 v1 = *reinterpret_cast<const float2*>(src + (size_t)(b + 1) * n_cols);
            const float2 v2 = *reinterpret_cast<const float2*>(src + (size_t)(b + 2) * n_cols);
            const float2 v3 = *reinterpret_cast<const float2*>(src + (size_t)(b + 3) * n_cols);
            t0 += v0.x; t1 += v0.y; t0 += v1.x; t1 += v1.y; t0 += v2.x; t1 += v2.y; t0 += v3.x; t1 += v3.y;
        }
        for (; b < b1; ++b) {
            const float2 v = *reinterpret_cast<const float2*>(src + (size_t)b * n_cols);
            t0 += v.x; t1 += v.y;
        }
    }
    part[q][threadIdx.x] = make_float2(t0, t1);
    __syncthreads();
    if (q != 0 || col >= n_cols) return;
    t0 = part[0][threadIdx.x].x + part[1][threadIdx.x].x + part[2][threadIdx.x].x + part[3][threadIdx.x].x;
    t1 = part[0][threadIdx.x].y + part[1][threadIdx.x].y + part[2][threadIdx.x].y + part[3][threadIdx.x].y;
    uint32_t* o = reinterpret_cast<uint32_t*>(out + (size_t)e * n_cols + col);
    if (accumulate) {
        float x0, x1;
        unpk(cvt_in2<BF16>(*o), x0, x1);
        t0 += x0; t1 += x1;
    }
    *o = cvt_pack<BF16>(t0, t1);
}

template <bool BF16>
int launch_bias_grad(const LinearBwdArgs& a, const HostSegs& hs, cudaStream_t st) {
    const bool narrow = ceil_div(a.out_feat, 128) * a.n_expert < 2 * sm_count();
    if (narrow) {
        dim3 grid((unsigned)ceil_div(a.out_feat, 64), (unsigned)a.n_expert);
        bias_grad_tc_kernel<BF16, 8><<<grid, 256, 0, st>>>((const uint16_t*)a.grad_y, a.seg_offsets, hs, (uint16_t*)a.grad_b,
                                                            a.n_rows, (int)a.out_feat, a.accumulate);
    } else {
        dim3 grid((unsigned)ceil_div(a.out_feat, 128), (unsigned)a.n_expert);
        bias_grad_tc_kernel<BF16, 16><<<grid, 256, 0, st>>>((const uint16_t*)a.grad_y, a.seg_offsets, hs, (uint16_t*)a.grad_b,
                                                             a.n_rows, (int)a.out_feat, a.accumulate);
    }
    FMOE_CHECK_LAUNCH();
    return 0;
}

}  // namespace

bool tc_forward_supported(const LinearArgs& a) {
    return shape_ok(a.n_rows, a.in_feat, a.out_feat, a.n_expert, a.dtype) && aligned16(a.x) && aligned16(a.weight) &&
           aligned16(a.y) && (!a.bias || aligned16(a.bias)) && (!a.pre_act || aligned16(a.pre_act));
}

bool tc_backward_supported(const LinearBwdArgs& a) {
    return shape_ok(a.n_rows, a.in_feat, a.out_feat, a.n_expert, a.dtype) && aligned16(a.grad_y) &&
           aligned16(a.weight) && (!a.x || aligned16(a.x)) && (!a.grad_x || aligned16(a.grad_x)) &&
           (!a.grad_w || aligned16(a.grad_w)) && (!a.act_pre || aligned16(a.act_pre)) &&
           (!a.grad_b || ((uintptr_t)a.grad_b & 1) == 0);
}

// fp32 partial column sums of the input gradient: one row of in_feat values per 32-row block
size_t tc_backward_scratch_bytes(int64_t n_rows, int64_t in_feat, int64_t, int n_expert, int) {
    return (size_t)(n_rows / 32 + n_expert + 1) * (size_t)in_feat * sizeof(float);
}

int tc_linear_forward(const LinearArgs& a, cudaStream_t st) {
    const bool bf16 = a.dtype == FMOE_BF16;
    CUtensorMap ma, mb;
    if (int rc = make_map(&ma, a.x, a.n_rows, a.in_feat, BM, bf16)) return rc;
    // Pairs of CTAs (256-row tiles) once there is enough work for them; each CTA of a
    // pair stages 128 of the tile's 256 weight rows.
    const bool pair = use_pairs(MODE_FWD, a.n_rows, a.n_expert, a.out_feat);
    if (int rc = make_map(&mb, a.weight, (int64_t)a.n_expert * a.out_feat, a.in_feat, pair ? 128 : BN, bf16)) return rc;
    Params p{};
    p.seg = a.seg_offsets; p.n_expert = a.n_expert; p.n_out = (int)a.out_feat; p.n_contr = (int)a.in_feat;
    p.w_rows = (int)a.out_feat; p.out = a.y; p.pre_out = a.pre_act; p.bias = a.bias; p.act = a.activation;
    p.is_bf16 = bf16; p.status = status_ptr(); p.n_rows = a.n_rows;
    const int tile_m = pair ? 256 : BM;
    const int64_t max_tiles = (ceil_div(a.n_rows, tile_m) + a.n_expert) * ceil_div(a.out_feat, BN);
    int reserve = 0;
    if (a.arrival) {
        p.arr_flags = a.arrival->flags; p.arr_seq = a.arrival->seq; p.arr_src_off = a.arrival->src_off;
        p.arr_world = a.arrival->world;
        reserve = a.arrival->reserve_sms;
    }
    if (a.done) {
        p.done = a.done->done; p.done_expected = a.done->expected; p.done_ready = a.done->ready;
        reserve = std::max(reserve, a.done->reserve_sms);
    }
    return pair ? launch<MODE_FWD, true>(ma, mb, a.host_segs, p, max_tiles, a.n_rows, st, reserve, a.remote, a.push)
                : launch<MODE_FWD, false>(ma, mb, a.host_segs, p, max_tiles, a.n_rows, st, reserve, a.remote, a.push);
}

// A side stream and a pair of events per device, created on first use: the bias
// gradient (an HBM-bound column sum with a small footprint) runs there, next to the
// tensor-core kernels of the same call, instead of after them.
struct SideStream {
    cudaStream_t stream = nullptr;
    cudaEvent_t fork = nullptr, join = nullptr;
};
int side_stream(SideStream** out) {
    static SideStream pool[64];
    static std::mutex mtx;
    int dev = 0;
    FMOE_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) dev = 0;
    std::lock_guard<std::mutex> lk(mtx);
    SideStream& s = pool[dev];
    if (!s.stream) {
        FMOE_CUDA_TRY(cudaStreamCreateWithFlags(&s.stream, cudaStreamNonBlocking));
        FMOE_CUDA_TRY(cudaEventCreateWithFlags(&s.fork, cudaEventDisableTiming));
        FMOE_CUDA_TRY(cudaEventCreateWithFlags(&s.join, cudaEventDisableTiming));
    }
    *out = &s;
    return 0;
}

int tc_linear_backward(const LinearBwdArgs& a, cudaStream_t st) {
    const bool bf16 = a.dtype == FMOE_BF16;
    SideStream* side = nullptr;
    const bool overlap_bias = a.grad_b && (a.grad_x || a.grad_w) && a.n_rows > 0;
    // grad_y still arriving: only the input-gradient product may start; everything else (the bias
    // gradient on the side stream included) is queued after the exchange has been closed
    const bool arriving = a.arrival != nullptr;
    bool closed = !arriving;
    if (arriving && !(a.grad_x && a.n_rows > 0)) {
        if (a.after_input_grad) { if (int rc = a.after_input_grad(a.after_ctx)) return rc; }
        closed = true;
    }
    auto queue_bias = [&]() -> int {
        if (int rc = side_stream(&side)) return rc;
        const HostSegs& hs = a.host_segs ? *a.host_segs : kNoSegs;
        FMOE_CUDA_TRY(cudaEventRecord(side->fork, st));
        FMOE_CUDA_TRY(cudaStreamWaitEvent(side->stream, side->fork, 0));
        if (int rc = bf16 ? launch_bias_grad<true>(a, hs, side->stream) : launch_bias_grad<false>(a, hs, side->stream))
            return rc;
        FMOE_CUDA_TRY(cudaEventRecord(side->join, side->stream));
        return 0;
    };
    if (overlap_bias && !closed) {
        // queued below, after the input-gradient product
    } else if (overlap_bias) {
        if (int rc = queue_bias()) return rc;
    }
    if (a.grad_x && a.n_rows > 0) {
        CUtensorMap ma, mb;
        if (int rc = make_map(&ma, a.grad_y, a.n_rows, a.out_feat, BM, bf16)) return rc;
        if (int rc = make_map(&mb, a.weight, (int64_t)a.n_expert * a.out_feat, a.in_feat, 64, bf16)) return rc;
        Params p{};
        p.seg = a.seg_offsets; p.n_expert = a.n_expert; p.n_out = (int)a.in_feat; p.n_contr = (int)a.out_feat;
        p.w_rows = (int)a.out_feat; p.out = a.grad_x; p.act_pre = a.act_pre; p.act = a.activation;
        p.is_bf16 = bf16; p.status = status_ptr(); p.n_rows = a.n_rows;
        if (a.grad_x_colsum) {
            FMOE_REQUIRE(a.scratch && aligned16(a.scratch) && ((uintptr_t)a.grad_x_colsum & 3) == 0,
                         "linear_backward: column sums of grad_x need the scratch buffer of fmoe_linear_scratch_bytes");
            p.colsum = (float*)a.scratch;
        }
        const bool pair = use_pairs(MODE_DGRAD, a.n_rows, a.n_expert, a.in_feat);
        const int64_t max_tiles = (ceil_div(a.n_rows, pair ? 256 : BM) + a.n_expert) * ceil_div(a.in_feat, BN);
        int reserve = 0;
        if (arriving && !closed) {
            p.arr_flags = a.arrival->flags; p.arr_seq = a.arrival->seq; p.arr_src_off = a.arrival->src_off;
            p.arr_world = a.arrival->world;
            reserve = a.arrival->reserve_sms;
        }
        if (a.done) {
            p.done = a.done->done; p.done_expected = a.done->expected; p.done_ready = a.done->ready;
            reserve = std::max(reserve, a.done->reserve_sms);
        }
        if (int rc = pair ? launch<MODE_DGRAD, true>(ma, mb, a.host_segs, p, max_tiles, a.n_rows, st, reserve, a.remote, a.push)
                          : launch<MODE_DGRAD, false>(ma, mb, a.host_segs, p, max_tiles, a.n_rows, st, reserve, a.remote, a.push))
            return rc;
        if (!closed) {
            if (a.after_input_grad) { if (int rc = a.after_input_grad(a.after_ctx)) return rc; }
            closed = true;
            if (overlap_bias) { if (int rc = queue_bias()) return rc; }
        }
        if (a.grad_x_colsum) {
            const HostSegs& hs = a.host_segs ? *a.host_segs : kNoSegs;
            dim3 grid((unsigned)ceil_div(a.in_feat, 256), (unsigned)a.n_expert);
            if (bf16) colsum_finish_kernel<true><<<grid, dim3(128, 4), 0, st>>>((const float*)a.scratch, a.seg_offsets, hs,
                                                                                (uint16_t*)a.grad_x_colsum, a.n_rows, (int)a.in_feat, 0);
            else colsum_finish_kernel<false><<<grid, dim3(128, 4), 0, st>>>((const float*)a.scratch, a.seg_offsets, hs,
                                                                            (uint16_t*)a.grad_x_colsum, a.n_rows, (int)a.in_feat, 0);
            FMOE_CHECK_LAUNCH();
        }
    }
    if (a.grad_w) {
        CUtensorMap ma, mb;
        // Tensor maps need at least one row; with no rows at all every expert is empty
        // and the kernel only writes zeros.
        const int64_t rows = std::max<int64_t>(a.n_rows, 1);
        if (int rc = make_map(&ma, a.grad_y, rows, a.out_feat, 64, bf16)) return rc;
        if (int rc = make_map(&mb, a.x, rows, a.in_feat, 64, bf16)) return rc;
        Params p{};
        p.seg = a.seg_offsets; p.n_expert = a.n_expert; p.n_out = (int)a.in_feat; p.n_contr = 0;
        p.out_rows_per_expert = (int)a.out_feat; p.out = a.grad_w; p.accumulate = a.accumulate;
        p.is_bf16 = bf16; p.status = status_ptr(); p.n_rows = a.n_rows;
        const bool pair = use_pairs(MODE_WGRAD, a.n_rows, a.n_expert, a.in_feat);
        const int64_t max_tiles = (int64_t)a.n_expert * ceil_div(a.out_feat, pair ? 256 : BM) * ceil_div(a.in_feat, BN);
        // (a push that forwards grad_x may still be running on its SMs)
        const int reserve = a.done ? a.done->reserve_sms : 0;
        if (int rc = pair ? launch<MODE_WGRAD, true>(ma, mb, a.host_segs, p, max_tiles, (int64_t)a.n_expert * a.out_feat, st, reserve)
                          : launch<MODE_WGRAD, false>(ma, mb, a.host_segs, p, max_tiles, (int64_t)a.n_expert * a.out_feat, st, reserve))
            return rc;
    }
    if (overlap_bias) {
        FMOE_CUDA_TRY(cudaStreamWaitEvent(st, side->join, 0));
    } else if (a.grad_b) {
        const HostSegs& hs = a.host_segs ? *a.host_segs : kNoSegs;
        if (int rc = bf16 ? launch_bias_grad<true>(a, hs, st) : launch_bias_grad<false>(a, hs, st)) return rc;
    }
    return 0;
}

int* device_status_ptr() { return status_ptr(); }
int gemm_form() { return forced_form(); }

int read_device_status(int* out) {
    int v = 0;
    FMOE_CUDA_TRY(cudaMemcpyFromSymbol(&v, g_status, sizeof(int)));
    *out = v;
    return 0;
}

}  // namespace fmoe

extern "C" int fmoe_gemm_set_form(int32_t form) {
    FMOE_REQUIRE(form >= FMOE_GEMM_AUTO && form <= FMOE_GEMM_SIMT, "gemm_set_form: unknown form %d", form);
    fmoe::g_form.store(form, std::memory_order_relaxed);
    return 0;
}

extern "C" int fmoe_gemm_set_sm_limit(int32_t n_sms) {
    FMOE_REQUIRE(n_sms >= 0, "gemm_set_sm_limit: n_sms=%d", n_sms);
    fmoe::g_sm_limit.store(n_sms, std::memory_order_relaxed);
    return 0;
}

extern "C" int fmoe_device_status_clear(void) {
    const int zero = 0;
    FMOE_CUDA_TRY(cudaMemcpyToSymbol(fmoe::g_status, &zero, sizeof(int)));
    return 0;
}

extern "C" int fmoe_device_status(int32_t* status_out) {
    FMOE_REQUIRE(status_out, "device_status: null pointer");
    int v = 0;
    if (int rc = fmoe::read_device_status(&v)) return rc;
    *status_out = v;
    return 0;
}
