// Block-scaled NVFP4 GEMM for sm_100a:  D[M,N] (bf16) = alpha * A[M,K] * B[N,K]^T.
//
// Semantics follow tirx_kernels/basic/nvfp4_gemm.py of the reference (operands and scale
// layout :47-66, :941-982; one E4M3 scale per 16 values along K, fp32 accumulation,
// alpha then bf16 in the epilogue :795-800).  The kernel itself is written from scratch:
//
//   * persistent CTAs (or CTA pairs), at most one per SM, walking a grouped tile order;
//   * warp 0: TMA producer of A and B - the operands of a 256-wide K slab land in a ring of
//             shared-memory stages, completion counted on mbarriers;
//   * warp 18: TMA producer of the scale-factor blocks of the same slab (a thread of its own:
//             issuing a TMA copy costs its thread on the order of a hundred cycles);
//   * warp 1: MMA issuer    - four tcgen05.mma.kind::mxf4nvf4.block_scale (K = 64 each) per
//             slab, accumulating into TMEM; tcgen05.commit releases the stage (the decode variant
//             has a second issuer, warp 19, with an accumulator of its own);
//   * warps 2-9: scale warps - two sets of four (one warp per 32-lane quarter of tensor
//             memory), each set owning the stages of one parity: ld.shared the slab's scale
//             factors and tcgen05.st them into the stage's tensor-memory columns;
//   * warps 10-17: epilogue - tcgen05.ld the accumulator (lane quarter x column half), scale by
//             alpha, convert to bf16, release tensor memory, then either store rows directly or
//             (CTA-pair variants) write them 128-byte-swizzled into a staging buffer and let the
//             TMA store 32 x 64 sub-tiles, once per destination buffer.  With several destinations
//             (this GPU's buffer and the peers' buffers mapped over NVLink) that store is the
//             output all-gather of a column-sharded projection.
//
// With CG == 2 two CTAs of a cluster share one 256 x BN tile: each loads its own 128 rows of A
// and half of B, the leader issues cta_group::2 MMAs for both.  No load uses cluster multicast:
// every TMA load is unicast into the issuing CTA's own shared memory, and cross-CTA signalling
// uses the cta_group::2 completion form and plain remote mbarrier arrives.  Peer GPUs are only
// ever written (TMA stores), never read.
//
// Every wait is bounded.  A wait that expires records a code in a device status word,
// raises a CTA-wide abort flag so the other roles drain, and the kernel exits normally
// (tensor memory released); the host reads the word through b2_nvfp4_gemm_status().
#include <cuda.h>

#include <atomic>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <unordered_map>
#include <vector>

#include "common.cuh"

namespace b2 {
namespace {

constexpr int kBlockM = 128;        // rows of A per CTA (TMEM lanes)
constexpr int kBlockK = 256;        // fp4 values per stage along K = 128 bytes = one swizzle row
constexpr int kThreads = 608;       // operand TMA warp, MMA warp, 2 x 4 scale warps, 8 epilogue warps, scale TMA warp
// The MMA role's waits on barriers that the peer CTA of a pair arrives on.  What those arrivals publish
// lives in tensor memory or was written by the TMA, none of it is read through the generic proxy by the
// waiting thread, and tcgen05.fence::after_thread_sync follows every wait, so the default (CTA-scope)
// acquire of mbarrier.try_wait is what the wait needs; the cluster-scope form costs the issuing thread
// on the order of a hundred cycles per K slab.
#ifndef B2_GEMM_CLUSTER_ACQUIRE
#define B2_GEMM_CLUSTER_ACQUIRE 0
#endif
constexpr bool kClusterAcquireWaits = B2_GEMM_CLUSTER_ACQUIRE != 0;
constexpr uint64_t kWaitBudgetNs = 1000ull * 1000ull * 1000ull;  // default budget of a wait: one second

struct GemmParams {
  const float* alpha;
  uint16_t* D;       // output (direct-store epilogue)
  int n_dest;        // TMA-store epilogue: buffers every tile is stored to (this GPU's own first)
  int ldd;           // elements between output rows (N, or world * N for the gathered layout)
  int col0;          // first output column of this GPU's slab inside the gathered row
  uint32_t* status;  // [0]: first failure code, [1]: detail; role timers from byte 64 on
  int profile;       // CTA 0 records per-role cycle counters when set
  int M, N, K;
  int splits;        // K is cut into `splits` ranges, each its own work item (1 = no split)
  float* partial;    // [splits][M][N] fp32 partial sums when splits > 1
  int tiles_m, tiles_n;  // in units of (cta_group * 128) rows and BN columns
  int group_n;           // tile-order grouping along N
  uint64_t wait_budget_ns;  // budget of a bounded wait (kWaitBudgetNs unless a test shortened it)
  int test_fault;        // test hook, 0 in production: 1 = the first slab of CTA 0 announces 16 bytes more
                         // than its copies deliver, so its barrier never completes (every copy still lands)
};

// ---- PTX wrappers -------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t mapa_shared(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
// Remote arrive without memory ordering: for hand-offs whose payload lives in tensor memory and
// has already been completed with tcgen05.wait, so no generic-proxy writes need publishing.
__device__ __forceinline__ void mbar_arrive_cluster_relaxed(uint32_t cluster_bar) {
  asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_local(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_try_wait_cluster_acquire(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{ .reg .pred p; mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;"
      " selp.u32 %0, 1, 0, p; }"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void prefetch_tmap(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}

template <int CG>
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y,
                                            uint32_t bar) {
  if constexpr (CG == 1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar)
        : "memory");
  } else {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar)
        : "memory");
  }
}
template <int CG>
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int x, int y,
                                            int z, uint32_t bar) {
  if constexpr (CG == 1) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(z), "r"(bar)
        : "memory");
  } else {
    asm volatile(
        "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(z), "r"(bar)
        : "memory");
  }
}

template <int CG>
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t cols) {
  if constexpr (CG == 1)
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
  else
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
}
template <int CG>
__device__ __forceinline__ void tmem_relinquish() {
  if constexpr (CG == 1)
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  else
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
template <int CG>
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t cols) {
  if constexpr (CG == 1)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
  else
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
template <int CG>
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                       uint32_t idesc, uint32_t sfa_tmem, uint32_t sfb_tmem,
                                       uint32_t accumulate) {
  if constexpr (CG == 1) {
    asm volatile(
        "{ .reg .pred p; setp.ne.b32 p, %6, 0;\n"
        "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%4], [%5], p; }"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(sfa_tmem), "r"(sfb_tmem), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{ .reg .pred p; setp.ne.b32 p, %6, 0;\n"
        "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%4], [%5], p; }"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(sfa_tmem), "r"(sfb_tmem), "r"(accumulate)
        : "memory");
  }
}
// Makes `bar` (a shared::cluster address, possibly in the peer CTA) track completion of all
// tcgen05 operations this thread issued so far.
template <int CG>
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  if constexpr (CG == 1)
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
  else
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// CTA pair: one commit that arrives on the barrier at the same shared-memory offset in both
// CTAs of the pair (a completion signal, not a load).
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
      "h"(static_cast<uint16_t>(3))
      : "memory");
}
// True in exactly one lane of a converged warp.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile("{ .reg .pred P; elect.sync _|P, 0xffffffff; selp.u32 %0, 1, 0, P; }" : "=r"(pred));
  return pred != 0;
}
// One K slab from the issuing thread's side: the four MMAs and the commit that hands the stage back, with the
// poll of the barrier the thread needs NEXT issued in front of them and its result read behind them.  A poll
// takes the thread 100-200 cycles even when the barrier completed long ago (by the time the MMA thread reaches
// a stage its operands and scales have been there for ~2000 cycles), and in one instruction stream that wait
// was serial with the ~50 cycles per MMA: the thread, not the ring or the tensor pipe, set the time per slab.
// Returns whether the next barrier's phase had completed.
template <int CG>
__device__ __forceinline__ uint32_t tc_slab_and_poll_next(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                                         uint32_t idesc, uint32_t sfa, uint32_t sfb,
                                                         uint32_t sfb_step, uint32_t accumulate_first,
                                                         uint32_t commit_bar, uint32_t next_bar,
                                                         uint32_t next_parity) {
  uint32_t ok;
#define B2_MMA_(cg, d, a, b, sa, sb, pr) \
  "tcgen05.mma.cta_group::" cg ".kind::mxf4nvf4.block_scale.scale_vec::4X [" d "], " a ", " b ", %10, [" sa "], [" sb "], " pr ";\n"
  if constexpr (CG == 1) {
    asm volatile(
        "{ .reg .pred p, q, t;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 q, [%21], %22;\n"
        "setp.ne.b32 p, %19, 0;\n"
        "setp.eq.b32 t, %10, %10;\n"
        B2_MMA_("1", "%1", "%2", "%6", "%11", "%15", "p")
        B2_MMA_("1", "%1", "%3", "%7", "%12", "%16", "t")
        B2_MMA_("1", "%1", "%4", "%8", "%13", "%17", "t")
        B2_MMA_("1", "%1", "%5", "%9", "%14", "%18", "t")
        "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%20];\n"
        "selp.u32 %0, 1, 0, q; }"
        : "=r"(ok)
        : "r"(d_tmem), "l"(a_desc), "l"(a_desc + 2), "l"(a_desc + 4), "l"(a_desc + 6), "l"(b_desc),
          "l"(b_desc + 2), "l"(b_desc + 4), "l"(b_desc + 6), "r"(idesc), "r"(sfa), "r"(sfa + 4), "r"(sfa + 8),
          "r"(sfa + 12), "r"(sfb), "r"(sfb + sfb_step), "r"(sfb + 2 * sfb_step), "r"(sfb + 3 * sfb_step),
          "r"(accumulate_first), "r"(commit_bar), "r"(next_bar), "r"(next_parity)
        : "memory");
  } else {
    asm volatile(
        "{ .reg .pred p, q, t;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 q, [%21], %22;\n"
        "setp.ne.b32 p, %19, 0;\n"
        "setp.eq.b32 t, %10, %10;\n"
        B2_MMA_("2", "%1", "%2", "%6", "%11", "%15", "p")
        B2_MMA_("2", "%1", "%3", "%7", "%12", "%16", "t")
        B2_MMA_("2", "%1", "%4", "%8", "%13", "%17", "t")
        B2_MMA_("2", "%1", "%5", "%9", "%14", "%18", "t")
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%20], %23;\n"
        "selp.u32 %0, 1, 0, q; }"
        : "=r"(ok)
        : "r"(d_tmem), "l"(a_desc), "l"(a_desc + 2), "l"(a_desc + 4), "l"(a_desc + 6), "l"(b_desc),
          "l"(b_desc + 2), "l"(b_desc + 4), "l"(b_desc + 6), "r"(idesc), "r"(sfa), "r"(sfa + 4), "r"(sfa + 8),
          "r"(sfa + 12), "r"(sfb), "r"(sfb + sfb_step), "r"(sfb + 2 * sfb_step), "r"(sfb + 3 * sfb_step),
          "r"(accumulate_first), "r"(commit_bar), "r"(next_bar), "r"(next_parity),
          "h"(static_cast<uint16_t>(3))
        : "memory");
  }
#undef B2_MMA_
  return ok;
}
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// ---- descriptors ----------------------------------------------------------------------------
// Shared-memory matrix descriptor (sm_100 format): start address >> 4 in bits [0,14), leading
// byte offset >> 4 in [16,30), stride byte offset >> 4 in [32,46), descriptor version 1 in
// [46,48), swizzle mode in [61,64) (0 none, 2 = 128-byte).
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo16, uint32_t sbo16,
                                              uint32_t layout) {
  return static_cast<uint64_t>((addr >> 4) & 0x3FFFu) | (static_cast<uint64_t>(lbo16 & 0x3FFFu) << 16) |
         (static_cast<uint64_t>(sbo16 & 0x3FFFu) << 32) | (1ull << 46) | (static_cast<uint64_t>(layout) << 61);
}
// K-major operand tile stored by TMA with 128-byte swizzle: rows of 128 B, 8-row groups 1024 B apart.
__device__ __forceinline__ uint64_t operand_desc(uint32_t addr) { return smem_desc(addr, 1, 64, 2); }
// Instruction descriptor of kind::mxf4nvf4 with block scaling: E2M1 operands (format 1) at bits 7
// and 10, both K-major, N >> 3 at bit 17, E4M3 scales (0) at bit 23, M >> 4 at bit 24.
__host__ __device__ constexpr uint32_t instr_desc(int m, int n) {
  return (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

// ---- shared memory ------------------------------------------------------------------------------
// AM: rows of A the TMA writes per stage.  The MMA always reads 128 rows; with AM < 128 (M <= AM) the
// rows past AM are whatever follows in the stage, which only reaches accumulator rows nobody reads,
// and the shared memory saved buys more stages in flight.
template <int CG, int BN, int STAGES, int TMA_OUT = 0, int AM = kBlockM>
struct SmemLayout {
  static constexpr int kBRows = BN / CG;                       // rows of B held by one CTA
  static constexpr int kChunks = BN / 128 > 0 ? BN / 128 : 1;  // 128-row scale chunks of B
  static constexpr int kABytes = AM * 128;
  static constexpr int kBBytes = kBRows * 128;
  static constexpr int kSfaBytes = 4 * 512;                    // 4 K-blocks of 64, 512 B each
  static constexpr int kSfbBytes = kChunks * 4 * 512;
  static constexpr int kStageBytes = kABytes + kBBytes + kSfaBytes + kSfbBytes;
  static constexpr int kSfCols = 16 + 16 * kChunks;            // TMEM columns of one stage's scales
  static constexpr int kBarrierBytes = 512;
  // output staging of the TMA-store epilogue (TMA_OUT > 0): every epilogue warp owns TMA_OUT
  // sub-tiles of 32 rows x 64 bf16 columns (4 KB, 128-byte rows, 128-byte swizzle) and pushes its
  // 32 x BN/2 part of the tile through them
  static constexpr int kStagingBytes = 8 * TMA_OUT * 4096;
  static_assert(TMA_OUT == 0 || (BN / 2 / 64) % TMA_OUT == 0, "sub-tiles per warp divide its columns");
  static constexpr int kRingBytes = STAGES * kStageBytes + kStagingBytes;
  static constexpr int kTotal = kRingBytes + kBarrierBytes + 1024;  // + alignment slack
  static_assert(kStageBytes % 1024 == 0, "stages and staging stay 1024-byte aligned");
  static_assert(AM == kBlockM || (CG == 1 && kStageBytes >= kBlockM * 128), "the MMA's 128-row window stays inside the stage");
  static_assert(kTotal <= 227 * 1024, "shared memory budget");
  static_assert(BN + STAGES * kSfCols <= 512, "tensor memory budget");
  static_assert((3 * STAGES + 2) * 8 + 16 <= kBarrierBytes, "barrier area");
};

struct WaitCtx {
  uint32_t* status;
  volatile uint32_t* abort_flag;  // in shared memory
  uint64_t budget_ns;
};

// Bounded mbarrier wait.  Returns false after recording `code` when the barrier never flips or
// another role of this CTA has already given up.  The waits on data arriving from memory (codes 3
// and 5) run out after the budget, the waits downstream of them (a free stage, a drained or a
// finished accumulator) after twice the budget, so that the status word names the role that
// stalled first rather than one that only waited for it.
template <bool kClusterAcquire = false>
__device__ __forceinline__ bool wait_or_abort(uint32_t bar, uint32_t parity, const WaitCtx& ctx,
                                              uint32_t code) {
  uint64_t started = 0;
  const uint64_t budget = (code == 3u || code == 5u) ? ctx.budget_ns : 2 * ctx.budget_ns;
  for (uint32_t i = 0;; ++i) {
    const bool ok = kClusterAcquire ? mbar_try_wait_cluster_acquire(bar, parity) : mbar_try_wait(bar, parity);
    if (ok) return true;
    if ((i & 63u) != 63u) continue;
    if (*ctx.abort_flag) return false;
    const uint64_t now = globaltimer_ns();
    if (started == 0) started = now;
    else if (now - started > budget) break;
    if (i > (1u << 26)) break;  // backstop in polls, should the timer not advance (seconds at the shortest poll)
  }
  if (atomicCAS(ctx.status, 0u, code) == 0u) ctx.status[1] = blockIdx.x;
  *ctx.abort_flag = 1u;
  return false;
}

__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int group_n, int& tm,
                                            int& tn) {
  const int per_group = group_n * tiles_m;
  const int g = t / per_group;
  const int first_n = g * group_n;
  const int width = min(group_n, tiles_n - first_n);
  const int local = t - g * per_group;
  tm = local / width;
  tn = first_n + local % width;
}

__device__ __forceinline__ void lds128(uint32_t addr, uint32_t* r) {
  asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
// registers -> tensor memory: lane i of the warp writes 16 consecutive columns of TMEM lane (base + i)
__device__ __forceinline__ void tmem_st_32x32_x16(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// Warp roles.  The scale and epilogue warps are placed so that (warp & 3) is the 32-lane quarter of
// tensor memory the warp is allowed to touch.
constexpr int kWarpProducer = 0, kWarpMma = 1, kWarpScale0 = 2, kWarpEpi0 = 10, kWarpScaleProducer = 18;

// Output tensor maps of the TMA-store epilogue: [0] this GPU's buffer, [1..] the peers' buffers.
template <bool TMA_OUT>
struct OutMaps {};
template <>
struct OutMaps<true> {
  CUtensorMap m[8];
};

// The output is written once and not read again by this kernel: its lines are marked evict-first so
// that they do not push the operands, which every tile row and column re-reads, out of L2.
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t policy;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
  return policy;
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t smem, int x, int y, uint64_t policy) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group.L2::cache_hint [%0, {%1, %2}], [%3], %4;" ::"l"(map),
               "r"(x), "r"(y), "r"(smem), "l"(policy)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void sts128(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

// MMAS: MMA-issuing warps.  Issuing one tcgen05.mma costs its thread about 75 cycles whatever the tile
// width, so a decode-sized problem that gives every CTA a narrow tile and all of K (no K ranges, no second
// kernel) is bound by that one thread: 128 MMAs of N = 64 take it longer than HBM takes to deliver the
// weights.  With MMAS == 2 a second warp issues the odd K slabs into a second accumulator (columns
// [BN, 2 BN) of tensor memory) and the epilogue adds the two.
template <int CG, int BN, int STAGES, int TMA_OUT, int AM, int MMAS>
__global__ void __launch_bounds__(kThreads + 32 * (MMAS - 1), 1)
    nvfp4_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                      const __grid_constant__ CUtensorMap map_sfa, const __grid_constant__ CUtensorMap map_sfb,
                      const __grid_constant__ GemmParams p, const __grid_constant__ OutMaps<(TMA_OUT > 0)> out_maps) {
  using L = SmemLayout<CG, BN, STAGES, TMA_OUT, AM>;
  static_assert(MMAS == 1 || (MMAS == 2 && CG == 1 && TMA_OUT == 0), "the second MMA warp exists for single-CTA tiles");
  static_assert(BN * MMAS + STAGES * L::kSfCols <= 512, "tensor memory budget");
  constexpr int kAccCols = BN * MMAS;  // accumulator columns in front of the stages' scale areas
  constexpr int kWarpMma2 = 19;
  constexpr int kTmemCols = 512;
  constexpr uint32_t kIdesc = instr_desc(kBlockM * CG, BN);
  constexpr uint32_t kOperandTx = static_cast<uint32_t>(L::kABytes + L::kBBytes) * CG;
  constexpr uint32_t kScaleTx = static_cast<uint32_t>(L::kSfaBytes + L::kSfbBytes);

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t bar_base = smem_base + L::kRingBytes;
  // full (on the leader): A and B of a stage landed in both CTAs of the group AND every scale warp
  // of the group has put the slab's scales into tensor memory (transaction bytes + one arrive per
  // scale warp); sfload: this CTA's scale blocks landed in shared memory; empty: the stage's MMAs
  // retired.
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto sfload_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto empty_bar = [&](int s) { return bar_base + 8u * (2 * STAGES + s); };
  const uint32_t tmem_full_bar = bar_base + 8u * (3 * STAGES);
  const uint32_t tmem_empty_bar = bar_base + 8u * (3 * STAGES + 1);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_gen + L::kRingBytes + 8 * (3 * STAGES + 2));
  volatile uint32_t* abort_flag = tmem_slot + 1;
  const WaitCtx ctx{p.status, abort_flag, p.wait_budget_ns};

  // Broadcast from lane 0: the value is the same in every lane anyway, but this way the compiler knows it, keeps
  // the role dispatch and everything computed from these in uniform registers and uniform control flow.
  constexpr bool kWarpWide = CG == 2;  // see the issuing roles below
  const int warp = kWarpWide ? __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0)
                             : static_cast<int>(threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const uint32_t rank = CG == 2 ? __shfl_sync(0xffffffffu, cluster_ctarank(), 0) : 0u;
  const bool leader = rank == 0;
  const int unit = CG == 2 ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
  const int num_units = CG == 2 ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);
  const int num_tiles = p.tiles_m * p.tiles_n * p.splits;  // work items: (tile, K range)
  const int k_slabs = p.K / kBlockK / p.splits;            // slabs per work item
  const bool prof = p.profile && blockIdx.x == 0 && lane == 0;
  unsigned long long* counters = reinterpret_cast<unsigned long long*>(p.status + 16);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1 + 4 * CG);  // the producer's expect_tx arrive + one arrive per scale warp of the group
      mbar_init(sfload_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    mbar_init(tmem_full_bar, MMAS);
    mbar_init(tmem_empty_bar, 8 * CG);  // one arrive per epilogue warp of every CTA in the group
    *abort_flag = 0u;
    fence_barrier_init();
    prefetch_tmap(&map_a);
    prefetch_tmap(&map_b);
    prefetch_tmap(&map_sfa);
    prefetch_tmap(&map_sfb);
  }
  if (warp == kWarpMma) {
    tmem_alloc<CG>(smem_u32(tmem_slot), kTmemCols);
    tmem_relinquish<CG>();
  }
  tc_fence_before();
  __syncthreads();
  if constexpr (CG == 2) cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = kWarpWide ? __shfl_sync(0xffffffffu, *tmem_slot, 0) : *tmem_slot;
  // Programmatic dependent launch, both ways.  This grid may have been launched before its predecessor on
  // the stream finished: everything above touched only this CTA's own shared and tensor memory, and nothing
  // below reads or writes global memory before the predecessor has completed and its writes are visible.
  // Then let the next launch start: with K ranges that is the kernel that adds the partial sums (resident
  // beside this grid, waiting), otherwise it is whatever follows with the same launch attribute - another
  // GEMM of a decode step is scheduled onto every SM the moment this grid's CTA leaves it, instead of after
  // the whole grid has drained and a launch has been processed.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  // The three issuing roles (operand copies, scale copies, MMAs) are, in the CTA-pair kernels, loops that the WHOLE warp runs,
  // with one elected lane issuing (kWarpWide).  TMA and tcgen05 instructions take their operands from uniform registers; what every
  // lane of a converged warp computes alike (ring position, barrier and shared-memory addresses, descriptors)
  // the compiler can keep there, whereas in a loop that only lane 0 runs every operand of every such
  // instruction is moved there first.  All lanes wait on the barriers (also the fastest way to be woken: a
  // lane waiting for its warp and handing the result on by shuffle takes twice as long) and agree on the
  // outcome by a vote, so the warp leaves the loop together when a wait gives up.
  if (warp == kWarpProducer) {
    if constexpr (kWarpWide) {
      // ================= TMA producer =================
      {
        int stage = 0;
        uint32_t phase = 0;
        bool alive = true;
        uint32_t excess_tx = (p.test_fault == 1 && blockIdx.x == 0) ? 16u : 0u;  // test hook, see GemmParams
        long long t_wait = 0, t_begin = prof ? clock64() : 0;
        for (int t = unit; t < num_tiles && alive; t += num_units) {
          int tm, tn;
          tile_coords(t / p.splits, p.tiles_m, p.tiles_n, p.group_n, tm, tn);
          const int row_a = (tm * CG + static_cast<int>(rank)) * kBlockM;
          const int row_b = tn * BN + static_cast<int>(rank) * L::kBRows;
          const int k_first = (t % p.splits) * k_slabs;
          for (int ks = k_first; ks < k_first + k_slabs; ++ks) {
            const long long w0 = prof ? clock64() : 0;
            if (!__all_sync(0xffffffffu, wait_or_abort(empty_bar(stage), phase ^ 1u, ctx, 1u))) { alive = false; break; }
            if (prof) t_wait += clock64() - w0;
            const uint32_t sbase = smem_base + stage * L::kStageBytes;
            // operand bytes of both CTAs of a pair are counted on the leader's barrier
            const uint32_t op_bar = CG == 2 ? mapa_shared(full_bar(stage), 0) : full_bar(stage);
            if (elect_one()) {
              if (leader) mbar_expect_tx(full_bar(stage), kOperandTx + excess_tx);
              tma_load_2d<CG>(sbase, &map_a, ks * 128, row_a, op_bar);
              tma_load_2d<CG>(sbase + L::kABytes, &map_b, ks * 128, row_b, op_bar);
            }
            __syncwarp();
            excess_tx = 0;
            if (++stage == STAGES) { stage = 0; phase ^= 1u; }
          }
        }
        if (prof) {
          counters[0] = t_wait;
          counters[1] = clock64() - t_begin;
        }
      }
    } else {
      // ================= TMA producer =================
      if (lane == 0) {
        int stage = 0;
        uint32_t phase = 0;
        bool alive = true;
        uint32_t excess_tx = (p.test_fault == 1 && blockIdx.x == 0) ? 16u : 0u;  // test hook, see GemmParams
        long long t_wait = 0, t_begin = prof ? clock64() : 0;
        for (int t = unit; t < num_tiles && alive; t += num_units) {
          int tm, tn;
          tile_coords(t / p.splits, p.tiles_m, p.tiles_n, p.group_n, tm, tn);
          const int row_a = (tm * CG + static_cast<int>(rank)) * kBlockM;
          const int row_b = tn * BN + static_cast<int>(rank) * L::kBRows;
          const int k_first = (t % p.splits) * k_slabs;
          for (int ks = k_first; ks < k_first + k_slabs; ++ks) {
            const long long w0 = prof ? clock64() : 0;
            if (!wait_or_abort(empty_bar(stage), phase ^ 1u, ctx, 1u)) { alive = false; break; }
            if (prof) t_wait += clock64() - w0;
            const uint32_t sbase = smem_base + stage * L::kStageBytes;
            // operand bytes of both CTAs of a pair are counted on the leader's barrier
            const uint32_t op_bar = CG == 2 ? mapa_shared(full_bar(stage), 0) : full_bar(stage);
            if (leader) mbar_expect_tx(full_bar(stage), kOperandTx + excess_tx);
            excess_tx = 0;
            tma_load_2d<CG>(sbase, &map_a, ks * 128, row_a, op_bar);
            tma_load_2d<CG>(sbase + L::kABytes, &map_b, ks * 128, row_b, op_bar);
            if (++stage == STAGES) { stage = 0; phase ^= 1u; }
          }
        }
        if (prof) {
          counters[0] = t_wait;
          counters[1] = clock64() - t_begin;
        }
      }
    }
  } else if (warp == kWarpMma || (MMAS == 2 && warp == kWarpMma2)) {
    if constexpr (kWarpWide) {
      // ================= MMA issuer(s) (leader CTA only) =================
      // Issuer `me` of MMAS takes the K slabs with (slab index in the tile) % MMAS == me and accumulates them
      // in its own tensor-memory columns.
      const int me = warp == kWarpMma ? 0 : 1;
      if (leader) {
        uint32_t acc_phase = 0;
        bool alive = true;
        int slab0 = 0;  // slabs of the tiles this CTA has finished: the ring position of the tile's first slab
        const bool mprof = prof && me == 0;
        long long t_full = 0, t_acc = 0, t_issue = 0, t_begin = mprof ? clock64() : 0;
        const uint64_t ns_begin = mprof ? globaltimer_ns() : 0;
        const uint32_t acc_tmem = tmem_base + static_cast<uint32_t>(me * BN);
        for (int t = unit; t < num_tiles && alive; t += num_units, slab0 += k_slabs) {
          const long long a0 = mprof ? clock64() : 0;
          if (!__all_sync(0xffffffffu,
                          wait_or_abort<kClusterAcquireWaits && CG == 2>(tmem_empty_bar, acc_phase ^ 1u, ctx, 2u)))
            break;
          if (mprof) t_acc += clock64() - a0;
          tc_fence_after();
          // A 64-wide tile uses half of a 128-row scale chunk of B: the MMA reads N / 32 scale columns from
          // the address it is given, so the upper half starts two columns in.
          uint32_t sfb_half = 0;
          if constexpr (BN == 64) {
            int tm, tn;
            tile_coords(t / p.splits, p.tiles_m, p.tiles_n, p.group_n, tm, tn);
            sfb_half = static_cast<uint32_t>(tn & 1) * 2u;
          }
          // ring position of this issuer's first slab of the tile; from there it moves MMAS stages per slab
          int stage = (slab0 + me) % STAGES;
          uint32_t phase = static_cast<uint32_t>((slab0 + me) / STAGES) & 1u;
          for (int ks = me; ks < k_slabs; ks += MMAS) {
            const long long w0 = mprof ? clock64() : 0;
            if (!__all_sync(0xffffffffu,
                            wait_or_abort<kClusterAcquireWaits && CG == 2>(full_bar(stage), phase, ctx, 3u))) {
              alive = false;
              break;
            }
            const long long w1 = mprof ? clock64() : 0;
            t_full += w1 - w0;
            tc_fence_after();
            const uint32_t sbase = smem_base + stage * L::kStageBytes;
            const uint32_t sf_tmem = tmem_base + kAccCols + stage * L::kSfCols;
            const uint64_t a_desc = operand_desc(sbase);
            const uint64_t b_desc = operand_desc(sbase + L::kABytes);
            if (elect_one()) {
  #pragma unroll
              for (int kb = 0; kb < 4; ++kb) {
                // 64 fp4 values = 32 bytes = 2 descriptor address units inside the swizzled row
                tc_mma<CG>(acc_tmem, a_desc + 2 * kb, b_desc + 2 * kb, kIdesc, sf_tmem + kb * 4,
                           sf_tmem + 16 + kb * 4 * L::kChunks + sfb_half, (ks >= MMAS || kb) ? 1u : 0u);
              }
              if constexpr (CG == 2) tc_commit_pair(empty_bar(stage));
              else tc_commit<CG>(empty_bar(stage));
            }
            __syncwarp();
            if (mprof) t_issue += clock64() - w1;
            stage += MMAS;
            if (stage >= STAGES) { stage -= STAGES; phase ^= 1u; }
          }
          if (!alive) break;
          if (elect_one()) {
            if constexpr (CG == 2) tc_commit_pair(tmem_full_bar);
            else tc_commit<CG>(tmem_full_bar);
          }
          __syncwarp();
          acc_phase ^= 1u;
        }
        if (mprof) {
          counters[2] = t_full;
          counters[3] = t_acc;
          counters[4] = clock64() - t_begin;
          counters[5] = t_issue;
          counters[11] = globaltimer_ns() - ns_begin;
        }
      }
    } else {
      // ================= MMA issuer(s) (leader CTA only) =================
      // Issuer `me` of MMAS takes the K slabs with (slab index in the tile) % MMAS == me and accumulates them
      // in its own tensor-memory columns.
      const int me = warp == kWarpMma ? 0 : 1;
      if (leader && lane == 0) {
        uint32_t acc_phase = 0;
        bool alive = true;
        int slab0 = 0;  // slabs of the tiles this CTA has finished: the ring position of the tile's first slab
        const bool mprof = prof && me == 0;
        long long t_full = 0, t_acc = 0, t_issue = 0, t_begin = mprof ? clock64() : 0;
        const uint64_t ns_begin = mprof ? globaltimer_ns() : 0;
        const uint32_t acc_tmem = tmem_base + static_cast<uint32_t>(me * BN);
        for (int t = unit; t < num_tiles && alive; t += num_units, slab0 += k_slabs) {
          const long long a0 = mprof ? clock64() : 0;
          if (!wait_or_abort<kClusterAcquireWaits && CG == 2>(tmem_empty_bar, acc_phase ^ 1u, ctx, 2u)) break;
          if (mprof) t_acc += clock64() - a0;
          tc_fence_after();
          // A 64-wide tile uses half of a 128-row scale chunk of B: the MMA reads N / 32 scale columns from
          // the address it is given, so the upper half starts two columns in.
          uint32_t sfb_half = 0;
          if constexpr (BN == 64) {
            int tm, tn;
            tile_coords(t / p.splits, p.tiles_m, p.tiles_n, p.group_n, tm, tn);
            sfb_half = static_cast<uint32_t>(tn & 1) * 2u;
          }
          // ring position of this issuer's first slab of the tile; from there it moves MMAS stages per slab
          int stage = (slab0 + me) % STAGES;
          uint32_t phase = static_cast<uint32_t>((slab0 + me) / STAGES) & 1u;
          bool polled = false;  // the poll issued with the previous slab already found this slab's barrier complete
          for (int ks = me; ks < k_slabs; ks += MMAS) {
            const long long w0 = mprof ? clock64() : 0;
            if (!polled && !wait_or_abort<kClusterAcquireWaits && CG == 2>(full_bar(stage), phase, ctx, 3u)) {
              alive = false;
              break;
            }
            const long long w1 = mprof ? clock64() : 0;
            t_full += w1 - w0;
            tc_fence_after();
            const uint32_t sbase = smem_base + stage * L::kStageBytes;
            const uint32_t sf_tmem = tmem_base + kAccCols + stage * L::kSfCols;
            int next_stage = stage + MMAS;
            uint32_t next_phase = phase;
            if (next_stage >= STAGES) { next_stage -= STAGES; next_phase ^= 1u; }
            const bool more = ks + MMAS < k_slabs;
            // 64 fp4 values = 32 bytes = 2 descriptor address units inside the swizzled row: the helper steps the
            // descriptors by 2, the scales of A by 4 columns and those of B by 4 per 128-row chunk per MMA.
            // After the tile's last slab there is nothing to poll: it polls this slab's own, completed barrier.
            const uint32_t ok = tc_slab_and_poll_next<CG>(
                acc_tmem, operand_desc(sbase), operand_desc(sbase + L::kABytes), kIdesc, sf_tmem,
                sf_tmem + 16 + sfb_half, 4 * L::kChunks, ks >= MMAS ? 1u : 0u, empty_bar(stage),
                full_bar(more ? next_stage : stage), more ? next_phase : phase);
            polled = more && ok != 0;
            stage = next_stage;
            phase = next_phase;
            if (mprof) t_issue += clock64() - w1;
          }
          if (!alive) break;
          if constexpr (CG == 2) tc_commit_pair(tmem_full_bar);
          else tc_commit<CG>(tmem_full_bar);
          acc_phase ^= 1u;
        }
        if (mprof) {
          counters[2] = t_full;
          counters[3] = t_acc;
          counters[4] = clock64() - t_begin;
          counters[5] = t_issue;
          counters[11] = globaltimer_ns() - ns_begin;
        }
      }
    }
  } else if (warp < kWarpEpi0) {
    // ================= scale warps: shared memory -> registers -> tensor memory =================
    // tcgen05.cp would do this copy with one shared-memory read instead of four, but every tcgen05
    // instruction costs the thread that issues it 35-70 cycles: the twelve copies of a slab plus their
    // commit take a thread ~760 cycles, and that delay sits on the path from "scales landed" to "MMA may
    // start".  Issued by the MMA thread the copies tripled its time per slab; issued by two threads of
    // their own (stages by parity) the kernel was still 6 % slower than with these warps, whose path
    // takes ~210 cycles (8192^3: 220.6 against 207.5 us; decode 13.8 against 11.8 us).
    // TMEM lane L, column 4*kb + j of a stage's scale area holds the four scales (one per 16-wide
    // K block of k-block kb) of tile row 32*j + L % 32, i.e. 16-byte row L % 32 of the 512-byte
    // swizzled block; every 32-lane quarter carries the same data.
    // Two sets of four warps share the K slabs, so one set's wait for its TMEM stores overlaps
    // the other set's shared-memory reads.  A set owns the stages of one parity: it then
    // observes every phase of the barriers it waits on (a waiter that skipped a phase could not
    // tell the phase it wants from the one two before it).
    const int quarter = warp & 3;
    const int set = (warp - kWarpScale0) >> 2;
    const bool sprof = prof && warp == kWarpScale0;
    long long t_wait = 0, t_body = 0;
    const int total_slabs = ((num_tiles - unit + num_units - 1) / num_units) * k_slabs;
    for (int n = 0; n < total_slabs; ++n) {
      const int stage = n % STAGES;
      if ((stage & 1) != set) continue;
      const uint32_t phase = static_cast<uint32_t>(n / STAGES) & 1u;
      const long long w0 = sprof ? clock64() : 0;
      if (!wait_or_abort(sfload_bar(stage), phase, ctx, 5u)) break;
      const long long w1 = sprof ? clock64() : 0;
      const uint32_t sfa_smem = smem_base + stage * L::kStageBytes + L::kABytes + L::kBBytes + lane * 16;
      const uint32_t sfb_smem = sfa_smem + L::kSfaBytes;
      uint32_t a[16], b[16 * L::kChunks];
#pragma unroll
      for (int kb = 0; kb < 4; ++kb) lds128(sfa_smem + kb * 512, a + 4 * kb);
#pragma unroll
      for (int kb = 0; kb < 4; ++kb)
#pragma unroll
        for (int c = 0; c < L::kChunks; ++c) lds128(sfb_smem + (c * 4 + kb) * 512, b + 4 * (kb * L::kChunks + c));
      const uint32_t dst = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + kAccCols + stage * L::kSfCols;
      tmem_st_32x32_x16(dst, a);
#pragma unroll
      for (int c = 0; c < L::kChunks; ++c) tmem_st_32x32_x16(dst + 16 + 16 * c, b + 16 * c);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (leader) mbar_arrive_local(full_bar(stage));
        else mbar_arrive_cluster_relaxed(mapa_shared(full_bar(stage), 0));
      }
      if (sprof) { t_wait += w1 - w0; t_body += clock64() - w1; }
    }
    if (sprof) {
      counters[9] = t_wait;
      counters[10] = t_body;
    }
  } else if (warp == kWarpScaleProducer) {
    if constexpr (kWarpWide) {
      // ================= TMA producer of the scale factors =================
      // A warp of its own: with the operand copies in the same issuing role that role was the slowest stage of
      // the pipeline.
      {
        int stage = 0;
        uint32_t phase = 0;
        bool alive = true;
        for (int t = unit; t < num_tiles && alive; t += num_units) {
          int tm, tn;
          tile_coords(t / p.splits, p.tiles_m, p.tiles_n, p.group_n, tm, tn);
          const int row_a = (tm * CG + static_cast<int>(rank)) * kBlockM;
          const int k_first = (t % p.splits) * k_slabs;
          for (int ks = k_first; ks < k_first + k_slabs; ++ks) {
            if (!__all_sync(0xffffffffu, wait_or_abort(empty_bar(stage), phase ^ 1u, ctx, 1u))) { alive = false; break; }
            const uint32_t sf_smem = smem_base + stage * L::kStageBytes + L::kABytes + L::kBBytes;
            if (elect_one()) {
              mbar_expect_tx(sfload_bar(stage), kScaleTx);
              tma_load_3d<1>(sf_smem, &map_sfa, 0, ks * 4, row_a / 128, sfload_bar(stage));
              tma_load_3d<1>(sf_smem + L::kSfaBytes, &map_sfb, 0, ks * 4, (tn * BN) / 128, sfload_bar(stage));
            }
            __syncwarp();
            if (++stage == STAGES) { stage = 0; phase ^= 1u; }
          }
        }
      }
    } else {
      // ================= TMA producer of the scale factors =================
      // A thread of its own: issuing a TMA copy costs its thread on the order of a hundred cycles, and
      // four of them in one thread per slab made that thread the slowest stage of the pipeline.
      if (lane == 0) {
        int stage = 0;
        uint32_t phase = 0;
        bool alive = true;
        for (int t = unit; t < num_tiles && alive; t += num_units) {
          int tm, tn;
          tile_coords(t / p.splits, p.tiles_m, p.tiles_n, p.group_n, tm, tn);
          const int row_a = (tm * CG + static_cast<int>(rank)) * kBlockM;
          const int k_first = (t % p.splits) * k_slabs;
          for (int ks = k_first; ks < k_first + k_slabs; ++ks) {
            if (!wait_or_abort(empty_bar(stage), phase ^ 1u, ctx, 1u)) { alive = false; break; }
            const uint32_t sf_smem = smem_base + stage * L::kStageBytes + L::kABytes + L::kBBytes;
            mbar_expect_tx(sfload_bar(stage), kScaleTx);
            tma_load_3d<1>(sf_smem, &map_sfa, 0, ks * 4, row_a / 128, sfload_bar(stage));
            tma_load_3d<1>(sf_smem + L::kSfaBytes, &map_sfb, 0, ks * 4, (tn * BN) / 128, sfload_bar(stage));
            if (++stage == STAGES) { stage = 0; phase ^= 1u; }
          }
        }
      }
    }
  } else {
    // ================= epilogue: 8 warps, lane quarter = warp & 3, column half = (warp - 10) / 4 ===========
    constexpr int kHalf = BN / 2;
    const int quarter = warp & 3;
    const int half = (warp - kWarpEpi0) >> 2;
    const float alpha = __ldg(p.alpha);
    const uint64_t store_policy = l2_policy_evict_first();
    uint32_t acc_phase = 0;
    const uint32_t empty_target = CG == 2 ? mapa_shared(tmem_empty_bar, 0) : tmem_empty_bar;
    const bool eprof = prof && warp == kWarpEpi0;
    long long t_wait = 0, t_body = 0, n_tiles = 0;
    // 32 accumulator columns of this warp's lane quarter, starting at tile column `col` (with two MMA
    // warps: the sum of their two accumulators)
    auto drain32 = [&](int col, uint32_t (&v)[32]) {
      const uint32_t addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + col;
      tmem_ld_32x32(addr, v);
      if constexpr (MMAS == 2) {
        uint32_t v2[32];
        tmem_ld_32x32(addr + BN, v2);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) + __uint_as_float(v2[i]));
      } else {
        tmem_ld_wait();
      }
    };
    for (int t = unit; t < num_tiles; t += num_units) {
      int tm, tn;
      tile_coords(t / p.splits, p.tiles_m, p.tiles_n, p.group_n, tm, tn);
      const long long w0 = eprof ? clock64() : 0;
      if (!wait_or_abort(tmem_full_bar, acc_phase, ctx, 4u)) break;
      const long long w1 = eprof ? clock64() : 0;
      t_wait += w1 - w0;
      tc_fence_after();
      const int row = (tm * CG + static_cast<int>(rank)) * kBlockM + quarter * 32 + lane;
      const int64_t doff = static_cast<int64_t>(row) * p.ldd + p.col0 + static_cast<int64_t>(tn) * BN + half * kHalf;
      uint16_t* drow = p.D + doff;
      // Drain this warp's part of the accumulator into registers as packed bf16, hand tensor memory
      // back to the MMA warp, and only then write to global memory: the next tile's MMAs overlap
      // the stores.
      if (p.splits > 1) {
        // split K: this work item's fp32 partial sums go to scratch; a second kernel adds the ranges
        if ((tm * CG + static_cast<int>(rank)) * kBlockM + quarter * 32 < p.M) {
          // (a decode-sized M leaves most lane quarters without a single row to drain)
          float* prow = p.partial + (static_cast<int64_t>(t % p.splits) * p.M + row) * p.N +
                        static_cast<int64_t>(tn) * BN + half * kHalf;
#pragma unroll 1
          for (int c0 = 0; c0 < kHalf; c0 += 32) {
            uint32_t v[32];
            drain32(half * kHalf + c0, v);
            if (row < p.M) {
              uint4* dst = reinterpret_cast<uint4*>(prow + c0);
#pragma unroll
              for (int i = 0; i < 8; ++i) dst[i] = make_uint4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          if (leader) mbar_arrive_local(tmem_empty_bar);
          else mbar_arrive_cluster_relaxed(empty_target);
        }
        acc_phase ^= 1u;
        if (eprof) { t_body += clock64() - w1; ++n_tiles; }
        continue;
      }
      if constexpr (TMA_OUT > 0) {
        // Drain to registers, hand tensor memory back, then push the rows through shared memory:
        // each lane owns one row and writes 16-byte chunks at their 128-byte-swizzled position
        // (conflict-free); one lane hands every 32 x 64 sub-tile to the TMA, once per destination
        // buffer.  Rows past M are clipped by the tensor map.  The stores run while the next tile is
        // multiplied; peers are reached by stores only.
        constexpr int kSubs = kHalf / 64;
        const uint32_t staging = smem_base + STAGES * L::kStageBytes +
                                 static_cast<uint32_t>(warp - kWarpEpi0) * TMA_OUT * 4096u;
        uint32_t packed[kHalf / 2];
#pragma unroll
        for (int c0 = 0; c0 < kHalf; c0 += 32) {
          uint32_t v[32];
          drain32(half * kHalf + c0, v);
#pragma unroll
          for (int i = 0; i < 16; ++i)
            packed[c0 / 2 + i] = pack_from_f32<BF16Tag>(__uint_as_float(v[2 * i]) * alpha,
                                                        __uint_as_float(v[2 * i + 1]) * alpha);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          if (leader) mbar_arrive_local(tmem_empty_bar);
          else mbar_arrive_cluster_relaxed(empty_target);
        }
        const int row0 = (tm * CG + static_cast<int>(rank)) * kBlockM + quarter * 32;
        const int x0 = p.col0 + tn * BN + half * kHalf;
#pragma unroll
        for (int sub = 0; sub < kSubs; ++sub) {
          if (sub % TMA_OUT == 0) {
            if (lane == 0) bulk_wait_read_all();  // earlier stores have read the staging
            __syncwarp();
          }
          const uint32_t buf = staging + (sub % TMA_OUT) * 4096u;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const uint32_t chunk = static_cast<uint32_t>(j) ^ (lane & 7u);
            sts128(buf + lane * 128u + chunk * 16u, packed[sub * 32 + 4 * j], packed[sub * 32 + 4 * j + 1],
                   packed[sub * 32 + 4 * j + 2], packed[sub * 32 + 4 * j + 3]);
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            if (row0 < p.M)
              for (int d = 0; d < p.n_dest; ++d) tma_store_2d(&out_maps.m[d], buf, x0 + sub * 64, row0, store_policy);
            bulk_commit();
          }
        }
      } else {
      uint32_t packed[kHalf / 2];
#pragma unroll
      for (int c0 = 0; c0 < kHalf; c0 += 32) {
        uint32_t v[32];
        drain32(half * kHalf + c0, v);
#pragma unroll
        for (int i = 0; i < 16; ++i)
          packed[c0 / 2 + i] = pack_from_f32<BF16Tag>(__uint_as_float(v[2 * i]) * alpha,
                                                      __uint_as_float(v[2 * i + 1]) * alpha);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (leader) mbar_arrive_local(tmem_empty_bar);
        else mbar_arrive_cluster_relaxed(empty_target);
      }
      if (row < p.M) {
        uint4* dst = reinterpret_cast<uint4*>(drow);
#pragma unroll
        for (int i = 0; i < kHalf / 8; ++i)
          dst[i] = make_uint4(packed[4 * i], packed[4 * i + 1], packed[4 * i + 2], packed[4 * i + 3]);
      }
      }
      acc_phase ^= 1u;
      if (eprof) { t_body += clock64() - w1; ++n_tiles; }
    }
    if constexpr (TMA_OUT > 0) {
      if (lane == 0) bulk_wait_all();  // every store has left shared memory and is written
    }
    if (eprof) {
      counters[6] = t_wait;
      counters[7] = t_body;
      counters[8] = n_tiles;
    }
  }

  // ---- teardown: nobody leaves while a peer may still signal into this CTA ----
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // give copies that may still be in flight time to land before shared memory is released
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
  }
  if constexpr (CG == 2) cluster_sync_all();
  if (warp == kWarpMma) {
    tc_fence_after();
    tmem_dealloc<CG>(tmem_base, kTmemCols);
  }
}

// ---- host ----------------------------------------------------------------------------------------
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                   CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                   CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult result;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &result) == cudaSuccess &&
        result == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  });
  return fn;
}

int encode_operand_map(CUtensorMap* map, const void* base, int rows, int k, int box_rows) {
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(k / 2), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(k / 2)};
  const cuuint32_t box[2] = {128, static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult r = encode_tiled_fn()(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims,
                                       strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                       CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                       CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled(operand) failed with %d", static_cast<int>(r));
    return B2_ERR_CUDA;
  }
  return B2_OK;
}

// The swizzled scale buffer is [rows/128][K/64][512 bytes]; viewed as uint16 (256, K/64, rows/128),
// one load of box (256, 4, chunks) lands in shared memory as [chunk][k-block][512 B].
int encode_scale_map(CUtensorMap* map, const void* base, int rows_padded, int k, int chunks) {
  const cuuint64_t dims[3] = {256, static_cast<cuuint64_t>(k / 64), static_cast<cuuint64_t>(rows_padded / 128)};
  const cuuint64_t strides[2] = {512, static_cast<cuuint64_t>(k) * 8};
  const cuuint32_t box[3] = {256, 4, static_cast<cuuint32_t>(chunks)};
  const cuuint32_t elem[3] = {1, 1, 1};
  const CUresult r = encode_tiled_fn()(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, const_cast<void*>(base), dims,
                                       strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                       CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                       CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled(scales) failed with %d", static_cast<int>(r));
    return B2_ERR_CUDA;
  }
  return B2_OK;
}

struct MapKey {
  const void *a, *b, *sfa, *sfb;
  int m, n, k, variant;
  bool operator==(const MapKey& o) const {
    return a == o.a && b == o.b && sfa == o.sfa && sfb == o.sfb && m == o.m && n == o.n && k == o.k &&
           variant == o.variant;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = 1469598103934665603ull;
    auto mix = [&](uint64_t v) { h = (h ^ v) * 1099511628211ull; };
    mix(reinterpret_cast<uint64_t>(k.a));
    mix(reinterpret_cast<uint64_t>(k.b));
    mix(reinterpret_cast<uint64_t>(k.sfa));
    mix(reinterpret_cast<uint64_t>(k.sfb));
    mix((static_cast<uint64_t>(k.m) << 32) ^ static_cast<uint64_t>(k.n));
    mix((static_cast<uint64_t>(k.k) << 8) ^ static_cast<uint64_t>(k.variant));
    return h;
  }
};
struct MapSet {
  CUtensorMap a, b, sfa, sfb;
};

std::mutex g_mu;
std::unordered_map<MapKey, MapSet, MapKeyHash> g_maps;
uint32_t* g_status[64] = {nullptr};
constexpr int kStatusWords = 64;  // 2 status words, padding, 12 64-bit role timers from word 16
std::atomic<int> g_profile{0};
std::atomic<unsigned long long> g_wait_budget_ns{kWaitBudgetNs};
std::atomic<int> g_test_fault{0};  // consumed by the next launch
// Launch the GEMM with the programmatic-dependent-launch attribute (B2_GEMM_PDL=0 turns it off).
int pdl_from_env() {
  const char* v = std::getenv("B2_GEMM_PDL");
  return (v && v[0] == '0') ? 0 : 1;
}
std::atomic<int> g_pdl{pdl_from_env()};


// Device status word of the current device, allocated (and zeroed) on first use.
int status_word(uint32_t** out) {
  int dev = 0;
  B2_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) {
    set_error("device ordinal %d out of range", dev);
    return B2_ERR_CUDA;
  }
  std::lock_guard<std::mutex> lock(g_mu);
  if (!g_status[dev]) {
    uint32_t* ptr = nullptr;
    B2_CUDA_TRY(cudaMalloc(&ptr, kStatusWords * sizeof(uint32_t)));
    B2_CUDA_TRY(cudaMemset(ptr, 0, kStatusWords * sizeof(uint32_t)));
    g_status[dev] = ptr;
  }
  *out = g_status[dev];
  return B2_OK;
}

// D = bf16(alpha * sum over K ranges of the fp32 partial sums), ranges added in index order.
__global__ void splitk_reduce_kernel(const float* __restrict__ partial, const float* __restrict__ alpha,
                                     uint16_t* __restrict__ D, int64_t mn, int splits) {
  asm volatile("griddepcontrol.wait;" ::: "memory");  // the GEMM grid has finished and its partial sums are visible
  const int64_t i = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) * 8;
  if (i >= mn) return;
  float acc[8];
  {
    const float4 a = *reinterpret_cast<const float4*>(partial + i), b = *reinterpret_cast<const float4*>(partial + i + 4);
    acc[0] = a.x; acc[1] = a.y; acc[2] = a.z; acc[3] = a.w; acc[4] = b.x; acc[5] = b.y; acc[6] = b.z; acc[7] = b.w;
  }
  for (int s = 1; s < splits; ++s) {
    const float* src = partial + s * mn + i;
    const float4 a = *reinterpret_cast<const float4*>(src), b = *reinterpret_cast<const float4*>(src + 4);
    acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w; acc[4] += b.x; acc[5] += b.y; acc[6] += b.z; acc[7] += b.w;
  }
  const float al = __ldg(alpha);
  uint4 out;
  out.x = pack_from_f32<BF16Tag>(acc[0] * al, acc[1] * al);
  out.y = pack_from_f32<BF16Tag>(acc[2] * al, acc[3] * al);
  out.z = pack_from_f32<BF16Tag>(acc[4] * al, acc[5] * al);
  out.w = pack_from_f32<BF16Tag>(acc[6] * al, acc[7] * al);
  *reinterpret_cast<uint4*>(D + i) = out;
}

template <int CG, int BN, int STAGES, int AM = kBlockM>
int encode_maps(MapSet* maps, const void* A, const void* B, const void* SFA, const void* SFB, int M, int N, int K) {
  using L = SmemLayout<CG, BN, STAGES, 0, AM>;
  const int m_padded = (M + 127) / 128 * 128, n_padded = (N + 127) / 128 * 128;
  if (int rc = encode_operand_map(&maps->a, A, M, K, AM)) return rc;
  if (int rc = encode_operand_map(&maps->b, B, N, K, L::kBRows)) return rc;
  if (int rc = encode_scale_map(&maps->sfa, SFA, m_padded, K, 1)) return rc;
  if (int rc = encode_scale_map(&maps->sfb, SFB, n_padded, K, L::kChunks)) return rc;
  return B2_OK;
}

// Launches the GEMM (and, with splits > 1, the reduction) on prepared tensor maps and scratch.
struct GatherTarget {  // the gathered output layout: row length and this GPU's first column in it
  int n_dest = 0;
  int ldd = 0;   // 0: N
  int col0 = 0;
};

// One 32-row x 64-column store box of a bf16 [M, ldd] output, 128-byte swizzled in shared memory.
int encode_output_map(CUtensorMap* map, void* base, int M, int ldd) {
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(ldd), static_cast<cuuint64_t>(M)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ldd) * 2};
  const cuuint32_t box[2] = {64, 32};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult r = encode_tiled_fn()(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, dims, strides, box, elem,
                                       CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                       CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled(output) failed with %d", static_cast<int>(r));
    return B2_ERR_CUDA;
  }
  return B2_OK;
}

template <int CG, int BN, int STAGES, int TMA_OUT = 0, int AM = kBlockM, int MMAS = 1>
int launch_kernels(const MapSet& maps, const float* alpha, void* D, int M, int N, int K, int splits,
                   uint32_t* status, float* partial, cudaStream_t stream, const GatherTarget& gather = GatherTarget(),
                   const OutMaps<(TMA_OUT > 0)>& out_maps = OutMaps<(TMA_OUT > 0)>()) {
  using L = SmemLayout<CG, BN, STAGES, TMA_OUT, AM>;
  auto kernel = nvfp4_gemm_kernel<CG, BN, STAGES, TMA_OUT, AM, MMAS>;
  GemmParams p;
  p.alpha = alpha;
  p.D = static_cast<uint16_t*>(D);
  p.n_dest = gather.n_dest;
  p.ldd = gather.ldd ? gather.ldd : N;
  p.col0 = gather.col0;
  p.status = status;
  p.profile = g_profile.load(std::memory_order_relaxed);
  p.M = M;
  p.N = N;
  p.K = K;
  p.splits = splits;
  p.partial = partial;
  p.tiles_m = (M + kBlockM * CG - 1) / (kBlockM * CG);
  p.tiles_n = N / BN;
  p.group_n = 8;
  p.wait_budget_ns = g_wait_budget_ns.load(std::memory_order_relaxed);
  p.test_fault = g_test_fault.exchange(0, std::memory_order_relaxed);
  const int sms = device_sm_count();
  if (sms <= 0) return B2_ERR_CUDA;
  // Persistent CTAs (pairs): as many as finish the work in the fewest rounds, and no more.  256 tiles on
  // 74 pairs take four rounds whether 74 or 64 pairs run them; with 64 every round is full and ten pairs
  // fewer compete for L2 and for the power budget.
  const int work = p.tiles_m * p.tiles_n * splits;
  const int rounds = (work + sms / CG - 1) / (sms / CG);
  const int units = (work + rounds - 1) / rounds;

  // The shared-memory limit of a kernel is an attribute per device: set it once for every device
  // ordinal this instantiation is launched on.
  {
    static bool configured[64] = {};  // per template instantiation, guarded by g_mu
    int dev = 0;
    B2_CUDA_TRY(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lock(g_mu);
    if (dev < 0 || dev >= 64 || !configured[dev]) {
      B2_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal));
      if (dev >= 0 && dev < 64) configured[dev] = true;
    }
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(units * CG);
  cfg.blockDim = dim3(kThreads + 32 * (MMAS - 1));
  cfg.dynamicSmemBytes = L::kTotal;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  cfg.attrs = attr;
  if (CG == 2) {
    attr[cfg.numAttrs].id = cudaLaunchAttributeClusterDimension;
    attr[cfg.numAttrs].val.clusterDim.x = 2;
    attr[cfg.numAttrs].val.clusterDim.y = 1;
    attr[cfg.numAttrs].val.clusterDim.z = 1;
    ++cfg.numAttrs;
  }
  if (g_pdl.load(std::memory_order_relaxed)) {
    // May start while the previous kernel on the stream is still running; see griddepcontrol.wait in the kernel.
    attr[cfg.numAttrs].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[cfg.numAttrs].val.programmaticStreamSerializationAllowed = 1;
    ++cfg.numAttrs;
  }
  B2_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, maps.a, maps.b, maps.sfa, maps.sfb, p, out_maps));
  if (splits > 1) {
    const int64_t mn = static_cast<int64_t>(M) * N;
    const int threads = 256;
    const int64_t blocks = (mn / 8 + threads - 1) / threads;
    cudaLaunchConfig_t rcfg = {};
    rcfg.gridDim = dim3(static_cast<unsigned>(blocks));
    rcfg.blockDim = dim3(threads);
    rcfg.stream = stream;
    cudaLaunchAttribute rattr[1];
    rattr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    rattr[0].val.programmaticStreamSerializationAllowed = 1;
    rcfg.attrs = rattr;
    rcfg.numAttrs = 1;
    B2_CUDA_TRY(cudaLaunchKernelEx(&rcfg, splitk_reduce_kernel, static_cast<const float*>(partial), alpha, p.D, mn, splits));
  }
  return B2_OK;
}

struct Scratch {
  float* ptr = nullptr;
  size_t bytes = 0;
  std::vector<void*> retired;  // outgrown buffers: earlier launches and captured graphs may still name them
};
Scratch g_scratch[64];
constexpr size_t kFirstScratchBytes = 32u << 20;  // covers 8 K ranges x 128 x 8192 fp32

// Per-device scratch for split-K partial sums.  The first request allocates 32 MiB (or what the
// request needs, if more); a larger request later allocates a new buffer and keeps the old one
// alive until the process exits, so nothing is ever freed under a launch in flight or a captured
// graph, and the launch path never takes the device-wide synchronisation of cudaFree.
int partial_scratch(size_t bytes, float** out) {
  int dev = 0;
  B2_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) {
    set_error("device ordinal %d out of range", dev);
    return B2_ERR_CUDA;
  }
  std::lock_guard<std::mutex> lock(g_mu);
  Scratch& sc = g_scratch[dev];
  if (sc.bytes < bytes) {
    const size_t want = bytes > kFirstScratchBytes ? bytes : kFirstScratchBytes;
    void* fresh = nullptr;
    B2_CUDA_TRY(cudaMalloc(&fresh, want));
    if (sc.ptr) sc.retired.push_back(sc.ptr);
    sc.ptr = static_cast<float*>(fresh);
    sc.bytes = want;
  }
  *out = sc.ptr;
  return B2_OK;
}

// K ranges for shapes with too few output tiles to occupy the GPU (decode-sized M): the largest
// power of two that keeps every SM at most one work item, divides the slab count and leaves at
// least four slabs per range.
int choose_splits(int tiles, int k_slabs, int units_available) {
  int splits = 1;
  while (splits < 8 && tiles * splits * 2 <= units_available && k_slabs % (splits * 2) == 0 &&
         k_slabs / (splits * 2) >= 4)
    splits *= 2;
  return splits;
}

// Status words and split-K scratch a caller-independent source provides (the array built into the
// library, for the entry point that must not allocate); null = the library's allocated ones.
struct FixedWorkspace {
  uint32_t* status;
  float* partial;
  size_t partial_bytes;
  const char* who;
};

template <int CG, int BN, int STAGES, int TMA_OUT = 0, int AM = kBlockM, int MMAS = 1>
int launch_variant(const void* A, const void* B, const void* SFA, const void* SFB, const float* alpha,
                   void* D, int M, int N, int K, int variant, cudaStream_t stream,
                   const FixedWorkspace* fixed = nullptr) {
  const int sms = device_sm_count();
  if (sms <= 0) return B2_ERR_CUDA;
  const int tiles = ((M + kBlockM * CG - 1) / (kBlockM * CG)) * (N / BN);
  const int splits = choose_splits(tiles, K / kBlockK, sms / CG);
  const size_t need = splits > 1 ? static_cast<size_t>(splits) * M * N * sizeof(float) : 0;
  uint32_t* status = nullptr;
  float* partial = nullptr;
  if (fixed) {
    if (need > fixed->partial_bytes) {
      set_error("%s: M=%d N=%d K=%d needs %zu bytes of partial sums (%d K ranges), the built-in scratch holds "
                "%zu; use b2_nvfp4_gemm", fixed->who, M, N, K, need, splits, fixed->partial_bytes);
      return B2_ERR_INVALID_ARGUMENT;
    }
    status = fixed->status;
    partial = fixed->partial;
  } else {
    if (int rc = status_word(&status)) return rc;
    if (need) {
      if (int rc = partial_scratch(need, &partial)) return rc;
    }
  }
  MapSet maps;
  {
    const MapKey key{A, B, SFA, SFB, M, N, K, variant};
    std::lock_guard<std::mutex> lock(g_mu);
    auto it = g_maps.find(key);
    if (it == g_maps.end()) {
      MapSet fresh;
      if (int rc = encode_maps<CG, BN, STAGES, AM>(&fresh, A, B, SFA, SFB, M, N, K)) return rc;
      if (g_maps.size() > 4096) g_maps.clear();
      it = g_maps.emplace(key, fresh).first;
    }
    maps = it->second;
  }
  if constexpr (TMA_OUT > 0) {
    OutMaps<true> out_maps;
    {
      const MapKey key{D, nullptr, nullptr, nullptr, M, N, 0, -1};
      std::lock_guard<std::mutex> lock(g_mu);
      auto it = g_maps.find(key);
      if (it == g_maps.end()) {
        MapSet fresh;
        if (int rc = encode_output_map(&fresh.a, D, M, N)) return rc;
        if (g_maps.size() > 4096) g_maps.clear();
        it = g_maps.emplace(key, fresh).first;
      }
      out_maps.m[0] = it->second.a;
    }
    GatherTarget target;
    target.n_dest = 1;
    return launch_kernels<CG, BN, STAGES, TMA_OUT>(maps, alpha, D, M, N, K, splits, status, partial, stream, target,
                                                out_maps);
  } else {
    return launch_kernels<CG, BN, STAGES, 0, AM, MMAS>(maps, alpha, D, M, N, K, splits, status, partial, stream);
  }
}

std::atomic<int> g_forced_variant{-1};  // test hook: -1 = automatic

// Automatic choice of the kernel variant (numbering of b2_nvfp4_gemm_set_variant).
int choose_variant(int M, int N, int K) {
  const int sms = device_sm_count();
  if (M <= 128) {
    // Decode-sized M: single-CTA tiles and K ranges to fill the GPU.  The time goes with the slabs
    // one CTA runs in series (waves x slabs per work item); a 256-wide slab costs about 1.8 of a
    // 128-wide one, and its four-fold partial sums only pay off while M is small.
    // M <= 32 and no more 64-wide tiles than SMs: every CTA takes one tile and all of K, two warps issue
    // its MMAs; no K ranges, no second kernel (16 x 8192 x 8192: 11.8 us against 13.1 with K ranges).
    if (sms > 0 && M <= 32 && N / 64 <= sms && K >= 512) return 7;
    // The same tiling with all 128 rows of A per stage for 32 < M <= 128 (128 x 8192 x 8192: 12.5 us against
    // 16.1 with 128-wide tiles and K ranges; 64 x 8192 x 8192: 12.2 against 14.5).
    if (sms > 0 && N / 64 <= sms && K >= 512) return 8;
    int variant = 0;
    if (sms > 0 && M <= 32 && N % 256 == 0) {
      const int k_slabs = K / kBlockK;
      auto serial_slabs = [&](int bn) {
        const int tiles = N / bn;
        const int splits = choose_splits(tiles, k_slabs, sms);
        return static_cast<double>((tiles * splits + sms - 1) / sms) * (k_slabs / splits);
      };
      if (1.8 * serial_slabs(256) < serial_slabs(128)) variant = 1;
    }
    if (M <= 32) variant += 4;  // 32 rows of A per stage, deeper ring
    return variant;
  }
  // At most one 128 x 128 tile per SM: single-CTA tiles in one wave, two warps issuing alternate K slabs into
  // two accumulators (256 x 8192 x 8192: 14.3 us against 15.9 with 256 x 128 pair tiles, 512 x 4096 x 4096:
  // 9.3 against 10.5; cold weights, launches in a CUDA graph).
  if (sms > 0 && static_cast<int64_t>((M + 127) / 128) * (N / 128) <= sms && K >= 512) return 9;
  int variant = N % 256 == 0 ? 2 : 3;
  if (variant == 2) {
    // few 256 x 256 tiles (fewer than half the CTA pairs busy): 256 x 128 tiles double the parallelism
    const int64_t tiles = static_cast<int64_t>((M + 255) / 256) * (N / 256);
    if (sms > 0 && tiles * 2 <= sms / 2) variant = 3;
  }
  return variant;
}

}  // namespace
}  // namespace b2

// Selects a kernel variant for the following calls of this process (-1 restores automatic
// selection).  0: single CTA, N tile 128; 1: single CTA, N tile 256; 2: CTA pair, N tile 256;
// 3: CTA pair, N tile 128; 4 and 5: 0 and 1 for M <= 32, loading 32 rows of A per stage into a deeper
// ring; 6: M <= 32, N tile 64; 7: 6 with two MMA-issuing warps; 8: 7 with all 128 rows of A per stage
// (M <= 128); 9: 0 with two MMA-issuing warps.  Used by the tests to exercise every variant on small shapes.
extern "C" int b2_nvfp4_gemm_set_variant(int variant) {
  if (variant < -1 || variant > 9) {
    b2::set_error("b2_nvfp4_gemm_set_variant: unknown variant %d", variant);
    return B2_ERR_INVALID_ARGUMENT;
  }
  b2::g_forced_variant.store(variant, std::memory_order_relaxed);
  return B2_OK;
}

extern "C" int b2_nvfp4_gemm(const void* A, const void* B, const void* SFA, const void* SFB,
                             const float* alpha_dev, void* D, int M, int N, int K, void* stream) {
  using namespace b2;
  if (!A || !B || !SFA || !SFB || !alpha_dev || !D) {
    set_error("b2_nvfp4_gemm: null pointer argument");
    return B2_ERR_INVALID_ARGUMENT;
  }
  if (M < 1 || N < 1 || K < 1 || K % 256 != 0 || N % 128 != 0) {
    set_error("b2_nvfp4_gemm: M=%d N=%d K=%d: need M >= 1, N %% 128 == 0, K %% 256 == 0", M, N, K);
    return B2_ERR_INVALID_ARGUMENT;
  }
  const uintptr_t all = reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) |
                        reinterpret_cast<uintptr_t>(SFA) | reinterpret_cast<uintptr_t>(SFB) |
                        reinterpret_cast<uintptr_t>(D);
  if (all & 15) {
    set_error("b2_nvfp4_gemm: all tensors must be 16-byte aligned");
    return B2_ERR_INVALID_ARGUMENT;
  }
  if (!encode_tiled_fn()) {
    set_error("b2_nvfp4_gemm: cuTensorMapEncodeTiled is not available from this driver");
    return B2_ERR_CUDA;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int variant = g_forced_variant.load(std::memory_order_relaxed);
  if (variant < 0) variant = choose_variant(M, N, K);
  if (variant == 7 && K < 512) variant = 6;  // the second MMA warp needs a K slab of its own
  if (variant == 9 && K < 512) variant = 0;
  if (variant == 8 && (K < 512 || M > 128)) {
    set_error("b2_nvfp4_gemm: variant 8 needs M <= 128 and K >= 512");
    return B2_ERR_INVALID_ARGUMENT;
  }
  if ((variant == 4 || variant == 5 || variant == 6 || variant == 7) && M > 32) {
    set_error("b2_nvfp4_gemm: variant %d needs M <= 32", variant);
    return B2_ERR_INVALID_ARGUMENT;
  }
  if ((variant == 1 || variant == 2 || variant == 5) && N % 256 != 0) {
    set_error("b2_nvfp4_gemm: variant %d needs N %% 256 == 0", variant);
    return B2_ERR_INVALID_ARGUMENT;
  }
  switch (variant) {
    case 0: return launch_variant<1, 128, 6>(A, B, SFA, SFB, alpha_dev, D, M, N, K, 0, s);
    case 1: return launch_variant<1, 256, 4>(A, B, SFA, SFB, alpha_dev, D, M, N, K, 1, s);
    case 2: return launch_variant<2, 256, 5, 1>(A, B, SFA, SFB, alpha_dev, D, M, N, K, 2, s);
    case 4: return launch_variant<1, 128, 9, 0, 32>(A, B, SFA, SFB, alpha_dev, D, M, N, K, 4, s);
    case 5: return launch_variant<1, 256, 5, 0, 32>(A, B, SFA, SFB, alpha_dev, D, M, N, K, 5, s);
    case 6: return launch_variant<1, 64, 13, 0, 32>(A, B, SFA, SFB, alpha_dev, D, M, N, K, 6, s);
    case 7: return launch_variant<1, 64, 11, 0, 32, 2>(A, B, SFA, SFB, alpha_dev, D, M, N, K, 7, s);
    case 8: return launch_variant<1, 64, 7, 0, 128, 2>(A, B, SFA, SFB, alpha_dev, D, M, N, K, 8, s);
    case 9: return launch_variant<1, 128, 6, 0, 128, 2>(A, B, SFA, SFB, alpha_dev, D, M, N, K, 9, s);
    default: return launch_variant<2, 128, 6, 1>(A, B, SFA, SFB, alpha_dev, D, M, N, K, 3, s);
  }
}

// Role timers of CTA 0 for the most recent profiled launch (SM cycles): producer wait-for-free-stage,
// producer total, MMA wait-for-data, MMA wait-for-accumulator, MMA total, MMA issue, epilogue
// wait-for-accumulator, epilogue body, tiles, scale-warp wait-for-load, scale-warp body, MMA total in nanoseconds.
// `enable` switches recording for later launches.
extern "C" int b2_nvfp4_gemm_role_timers(int enable, unsigned long long* out12, void* stream) {
  using namespace b2;
  uint32_t* status = nullptr;
  if (int rc = status_word(&status)) return rc;
  g_profile.store(enable ? 1 : 0, std::memory_order_relaxed);
  if (out12) {
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    B2_CUDA_TRY(cudaMemcpyAsync(out12, status + 16, 12 * sizeof(unsigned long long), cudaMemcpyDeviceToHost, s));
    B2_CUDA_TRY(cudaStreamSynchronize(s));
  }
  return B2_OK;
}

namespace b2 {
namespace {
// Reads and clears the two status words at `status`; `who` prefixes the message.
int read_status(uint32_t* status, const char* who, cudaStream_t s) {
  uint32_t host[2] = {0, 0};
  B2_CUDA_TRY(cudaMemcpyAsync(host, status, sizeof(host), cudaMemcpyDeviceToHost, s));
  B2_CUDA_TRY(cudaStreamSynchronize(s));
  if (host[0] == 0) return B2_OK;
  B2_CUDA_TRY(cudaMemsetAsync(status, 0, sizeof(host), s));
  static const char* const kWhat[] = {"",
                                      "producer waiting for a free stage",
                                      "MMA waiting for a drained accumulator",
                                      "MMA waiting for loaded operands and scale factors in tensor memory",
                                      "epilogue waiting for the accumulator",
                                      "scale warp waiting for loaded scale factors",
                                      "(unused)"};
  set_error("%s: bounded wait expired (%s) in CTA %u", who, host[0] < 7 ? kWhat[host[0]] : "unknown", host[1]);
  return B2_ERR_DEVICE_TIMEOUT;
}
}  // namespace
}  // namespace b2

extern "C" int b2_nvfp4_gemm_status(void* stream) {
  using namespace b2;
  uint32_t* status = nullptr;
  if (int rc = status_word(&status)) return rc;
  return read_status(status, "b2_nvfp4_gemm", static_cast<cudaStream_t>(stream));
}

// ---- decode-sized GEMM for callers that must not allocate ---------------------------------------
//
// Some hosts of this library run where device allocation is off the table: a serving loop that
// has handed every byte of HBM to its own pool and treats a cudaMalloc from a plugin as a bug, a
// caller inside a latency-critical section where the implicit device synchronisation of
// cudaMalloc / cudaFree would stall every stream, or a sandboxed plugin host that simply forbids
// the call.  b2_nvfp4_gemm allocates on such a caller's behalf (its status word on first use,
// and a scratch buffer for the partial sums of its split-K path).  The entry point below does
// the same decode-sized product with all of that scratch placed in one array that is part of the
// library image itself.
namespace b2 {
namespace {

constexpr size_t kBuiltinPartialBytes = 4u << 20;  // room for the fp32 partial sums: 4 MiB
constexpr size_t kBuiltinStatusBytes = 256;        // status words and role timers
// Lives in every GPU context that loads the library, until the process exits.
static __device__ __align__(256) unsigned char g_builtin_scratch[kBuiltinPartialBytes + kBuiltinStatusBytes];

// Device address of the array per device ordinal.  In host code `g_builtin_scratch` names a
// host-side shadow of the symbol, not device memory, so the address a kernel may use has to be
// asked for, once per device and with that device current.
unsigned char* g_builtin_base[64] = {nullptr};

int builtin_scratch(unsigned char** out) {
  int dev = 0;
  B2_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) {
    set_error("device ordinal %d out of range", dev);
    return B2_ERR_CUDA;
  }
  std::lock_guard<std::mutex> lock(g_mu);
  if (!g_builtin_base[dev]) {
    void* ptr = nullptr;
    B2_CUDA_TRY(cudaGetSymbolAddress(&ptr, g_builtin_scratch));
    g_builtin_base[dev] = static_cast<unsigned char*>(ptr);
  }
  *out = g_builtin_base[dev];
  return B2_OK;
}

}  // namespace
}  // namespace b2

// D[M,N] (bf16) = alpha * A[M,K] * B[N,K]^T for M <= 128: the operands, the kernel variant, the K
// ranges and therefore the bits of the result are those of b2_nvfp4_gemm, without any device
// allocation: no cudaMalloc, cudaFree or allocating library routine is called, here or on first
// use.  The split-K partial sums and the kernel's status words live in an array built into the
// library (4 MiB + 256 B per GPU that loads it).
//
//  * The first call on a device looks the array's device address up (cudaGetSymbolAddress) and
//    sets the kernel's shared-memory attribute; make that first call before any stream capture.
//  * A problem whose partial sums (K ranges x M x N x 4 bytes) exceed 4 MiB is rejected with
//    B2_ERR_INVALID_ARGUMENT and nothing is launched.
//  * Every call on a device uses the same array, which keeps the previous call's contents.  Each
//    call overwrites all partial sums it later reads, so nothing needs clearing, but two calls
//    that overlap on the GPU (different streams, or graphs replayed concurrently) race on it:
//    keep calls of this entry point on one device in stream order.
//  * A bounded wait that expires still ends the kernel cleanly; its code goes to the built-in
//    status words, which b2_nvfp4_gemm_small_m_noalloc_status reads and clears.
extern "C" int b2_nvfp4_gemm_small_m_noalloc(const void* A, const void* B, const void* SFA, const void* SFB,
                                             const float* alpha_dev, void* D, int M, int N, int K,
                                             void* stream) {
  using namespace b2;
  if (!A || !B || !SFA || !SFB || !alpha_dev || !D) {
    set_error("b2_nvfp4_gemm_small_m_noalloc: null pointer argument");
    return B2_ERR_INVALID_ARGUMENT;
  }
  if (M < 1 || M > kBlockM || N < 1 || K < 1 || K % 256 != 0 || N % 128 != 0) {
    set_error("b2_nvfp4_gemm_small_m_noalloc: M=%d N=%d K=%d: need 1 <= M <= 128, N %% 128 == 0, K %% 256 == 0",
              M, N, K);
    return B2_ERR_INVALID_ARGUMENT;
  }
  const uintptr_t all = reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) |
                        reinterpret_cast<uintptr_t>(SFA) | reinterpret_cast<uintptr_t>(SFB) |
                        reinterpret_cast<uintptr_t>(D);
  if (all & 15) {
    set_error("b2_nvfp4_gemm_small_m_noalloc: all tensors must be 16-byte aligned");
    return B2_ERR_INVALID_ARGUMENT;
  }
  if (!encode_tiled_fn()) {
    set_error("b2_nvfp4_gemm_small_m_noalloc: cuTensorMapEncodeTiled is not available from this driver");
    return B2_ERR_CUDA;
  }
  unsigned char* base = nullptr;
  if (int rc = builtin_scratch(&base)) return rc;
  const FixedWorkspace ws{reinterpret_cast<uint32_t*>(base + kBuiltinPartialBytes), reinterpret_cast<float*>(base),
                          kBuiltinPartialBytes, "b2_nvfp4_gemm_small_m_noalloc"};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (choose_variant(M, N, K)) {
    case 0: return launch_variant<1, 128, 6>(A, B, SFA, SFB, alpha_dev, D, M, N, K, 0, s, &ws);
    case 1: return launch_variant<1, 256, 4>(A, B, SFA, SFB, alpha_dev, D, M, N, K, 1, s, &ws);
    case 4: return launch_variant<1, 128, 9, 0, 32>(A, B, SFA, SFB, alpha_dev, D, M, N, K, 4, s, &ws);
    case 7: return launch_variant<1, 64, 11, 0, 32, 2>(A, B, SFA, SFB, alpha_dev, D, M, N, K, 7, s, &ws);
    case 8: return launch_variant<1, 64, 7, 0, 128, 2>(A, B, SFA, SFB, alpha_dev, D, M, N, K, 8, s, &ws);
    default: return launch_variant<1, 256, 5, 0, 32>(A, B, SFA, SFB, alpha_dev, D, M, N, K, 5, s, &ws);
  }
}

// Status of the launches of b2_nvfp4_gemm_small_m_noalloc on the current device: synchronises
// `stream`, returns B2_OK or B2_ERR_DEVICE_TIMEOUT (detail in b2_last_error()) and clears the
// words.  Allocates nothing: an 8-byte copy out of the built-in array and, after a failure, an
// 8-byte memset.
extern "C" int b2_nvfp4_gemm_small_m_noalloc_status(void* stream) {
  using namespace b2;
  unsigned char* base = nullptr;
  if (int rc = builtin_scratch(&base)) return rc;
  return read_status(reinterpret_cast<uint32_t*>(base + kBuiltinPartialBytes), "b2_nvfp4_gemm_small_m_noalloc",
                     static_cast<cudaStream_t>(stream));
}

// Test hooks of the bounded waits.  `milliseconds` > 0 shortens the budget of every device-side
// wait of later launches (0 restores the one-second default).  `fault` = 1 makes the NEXT launch
// announce, for the first K slab of CTA 0, 16 bytes more than its copies deliver: every copy lands,
// nothing stays in flight, the slab's barrier simply never completes, the MMA role's wait runs out
// and the kernel ends through its abort path.  Both are off unless a test turns them on.
extern "C" int b2_nvfp4_gemm_set_wait_budget_ms(int milliseconds) {
  if (milliseconds < 0 || milliseconds > 10000) {
    b2::set_error("b2_nvfp4_gemm_set_wait_budget_ms: %d ms out of range [0, 10000]", milliseconds);
    return B2_ERR_INVALID_ARGUMENT;
  }
  b2::g_wait_budget_ns.store(milliseconds ? 1000000ull * static_cast<unsigned long long>(milliseconds) : b2::kWaitBudgetNs,
                             std::memory_order_relaxed);
  return B2_OK;
}

extern "C" int b2_nvfp4_gemm_inject_test_fault(int fault) {
  if (fault < 0 || fault > 1) {
    b2::set_error("b2_nvfp4_gemm_inject_test_fault: unknown fault %d", fault);
    return B2_ERR_INVALID_ARGUMENT;
  }
  b2::g_test_fault.store(fault, std::memory_order_relaxed);
  return B2_OK;
}

// ---- sharded projection: GEMM with the output all-gather fused into its epilogue ---------------
//
// Every GPU owns one [M, world * N] bf16 buffer allocated with b2_peer_alloc and mapped into
// the other processes through CUDA IPC.  GPU `rank` multiplies by its N-row slab of the weight and
// its epilogue stores each finished tile into column range [rank * N, (rank + 1) * N) of ALL
// `world` buffers (its own through `D_all[rank]`, the others over NVLink).  Only stores cross the
// link; there is no remote load and no multicast.  The caller orders a cross-rank barrier after the
// launch before anyone reads the gathered rows.
extern "C" int b2_peer_alloc(void** ptr, int64_t bytes) {
  using namespace b2;
  if (!ptr || bytes <= 0) {
    set_error("b2_peer_alloc: bad arguments");
    return B2_ERR_INVALID_ARGUMENT;
  }
  B2_CUDA_TRY(cudaMalloc(ptr, static_cast<size_t>(bytes)));
  return B2_OK;
}

extern "C" int b2_peer_free(void* ptr) {
  using namespace b2;
  B2_CUDA_TRY(cudaFree(ptr));
  return B2_OK;
}

extern "C" int b2_peer_export(void* ptr, unsigned char* handle64) {
  using namespace b2;
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  if (!ptr || !handle64) {
    set_error("b2_peer_export: null argument");
    return B2_ERR_INVALID_ARGUMENT;
  }
  cudaIpcMemHandle_t handle;
  B2_CUDA_TRY(cudaIpcGetMemHandle(&handle, ptr));
  memcpy(handle64, &handle, 64);
  return B2_OK;
}

extern "C" int b2_peer_open(const unsigned char* handle64, void** ptr) {
  using namespace b2;
  if (!ptr || !handle64) {
    set_error("b2_peer_open: null argument");
    return B2_ERR_INVALID_ARGUMENT;
  }
  cudaIpcMemHandle_t handle;
  memcpy(&handle, handle64, 64);
  B2_CUDA_TRY(cudaIpcOpenMemHandle(ptr, handle, cudaIpcMemLazyEnablePeerAccess));
  return B2_OK;
}

extern "C" int b2_peer_close(void* ptr) {
  using namespace b2;
  B2_CUDA_TRY(cudaIpcCloseMemHandle(ptr));
  return B2_OK;
}

extern "C" int b2_nvfp4_gemm_allgather(const void* A, const void* B, const void* SFA, const void* SFB,
                                       const float* alpha_dev, void* const* D_all, int world, int rank,
                                       int M, int N, int K, void* stream) {
  using namespace b2;
  if (!A || !B || !SFA || !SFB || !alpha_dev || !D_all) {
    set_error("b2_nvfp4_gemm_allgather: null pointer argument");
    return B2_ERR_INVALID_ARGUMENT;
  }
  if (world < 1 || world > 8 || rank < 0 || rank >= world) {
    set_error("b2_nvfp4_gemm_allgather: rank %d of world %d (1..8 GPUs of one box)", rank, world);
    return B2_ERR_INVALID_ARGUMENT;
  }
  if (M <= 128 || N < 1 || K < 1 || K % 256 != 0 || N % 128 != 0) {
    set_error("b2_nvfp4_gemm_allgather: M=%d N=%d K=%d: need M > 128, N %% 128 == 0, K %% 256 == 0", M, N, K);
    return B2_ERR_INVALID_ARGUMENT;
  }
  for (int g = 0; g < world; ++g) {
    if (!D_all[g] || (reinterpret_cast<uintptr_t>(D_all[g]) & 31)) {
      set_error("b2_nvfp4_gemm_allgather: output buffer %d is null or not 32-byte aligned", g);
      return B2_ERR_INVALID_ARGUMENT;
    }
  }
  if (!encode_tiled_fn()) {
    set_error("b2_nvfp4_gemm_allgather: cuTensorMapEncodeTiled is not available from this driver");
    return B2_ERR_CUDA;
  }
  uint32_t* status = nullptr;
  if (int rc = status_word(&status)) return rc;
  // destination 0 is this GPU's buffer, then the peers in ring order starting after this rank, so
  // that the GPUs do not all write to the same one at the same time
  OutMaps<true> out_maps;
  for (int i = 0; i < world; ++i)
    if (int rc = encode_output_map(&out_maps.m[i], D_all[(rank + i) % world], M, world * N)) return rc;
  GatherTarget gather;
  gather.n_dest = world;
  gather.ldd = world * N;
  gather.col0 = rank * N;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  MapSet maps;
  if (N % 256 == 0) {
    if (int rc = encode_maps<2, 256, 5>(&maps, A, B, SFA, SFB, M, N, K)) return rc;
    return launch_kernels<2, 256, 5, 1>(maps, alpha_dev, D_all[rank], M, N, K, 1, status, nullptr, s, gather,
                                           out_maps);
  }
  if (int rc = encode_maps<2, 128, 6>(&maps, A, B, SFA, SFB, M, N, K)) return rc;
  return launch_kernels<2, 128, 6, 1>(maps, alpha_dev, D_all[rank], M, N, K, 1, status, nullptr, s, gather,
                                         out_maps);
}
