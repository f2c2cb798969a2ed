// Thin inline-PTX wrappers for the Blackwell (sm_100a) primitives used by every kernel in
// this tree: mbarrier, TMA tiled loads (never with cluster multicast), tcgen05 MMA / TMEM,
// and system-scope release/acquire flags for peer-to-peer signalling over NVLink.
//
// Every wait in this header is bounded: it polls until a wall-clock budget (read from
// %globaltimer) runs out and then returns false so that the caller can record a status
// word, drain its own copies, free TMEM and return.  Nothing here traps or spins forever.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

namespace fm {

// ---------------------------------------------------------------------------------------
// Status word written by kernels that gave up on a wait.  Layout (int32[8]):
//   [0] code (0 = ok), [1] kernel id, [2] block, [3] what was waited on, [4] expected,
//   [5] observed, [6..7] spare.
// ---------------------------------------------------------------------------------------
enum StatusCode : int {
  kStatusOk = 0,
  kStatusMbarTimeout = 1,   // an mbarrier inside the CTA never completed its phase
  kStatusFlagTimeout = 2,   // a peer / producer flag never reached the expected value
  kStatusBadArgs = 3,
};

__device__ __forceinline__ void report_status(int* status, int code, int kernel_id, int what,
                                              int expected, int observed) {
  if (status == nullptr) return;
  if (atomicCAS(status, 0, code) == 0) {
    status[1] = kernel_id;
    status[2] = (int)blockIdx.x;
    status[3] = what;
    status[4] = expected;
    status[5] = observed;
    __threadfence_system();
  }
}

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n\t.reg .pred P;\n\t"
      "elect.sync _|P, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, P;\n\t}\n"
      : "=r"(pred));
  return pred != 0;
}

// ---------------------------------------------------------------------------------------
// mbarrier
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred P;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, P;\n\t}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait.  `abort_flag` is a CTA-shared word: once any role of the CTA has given up,
// every other wait returns false immediately so that the whole CTA unwinds together.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, uint64_t timeout_ns,
                                          volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = global_timer_ns();
  uint32_t spins = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((++spins & 63u) == 0) {
      if (*abort_flag) return false;
      if (global_timer_ns() - t0 > timeout_ns) {
        *abort_flag = 1;
        return false;
      }
    }
  }
}

// Fire-and-forget vector reduction (no return value, so the issuing warp never waits for it).
__device__ __forceinline__ void red_add_v4_f32(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};"
               :: "l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---------------------------------------------------------------------------------------
// TMA (tiled bulk tensor copies; the loads below never carry a multicast qualifier)
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* m, uint64_t* bar,
                                            int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)),
        "r"(c0), "r"(c1)
      : "memory");
}
// Tiled reduction shared -> global (element-wise add into the tensor; rows / columns outside the
// tensor are dropped).  The innermost coordinate times the element size must be a multiple of 16
// bytes and no coordinate may be negative.  Completion is tracked by bulk async-groups.
__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap* m, const void* smem_src, int c0, int c1) {
  asm volatile(
      "cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];"
      ::"l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(smem_src)), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void bulk_commit_group() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
// Wait until at most N of this thread's bulk groups still READ their shared-memory source.
template <int N>
__device__ __forceinline__ void bulk_wait_group_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
// Wait until at most N of this thread's bulk groups are incomplete (writes performed).
template <int N>
__device__ __forceinline__ void bulk_wait_group() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* m, uint64_t* bar,
                                            int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)),
        "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}

// ---------------------------------------------------------------------------------------
// tcgen05 / TMEM
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_slot, uint32_t ncols) {  // whole warp
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(smem_slot)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {  // whole warp
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// D[tmem] (+)= A[smem] * B[smem]; one thread issues for the CTA.
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                          uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on an mbarrier once every MMA issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// 32 lanes x 32 consecutive fp32 columns: thread i of the warp receives row (lane base + i).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
        "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
        "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

// Shared-memory operand descriptor for a 128-byte-swizzled tile (the only swizzle used here).
//   K-major tile : rows of 128 B (64 bf16 along K); 8-row groups 1024 B apart -> SBO = 1024.
//   MN-major tile: K rows of 128 B (64 bf16 along M or N); 8-K-row groups 1024 B apart
//                  (SBO = 1024); successive 64-element MN blocks `lbo` bytes apart.
__device__ __forceinline__ uint64_t umma_smem_desc(uint32_t smem_addr, uint32_t lbo_bytes,
                                                   uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= (uint64_t)1 << 46;  // descriptor version for sm_100
  d |= (uint64_t)2 << 61;  // SWIZZLE_128B
  return d;
}
// Instruction descriptor: bf16 x bf16 -> fp32, M = 128, N = n.
__host__ __device__ constexpr uint32_t umma_idesc_bf16(int m, int n, bool a_mn_major,
                                                       bool b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((a_mn_major ? 1u : 0u) << 15) |
         ((b_mn_major ? 1u : 0u) << 16) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// ---------------------------------------------------------------------------------------
// System-scope flags (a producer on another GPU publishes data, then the flag)
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void flag_release_add(int* flag, int v) {
  asm volatile("red.release.sys.global.add.s32 [%0], %1;" ::"l"(flag), "r"(v) : "memory");
}
__device__ __forceinline__ void flag_release_store(int* flag, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(flag), "r"(v) : "memory");
}
__device__ __forceinline__ int flag_acquire_load(const int* flag) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
  return v;
}
// Bounded wait until *flag >= expected.  Returns false on timeout (or CTA abort).
__device__ __forceinline__ bool flag_wait_ge(const int* flag, int expected, uint64_t timeout_ns,
                                             volatile int* abort_flag, int* observed) {
  int v = flag_acquire_load(flag);
  if (v >= expected) return true;
  const uint64_t t0 = global_timer_ns();
  uint32_t spins = 0;
  while (true) {
    v = flag_acquire_load(flag);
    if (v >= expected) return true;
    __nanosleep(64);
    if ((++spins & 15u) == 0) {
      if (abort_flag != nullptr && *abort_flag) break;
      if (global_timer_ns() - t0 > timeout_ns) {
        if (abort_flag != nullptr) *abort_flag = 1;
        break;
      }
    }
  }
  if (observed) *observed = v;
  return false;
}

// Prologue of a kernel that consumes rows pushed by peers: the first `n` threads of every CTA wait,
// bounded, until the `n` per-source arrival counters have reached `expected`; the others wait at
// the CTA barrier.  CTA 0 reports a timeout and adds the time its slowest thread waited to
// `wait_ns` (communication the step could not hide).  Replaces a stand-alone wait kernel in front
// of the consumer.  Needs n <= blockDim.x.
__device__ __forceinline__ void wait_counters_cta(const int* flags, int n, int expected,
                                                  unsigned long long* wait_ns, uint64_t timeout_ns,
                                                  int* status, int kernel_id) {
  __shared__ unsigned long long slowest_wait;
  if (threadIdx.x == 0) slowest_wait = 0;
  __syncthreads();
  if ((int)threadIdx.x < n) {
    int observed = 0;
    const uint64_t t0 = global_timer_ns();
    if (!flag_wait_ge(flags + threadIdx.x, expected, timeout_ns, nullptr, &observed) && blockIdx.x == 0)
      report_status(status, kStatusFlagTimeout, kernel_id, (int)threadIdx.x, expected, observed);
    if (wait_ns != nullptr && blockIdx.x == 0)
      atomicMax(&slowest_wait, (unsigned long long)(global_timer_ns() - t0));
  }
  __syncthreads();
  if (threadIdx.x == 0 && blockIdx.x == 0 && wait_ns != nullptr) atomicAdd(wait_ns, slowest_wait);
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

}  // namespace fm

// ---------------------------------------------------------------------------------------
// CTA-pair (cta_group::2) primitives: two CTAs of a cluster share one 256-row MMA.  Loads
// carry no multicast; each CTA fetches its own operand halves into its own shared memory and
// signals the leader's barrier.
// ---------------------------------------------------------------------------------------
namespace fm {

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Address of the same shared-memory location in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// Address bit that distinguishes the two CTAs of a pair inside the cluster shared window;
// clearing it turns a barrier address of either CTA into the leader's.
constexpr uint32_t kPeerBitMask = 0xFEFFFFFFu;

__device__ __forceinline__ void tma2_load_2d(void* smem_dst, const CUtensorMap* m, uint64_t* leader_bar,
                                             int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)),
        "r"(smem_u32(leader_bar) & kPeerBitMask), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tma2_load_3d(void* smem_dst, const CUtensorMap* m, uint64_t* leader_bar,
                                             int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)),
        "r"(smem_u32(leader_bar) & kPeerBitMask), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc2(uint32_t* smem_slot, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_slot)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma2_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// accumulating form with a constant predicate (see the fast issue path below)
__device__ __forceinline__ void umma2_bf16_acc(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.eq.u32 p, 1, 1;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc)
      : "memory");
}
// Arrive on the barrier at this shared-memory offset in every CTA of `cta_mask` once the MMAs
// issued so far have completed.
__device__ __forceinline__ void umma2_commit_mc(uint64_t* bar, uint16_t cta_mask) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(smem_u32(bar)), "h"(cta_mask)
      : "memory");
}

}  // namespace fm

// ---------------------------------------------------------------------------------------
// TMEM stores and MMA with the A operand in TMEM (used by flash attention: the probability
// block is written back over the score block and multiplied with V from there).
// ---------------------------------------------------------------------------------------
namespace fm {

__device__ __forceinline__ void tmem_st_wait() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
// 32 lanes x 16 consecutive 32-bit columns.
__device__ __forceinline__ void tmem_st_32x16(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
        "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]),
        "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
        "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]),
        "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]),
        "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]),
        "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
// ---------------------------------------------------------------------------------------
// Fast issue path.  One thread issues every MMA of a CTA, and that thread executes scalar code
// at roughly one dependent instruction per 5 cycles: building two 64-bit descriptors and a
// predicate per MMA (about 30 instructions) costs more than the 64 cycles a 128 x 128 x 16
// product takes on the tensor core (measured: 150 cycles per MMA with descriptors built in the
// loop, 65 with the low descriptor words precomputed and straight-line issue).  Within a tile
// only the start address changes between k-steps, and it sits in the low word, so an issue loop
// keeps the low words of the eight k-steps in registers, adds a stage offset and joins them
// with the constant high word.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t umma_desc_lo(uint32_t smem_addr, uint32_t lbo_bytes) {
  return ((smem_addr & 0x3FFFFu) >> 4) | (((lbo_bytes >> 4) & 0x3FFFu) << 16);
}
// high word: SBO, descriptor version, SWIZZLE_128B
__host__ __device__ constexpr uint32_t umma_desc_hi(uint32_t sbo_bytes) {
  return ((sbo_bytes >> 4) & 0x3FFFu) | (1u << 14) | (2u << 29);
}
__device__ __forceinline__ uint64_t umma_desc_join(uint32_t lo, uint32_t hi) {
  uint64_t d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(lo), "r"(hi));
  return d;
}
// Low words of the eight k-steps (16 elements each) of a [128 x 128] bf16 operand stored as two
// 128-byte-swizzled [128 rows x 64] slabs `slab_bytes` apart.
//   K-major (rows = M or N index, 64 k per slab): step kk starts 32 bytes further along the row.
//   MN-major (rows = k index, 64 M/N per slab): step kk starts 16 rows further; LBO = slab pitch.
__device__ __forceinline__ void umma_lo_k_major(uint32_t base, uint32_t slab_bytes, uint32_t (&lo)[8]) {
#pragma unroll
  for (int kk = 0; kk < 8; ++kk) lo[kk] = umma_desc_lo(base + (kk >> 2) * slab_bytes + (kk & 3) * 32, 0);
}
__device__ __forceinline__ void umma_lo_mn_major(uint32_t base, uint32_t slab_bytes, uint32_t (&lo)[8]) {
#pragma unroll
  for (int kk = 0; kk < 8; ++kk) lo[kk] = umma_desc_lo(base + kk * 2048, slab_bytes);
}
// accumulating MMA with a constant predicate (no register, no setp on a register)
__device__ __forceinline__ void umma_bf16_acc(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.eq.u32 p, 1, 1;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc)
      : "memory");
}
__device__ __forceinline__ void umma_bf16_ts_acc(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.eq.u32 p, 1, 1;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}\n"
      ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc)
      : "memory");
}
__device__ __forceinline__ void umma_bf16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b,
                                             uint32_t idesc, uint32_t accumulate);
// D (+)= A B over the eight k-steps of a 128-deep product.  `a_add` / `b_add`: stage offset of
// the operand in 16-byte units; `first_acc`: whether the first step accumulates onto D.
__device__ __forceinline__ void umma8_ss(uint32_t tmem_d, const uint32_t (&a_lo)[8], uint32_t a_add,
                                         const uint32_t (&b_lo)[8], uint32_t b_add, uint32_t idesc,
                                         uint32_t first_acc) {
  constexpr uint32_t hi = umma_desc_hi(1024);
  umma_bf16(tmem_d, umma_desc_join(a_lo[0] + a_add, hi), umma_desc_join(b_lo[0] + b_add, hi), idesc, first_acc);
#pragma unroll
  for (int kk = 1; kk < 8; ++kk)
    umma_bf16_acc(tmem_d, umma_desc_join(a_lo[kk] + a_add, hi), umma_desc_join(b_lo[kk] + b_add, hi), idesc);
}
// The same with A in TMEM: step kk reads eight 32-bit columns (16 bf16) starting at column
// (kk / 4) * group_cols + (kk % 4) * 8 of `tmem_a` (group_cols = 32: 64 contiguous columns).
__device__ __forceinline__ void umma8_ts(uint32_t tmem_d, uint32_t tmem_a, uint32_t group_cols,
                                         const uint32_t (&b_lo)[8], uint32_t b_add, uint32_t idesc,
                                         uint32_t first_acc) {
  constexpr uint32_t hi = umma_desc_hi(1024);
  umma_bf16_ts(tmem_d, tmem_a, umma_desc_join(b_lo[0] + b_add, hi), idesc, first_acc);
#pragma unroll
  for (int kk = 1; kk < 8; ++kk)
    umma_bf16_ts_acc(tmem_d, tmem_a + (kk >> 2) * group_cols + (kk & 3) * 8,
                     umma_desc_join(b_lo[kk] + b_add, hi), idesc);
}

// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void umma_bf16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b,
                                             uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}\n"
      ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

}  // namespace fm
