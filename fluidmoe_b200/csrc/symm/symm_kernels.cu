// Device-initiated primitives over symmetric memory: barrier, all-to-all push / wait, two-shot
// all-reduce.  Data moves with ordinary 16-byte loads and stores on peer pointers (NVLink);
// completion is published with system-scope release operations and observed with bounded
// acquire polls.  No kernel here waits without a time limit.
#include <stdio.h>

#include "../include/fm_symm.h"
#include "../include/sm100_ptx.cuh"

extern "C" void fm_set_error(const char* msg);

namespace fm {

constexpr int kKernelIdBarrier = 10;
constexpr int kKernelIdA2AWait = 11;
constexpr int kKernelIdAllReduce = 12;
constexpr int kKernelIdWaitFlag = 13;

__global__ void symm_barrier_kernel(int* const* flag_ptrs, int my_rank, int nranks, int epoch,
                                    unsigned long long timeout_ns, int* status) {
  const int p = threadIdx.x;
  if (p >= nranks) return;
  __threadfence_system();
  // Tell rank p that I arrived at `epoch` ...
  flag_release_store(flag_ptrs[p] + my_rank, epoch);
  // ... and wait until rank p told me the same.
  int observed = 0;
  if (!flag_wait_ge(flag_ptrs[my_rank] + p, epoch, timeout_ns, nullptr, &observed))
    report_status(status, kStatusFlagTimeout, kKernelIdBarrier, p, epoch, observed);
}

__global__ void a2a_push_kernel(const uint8_t* send, const long long* send_offs,
                                const long long* send_bytes, void* const* recv_ptrs,
                                const long long* dst_offs, int* const* flag_ptrs,
                                int* local_counters, int my_rank, int nranks, int epoch) {
  // Peers are visited starting from my right-hand neighbour so that the ranks do not all write
  // to the same destination at once.
  for (int i = 0; i < nranks; ++i) {
    const int p = (my_rank + 1 + i) % nranks;
    const uint4* src = reinterpret_cast<const uint4*>(send + send_offs[p]);
    uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(recv_ptrs[p]) + dst_offs[p]);
    const long long n = send_bytes[p] / 16;
    for (long long j = (long long)blockIdx.x * blockDim.x + threadIdx.x; j < n;
         j += (long long)gridDim.x * blockDim.x)
      dst[j] = src[j];
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
      // The last CTA to finish peer p's slice publishes it.
      const int done = atomicAdd(&local_counters[p], 1) + 1;
      if (done == (int)gridDim.x) {
        local_counters[p] = 0;
        __threadfence_system();
        flag_release_store(flag_ptrs[p] + my_rank, epoch);
      }
    }
  }
}

__global__ void put_signal_kernel(const uint4* src, long long nvec, uint4* dst, int* flag,
                                  int value, int* local_counter) {
  for (long long j = (long long)blockIdx.x * blockDim.x + threadIdx.x; j < nvec;
       j += (long long)gridDim.x * blockDim.x)
    dst[j] = src[j];
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int done = atomicAdd(local_counter, 1) + 1;
    if (done == (int)gridDim.x) {
      *local_counter = 0;
      __threadfence_system();
      flag_release_store(flag, value);
    }
  }
}

// Fused permute + dispatch: slot s of the sender's permuted order (global-expert-major,
// `cap` slots per expert, `nle` experts per rank) is the row x[sorted_idx[s]].  It is stored
// straight into the destination rank's expert-major buffer at row (j * P + me) * cap + i, its
// routing probability into the matching fp32 slot, and the destination's arrival counter of the
// 128-row block that contains the row is bumped with a system-scope release.  One warp moves one
// row with 16-byte accesses.  Takes the place of the permute + dispatch all-to-all rounds of
// fluid/moe/forward.py:446-461,623-733 (and, with probs == nullptr, of the combine-gradient
// all-to-all of fluid/moe/backward.py:758-801).
__global__ void permute_dispatch_kernel(const __nv_bfloat16* __restrict__ x,
                                        const long long* __restrict__ sorted_idx,
                                        const float* __restrict__ probs,
                                        __nv_bfloat16* const* __restrict__ dst_tokens,
                                        float* const* __restrict__ dst_probs,
                                        int* const* __restrict__ dst_flags, long long total_slots,
                                        int H, int cap, int nle, int P, int me,
                                        int blocks_per_group) {
  const int nvec = H / 8;
  const int lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  const long long S = (long long)nle * cap;
  // A warp takes kRowsPerFence consecutive slots; the system-scope fence and the counter update
  // are issued once per run of rows that share a counter, not once per row.
  constexpr int kRowsPerFence = 8;
  const long long nchunks = (total_slots + kRowsPerFence - 1) / kRowsPerFence;
  for (long long c = (long long)blockIdx.x * warps_per_block + (threadIdx.x >> 5); c < nchunks;
       c += (long long)gridDim.x * warps_per_block) {
    int* pending_flag = nullptr;
    int pending = 0;
    const long long s_end = min(total_slots, (c + 1) * kRowsPerFence);
    for (long long s = c * kRowsPerFence; s < s_end; ++s) {
      // Visit destinations starting from my right-hand neighbour (the local copy comes last).
      const long long dst_rank_seq = s / S;
      const int p = (int)((me + 1 + dst_rank_seq) % P);
      const long long within = s % S;
      const int j = (int)(within / cap);
      const int i = (int)(within % cap);
      const long long src_slot = (long long)p * S + within;
      const long long tok = sorted_idx[src_slot];
      const long long row_in_group = (long long)me * cap + i;
      const long long drow = (long long)j * P * cap + row_in_group;
      int* flag = dst_flags[p] + j * blocks_per_group + (int)(row_in_group / 128);
      if (flag != pending_flag && pending > 0) {
        __syncwarp();
        if (lane == 0) {
          __threadfence_system();
          flag_release_add(pending_flag, pending);
        }
        pending = 0;
      }
      pending_flag = flag;
      const uint4* src = reinterpret_cast<const uint4*>(x + tok * H);
      uint4* dst = reinterpret_cast<uint4*>(dst_tokens[p] + drow * H);
      for (int v = lane; v < nvec; v += 32) dst[v] = src[v];
      if (lane == 0 && probs != nullptr) dst_probs[p][drow] = probs[src_slot];
      ++pending;
    }
    if (pending > 0) {
      __syncwarp();
      if (lane == 0) {
        __threadfence_system();
        flag_release_add(pending_flag, pending);
      }
    }
  }
}

// HP->SP push: `src` is [P * rows_blk, W] (rows of block p belong to rank p).  Row i of block p
// is stored into rank p's buffer at row i, columns [me * W, (me + 1) * W) (leading dimension
// P * W), and rank p's counter flags[p][me * row_blocks + i / 128] grows by one.  One warp per row.
// Replaces the HP->SP pairwise rounds of fluid/attention/forward.py:435-452 (and the HP->SP
// all-to-all of fluid/attention/backward.py:294-349).
__global__ void rows_push_kernel(const __nv_bfloat16* __restrict__ src,
                                 __nv_bfloat16* const* __restrict__ dst_base,
                                 int* const* __restrict__ dst_flags, long long rows_blk, int W, int P,
                                 int me, int row_blocks) {
  const int nvec = W / 8;
  const int lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  const long long total = rows_blk * P;
  constexpr int kRowsPerFence = 8;   // one fence + counter update per run of rows sharing a counter
  const long long nchunks = (total + kRowsPerFence - 1) / kRowsPerFence;
  for (long long c = (long long)blockIdx.x * warps_per_block + (threadIdx.x >> 5); c < nchunks;
       c += (long long)gridDim.x * warps_per_block) {
    int* pending_flag = nullptr;
    int pending = 0;
    const long long s_end = min(total, (c + 1) * kRowsPerFence);
    for (long long s = c * kRowsPerFence; s < s_end; ++s) {
      const int p = (int)((me + 1 + s / rows_blk) % P);   // right-hand neighbour first, self last
      const long long i = s % rows_blk;
      int* flag = dst_flags[p] + me * row_blocks + (int)(i / 128);
      if (flag != pending_flag && pending > 0) {
        __syncwarp();
        if (lane == 0) {
          __threadfence_system();
          flag_release_add(pending_flag, pending);
        }
        pending = 0;
      }
      pending_flag = flag;
      const uint4* from = reinterpret_cast<const uint4*>(src + ((long long)p * rows_blk + i) * W);
      uint4* to = reinterpret_cast<uint4*>(dst_base[p] + i * (long long)P * W + (long long)me * W);
      for (int v = lane; v < nvec; v += 32) to[v] = from[v];
      ++pending;
    }
    if (pending > 0) {
      __syncwarp();
      if (lane == 0) {
        __threadfence_system();
        flag_release_add(pending_flag, pending);
      }
    }
  }
}

// Thread p waits until the arrival word of source p reached `epoch` (or `expected[p]`, when the
// amount every source sends is only known on the device).  With `wait_ns` the time the slowest
// thread waited is added to a device counter: this kernel sits alone on its stream, so that time
// is communication the step could not hide.
__global__ void a2a_wait_kernel(const int* my_flags, int my_rank, int nranks, int epoch,
                                const int* expected, unsigned long long* wait_ns,
                                unsigned long long timeout_ns, int* status) {
  __shared__ unsigned long long slowest;
  const int p = threadIdx.x;
  if (p == 0) slowest = 0;
  __syncthreads();
  if (p < nranks) {
    const int want = expected ? expected[p] : epoch;
    int observed = 0;
    const uint64_t t0 = wait_ns ? global_timer_ns() : 0;
    if (!flag_wait_ge(my_flags + p, want, timeout_ns, nullptr, &observed))
      report_status(status, kStatusFlagTimeout, kKernelIdA2AWait, p, want, observed);
    if (wait_ns) atomicMax(&slowest, (unsigned long long)(global_timer_ns() - t0));
  }
  __syncthreads();
  if (p == 0 && wait_ns) atomicAdd(wait_ns, slowest);
}

__global__ void wait_flag_kernel(const int* flag, int expected, unsigned long long timeout_ns,
                                 int* status) {
  int observed = 0;
  if (!flag_wait_ge(flag, expected, timeout_ns, nullptr, &observed))
    report_status(status, kStatusFlagTimeout, kKernelIdWaitFlag, 0, expected, observed);
}

// Two-shot all-reduce.  Phase 0: barrier (everyone's data is written).  Phase 1: rank r sums
// chunk r over all peers and stores the scaled result into every peer's buffer.  Phase 2:
// barrier (everyone's results are visible).  Barriers are done by CTA 0 with a grid-wide
// hand-off through a local counter, so the kernel needs all its CTAs resident: the host caps
// the grid at the SM count.
template <class T>
struct Vec16;
template <>
struct Vec16<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void load(const float* p, float* v) {
    const float4 x = *reinterpret_cast<const float4*>(p);
    v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
  }
  static __device__ __forceinline__ void store(float* p, const float* v) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  }
};
template <>
struct Vec16<__nv_bfloat16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* v) {
    const uint4 x = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&w[i]);
      v[2 * i] = __low2float(b);
      v[2 * i + 1] = __high2float(b);
    }
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float* v) {
    uint4 x;
    x.x = pack_bf16x2(v[0], v[1]); x.y = pack_bf16x2(v[2], v[3]);
    x.z = pack_bf16x2(v[4], v[5]); x.w = pack_bf16x2(v[6], v[7]);
    *reinterpret_cast<uint4*>(p) = x;
  }
};

__device__ __forceinline__ bool grid_peer_barrier(int* const* flag_ptrs, int my_rank, int nranks,
                                                  int epoch, int* local_sync, int phase_target,
                                                  unsigned long long timeout_ns, int* status) {
  // 1. all CTAs of this rank arrive
  __threadfence_system();
  __syncthreads();
  __shared__ int ok_s;
  if (threadIdx.x == 0) {
    ok_s = 1;
    atomicAdd(local_sync, 1);
  }
  if (blockIdx.x == 0) {
    if (threadIdx.x == 0) {
      int observed = 0;
      if (!flag_wait_ge(local_sync, phase_target * (int)gridDim.x, timeout_ns, nullptr, &observed)) {
        report_status(status, kStatusFlagTimeout, kKernelIdAllReduce, -1, phase_target, observed);
        ok_s = 0;
      }
    }
    __syncthreads();
    // 2. CTA 0 exchanges the epoch with every peer
    if ((int)threadIdx.x < nranks) {
      __threadfence_system();
      flag_release_store(flag_ptrs[threadIdx.x] + my_rank, epoch);
      int observed = 0;
      if (!flag_wait_ge(flag_ptrs[my_rank] + threadIdx.x, epoch, timeout_ns, nullptr, &observed)) {
        report_status(status, kStatusFlagTimeout, kKernelIdAllReduce, threadIdx.x, epoch, observed);
      }
    }
    __syncthreads();
    // 3. release the other CTAs of this rank
    if (threadIdx.x == 0) flag_release_store(local_sync + 1, epoch);
  }
  if (threadIdx.x == 0) {
    int observed = 0;
    if (!flag_wait_ge(local_sync + 1, epoch, timeout_ns, nullptr, &observed)) ok_s = 0;
  }
  __syncthreads();
  return ok_s != 0;
}

template <class T>
__global__ void allreduce_p2p_kernel(T* const* bufs_in, long long elem_offset, long long count, float scale,
                                     int* const* flag_ptrs, int my_rank, int nranks, int epoch,
                                     unsigned long long timeout_ns, int* status) {
  constexpr int VN = Vec16<T>::N;
  constexpr int kMaxRanks = 32;
  // the slice [elem_offset, elem_offset + count) of every rank's buffer
  __shared__ T* bufs[kMaxRanks];
  if (threadIdx.x < nranks) bufs[threadIdx.x] = bufs_in[threadIdx.x] + elem_offset;
  __syncthreads();
  // local_sync words live right after the nranks barrier words of my flag block.
  int* local_sync = flag_ptrs[my_rank] + nranks;
  if (!grid_peer_barrier(flag_ptrs, my_rank, nranks, 2 * epoch - 1, local_sync, 2 * epoch - 1,
                         timeout_ns, status))
    return;
  const long long nvec = count / VN;
  const long long per = (nvec + nranks - 1) / nranks;
  const long long lo = per * my_rank;
  const long long hi = min(nvec, lo + per);
  for (long long j = lo + (long long)blockIdx.x * blockDim.x + threadIdx.x; j < hi;
       j += (long long)gridDim.x * blockDim.x) {
    float acc[VN];
#pragma unroll
    for (int i = 0; i < VN; ++i) acc[i] = 0.f;
    for (int p = 0; p < nranks; ++p) {
      float v[VN];
      Vec16<T>::load(bufs[(my_rank + p) % nranks] + j * VN, v);
#pragma unroll
      for (int i = 0; i < VN; ++i) acc[i] += v[i];
    }
#pragma unroll
    for (int i = 0; i < VN; ++i) acc[i] *= scale;
    for (int p = 0; p < nranks; ++p) Vec16<T>::store(bufs[(my_rank + p) % nranks] + j * VN, acc);
  }
  // tail elements (count not a multiple of the vector width): rank 0 handles them
  if (my_rank == 0 && blockIdx.x == 0 && threadIdx.x < (int)(count - nvec * VN)) {
    const long long j = nvec * VN + threadIdx.x;
    float acc = 0.f;
    for (int p = 0; p < nranks; ++p) acc += (float)bufs[p][j];
    for (int p = 0; p < nranks; ++p) bufs[p][j] = (T)(acc * scale);
  }
  grid_peer_barrier(flag_ptrs, my_rank, nranks, 2 * epoch, local_sync, 2 * epoch, timeout_ns,
                    status);
}

// In-switch all-reduce (NVLS): `mc` is the multicast address of a buffer that every rank of the
// group has bound to one NVLink multicast object.  Rank r owns the r-th slice of the buffer:
// `multimem.ld_reduce` returns the sum over all ranks (the NVSwitch adds the copies), the thread
// scales it, and `multimem.st` writes the result into every rank's copy.  The same bounded
// peer barrier as the two-shot kernel brackets the data phase.
__global__ void allreduce_nvls_kernel(float* mc, long long count, float scale, int* const* flag_ptrs,
                                      int my_rank, int nranks, int epoch, unsigned long long timeout_ns,
                                      int* status) {
  int* local_sync = flag_ptrs[my_rank] + nranks;
  if (!grid_peer_barrier(flag_ptrs, my_rank, nranks, 2 * epoch - 1, local_sync, 2 * epoch - 1,
                         timeout_ns, status))
    return;
  const long long nvec = count / 4;
  const long long per = (nvec + nranks - 1) / nranks;
  const long long lo = per * my_rank;
  const long long hi = min(nvec, lo + per);
  for (long long j = lo + (long long)blockIdx.x * blockDim.x + threadIdx.x; j < hi;
       j += (long long)gridDim.x * blockDim.x) {
    float4 v;
    float* addr = mc + j * 4;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(addr) : "memory");
    v.x *= scale; v.y *= scale; v.z *= scale; v.w *= scale;
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};"
                 :: "l"(addr), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
  }
  // tail (count not a multiple of 4): rank 0, one element at a time
  if (my_rank == 0 && blockIdx.x == 0 && threadIdx.x < (int)(count - nvec * 4)) {
    float* addr = mc + nvec * 4 + threadIdx.x;
    float v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.f32 %0, [%1];" : "=f"(v) : "l"(addr) : "memory");
    v *= scale;
    asm volatile("multimem.st.relaxed.sys.global.f32 [%0], %1;" :: "l"(addr), "f"(v) : "memory");
  }
  __threadfence_system();
  grid_peer_barrier(flag_ptrs, my_rank, nranks, 2 * epoch, local_sync, 2 * epoch, timeout_ns, status);
}

}  // namespace fm

static int launch_check(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    char buf[256];
    snprintf(buf, sizeof(buf), "%s: %s", what, cudaGetErrorString(e));
    fm_set_error(buf);
    return (int)e;
  }
  return 0;
}

extern "C" int fm_symm_barrier(int* const* flag_ptrs_dev, int my_rank, int nranks, int epoch,
                               unsigned long long timeout_ns, int* status, cudaStream_t stream) {
  fm::symm_barrier_kernel<<<1, 32 * ((nranks + 31) / 32), 0, stream>>>(
      flag_ptrs_dev, my_rank, nranks, epoch, timeout_ns ? timeout_ns : 4000000000ull, status);
  return launch_check("symm_barrier");
}

extern "C" int fm_a2a_push(const void* send, const long long* send_offs,
                           const long long* send_bytes, void* const* recv_ptrs,
                           const long long* dst_offs, int* const* flag_ptrs, int* local_counters,
                           int my_rank, int nranks, int epoch, int num_ctas, cudaStream_t stream) {
  if (num_ctas <= 0) num_ctas = 64;
  fm::a2a_push_kernel<<<num_ctas, 512, 0, stream>>>(
      reinterpret_cast<const uint8_t*>(send), send_offs, send_bytes, recv_ptrs, dst_offs,
      flag_ptrs, local_counters, my_rank, nranks, epoch);
  return launch_check("a2a_push");
}

extern "C" int fm_put_signal(const void* src, long long bytes, void* dst, int* flag, int value,
                             int num_ctas, int* local_counter, cudaStream_t stream) {
  if (bytes % 16 != 0) {
    fm_set_error("put_signal: size must be a multiple of 16 bytes");
    return -1;
  }
  if (num_ctas <= 0) num_ctas = 16;
  fm::put_signal_kernel<<<num_ctas, 512, 0, stream>>>(reinterpret_cast<const uint4*>(src),
                                                      bytes / 16, reinterpret_cast<uint4*>(dst),
                                                      flag, value, local_counter);
  return launch_check("put_signal");
}

extern "C" int fm_permute_dispatch(const void* x, const long long* sorted_idx, const float* probs,
                                   void* const* dst_tokens, float* const* dst_probs,
                                   int* const* dst_flags, long long total_slots, int H, int cap,
                                   int nle, int P, int me, int blocks_per_group, int num_ctas,
                                   cudaStream_t stream) {
  if (H % 8 != 0) {
    fm_set_error("permute_dispatch: H must be a multiple of 8");
    return -1;
  }
  if (num_ctas <= 0) num_ctas = 148 * 2;
  fm::permute_dispatch_kernel<<<num_ctas, 256, 0, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), sorted_idx, probs,
      reinterpret_cast<__nv_bfloat16* const*>(dst_tokens), dst_probs, dst_flags, total_slots, H, cap,
      nle, P, me, blocks_per_group);
  return launch_check("permute_dispatch");
}

extern "C" int fm_rows_push(const void* src, void* const* dst_base, int* const* dst_flags,
                            long long rows_blk, int W, int P, int me, int row_blocks, int num_ctas,
                            cudaStream_t stream) {
  if (W % 8 != 0) {
    fm_set_error("rows_push: row width must be a multiple of 8");
    return -1;
  }
  if (num_ctas <= 0) num_ctas = 148 * 2;
  fm::rows_push_kernel<<<num_ctas, 256, 0, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(src), reinterpret_cast<__nv_bfloat16* const*>(dst_base),
      dst_flags, rows_blk, W, P, me, row_blocks);
  return launch_check("rows_push");
}

extern "C" int fm_a2a_wait(const int* my_flags, int my_rank, int nranks, int epoch,
                           unsigned long long timeout_ns, int* status, cudaStream_t stream) {
  fm::a2a_wait_kernel<<<1, 32 * ((nranks + 31) / 32), 0, stream>>>(
      my_flags, my_rank, nranks, epoch, nullptr, nullptr, timeout_ns ? timeout_ns : 4000000000ull, status);
  return launch_check("a2a_wait");
}

extern "C" int fm_a2a_wait_counts(const int* my_flags, int nranks, int epoch, const int* expected,
                                  unsigned long long* wait_ns, unsigned long long timeout_ns, int* status,
                                  cudaStream_t stream) {
  fm::a2a_wait_kernel<<<1, 32 * ((nranks + 31) / 32), 0, stream>>>(
      my_flags, 0, nranks, epoch, expected, wait_ns, timeout_ns ? timeout_ns : 4000000000ull, status);
  return launch_check("a2a_wait_counts");
}

extern "C" int fm_wait_flag(const int* flag, int expected, unsigned long long timeout_ns,
                            int* status, cudaStream_t stream) {
  fm::wait_flag_kernel<<<1, 1, 0, stream>>>(flag, expected, timeout_ns, status);
  return launch_check("wait_flag");
}

extern "C" int fm_allreduce_p2p(void* const* buf_ptrs_dev, long long count, int dtype_fp32,
                                float scale, int* const* flag_ptrs_dev, int my_rank, int nranks,
                                int epoch, int num_ctas, unsigned long long timeout_ns,
                                int* status, cudaStream_t stream) {
  return fm_allreduce_p2p_slice(buf_ptrs_dev, 0, count, dtype_fp32, scale, flag_ptrs_dev, my_rank, nranks,
                                epoch, num_ctas, timeout_ns, status, stream);
}

extern "C" int fm_allreduce_p2p_slice(void* const* buf_ptrs_dev, long long elem_offset, long long count,
                                      int dtype_fp32, float scale, int* const* flag_ptrs_dev, int my_rank,
                                      int nranks, int epoch, int num_ctas, unsigned long long timeout_ns,
                                      int* status, cudaStream_t stream) {
  if (nranks > 32) {
    fm_set_error("allreduce_p2p: at most 32 ranks");
    return -1;
  }
  if ((elem_offset * (dtype_fp32 ? 4 : 2)) % 16 != 0) {
    fm_set_error("allreduce_p2p: the slice must start on a 16-byte boundary");
    return -1;
  }
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (num_ctas <= 0 || num_ctas > sms) num_ctas = sms / 2 > 0 ? sms / 2 : 1;
  const unsigned long long to = timeout_ns ? timeout_ns : 4000000000ull;
  if (dtype_fp32)
    fm::allreduce_p2p_kernel<float><<<num_ctas, 512, 0, stream>>>(
        reinterpret_cast<float* const*>(buf_ptrs_dev), elem_offset, count, scale, flag_ptrs_dev, my_rank,
        nranks, epoch, to, status);
  else
    fm::allreduce_p2p_kernel<__nv_bfloat16><<<num_ctas, 512, 0, stream>>>(
        reinterpret_cast<__nv_bfloat16* const*>(buf_ptrs_dev), elem_offset, count, scale, flag_ptrs_dev,
        my_rank, nranks, epoch, to, status);
  return launch_check("allreduce_p2p");
}

extern "C" int fm_allreduce_nvls(float* multicast_ptr, long long count, float scale,
                                 int* const* flag_ptrs_dev, int my_rank, int nranks, int epoch,
                                 int num_ctas, unsigned long long timeout_ns, int* status,
                                 cudaStream_t stream) {
  if (multicast_ptr == nullptr || (reinterpret_cast<uintptr_t>(multicast_ptr) & 15) != 0) {
    fm_set_error("allreduce_nvls: needs a 16-byte aligned multicast address");
    return -1;
  }
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (num_ctas <= 0 || num_ctas > sms) num_ctas = sms / 4 > 0 ? sms / 4 : 1;
  fm::allreduce_nvls_kernel<<<num_ctas, 512, 0, stream>>>(multicast_ptr, count, scale, flag_ptrs_dev, my_rank,
                                                         nranks, epoch, timeout_ns ? timeout_ns : 4000000000ull,
                                                         status);
  return launch_check("allreduce_nvls");
}
