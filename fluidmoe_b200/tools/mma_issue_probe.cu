// Stand-alone probe of the tcgen05.mma issue path on sm_100a.
//
// One thread of one CTA issues 128 x N x 16 bf16 products back to back (descriptors complete in
// registers, straight-line code, mode chosen at compile time) and the probe reports cycles per
// MMA for: both operands in shared memory (SS) or A in TMEM (TS); N = 64 / 128 / 256; one or
// several accumulators; a commit every eight MMAs; three other warps loading and storing TMEM
// meanwhile.  It answers what the tensor core itself sustains, so that a kernel's issue loop can
// be judged against it.  Every wait is bounded.
//
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -I fluidmoe_b200/csrc/include \
//        -o /tmp/mma_issue_probe fluidmoe_b200/tools/mma_issue_probe.cu -lcuda && /tmp/mma_issue_probe 64
// or  python -m fluidmoe_b200.tools.kernel_bench mma_issue
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cstdio>
#include <cstdlib>
#include "sm100_ptx.cuh"
using namespace fm;
constexpr int kTile = 32768;
struct Res { long long cyc[16]; };

__device__ __forceinline__ void mma_ss(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.eq.u32 p, 1, 1;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
               ::"r"(d), "l"(a), "l"(b), "r"(idesc) : "memory");
}
__device__ __forceinline__ void mma_ts(uint32_t d, uint32_t a, uint64_t b, uint32_t idesc) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.eq.u32 p, 1, 1;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}\n"
               ::"r"(d), "r"(a), "l"(b), "r"(idesc) : "memory");
}

// TS: A from TMEM; N; NACC accumulators used round-robin (each N columns wide... capped to fit 384 columns)
template <bool TS, int N, int NACC, bool COMMIT = false>
__device__ long long run(uint32_t tb, uint32_t a_addr, uint32_t b_addr, uint64_t* bar, uint32_t& phase, int reps,
                         volatile int* abort_flag) {
  const uint32_t idesc = umma_idesc_bf16(128, N, false, false);
  uint64_t da[8], db[8];
#pragma unroll
  for (int kk = 0; kk < 8; ++kk) {
    da[kk] = umma_smem_desc(a_addr + (kk >> 2) * (kTile / 2) + (kk & 3) * 32, 0, 1024);
    db[kk] = umma_smem_desc(b_addr + (kk >> 2) * (N * 128) + (kk & 3) * 32, 0, 1024);
  }
  long long t0 = clock64();
#pragma unroll 1
  for (int r = 0; r < reps; ++r) {
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
      const uint32_t d = tb + (kk % NACC) * N;
      if (TS) mma_ts(d, tb + 448 + kk * 8, db[kk], idesc);
      else mma_ss(d, da[kk], db[kk], idesc);
    }
    if (COMMIT) umma_commit(bar + 1);     // nobody waits on this one
  }
  umma_commit(bar);
  if (!mbar_wait(bar, phase, 2000000000ull, abort_flag)) return -1;
  phase ^= 1;
  tc_fence_after_sync();
  return clock64() - t0;
}

__global__ void __launch_bounds__(128, 1) bench(Res* out, int reps) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + kTile;
  uint64_t* bar = reinterpret_cast<uint64_t*>(smem + 3 * kTile);
  uint32_t* slot = reinterpret_cast<uint32_t*>(bar + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(slot + 1);
  volatile int* run_flag = abort_flag + 1;
  const int warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < 3 * kTile / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(smem)[i] = 0x3c003c00u;
  if (threadIdx.x == 0) { mbar_init(bar, 1); mbar_init(bar + 1, 1); *abort_flag = 0; *run_flag = 0; mbar_fence_init(); }
  if (warp == 0) { tmem_alloc(slot, 512); tmem_relinquish(); }
  fence_proxy_async_smem();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tb = *slot;
  if (threadIdx.x == 0) {
    const uint32_t a = smem_u32(sA), b = smem_u32(sB);
    uint32_t ph = 0;
    long long c[16];
    c[0] = run<false, 128, 1>(tb, a, b, bar, ph, reps, abort_flag);
    c[1] = run<false, 128, 2>(tb, a, b, bar, ph, reps, abort_flag);
    c[2] = run<true, 128, 1>(tb, a, b, bar, ph, reps, abort_flag);
    c[3] = run<true, 128, 2>(tb, a, b, bar, ph, reps, abort_flag);
    c[4] = run<false, 256, 1>(tb, a, b, bar, ph, reps, abort_flag);
    c[5] = run<true, 256, 1>(tb, a, b, bar, ph, reps, abort_flag);
    c[6] = run<false, 64, 1>(tb, a, b, bar, ph, reps, abort_flag);
    c[7] = run<false, 64, 4>(tb, a, b, bar, ph, reps, abort_flag);
    c[8] = run<true, 64, 4>(tb, a, b, bar, ph, reps, abort_flag);
    c[9] = run<false, 128, 3>(tb, a, b, bar, ph, reps, abort_flag);
    c[10] = run<false, 128, 1, true>(tb, a, b, bar, ph, reps, abort_flag);
    c[11] = run<true, 128, 1, true>(tb, a, b, bar, ph, reps, abort_flag);
    // with the other three warps hammering TMEM loads / stores on columns 256..383
    *run_flag = 1;
    __threadfence_block();
    c[12] = run<false, 128, 1, true>(tb, a, b, bar, ph, reps, abort_flag);
    c[13] = run<true, 128, 1, true>(tb, a, b, bar, ph, reps, abort_flag);
    *run_flag = 2;
    if (blockIdx.x == 0) for (int i = 0; i < 14; ++i) out->cyc[i] = c[i];
  } else if (warp >= 1) {
    // wait for run_flag 1, then ld/st until 2 (bounded)
    const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;
    long long spins = 0;
    while (*run_flag == 0 && ++spins < 200000000ll) __nanosleep(200);
    long long iters = 0;
    while (*run_flag == 1 && ++iters < 4000000ll) {
      uint32_t v[32];
      tmem_ld_32x32(tb + 256 + lane_addr, v);
      tmem_ld_wait();
      tmem_st_32x32(tb + 320 + lane_addr, v);
      tmem_st_wait();
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) { tc_fence_after_sync(); tmem_dealloc(tb, 512); }
}

int main(int argc, char** argv) {
  int reps = argc > 1 ? atoi(argv[1]) : 64;
  Res* d; cudaMalloc(&d, sizeof(Res)); cudaMemset(d, 0, sizeof(Res));
  const int smem = 3 * kTile + 1024 + 256;
  cudaFuncSetAttribute(bench, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  const char* names[14] = {"SS N=128 1 acc", "SS N=128 2 acc", "TS N=128 1 acc", "TS N=128 2 acc", "SS N=256", "TS N=256",
                           "SS N=64 1 acc", "SS N=64 4 acc", "TS N=64 4 acc", "SS N=128 3 acc",
                           "SS N=128 commit/8", "TS N=128 commit/8", "SS commit/8 + tmem traffic", "TS commit/8 + tmem traffic"};
  const int nom[14] = {64, 64, 64, 64, 128, 128, 32, 32, 32, 64, 64, 64, 64, 64};
  for (int grid : {1}) {
    for (int it = 0; it < 2; ++it) {
      bench<<<grid, 128, smem>>>(d, reps);
      cudaError_t e = cudaDeviceSynchronize();
      if (e != cudaSuccess) { printf("error %s\n", cudaGetErrorString(e)); return 1; }
    }
    Res h; cudaMemcpy(&h, d, sizeof(Res), cudaMemcpyDeviceToHost);
    for (int m = 0; m < 14; ++m)
      printf("grid %3d  %-18s %8lld cycles, %6.1f per MMA (nominal %d)\n", grid, names[m], h.cyc[m], (double)h.cyc[m] / (reps * 8), nom[m]);
  }
  return 0;
}
