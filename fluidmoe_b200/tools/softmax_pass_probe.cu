// Stand-alone probe of the attention softmax's exponential pass: one thread = one query row of
// 128 scores in registers; per pass 128 x (fma, ex2, add) and 64 bf16x2 packs, as in the forward
// kernel.  Reports cycles per pass for 1, 2 and 4 warps per scheduler and for variants without
// the exponential, without the pack, with the exponential alone and with half-precision packed
// exponentials.  It shows how many warps a scheduler needs before the special-function unit
// (16 results per clock and SM) becomes the limit rather than dependent-instruction latency.
//
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -o /tmp/softmax_pass_probe \
//        fluidmoe_b200/tools/softmax_pass_probe.cu && /tmp/softmax_pass_probe
// or  python -m fluidmoe_b200.tools.kernel_bench softmax_pass
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cstdio>
#include <cstdlib>
#include <cstdint>
__device__ __forceinline__ float fast_exp2(float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) { uint32_t r; asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo)); return r; }
__device__ __forceinline__ uint32_t ex2_h2(uint32_t x) { uint32_t y; asm("ex2.approx.f16x2 %0, %1;" : "=r"(y) : "r"(x)); return y; }
__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) { uint32_t r; asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo)); return r; }

template <int MODE>
__global__ void bench(const float* in, float* out, long long* cyc, int reps) {
  float sv[128];
#pragma unroll
  for (int i = 0; i < 128; ++i) sv[i] = in[(threadIdx.x * 128 + i) & 4095];
  float acc = 0.f; uint32_t sink = 0;
  const float sc = in[0], nm = in[1];
  __syncthreads();
  long long t0 = clock64();
#pragma unroll 1
  for (int r = 0; r < reps; ++r) {
    float l[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) l[k] = 0.f;
#pragma unroll
    for (int i = 0; i < 64; ++i) {
      float x0 = fmaf(sv[2 * i], sc, nm), x1 = fmaf(sv[2 * i + 1], sc, nm);
      float p0, p1;
      if (MODE == 0) { p0 = fast_exp2(x0); p1 = fast_exp2(x1); l[i & 7] += p0; l[(i + 4) & 7] += p1; sink ^= pack_bf16x2(p0, p1); }
      if (MODE == 1) { p0 = x0; p1 = x1; l[i & 7] += p0; l[(i + 4) & 7] += p1; sink ^= pack_bf16x2(p0, p1); }      // no ex2
      if (MODE == 2) { p0 = fast_exp2(x0); p1 = fast_exp2(x1); l[i & 7] += p0; l[(i + 4) & 7] += p1; }             // no cvt
      if (MODE == 3) { p0 = fast_exp2(x0); p1 = fast_exp2(x1); sink ^= __float_as_uint(p0) ^ __float_as_uint(p1); } // ex2 only (+fma)
      if (MODE == 4) { uint32_t h = ex2_h2(pack_h2(x0, x1)); sink ^= h; }                                          // half2 ex2
    }
    acc += ((l[0] + l[1]) + (l[2] + l[3])) + ((l[4] + l[5]) + (l[6] + l[7]));
    // make the next repetition depend on this one a little
    sv[r & 127] += acc * 1e-30f;
  }
  long long t1 = clock64();
  out[blockIdx.x * blockDim.x + threadIdx.x] = acc + __uint_as_float(sink);
  if (threadIdx.x == 0 && blockIdx.x == 0) cyc[MODE] = t1 - t0;
}
int main(int argc, char** argv) {
  int reps = 256;
  float *in, *out; long long* cyc;
  cudaMalloc(&in, 4096 * 4); cudaMalloc(&out, 1 << 20); cudaMalloc(&cyc, 64);
  float h[4096]; for (int i = 0; i < 4096; ++i) h[i] = -(float)(i % 37) * 0.1f; h[0] = 0.125f; h[1] = -1.0f;
  cudaMemcpy(in, h, sizeof(h), cudaMemcpyHostToDevice);
  const char* names[5] = {"fma+ex2+fadd+cvt (the kernel's pass)", "no ex2", "no cvt", "fma+ex2 only", "fma+cvt.f16x2+ex2.f16x2"};
  for (int threads : {128, 256, 512}) {
    for (int it = 0; it < 2; ++it) {
      bench<0><<<1, threads>>>(in, out, cyc, reps); bench<1><<<1, threads>>>(in, out, cyc, reps); bench<2><<<1, threads>>>(in, out, cyc, reps);
      bench<3><<<1, threads>>>(in, out, cyc, reps); bench<4><<<1, threads>>>(in, out, cyc, reps);
      if (cudaDeviceSynchronize() != cudaSuccess) { printf("error\n"); return 1; }
    }
    long long c[8]; cudaMemcpy(c, cyc, 40, cudaMemcpyDeviceToHost);
    for (int m = 0; m < 5; ++m) printf("%d warps/scheduler  %-40s %7.1f cycles per 128-value row pass\n", threads / 128, names[m], (double)c[m] / reps);
  }
  return 0;
}
