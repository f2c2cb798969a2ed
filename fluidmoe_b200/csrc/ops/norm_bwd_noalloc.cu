// Normalisation backward that allocates nothing: the partial weight / bias gradients live in a
// scratch array that is part of the library image (see include/fm_noalloc.h for the contract
// and for who needs this).  The arithmetic is the same as fm_norm_bwd in elementwise.cu; the
// kernels are repeated here so that the regular path is left untouched.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../include/fm_noalloc.h"
#include "../include/sm100_ptx.cuh"

extern "C" void fm_set_error(const char* msg);

namespace fm_noalloc {

constexpr int kThreads = 256;
constexpr int kChunks = FM_NOALLOC_MAX_H / (8 * kThreads);  // 16-byte chunks per thread per row
static_assert(kChunks * 8 * kThreads == FM_NOALLOC_MAX_H, "FM_NOALLOC_MAX_H must be 2048 * n");

// Scratch for the per-CTA partial sums: [FM_NOALLOC_MAX_BLOCKS][2][FM_NOALLOC_MAX_H] floats.
// In host code this name is only a handle: the device address is fetched with
// cudaGetSymbolAddress below and handed to the kernels as an ordinary pointer.
static __device__ __align__(256) float g_scratch[(size_t)FM_NOALLOC_MAX_BLOCKS * 2 * FM_NOALLOC_MAX_H];

__device__ __forceinline__ void unpack8(const uint4& p, float* v) {
  const uint32_t w[4] = {p.x, p.y, p.z, p.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&w[j]);
    v[2 * j] = __low2float(b);
    v[2 * j + 1] = __high2float(b);
  }
}
__device__ __forceinline__ uint4 pack8(const float* v) {
  uint4 p;
  p.x = fm::pack_bf16x2(v[0], v[1]);
  p.y = fm::pack_bf16x2(v[2], v[3]);
  p.z = fm::pack_bf16x2(v[4], v[5]);
  p.w = fm::pack_bf16x2(v[6], v[7]);
  return p;
}
__device__ __forceinline__ float block_sum(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int i = 0; i < kThreads / 32; ++i) t += red[i];
  return t;
}

// Rows blockIdx.x, blockIdx.x + gridDim.x, ...; a thread keeps the gradient sums of its own
// columns in registers and writes them once to scratch[blockIdx.x][0 or 1][column].
__global__ void __launch_bounds__(kThreads)
bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
           const __nv_bfloat16* __restrict__ w, const float* __restrict__ mean,
           const float* __restrict__ rstd, const __nv_bfloat16* __restrict__ res_grad,
           __nv_bfloat16* __restrict__ dx, float* __restrict__ scratch, int T, int H, int kind) {
  __shared__ float red[kThreads / 32];
  const int nvec = H / 8;
  float dg[kChunks][8], db[kChunks][8], g[kChunks][8];
#pragma unroll
  for (int c = 0; c < kChunks; ++c) {
    const int i = threadIdx.x + c * kThreads;
    if (i < nvec) unpack8(reinterpret_cast<const uint4*>(w)[i], g[c]);
#pragma unroll
    for (int j = 0; j < 8; ++j) dg[c][j] = db[c][j] = 0.f;
  }
  for (long long r = blockIdx.x; r < T; r += gridDim.x) {
    const float mu = kind == 0 ? mean[r] : 0.f;
    const float rs = rstd[r];
    float xh[kChunks][8], gy[kChunks][8];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int c = 0; c < kChunks; ++c) {
      const int i = threadIdx.x + c * kThreads;
      if (i < nvec) {
        float xv[8], dv[8];
        unpack8(reinterpret_cast<const uint4*>(x + r * H)[i], xv);
        unpack8(reinterpret_cast<const uint4*>(dy + r * H)[i], dv);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xh[c][j] = (xv[j] - mu) * rs;
          gy[c][j] = dv[j] * g[c][j];
          s1 += gy[c][j] * xh[c][j];
          s2 += gy[c][j];
          dg[c][j] += dv[j] * xh[c][j];
          db[c][j] += dv[j];
        }
      }
    }
    const float c1 = block_sum(s1, red) / H;
    const float c2 = kind == 0 ? block_sum(s2, red) / H : 0.f;
#pragma unroll
    for (int c = 0; c < kChunks; ++c) {
      const int i = threadIdx.x + c * kThreads;
      if (i < nvec) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = (gy[c][j] - c2 - xh[c][j] * c1) * rs;
        if (res_grad != nullptr) {
          float rg[8];
          unpack8(reinterpret_cast<const uint4*>(res_grad + r * H)[i], rg);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += rg[j];
        }
        reinterpret_cast<uint4*>(dx + r * H)[i] = pack8(o);
      }
    }
  }
  float* pg = scratch + (size_t)blockIdx.x * 2 * H;
#pragma unroll
  for (int c = 0; c < kChunks; ++c) {
    const int i = threadIdx.x + c * kThreads;
    if (i < nvec) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        pg[i * 8 + j] = dg[c][j];
        pg[H + i * 8 + j] = db[c][j];
      }
    }
  }
}

__global__ void reduce_kernel(const float* __restrict__ scratch, float* __restrict__ dw,
                              float* __restrict__ db, int nblocks, int H) {
  const int col = blockIdx.x * blockDim.x + threadIdx.x;
  if (col >= 2 * H) return;
  float s = 0.f;
  for (int b = 0; b < nblocks; ++b) s += scratch[(size_t)b * 2 * H + col];
  if (col < H)
    dw[col] = s;
  else if (db != nullptr)
    db[col - H] = s;
}

constexpr int kMaxDevices = 64;
static float* g_scratch_addr[kMaxDevices] = {nullptr};

// Device address of the scratch array on the current device, looked up once per device.
static float* scratch_for_current_device() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    fm_set_error("norm_bwd_static: cannot identify the current device");
    return nullptr;
  }
  if (g_scratch_addr[dev] == nullptr) {
    float* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_scratch);
    if (e != cudaSuccess || p == nullptr) {
      char buf[256];
      snprintf(buf, sizeof(buf), "norm_bwd_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
      fm_set_error(buf);
      (void)cudaGetLastError();
      return nullptr;
    }
    g_scratch_addr[dev] = p;
  }
  return g_scratch_addr[dev];
}

}  // namespace fm_noalloc

extern "C" int fm_norm_bwd_static(const void* dy, const void* x, const void* w, const float* mean,
                                  const float* rstd, const void* res_grad, void* dx, float* dw,
                                  float* db, int T, int H, int kind, cudaStream_t stream) {
  using namespace fm_noalloc;
  if (T <= 0) {
    char buf[120];
    snprintf(buf, sizeof(buf), "norm_bwd_static: T=%d rows; at least one row is needed", T);
    fm_set_error(buf);
    return -1;
  }
  if (H <= 0 || H % 8 != 0 || H > FM_NOALLOC_MAX_H) {
    char buf[200];
    snprintf(buf, sizeof(buf),
             "norm_bwd_static: H=%d is not supported (a multiple of 8, at most %d; the scratch array has a fixed size)",
             H, FM_NOALLOC_MAX_H);
    fm_set_error(buf);
    return -1;
  }
  if (kind == 0 && mean == nullptr) {
    fm_set_error("norm_bwd_static: LayerNorm needs the saved mean");
    return -1;
  }
  float* scratch = scratch_for_current_device();
  if (scratch == nullptr) return -2;
  {
    // the scratch looked up above belongs to the current device; the buffers must live there too
    int dev = -1;
    cudaPointerAttributes attr;
    if (cudaGetDevice(&dev) == cudaSuccess && cudaPointerGetAttributes(&attr, dx) == cudaSuccess &&
        attr.type == cudaMemoryTypeDevice && attr.device != dev) {
      char buf[160];
      snprintf(buf, sizeof(buf), "norm_bwd_static: dx lives on device %d but device %d is current", attr.device, dev);
      fm_set_error(buf);
      return -3;
    }
    (void)cudaGetLastError();
  }
  using bf = __nv_bfloat16;
  const int nb = T < FM_NOALLOC_MAX_BLOCKS ? T : FM_NOALLOC_MAX_BLOCKS;
  bwd_kernel<<<nb, kThreads, 0, stream>>>((const bf*)dy, (const bf*)x, (const bf*)w, mean, rstd,
                                          (const bf*)res_grad, (bf*)dx, scratch, T, H, kind);
  cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) {
    reduce_kernel<<<(2 * H + 255) / 256, 256, 0, stream>>>(scratch, dw, db, nb, H);
    e = cudaGetLastError();
  }
  if (e != cudaSuccess) {
    fm_set_error(cudaGetErrorString(e));
    return (int)e;
  }
  return 0;
}
