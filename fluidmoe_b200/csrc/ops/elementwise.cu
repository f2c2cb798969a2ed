// Memory-bound kernels of the layer: normalisation, rotary embedding, router top-k softmax,
// token permute / un-permute, and the fused Adam step.  All activations are bf16 with fp32
// arithmetic; every kernel moves 16 bytes per thread per access and touches each element once
// where the math allows it.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>
#include <stdio.h>

#include "../include/fm_ops.h"
#include "../include/sm100_ptx.cuh"

extern "C" void fm_set_error(const char* msg);

namespace fm {

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
  p.x = pack_bf16x2(v[0], v[1]);
  p.y = pack_bf16x2(v[2], v[3]);
  p.z = pack_bf16x2(v[4], v[5]);
  p.w = pack_bf16x2(v[6], v[7]);
  return p;
}

template <int THREADS>
__device__ __forceinline__ float block_sum(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int i = 0; i < THREADS / 32; ++i) t += red[i];
  return t;
}

// --------------------------------------------------------------------------------------------
// Normalisation forward.  One CTA per row; the row is cached in shared memory so global memory
// is read once.  kind: 0 = LayerNorm (mean and rstd saved), 1 = RMSNorm (rstd saved).
// --------------------------------------------------------------------------------------------
constexpr int kNormThreads = 256;

__global__ void __launch_bounds__(kNormThreads)
norm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                const __nv_bfloat16* __restrict__ b, __nv_bfloat16* __restrict__ y,
                float* __restrict__ mean_out, float* __restrict__ rstd_out, int H, float eps,
                int kind) {
  extern __shared__ uint4 row_s[];
  __shared__ float red[kNormThreads / 32];
  const long long r = blockIdx.x;
  const int nvec = H / 8;
  const uint4* xr = reinterpret_cast<const uint4*>(x + r * H);
  float s = 0.f;
  for (int i = threadIdx.x; i < nvec; i += kNormThreads) {
    const uint4 p = xr[i];
    row_s[i] = p;
    float v[8];
    unpack8(p, v);
    if (kind == 0) {
#pragma unroll
      for (int j = 0; j < 8; ++j) s += v[j];
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) s += v[j] * v[j];
    }
  }
  s = block_sum<kNormThreads>(s, red);
  float mean = 0.f, rstd;
  if (kind == 0) {
    mean = s / H;
    float q = 0.f;
    for (int i = threadIdx.x; i < nvec; i += kNormThreads) {
      float v[8];
      unpack8(row_s[i], v);
#pragma unroll
      for (int j = 0; j < 8; ++j) q += (v[j] - mean) * (v[j] - mean);
    }
    q = block_sum<kNormThreads>(q, red);
    rstd = rsqrtf(q / H + eps);
  } else {
    rstd = rsqrtf(s / H + eps);
  }
  if (threadIdx.x == 0) {
    if (mean_out) mean_out[r] = mean;
    rstd_out[r] = rstd;
  }
  uint4* yr = reinterpret_cast<uint4*>(y + r * H);
  const uint4* wv = reinterpret_cast<const uint4*>(w);
  const uint4* bv = reinterpret_cast<const uint4*>(b);
  for (int i = threadIdx.x; i < nvec; i += kNormThreads) {
    float v[8], g[8], o[8];
    unpack8(row_s[i], v);
    unpack8(wv[i], g);
    if (b != nullptr) {
      float bb[8];
      unpack8(bv[i], bb);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = (v[j] - mean) * rstd * g[j] + bb[j];
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = (v[j] - mean) * rstd * g[j];
    }
    yr[i] = pack8(o);
  }
}

// --------------------------------------------------------------------------------------------
// Normalisation backward.  Each CTA walks rows blockIdx.x, +gridDim.x, ...; a thread owns the
// same columns in every row, so the weight / bias gradients accumulate in registers and are
// written once per CTA to a partial buffer [gridDim.x, 2, H] that a second kernel reduces.
// dx optionally adds the gradient that reaches the input through the residual branch.
// --------------------------------------------------------------------------------------------
constexpr int kNormBwdChunks = 4;  // columns per thread = 8 * chunks  ->  H <= 8192

// kChunks (1, 2 or 4) is chosen from H: the per-thread arrays below are sized by it, and with
// four chunks the kernel needs 195 registers, which leaves one CTA of eight warps per SM and makes
// it latency-bound (0.31 of the copy bandwidth at H = 4096); two chunks fit two CTAs per SM.
template <int kChunks>
__global__ void __launch_bounds__(kNormThreads, kChunks <= 2 ? 2 : 1)
norm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                const __nv_bfloat16* __restrict__ w, const float* __restrict__ mean,
                const float* __restrict__ rstd, const __nv_bfloat16* __restrict__ res_grad,
                __nv_bfloat16* __restrict__ dx, float* __restrict__ partial, int T, int H,
                int kind) {
  __shared__ float red[kNormThreads / 32];
  const int nvec = H / 8;
  float dg[kChunks][8], db[kChunks][8], g[kChunks][8];
#pragma unroll
  for (int c = 0; c < kChunks; ++c) {
    const int i = threadIdx.x + c * kNormThreads;
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
      const int i = threadIdx.x + c * kNormThreads;
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
    const float c1 = block_sum<kNormThreads>(s1, red) / H;
    const float c2 = kind == 0 ? block_sum<kNormThreads>(s2, red) / H : 0.f;
#pragma unroll
    for (int c = 0; c < kChunks; ++c) {
      const int i = threadIdx.x + c * kNormThreads;
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
  float* pg = partial + (long long)blockIdx.x * 2 * H;
#pragma unroll
  for (int c = 0; c < kChunks; ++c) {
    const int i = threadIdx.x + c * kNormThreads;
    if (i < nvec) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        pg[i * 8 + j] = dg[c][j];
        pg[H + i * 8 + j] = db[c][j];
      }
    }
  }
}

// Column sums of the partial buffer: a CTA owns 32 columns, its eight warps take every eighth
// partial row each and the eight sums meet in shared memory.
__global__ void __launch_bounds__(256)
norm_bwd_reduce_kernel(const float* __restrict__ partial, float* __restrict__ dw,
                       float* __restrict__ db, int nblocks, int H) {
  __shared__ float part[8][33];
  const int lane = threadIdx.x & 31, grp = threadIdx.x >> 5;
  const int col = blockIdx.x * 32 + lane;
  float s = 0.f;
  if (col < 2 * H)
    for (int b = grp; b < nblocks; b += 8) s += partial[(long long)b * 2 * H + col];
  part[grp][lane] = s;
  __syncthreads();
  if (grp == 0 && col < 2 * H) {
#pragma unroll
    for (int g2 = 1; g2 < 8; ++g2) s += part[g2][lane];
    if (col < H)
      dw[col] = s;
    else if (db != nullptr)
      db[col - H] = s;
  }
}

// --------------------------------------------------------------------------------------------
// Rotary embedding in place on the packed QKV buffer [rows, heads_per_row, d]: heads
// 0 .. rope_heads-1 of every row are rotated (the query heads and the key head of a KV group),
// the rest (the value head) is left alone.  Position of a row = row / rows_per_pos.
// sign = +1 forward, -1 backward (transposed rotation).
// --------------------------------------------------------------------------------------------
constexpr int kKernelIdRopeWait = 16;
__global__ void rope_packed_kernel(__nv_bfloat16* __restrict__ t, const float* __restrict__ freqs,
                                   long long rows, int heads_per_row, int rope_heads, int d,
                                   int rot, int rows_per_pos, int backward, const int* wait_flags,
                                   int wait_n, int wait_expected, unsigned long long* wait_ns,
                                   unsigned long long timeout_ns, int* status) {
  // first consumer of the projection buffer that peers fill: wait for their rows here
  if (wait_flags != nullptr)
    wait_counters_cta(wait_flags, wait_n, wait_expected, wait_ns, timeout_ns, status, kKernelIdRopeWait);
  const int half = rot / 2;
  const int vec_per_head = half / 8;
  const long long total = rows * rope_heads * vec_per_head;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int vi = (int)(idx % vec_per_head);
    const long long rh = idx / vec_per_head;
    const int h = (int)(rh % rope_heads);
    const long long row = rh / rope_heads;
    const long long pos = row / rows_per_pos;
    __nv_bfloat16* base = t + (row * heads_per_row + h) * d;
    uint4* p1 = reinterpret_cast<uint4*>(base + vi * 8);
    uint4* p2 = reinterpret_cast<uint4*>(base + half + vi * 8);
    float a[8], b[8], o1[8], o2[8];
    unpack8(*p1, a);
    unpack8(*p2, b);
    // `freqs` holds (cos, sin) pairs of the angles, [position][rot][2]: the table is computed once
    // per sequence on the host side instead of two sincosf per value here (which made the kernel
    // compute-bound at 0.41 of the copy bandwidth)
    const float2* f1 = reinterpret_cast<const float2*>(freqs) + pos * rot + vi * 8;
    const float2* f2 = f1 + half;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float2 cs1 = f1[j], cs2 = f2[j];
      const float c1 = cs1.x, s1 = cs1.y, c2 = cs2.x, s2 = cs2.y;
      if (!backward) {
        o1[j] = a[j] * c1 - b[j] * s1;
        o2[j] = b[j] * c2 + a[j] * s2;
      } else {
        o1[j] = a[j] * c1 + b[j] * s2;
        o2[j] = b[j] * c2 - a[j] * s1;
      }
    }
    *p1 = pack8(o1);
    *p2 = pack8(o2);
  }
}

// --------------------------------------------------------------------------------------------
// Router: top-k over experts then softmax over the k winners (fp32).  One thread per token.
// Ties go to the lower expert index.
// --------------------------------------------------------------------------------------------
__global__ void topk_softmax_kernel(const float* __restrict__ logits, long long* __restrict__ idx_out,
                                    float* __restrict__ prob_out, int T, int E, int k) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= T) return;
  const float* l = logits + (long long)t * E;
  float vals[16];
  int ids[16];
  for (int j = 0; j < k; ++j) {
    float best = -INFINITY;
    int bi = -1;
    for (int e = 0; e < E; ++e) {
      const float v = l[e];
      bool taken = false;
      for (int q = 0; q < j; ++q) taken |= (ids[q] == e);
      if (!taken && (v > best || bi < 0)) {
        best = v;
        bi = e;
      }
    }
    vals[j] = best;
    ids[j] = bi;
  }
  float m = vals[0], s = 0.f;
  for (int j = 0; j < k; ++j) s += __expf(vals[j] - m);
  for (int j = 0; j < k; ++j) {
    idx_out[(long long)t * k + j] = ids[j];
    prob_out[(long long)t * k + j] = __expf(vals[j] - m) / s;
  }
}

// --------------------------------------------------------------------------------------------
// Permute: out[s] = x[idx[s]] (one warp per row, 16-byte accesses).
// --------------------------------------------------------------------------------------------
__global__ void gather_rows_kernel(const __nv_bfloat16* __restrict__ x,
                                   const long long* __restrict__ idx,
                                   __nv_bfloat16* __restrict__ out, long long rows, int H) {
  const int nvec = H / 8;
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  for (long long s = (long long)blockIdx.x * warps_per_block + (threadIdx.x >> 5); s < rows;
       s += (long long)gridDim.x * warps_per_block) {
    const uint4* src = reinterpret_cast<const uint4*>(x + idx[s] * H);
    uint4* dst = reinterpret_cast<uint4*>(out + s * H);
    for (int i = lane; i < nvec; i += 32) dst[i] = src[i];
  }
}

// --------------------------------------------------------------------------------------------
// Un-permute: out[t] = residual[t] + sum_j rows[slot[t, j]], fp32 accumulation, slots < 0
// skipped.  Deterministic (a gather, not a scatter-add).
// --------------------------------------------------------------------------------------------
constexpr int kKernelIdUnpermuteWait = 15;
// Optionally the kernel first waits, bounded, until the arrival counters of the `wait_n` sources
// have reached `wait_expected` (rows pushed by peers into `rows`): the consumer polls its own
// counters instead of a stand-alone wait kernel in front of it.  The time the slowest thread of CTA 0
// waited is added to `wait_ns` (communication the step could not hide).
__global__ void unpermute_reduce_kernel(const __nv_bfloat16* __restrict__ rows,
                                        const int* __restrict__ slot,
                                        const __nv_bfloat16* __restrict__ residual,
                                        __nv_bfloat16* __restrict__ out, int T, int k, int H,
                                        const int* wait_flags, int wait_n, int wait_expected,
                                        unsigned long long* wait_ns, unsigned long long timeout_ns,
                                        int* status) {
  if (wait_flags != nullptr)
    wait_counters_cta(wait_flags, wait_n, wait_expected, wait_ns, timeout_ns, status, kKernelIdUnpermuteWait);
  const int nvec = H / 8;
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  for (long long t = (long long)blockIdx.x * warps_per_block + (threadIdx.x >> 5); t < T;
       t += (long long)gridDim.x * warps_per_block) {
    int sl[16];
    for (int j = 0; j < k; ++j) sl[j] = slot[t * k + j];
    for (int i = lane; i < nvec; i += 32) {
      float acc[8];
      if (residual != nullptr) {
        unpack8(reinterpret_cast<const uint4*>(residual + t * H)[i], acc);
      } else {
#pragma unroll
        for (int q = 0; q < 8; ++q) acc[q] = 0.f;
      }
      for (int j = 0; j < k; ++j) {
        if (sl[j] < 0) continue;
        float v[8];
        unpack8(reinterpret_cast<const uint4*>(rows + (long long)sl[j] * H)[i], v);
#pragma unroll
        for (int q = 0; q < 8; ++q) acc[q] += v[q];
      }
      reinterpret_cast<uint4*>(out + t * H)[i] = pack8(acc);
    }
  }
}

// --------------------------------------------------------------------------------------------
// Fused Adam(W) on a flat slice: fp32 gradient, fp32 moments, bf16 parameter updated in place
// (optionally through an fp32 master copy).  The gradient may be zeroed in the same pass.
// --------------------------------------------------------------------------------------------
template <class ST>
struct Vec4;
template <>
struct Vec4<float> {
  static __device__ __forceinline__ void load(const float* p, float* v) {
    const float4 x = *reinterpret_cast<const float4*>(p);
    v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
  }
  static __device__ __forceinline__ void store(float* p, const float* v) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  }
};
template <>
struct Vec4<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* v) {
    const uint2 x = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&x.x);
    const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&x.y);
    v[0] = __low2float(a); v[1] = __high2float(a); v[2] = __low2float(b); v[3] = __high2float(b);
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float* v) {
    uint2 x;
    x.x = pack_bf16x2(v[0], v[1]);
    x.y = pack_bf16x2(v[2], v[3]);
    *reinterpret_cast<uint2*>(p) = x;
  }
};

// n must be a multiple of 4 and all pointers 16-byte aligned (the host falls back to the tail
// kernel otherwise); every thread handles 4 consecutive elements per iteration with one vector
// access per array.
template <class ST>
__global__ void __launch_bounds__(512)
adam_kernel(__nv_bfloat16* __restrict__ p, float* __restrict__ master, float* __restrict__ g,
            ST* __restrict__ m, ST* __restrict__ v, long long n4, float lr, float beta1, float beta2,
            float eps, float weight_decay, float rbc1, float rbc2, float grad_scale, int zero_grad) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4;
       i += (long long)gridDim.x * blockDim.x) {
    const long long q = i * 4;
    float gr[4], w[4], mm[4], vv[4];
    Vec4<float>::load(g + q, gr);
    Vec4<ST>::load(m + q, mm);
    Vec4<ST>::load(v + q, vv);
    if (master)
      Vec4<float>::load(master + q, w);
    else
      Vec4<__nv_bfloat16>::load(p + q, w);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float gj = gr[j] * grad_scale;
      mm[j] = beta1 * mm[j] + (1.f - beta1) * gj;
      vv[j] = beta2 * vv[j] + (1.f - beta2) * gj * gj;
      const float upd = (mm[j] * rbc1) / (sqrtf(vv[j] * rbc2) + eps) + weight_decay * w[j];
      w[j] -= lr * upd;
    }
    Vec4<ST>::store(m + q, mm);
    Vec4<ST>::store(v + q, vv);
    if (master) Vec4<float>::store(master + q, w);
    Vec4<__nv_bfloat16>::store(p + q, w);
    if (zero_grad) *reinterpret_cast<float4*>(g + q) = make_float4(0.f, 0.f, 0.f, 0.f);
  }
}

// Background form of the Adam step for bf16 parameters with bf16 moments: 128-thread CTAs with at
// most 80 registers, so that one CTA fits on an SM BESIDE a resident tensor-core kernel (GEMM /
// attention CTAs leave about 11 K registers and no shared memory is needed here).  Every thread
// keeps four independent 4-element groups in flight per iteration to cover DRAM latency with so
// few threads.  Launched on a side stream, it runs under the tensor-bound kernels of the
// following layers.  n4 = number of 4-element groups; pointers 16-byte aligned (8 for bf16).
__global__ void __launch_bounds__(128, 6)   // at most 80 registers: 10 K per CTA
adam_background_kernel(__nv_bfloat16* __restrict__ p, const float* __restrict__ g,
                       __nv_bfloat16* __restrict__ m, __nv_bfloat16* __restrict__ v, long long n4, float lr,
                       float beta1, float beta2, float eps, float weight_decay, float rbc1, float rbc2,
                       float grad_scale) {
  constexpr int U = 4;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i0 = (long long)blockIdx.x * blockDim.x + threadIdx.x; i0 < n4; i0 += stride * U) {
    float4 gr[U];
    uint2 pw[U], pm[U], pv[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = i0 + u * stride;
      if (i < n4) {
        gr[u] = *reinterpret_cast<const float4*>(g + i * 4);
        pw[u] = *reinterpret_cast<const uint2*>(p + i * 4);
        pm[u] = *reinterpret_cast<const uint2*>(m + i * 4);
        pv[u] = *reinterpret_cast<const uint2*>(v + i * 4);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = i0 + u * stride;
      if (i < n4) {
        const float gg[4] = {gr[u].x, gr[u].y, gr[u].z, gr[u].w};
        uint32_t* ww = reinterpret_cast<uint32_t*>(&pw[u]);
        uint32_t* wm = reinterpret_cast<uint32_t*>(&pm[u]);
        uint32_t* wv = reinterpret_cast<uint32_t*>(&pv[u]);
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          float w2[2] = {__uint_as_float(ww[q] << 16), __uint_as_float(ww[q] & 0xffff0000u)};
          float m2[2] = {__uint_as_float(wm[q] << 16), __uint_as_float(wm[q] & 0xffff0000u)};
          float v2[2] = {__uint_as_float(wv[q] << 16), __uint_as_float(wv[q] & 0xffff0000u)};
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const float gj = gg[2 * q + e] * grad_scale;
            m2[e] = beta1 * m2[e] + (1.f - beta1) * gj;
            v2[e] = beta2 * v2[e] + (1.f - beta2) * gj * gj;
            w2[e] -= lr * ((m2[e] * rbc1) / (sqrtf(v2[e] * rbc2) + eps) + weight_decay * w2[e]);
          }
          ww[q] = pack_bf16x2(w2[0], w2[1]);
          wm[q] = pack_bf16x2(m2[0], m2[1]);
          wv[q] = pack_bf16x2(v2[0], v2[1]);
        }
        *reinterpret_cast<uint2*>(m + i * 4) = pm[u];
        *reinterpret_cast<uint2*>(v + i * 4) = pv[u];
        *reinterpret_cast<uint2*>(p + i * 4) = pw[u];
      }
    }
  }
}

template <class ST>
__global__ void adam_tail_kernel(__nv_bfloat16* p, float* master, float* g, ST* m, ST* v,
                                 long long lo, long long n, float lr, float beta1, float beta2,
                                 float eps, float weight_decay, float rbc1, float rbc2,
                                 float grad_scale, int zero_grad) {
  const long long q = lo + (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (q >= n) return;
  const float gj = g[q] * grad_scale;
  float w = master ? master[q] : __bfloat162float(p[q]);
  const float mi = beta1 * (float)m[q] + (1.f - beta1) * gj;
  const float vi = beta2 * (float)v[q] + (1.f - beta2) * gj * gj;
  m[q] = (ST)mi;
  v[q] = (ST)vi;
  w -= lr * ((mi * rbc1) / (sqrtf(vi * rbc2) + eps) + weight_decay * w);
  if (master) master[q] = w;
  p[q] = __float2bfloat16(w);
  if (zero_grad) g[q] = 0.f;
}

// --------------------------------------------------------------------------------------------
// Router backward: gradient of the loss w.r.t. the router logits [T, E] (fp32).  One thread per
// token gathers the gradient of its k slot probabilities (dropped choices have slot -1 and
// contribute nothing), adds the load-balancing term coef * tokens_per_expert[e], runs the backward
// of the softmax over the k selected logits, scatters into a zeroed row and adds the z-loss term
// zc * logsumexp(logits) * softmax(logits).  Reference: fluid/moe/backward.py:1461-1530.
// --------------------------------------------------------------------------------------------
__global__ void router_bwd_kernel(const float* __restrict__ dprobs_slots, const int* __restrict__ slot_of_token,
                                  const long long* __restrict__ top_idx, const float* __restrict__ top_probs,
                                  const float* __restrict__ logits, const float* __restrict__ tpe,
                                  float aux_coef, float z_coef, int T, int k, int E,
                                  float* __restrict__ dlogits) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= T) return;
  float* out = dlogits + (long long)t * E;
  if (z_coef != 0.f) {
    const float* lg = logits + (long long)t * E;
    float mx = -INFINITY;
    for (int e = 0; e < E; ++e) mx = fmaxf(mx, lg[e]);
    float sum = 0.f;
    for (int e = 0; e < E; ++e) sum += __expf(lg[e] - mx);
    const float lse = mx + __logf(sum);
    const float f = z_coef * lse / sum;
    for (int e = 0; e < E; ++e) out[e] = f * __expf(lg[e] - mx);
  } else {
    for (int e = 0; e < E; ++e) out[e] = 0.f;
  }
  float dot = 0.f;
  for (int j = 0; j < k; ++j) {
    const int slot = slot_of_token[(long long)t * k + j];
    float g = slot >= 0 ? dprobs_slots[slot] : 0.f;
    if (tpe != nullptr) g += aux_coef * tpe[top_idx[(long long)t * k + j]];
    dot += top_probs[(long long)t * k + j] * g;
  }
  for (int j = 0; j < k; ++j) {
    const int slot = slot_of_token[(long long)t * k + j];
    const long long e = top_idx[(long long)t * k + j];
    float g = slot >= 0 ? dprobs_slots[slot] : 0.f;
    if (tpe != nullptr) g += aux_coef * tpe[e];
    out[e] += top_probs[(long long)t * k + j] * (g - dot);
  }
}

// --------------------------------------------------------------------------------------------
// Routing plan for fixed (padded) capacity.  One CTA per expert:
//   1. count the tokens routed to the expert;
//   2. if there are more than `cap`, find the cap-th largest probability by radix select on the
//      float bits (probabilities are positive, so the unsigned order is the numeric order) and
//      keep ties in ascending token order;
//   3. walk the tokens in order and assign slots: kept tokens, plus the first (cap - kept)
//      tokens that are NOT routed to this expert as padding (probability 0), all in ascending
//      token order.
// Outputs have static shapes; nothing is read back by the host.
// --------------------------------------------------------------------------------------------
constexpr int kPlanThreads = 512;

__device__ __forceinline__ int block_excl_scan(int v, int* total, int* smem /* [32] */) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int x = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int y = __shfl_up_sync(0xffffffffu, x, o);
    if (lane >= o) x += y;
  }
  __syncthreads();
  if (lane == 31) smem[warp] = x;
  __syncthreads();
  if (warp == 0) {
    int w = lane < kPlanThreads / 32 ? smem[lane] : 0;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int y = __shfl_up_sync(0xffffffffu, w, o);
      if (lane >= o) w += y;
    }
    smem[lane] = w;  // inclusive warp totals
  }
  __syncthreads();
  const int base = warp == 0 ? 0 : smem[warp - 1];
  *total = smem[kPlanThreads / 32 - 1];
  return base + x - v;
}

__global__ void __launch_bounds__(kPlanThreads)
moe_plan_kernel(const long long* __restrict__ top_idx, const float* __restrict__ top_probs, int T,
                int k, int E, int cap, long long* __restrict__ sorted_indices,
                float* __restrict__ slot_probs, int* __restrict__ slot_of_token,
                int* __restrict__ routed_per_expert) {
  __shared__ int hist[256];
  __shared__ int scan_s[32];
  __shared__ int sh_count, sh_prefix, sh_quota;
  const int e = blockIdx.x;
  const int tid = threadIdx.x;

  auto lookup = [&](int t, int& j_out) -> float {
    for (int j = 0; j < k; ++j)
      if ((int)top_idx[(long long)t * k + j] == e) {
        j_out = j;
        return top_probs[(long long)t * k + j];
      }
    j_out = -1;
    return 0.f;
  };

  // ---- 1. count ----
  if (tid == 0) sh_count = 0;
  __syncthreads();
  int local = 0;
  for (int t = tid; t < T; t += kPlanThreads) {
    int j;
    lookup(t, j);
    local += j >= 0;
  }
  atomicAdd(&sh_count, local);
  __syncthreads();
  const int count = sh_count;
  const int kept_total = min(count, cap);

  // ---- 2. threshold by radix select (only when tokens must be dropped) ----
  uint32_t thr_bits = 0;   // keep prob > thr, plus `quota` tokens with prob == thr
  int quota = 0;
  if (count > cap) {
    uint32_t prefix = 0, mask = 0;
    int want = cap;  // rank (1-based, from the top) of the threshold element
    for (int shift = 24; shift >= 0; shift -= 8) {
      for (int i = tid; i < 256; i += kPlanThreads) hist[i] = 0;
      __syncthreads();
      for (int t = tid; t < T; t += kPlanThreads) {
        int j;
        const float pr = lookup(t, j);
        if (j < 0) continue;
        const uint32_t b = __float_as_uint(pr);
        if ((b & mask) == prefix) atomicAdd(&hist[(b >> shift) & 255], 1);
      }
      __syncthreads();
      if (tid == 0) {
        int acc = 0, bin = 255;
        for (; bin >= 0; --bin) {
          if (acc + hist[bin] >= want) break;
          acc += hist[bin];
        }
        sh_prefix = bin;
        sh_quota = want - acc;  // rank of the threshold inside the chosen bin
      }
      __syncthreads();
      prefix |= (uint32_t)sh_prefix << shift;
      mask |= 255u << shift;
      want = sh_quota;
      __syncthreads();
    }
    thr_bits = prefix;
    quota = want;  // number of elements equal to the threshold that are kept
  }

  // ---- 3. ordered slot assignment ----
  int ties_seen = 0, sel_seen = 0, nonrouted_seen = 0;
  const int pad_budget = cap - kept_total;
  for (int t0 = 0; t0 < T; t0 += kPlanThreads) {
    const int t = t0 + tid;
    int j = -1;
    float pr = 0.f;
    bool valid = t < T;
    if (valid) pr = lookup(t, j);
    const bool routed = valid && j >= 0;
    const uint32_t b = __float_as_uint(pr);
    const bool above = routed && (count <= cap || b > thr_bits);
    const bool tie = routed && count > cap && b == thr_bits;
    int tot;
    const int tie_rank = block_excl_scan(tie ? 1 : 0, &tot, scan_s) + ties_seen;
    ties_seen += tot;
    const bool kept = above || (tie && tie_rank < quota);
    const bool nonrouted = valid && !routed;
    const int nr_rank = block_excl_scan(nonrouted ? 1 : 0, &tot, scan_s) + nonrouted_seen;
    nonrouted_seen += tot;
    const bool selected = kept || (nonrouted && nr_rank < pad_budget);
    const int pos = block_excl_scan(selected ? 1 : 0, &tot, scan_s) + sel_seen;
    sel_seen += tot;
    if (selected && pos < cap) {
      const long long slot = (long long)e * cap + pos;
      sorted_indices[slot] = t;
      slot_probs[slot] = kept ? pr : 0.f;
      if (kept) slot_of_token[(long long)t * k + j] = (int)slot;
    }
    if (routed && !kept) slot_of_token[(long long)t * k + j] = -1;
  }
  if (tid == 0) routed_per_expert[e] = kept_total;
}

// --------------------------------------------------------------------------------------------
// Cross-entropy over bf16 logits, forward and backward in one kernel: one CTA per row makes one
// pass for the running max / sum (log-sum-exp) and one pass that overwrites the logits with
// dlogits = (softmax - onehot) * grad_scale.  Rows whose label is negative are ignored (loss 0,
// zero gradient).  loss_out[row] = lse - logit[label].
// --------------------------------------------------------------------------------------------
constexpr int kCeThreads = 512;

__global__ void __launch_bounds__(kCeThreads)
cross_entropy_kernel(__nv_bfloat16* __restrict__ logits, const long long* __restrict__ labels,
                     float* __restrict__ loss_out, int V, float grad_scale) {
  __shared__ float red[kCeThreads / 32];
  __shared__ float bcast[2];
  const long long r = blockIdx.x;
  __nv_bfloat16* row = logits + r * V;
  const long long label = labels[r];
  const int nvec = V / 8;
  float m = -INFINITY, s = 0.f;
  for (int i = threadIdx.x; i < nvec; i += kCeThreads) {
    float v[8];
    unpack8(reinterpret_cast<const uint4*>(row)[i], v);
    float mx = v[0];
#pragma unroll
    for (int j = 1; j < 8; ++j) mx = fmaxf(mx, v[j]);
    if (mx > m) {
      s *= __expf(m - mx);
      m = mx;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) s += __expf(v[j] - m);
  }
  for (int i = nvec * 8 + threadIdx.x; i < V; i += kCeThreads) {
    const float x = __bfloat162float(row[i]);
    if (x > m) {
      s *= __expf(m - x);
      m = x;
    }
    s += __expf(x - m);
  }
  // block reduce of (m, s)
  float gm = m;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) gm = fmaxf(gm, __shfl_xor_sync(0xffffffffu, gm, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = gm;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = red[0];
    for (int i = 1; i < kCeThreads / 32; ++i) t = fmaxf(t, red[i]);
    bcast[0] = t;
  }
  __syncthreads();
  gm = bcast[0];
  const float total = block_sum<kCeThreads>(m == -INFINITY ? 0.f : s * __expf(m - gm), red);
  const float lse = gm + __logf(total);
  if (threadIdx.x == 0)
    loss_out[r] = label >= 0 ? lse - __bfloat162float(row[label]) : 0.f;
  __syncthreads();
  const float scale = label >= 0 ? grad_scale : 0.f;
  for (int i = threadIdx.x; i < nvec; i += kCeThreads) {
    float v[8];
    unpack8(reinterpret_cast<const uint4*>(row)[i], v);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float pr = __expf(v[j] - lse);
      v[j] = (pr - ((long long)(i * 8 + j) == label ? 1.f : 0.f)) * scale;
    }
    reinterpret_cast<uint4*>(row)[i] = pack8(v);
  }
  for (int i = nvec * 8 + threadIdx.x; i < V; i += kCeThreads) {
    const float pr = __expf(__bfloat162float(row[i]) - lse);
    row[i] = __float2bfloat16((pr - ((long long)i == label ? 1.f : 0.f)) * scale);
  }
}

}  // namespace fm

static int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    char buf[256];
    snprintf(buf, sizeof(buf), "%s: %s", what, cudaGetErrorString(e));
    fm_set_error(buf);
    return (int)e;
  }
  return 0;
}
static int grid_for(long long work, int per_block, int cap = 148 * 16) {
  long long g = (work + per_block - 1) / per_block;
  if (g < 1) g = 1;
  if (g > cap) g = cap;
  return (int)g;
}

extern "C" int fm_norm_fwd(const void* x, const void* w, const void* b, void* y, float* mean,
                           float* rstd, int T, int H, float eps, int kind, cudaStream_t s) {
  if (H % 8 != 0 || H > 24576) {
    fm_set_error("norm_fwd: H must be a multiple of 8 and at most 24576");
    return -1;
  }
  using bf = __nv_bfloat16;
  fm::norm_fwd_kernel<<<T, fm::kNormThreads, (size_t)H * 2, s>>>(
      (const bf*)x, (const bf*)w, (const bf*)b, (bf*)y, mean, rstd, H, eps, kind);
  return check_launch("norm_fwd");
}

extern "C" int fm_norm_bwd_blocks(int T) { return T < 592 ? T : 592; }

extern "C" int fm_norm_bwd(const void* dy, const void* x, const void* w, const float* mean,
                           const float* rstd, const void* res_grad, void* dx, float* partial,
                           float* dw, float* db, int T, int H, int kind, cudaStream_t s) {
  if (H % 8 != 0 || H > 8 * fm::kNormBwdChunks * fm::kNormThreads) {
    fm_set_error("norm_bwd: H must be a multiple of 8 and at most 8192");
    return -1;
  }
  using bf = __nv_bfloat16;
  const int nb = fm_norm_bwd_blocks(T);
  const int nvec = H / 8;
  auto launch = [&](auto kernel) {
    kernel<<<nb, fm::kNormThreads, 0, s>>>((const bf*)dy, (const bf*)x, (const bf*)w, mean, rstd,
                                           (const bf*)res_grad, (bf*)dx, partial, T, H, kind);
  };
  if (nvec <= fm::kNormThreads) launch(fm::norm_bwd_kernel<1>);
  else if (nvec <= 2 * fm::kNormThreads) launch(fm::norm_bwd_kernel<2>);
  else launch(fm::norm_bwd_kernel<4>);
  int rc = check_launch("norm_bwd");
  if (rc) return rc;
  fm::norm_bwd_reduce_kernel<<<(2 * H + 31) / 32, 256, 0, s>>>(partial, dw, db, nb, H);
  return check_launch("norm_bwd_reduce");
}

extern "C" int fm_rope_packed(void* t, const float* freqs, long long rows, int heads_per_row,
                              int rope_heads, int d, int rot, int rows_per_pos, int backward,
                              cudaStream_t s) {
  if (rot % 16 != 0 || d % 8 != 0 || rot > d) {
    fm_set_error("rope: rot_dim must be a multiple of 16 and at most head_dim");
    return -1;
  }
  return fm_rope_packed_gated(t, freqs, rows, heads_per_row, rope_heads, d, rot, rows_per_pos, backward, nullptr,
                              0, 0, nullptr, 0, nullptr, s);
}

extern "C" int fm_rope_packed_gated(void* t, const float* freqs, long long rows, int heads_per_row,
                                    int rope_heads, int d, int rot, int rows_per_pos, int backward,
                                    const int* wait_flags, int wait_n, int wait_expected,
                                    unsigned long long* wait_ns, unsigned long long timeout_ns, int* status,
                                    cudaStream_t s) {
  if (rot % 16 != 0 || d % 8 != 0 || rot > d || wait_n > 256) {
    fm_set_error("rope: rot_dim must be a multiple of 16 and at most head_dim (and at most 256 sources)");
    return -1;
  }
  const long long total = rows * rope_heads * (rot / 16);
  fm::rope_packed_kernel<<<grid_for(total, 256), 256, 0, s>>>(
      (__nv_bfloat16*)t, freqs, rows, heads_per_row, rope_heads, d, rot, rows_per_pos, backward, wait_flags,
      wait_n, wait_expected, wait_ns, timeout_ns ? timeout_ns : 4000000000ull, status);
  return check_launch("rope_packed");
}

extern "C" int fm_topk_softmax(const float* logits, long long* idx, float* probs, int T, int E,
                               int k, cudaStream_t s) {
  if (k > 16 || k > E) {
    fm_set_error("topk_softmax: k must be at most 16 and at most the number of experts");
    return -1;
  }
  fm::topk_softmax_kernel<<<(T + 127) / 128, 128, 0, s>>>(logits, idx, probs, T, E, k);
  return check_launch("topk_softmax");
}

extern "C" int fm_gather_rows(const void* x, const long long* idx, void* out, long long rows, int H,
                              cudaStream_t s) {
  if (H % 8 != 0) {
    fm_set_error("gather_rows: H must be a multiple of 8");
    return -1;
  }
  fm::gather_rows_kernel<<<grid_for(rows, 8), 256, 0, s>>>((const __nv_bfloat16*)x, idx,
                                                          (__nv_bfloat16*)out, rows, H);
  return check_launch("gather_rows");
}

extern "C" int fm_unpermute_reduce(const void* rows, const int* slot, const void* residual,
                                   void* out, int T, int k, int H, cudaStream_t s) {
  if (H % 8 != 0 || k > 16) {
    fm_set_error("unpermute_reduce: H must be a multiple of 8 and k at most 16");
    return -1;
  }
  fm::unpermute_reduce_kernel<<<grid_for(T, 8), 256, 0, s>>>(
      (const __nv_bfloat16*)rows, slot, (const __nv_bfloat16*)residual, (__nv_bfloat16*)out, T, k,
      H, nullptr, 0, 0, nullptr, 0, nullptr);
  return check_launch("unpermute_reduce");
}

extern "C" int fm_unpermute_reduce_gated(const void* rows, const int* slot, const void* residual,
                                         void* out, int T, int k, int H, const int* wait_flags, int wait_n,
                                         int wait_expected, unsigned long long* wait_ns,
                                         unsigned long long timeout_ns, int* status, cudaStream_t s) {
  if (H % 8 != 0 || k > 16 || wait_n > 256) {
    fm_set_error("unpermute_reduce_gated: H must be a multiple of 8, k at most 16, at most 256 sources");
    return -1;
  }
  fm::unpermute_reduce_kernel<<<grid_for(T, 8), 256, 0, s>>>(
      (const __nv_bfloat16*)rows, slot, (const __nv_bfloat16*)residual, (__nv_bfloat16*)out, T, k,
      H, wait_flags, wait_n, wait_expected, wait_ns, timeout_ns ? timeout_ns : 4000000000ull, status);
  return check_launch("unpermute_reduce_gated");
}

extern "C" int fm_adam(void* p, float* master, float* g, void* m, void* v, long long n, float lr,
                       float beta1, float beta2, float eps, float weight_decay, int step,
                       float grad_scale, int zero_grad, int state_bf16, cudaStream_t s) {
  const float rbc1 = 1.f / (1.f - powf(beta1, (float)step));
  const float rbc2 = 1.f / (1.f - powf(beta2, (float)step));
  using bf = __nv_bfloat16;
  const bool aligned = ((reinterpret_cast<uintptr_t>(p) & 7) == 0) &&
                       ((reinterpret_cast<uintptr_t>(g) & 15) == 0) &&
                       ((reinterpret_cast<uintptr_t>(m) & 15) == 0) &&
                       ((reinterpret_cast<uintptr_t>(v) & 15) == 0) &&
                       (master == nullptr || (reinterpret_cast<uintptr_t>(master) & 15) == 0);
  const long long n4 = aligned ? n / 4 : 0;
  if (n4 > 0) {
    const int grid = grid_for(n4, 512, 148 * 8);
    if (state_bf16)
      fm::adam_kernel<bf><<<grid, 512, 0, s>>>((bf*)p, master, g, (bf*)m, (bf*)v, n4, lr, beta1, beta2,
                                              eps, weight_decay, rbc1, rbc2, grad_scale, zero_grad);
    else
      fm::adam_kernel<float><<<grid, 512, 0, s>>>((bf*)p, master, g, (float*)m, (float*)v, n4, lr,
                                                 beta1, beta2, eps, weight_decay, rbc1, rbc2,
                                                 grad_scale, zero_grad);
    int rc = check_launch("adam");
    if (rc) return rc;
  }
  const long long lo = n4 * 4;
  if (lo < n) {
    const int grid = (int)((n - lo + 255) / 256);
    if (state_bf16)
      fm::adam_tail_kernel<bf><<<grid, 256, 0, s>>>((bf*)p, master, g, (bf*)m, (bf*)v, lo, n, lr, beta1,
                                                   beta2, eps, weight_decay, rbc1, rbc2, grad_scale,
                                                   zero_grad);
    else
      fm::adam_tail_kernel<float><<<grid, 256, 0, s>>>((bf*)p, master, g, (float*)m, (float*)v, lo, n,
                                                      lr, beta1, beta2, eps, weight_decay, rbc1, rbc2,
                                                      grad_scale, zero_grad);
    return check_launch("adam_tail");
  }
  return 0;
}

extern "C" int fm_router_bwd(const float* dprobs_slots, const int* slot_of_token, const long long* top_idx,
                             const float* top_probs, const float* logits, const float* tpe, float aux_coef,
                             float z_coef, int T, int k, int E, float* dlogits, cudaStream_t s) {
  if (z_coef != 0.f && logits == nullptr) {
    fm_set_error("router_bwd: the z-loss term needs the logits");
    return -1;
  }
  fm::router_bwd_kernel<<<(T + 127) / 128, 128, 0, s>>>(dprobs_slots, slot_of_token, top_idx, top_probs, logits,
                                                       tpe, aux_coef, z_coef, T, k, E, dlogits);
  return check_launch("router_bwd");
}

extern "C" int fm_adam_background(void* p, const float* g, void* m, void* v, long long n, float lr, float beta1,
                                  float beta2, float eps, float weight_decay, int step, float grad_scale,
                                  int num_ctas, cudaStream_t s) {
  using bf = __nv_bfloat16;
  if ((n & 3) != 0 || (reinterpret_cast<uintptr_t>(p) & 7) || (reinterpret_cast<uintptr_t>(g) & 15) ||
      (reinterpret_cast<uintptr_t>(m) & 7) || (reinterpret_cast<uintptr_t>(v) & 7)) {
    fm_set_error("adam_background: needs a multiple of 4 elements and aligned pointers");
    return -1;
  }
  const float rbc1 = 1.f / (1.f - powf(beta1, (float)step));
  const float rbc2 = 1.f / (1.f - powf(beta2, (float)step));
  if (num_ctas <= 0) num_ctas = 148;
  fm::adam_background_kernel<<<num_ctas, 128, 0, s>>>((bf*)p, g, (bf*)m, (bf*)v, n / 4, lr, beta1, beta2, eps,
                                                     weight_decay, rbc1, rbc2, grad_scale);
  return check_launch("adam_background");
}

extern "C" int fm_moe_plan(const long long* top_idx, const float* top_probs, int T, int k, int E,
                           int cap, long long* sorted_indices, float* slot_probs, int* slot_of_token,
                           int* routed_per_expert, cudaStream_t s) {
  if (k > 16 || cap > T) {
    fm_set_error("moe_plan: k must be at most 16 and the capacity at most the number of tokens");
    return -1;
  }
  fm::moe_plan_kernel<<<E, fm::kPlanThreads, 0, s>>>(top_idx, top_probs, T, k, E, cap, sorted_indices,
                                                    slot_probs, slot_of_token, routed_per_expert);
  return check_launch("moe_plan");
}

extern "C" int fm_cross_entropy(void* logits, const long long* labels, float* loss_out, int T, int V,
                                float grad_scale, cudaStream_t s) {
  if ((reinterpret_cast<uintptr_t>(logits) & 15) != 0 || (V % 8) != 0) {
    fm_set_error("cross_entropy: logits must be 16-byte aligned with V a multiple of 8");
    return -1;
  }
  fm::cross_entropy_kernel<<<T, fm::kCeThreads, 0, s>>>((__nv_bfloat16*)logits, labels, loss_out, V,
                                                      grad_scale);
  return check_launch("cross_entropy");
}
