// Epilogues and host launcher of the tcgen05 GEMM (see gemm_sm100.cuh for the main loop).
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <map>
#include <mutex>
#include <utility>

#include "../include/fm_api.h"
#include "gemm_sm100.cuh"

namespace fm {

// ----------------------------------------------------------------------------------------
// helpers
// ----------------------------------------------------------------------------------------
__device__ __forceinline__ float gelu_f(float x) {
  return 0.5f * x * (1.0f + erff(x * 0.70710678118654752f));
}
__device__ __forceinline__ float dgelu_f(float x) {
  const float cdf = 0.5f * (1.0f + erff(x * 0.70710678118654752f));
  const float pdf = 0.3989422804014327f * __expf(-0.5f * x * x);
  return cdf + x * pdf;
}
// Hardware reciprocal (1 ulp): the epilogue warps are latency-bound and the result is rounded to bf16.
__device__ __forceinline__ float sigmoid_f(float x) { return __fdividef(1.0f, 1.0f + __expf(-x)); }
__device__ __forceinline__ float silu_f(float x) { return x * sigmoid_f(x); }
__device__ __forceinline__ float dsilu_f(float x) {
  const float s = sigmoid_f(x);
  return s * (1.0f + x * (1.0f - s));
}
__device__ __forceinline__ float act_f(int kind, float x) {
  return kind == FM_ACT_GELU ? gelu_f(x) : (kind == FM_ACT_SILU ? silu_f(x) : x);
}
__device__ __forceinline__ float dact_f(int kind, float x) {
  return kind == FM_ACT_GELU ? dgelu_f(x) : (kind == FM_ACT_SILU ? dsilu_f(x) : 1.0f);
}

__device__ __forceinline__ void load_acc(uint32_t taddr, float* v, bool zero) {
  if (zero) {
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = 0.f;
    return;
  }
  uint32_t r[32];
  tmem_ld_32x32(taddr, r);
  tmem_ld_wait();
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// Store 32 consecutive values of one row as bf16.  `ncols` = columns that exist (<= 32).
__device__ __forceinline__ void store_row_bf16(__nv_bfloat16* dst, const float* v, int ncols) {
  if (ncols >= 32 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint4 p;
      p.x = pack_bf16x2(v[8 * i + 0], v[8 * i + 1]);
      p.y = pack_bf16x2(v[8 * i + 2], v[8 * i + 3]);
      p.z = pack_bf16x2(v[8 * i + 4], v[8 * i + 5]);
      p.w = pack_bf16x2(v[8 * i + 6], v[8 * i + 7]);
      reinterpret_cast<uint4*>(dst)[i] = p;
    }
  } else {
    for (int i = 0; i < 32 && i < ncols; ++i) dst[i] = __float2bfloat16(v[i]);
  }
}
__device__ __forceinline__ void load_row_bf16(const __nv_bfloat16* src, float* v, int ncols) {
  if (ncols >= 32 && (reinterpret_cast<uintptr_t>(src) & 15) == 0) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint4 p = reinterpret_cast<const uint4*>(src)[i];
      const uint32_t w[4] = {p.x, p.y, p.z, p.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&w[j]);
        v[8 * i + 2 * j] = __low2float(b);
        v[8 * i + 2 * j + 1] = __high2float(b);
      }
    }
  } else {
    for (int i = 0; i < 32; ++i) v[i] = i < ncols ? __bfloat162float(src[i]) : 0.f;
  }
}

// ----------------------------------------------------------------------------------------
// Coalesced epilogue stores.  After tcgen05.ld every lane holds 32 consecutive columns of ONE
// row, so a direct store makes each warp instruction touch 32 different rows.  Instead the
// warp writes its 32 x 32 block to a padded shared-memory stage and reads it back so that a
// group of lanes covers one row segment contiguously: every global store instruction then
// writes whole 32-byte sectors (fp32: 8 lanes x 16 B per row, 4 rows per instruction; bf16:
// 4 lanes x 16 B per row, 8 rows per instruction).
// ----------------------------------------------------------------------------------------
constexpr int kStgLd = 36;  // floats per staged row (16-byte aligned, conflict-free)

__device__ __forceinline__ void stage_put(float* stg, int lane, const float* v) {
  __syncwarp();
#pragma unroll
  for (int i = 0; i < 8; ++i)
    *reinterpret_cast<float4*>(stg + lane * kStgLd + 4 * i) =
        make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
  __syncwarp();
}
// The inverse: rows were filled cooperatively, every lane takes its own row back.
__device__ __forceinline__ void stage_get(const float* stg, int lane, float* v) {
  __syncwarp();
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float4 x = *reinterpret_cast<const float4*>(stg + lane * kStgLd + 4 * i);
    v[4 * i] = x.x; v[4 * i + 1] = x.y; v[4 * i + 2] = x.z; v[4 * i + 3] = x.w;
  }
  __syncwarp();
}

// bf16 rows at base + rr * ld (rr = 0..rows_ok-1), 32 columns each; base 16-byte aligned, ld % 8 == 0.
__device__ __forceinline__ void staged_store_bf16(float* stg, int lane, const float* v, int rows_ok,
                                                  __nv_bfloat16* base, long long ld) {
  stage_put(stg, lane, v);
  const int sub = lane >> 2, c8 = (lane & 3) * 8;
#pragma unroll
  for (int pass = 0; pass < 4; ++pass) {
    const int rr = pass * 8 + sub;
    if (rr < rows_ok) {
      const float4 a = *reinterpret_cast<const float4*>(stg + rr * kStgLd + c8);
      const float4 b = *reinterpret_cast<const float4*>(stg + rr * kStgLd + c8 + 4);
      uint4 p;
      p.x = pack_bf16x2(a.x, a.y); p.y = pack_bf16x2(a.z, a.w);
      p.z = pack_bf16x2(b.x, b.y); p.w = pack_bf16x2(b.z, b.w);
      *reinterpret_cast<uint4*>(base + rr * ld + c8) = p;
    }
  }
}
// Same with an arbitrary destination per row: `my_row_ptr` is the destination of THIS lane's
// row (null = skip); the other lanes fetch it with a shuffle.
__device__ __forceinline__ void staged_store_bf16_scatter(float* stg, int lane, const float* v,
                                                          __nv_bfloat16* my_row_ptr) {
  stage_put(stg, lane, v);
  const int sub = lane >> 2, c8 = (lane & 3) * 8;
  const unsigned long long mine = reinterpret_cast<unsigned long long>(my_row_ptr);
#pragma unroll
  for (int pass = 0; pass < 4; ++pass) {
    const int rr = pass * 8 + sub;
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(__shfl_sync(0xffffffffu, mine, rr));
    if (dst != nullptr) {
      const float4 a = *reinterpret_cast<const float4*>(stg + rr * kStgLd + c8);
      const float4 b = *reinterpret_cast<const float4*>(stg + rr * kStgLd + c8 + 4);
      uint4 p;
      p.x = pack_bf16x2(a.x, a.y); p.y = pack_bf16x2(a.z, a.w);
      p.z = pack_bf16x2(b.x, b.y); p.w = pack_bf16x2(b.z, b.w);
      *reinterpret_cast<uint4*>(dst + c8) = p;
    }
  }
}
// fp32 rows, optional accumulate; base 16-byte aligned, ld % 4 == 0.
__device__ __forceinline__ void staged_store_f32(float* stg, int lane, const float* v, int rows_ok,
                                                 float* base, long long ld, bool accumulate) {
  stage_put(stg, lane, v);
  const int sub = lane >> 3, c4 = (lane & 7) * 4;
#pragma unroll
  for (int pass = 0; pass < 8; ++pass) {
    const int rr = pass * 4 + sub;
    if (rr < rows_ok) {
      float4 x = *reinterpret_cast<const float4*>(stg + rr * kStgLd + c4);
      float4* dst = reinterpret_cast<float4*>(base + rr * ld + c4);
      if (accumulate) {
        const float4 o = *dst;
        x.x += o.x; x.y += o.y; x.z += o.z; x.w += o.w;
      }
      *dst = x;
    }
  }
}
// Coalesced load of 32 bf16 rows x 32 columns into the stage; every lane then reads its row.
__device__ __forceinline__ void staged_load_bf16(float* stg, int lane, float* v, int rows_ok,
                                                 const __nv_bfloat16* base, long long ld) {
  __syncwarp();
  const int sub = lane >> 2, c8 = (lane & 3) * 8;
#pragma unroll
  for (int pass = 0; pass < 4; ++pass) {
    const int rr = pass * 8 + sub;
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;
    if (rr < rows_ok) {
      const uint4 p = *reinterpret_cast<const uint4*>(base + rr * ld + c8);
      const __nv_bfloat162 p0 = *reinterpret_cast<const __nv_bfloat162*>(&p.x);
      const __nv_bfloat162 p1 = *reinterpret_cast<const __nv_bfloat162*>(&p.y);
      const __nv_bfloat162 p2 = *reinterpret_cast<const __nv_bfloat162*>(&p.z);
      const __nv_bfloat162 p3 = *reinterpret_cast<const __nv_bfloat162*>(&p.w);
      a = make_float4(__low2float(p0), __high2float(p0), __low2float(p1), __high2float(p1));
      b = make_float4(__low2float(p2), __high2float(p2), __low2float(p3), __high2float(p3));
    }
    *reinterpret_cast<float4*>(stg + rr * kStgLd + c8) = a;
    *reinterpret_cast<float4*>(stg + rr * kStgLd + c8 + 4) = b;
  }
  stage_get(stg, lane, v);
}
__device__ __forceinline__ bool aligned16(const void* p) {
  return (reinterpret_cast<uintptr_t>(p) & 15) == 0;
}

// ----------------------------------------------------------------------------------------
// Epilogue 0: plain store (bf16 or fp32, optional accumulate; the fp32-accumulate form is the
// weight-gradient epilogue that adds straight into a flat gradient buffer).
// ----------------------------------------------------------------------------------------
struct EpiStore {
  void* C;
  long long ldc;
  long long group_stride;
  int out_fp32;
  int accumulate;
  float alpha;

  template <int BN>
  __device__ __forceinline__ void run(const Tile& t, const GemmArgs& a, uint32_t taddr, int r,
                                      bool zero, int chalf, float* stg) const {
    const int lane = r & 31;
    const long long row = a.mode == 0 ? (long long)t.row_base + t.m0 + r : (long long)t.m0 + r;
    const long long row0 = row - lane;   // first row of this warp
    const long long goff = a.mode == 0 ? 0 : (long long)t.g * group_stride;
    const bool row_ok = r < t.rows_valid;
    const int rows_ok = max(0, min(32, t.rows_valid - (r - lane)));
#pragma unroll 1
    for (int c = chalf * (BN / 64); c < (chalf + 1) * (BN / 64); ++c) {
      const int col = t.n_tile * BN + c * 32;
      if (col >= a.N) break;
      float v[32];
      load_acc(taddr + c * 32, v, zero);
      if (rows_ok == 0) continue;
      const int ncols = min(32, a.N - col);
      if (alpha != 1.0f) {
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] *= alpha;
      }
      if (out_fp32) {
        float* base = reinterpret_cast<float*>(C) + goff + row0 * ldc + col;
        if (ncols == 32 && (ldc & 3) == 0 && aligned16(base)) {
          staged_store_f32(stg, lane, v, rows_ok, base, ldc, accumulate != 0);
        } else if (row_ok) {
          float* dst = base + (long long)lane * ldc;
          for (int i = 0; i < ncols; ++i) dst[i] = accumulate ? dst[i] + v[i] : v[i];
        }
      } else {
        __nv_bfloat16* base = reinterpret_cast<__nv_bfloat16*>(C) + goff + row0 * ldc + col;
        if (ncols == 32 && (ldc & 7) == 0 && aligned16(base)) {
          if (accumulate) {
            float p[32];
            staged_load_bf16(stg, lane, p, rows_ok, base, ldc);
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] += p[i];
          }
          staged_store_bf16(stg, lane, v, rows_ok, base, ldc);
        } else if (row_ok) {
          __nv_bfloat16* dst = base + (long long)lane * ldc;
          if (accumulate) {
            float p[32];
            load_row_bf16(dst, p, ncols);
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] += p[i];
          }
          store_row_bf16(dst, v, ncols);
        }
      }
    }
  }
  __device__ __forceinline__ void tile_done(const Tile&, const GemmArgs&, int) const {}
};

// Store one 32 x 32 block of bf16 rows (consecutive rows, leading dimension ld), coalesced when
// the block is full-width and aligned, per-row otherwise.
__device__ __forceinline__ void put_block_bf16(float* stg, int lane, const float* v, int rows_ok,
                                               bool row_ok, __nv_bfloat16* base, long long ld, int ncols) {
  if (ncols == 32 && (ld & 7) == 0 && aligned16(base))
    staged_store_bf16(stg, lane, v, rows_ok, base, ld);
  else if (row_ok)
    store_row_bf16(base + (long long)lane * ld, v, ncols);
}
__device__ __forceinline__ void get_block_bf16(float* stg, int lane, float* v, int rows_ok, bool row_ok,
                                               const __nv_bfloat16* base, long long ld, int ncols) {
  if (ncols == 32 && (ld & 7) == 0 && aligned16(base)) {
    staged_load_bf16(stg, lane, v, rows_ok, base, ld);
  } else if (row_ok) {
    load_row_bf16(base + (long long)lane * ld, v, ncols);
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = 0.f;
  }
}

// ----------------------------------------------------------------------------------------
// Epilogue 5: optimizer in the weight-gradient epilogue.  The accumulator tile IS the gradient
// of the matching tile of a bf16 parameter; instead of storing it, the epilogue reads the
// parameter and its two bf16 Adam moments, applies the AdamW update and writes the three back
// (12 bytes of traffic per element instead of a 4-byte gradient store here plus a 16-byte
// optimizer pass later).  Only valid when the gradient is complete after this GEMM: a single
// micro-batch per step and no data-parallel reduction of this parameter.
// ----------------------------------------------------------------------------------------
struct EpiAdam {
  __nv_bfloat16* P;
  __nv_bfloat16* Mo;
  __nv_bfloat16* Vo;
  long long ld;
  long long group_stride;
  float alpha;   // gradient scale
  float lr, beta1, beta2, eps, weight_decay, rbc1, rbc2;

  // One AdamW step on 8 consecutive elements held as bf16 pairs.  The epilogue has only eight
  // warps per SM to hide latency with, so the square root and the division use the hardware
  // approximations (2 ulp; parameter and moments are rounded to bf16 right after).
  static __device__ __forceinline__ float sqrt_approx(float x) {
    float y;
    asm("sqrt.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
  }
  static __device__ __forceinline__ float rcp_approx(float x) {
    float y;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
  }
  // The arithmetic runs on packed fp32 pairs (fma.rn.f32x2 and friends, one issue slot per two
  // elements): the eight epilogue warps are bound by instruction issue and dependency latency, not
  // by the memory system, so halving the fp32 instruction count is what shortens the epilogue.
  __device__ __forceinline__ void update8(const float* gg, uint4& pw, uint4& pm, uint4& pv) const {
    uint32_t* ww = reinterpret_cast<uint32_t*>(&pw);
    uint32_t* wm = reinterpret_cast<uint32_t*>(&pm);
    uint32_t* wv = reinterpret_cast<uint32_t*>(&pv);
    const float c1 = (1.f - beta1) * alpha, c2 = (1.f - beta2) * alpha * alpha;
    const float step_m = lr * rbc1, decay = 1.f - lr * weight_decay;
    const float2 kB1 = make_float2(beta1, beta1), kB2 = make_float2(beta2, beta2);
    const float2 kC1 = make_float2(c1, c1), kC2 = make_float2(c2, c2);
    const float2 kR2 = make_float2(rbc2, rbc2), kEps = make_float2(eps, eps);
    const float2 kNs = make_float2(-step_m, -step_m), kDec = make_float2(decay, decay);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      // bf16 -> fp32 is a 16-bit shift of the bit pattern
      float2 w2 = make_float2(__uint_as_float(ww[q] << 16), __uint_as_float(ww[q] & 0xffff0000u));
      float2 m2 = make_float2(__uint_as_float(wm[q] << 16), __uint_as_float(wm[q] & 0xffff0000u));
      float2 v2 = make_float2(__uint_as_float(wv[q] << 16), __uint_as_float(wv[q] & 0xffff0000u));
      const float2 g2 = make_float2(gg[2 * q], gg[2 * q + 1]);
      m2 = __ffma2_rn(kB1, m2, __fmul2_rn(kC1, g2));
      v2 = __ffma2_rn(kB2, v2, __fmul2_rn(kC2, __fmul2_rn(g2, g2)));
      float2 s2 = __fmul2_rn(v2, kR2);
      s2.x = sqrt_approx(s2.x);
      s2.y = sqrt_approx(s2.y);
      s2 = __fadd2_rn(s2, kEps);
      const float2 r2 = make_float2(rcp_approx(s2.x), rcp_approx(s2.y));
      w2 = __ffma2_rn(__fmul2_rn(kNs, m2), r2, __fmul2_rn(kDec, w2));
      ww[q] = pack_bf16x2(w2.x, w2.y);
      wm[q] = pack_bf16x2(m2.x, m2.y);
      wv[q] = pack_bf16x2(v2.x, v2.y);
    }
  }

  static constexpr bool kPrefetch = true;
  // Called one tile ahead: pull this warp's part of parameter and moments (32 rows x BN/2
  // columns of three bf16 arrays) into L2 while the tensor core still works on the tile.
  template <int BN>
  __device__ __forceinline__ void prefetch(const Tile& t, const GemmArgs& a, int r, int chalf) const {
    const int lane = r & 31;
    if (r >= t.rows_valid) return;
    const long long row = a.mode == 0 ? (long long)t.row_base + t.m0 + r : (long long)t.m0 + r;
    const long long goff = a.mode == 0 ? 0 : (long long)t.g * group_stride;
    const int col0 = t.n_tile * BN + chalf * (BN / 2);
    const long long off = goff + row * ld + col0;
    (void)lane;
#pragma unroll
    for (int l = 0; l < BN / 2; l += 64) {     // 64 bf16 = one 128-byte line
      if (col0 + l >= a.N) break;
      asm volatile("prefetch.global.L2::evict_last [%0];" ::"l"(P + off + l));
      asm volatile("prefetch.global.L2::evict_last [%0];" ::"l"(Mo + off + l));
      asm volatile("prefetch.global.L2::evict_last [%0];" ::"l"(Vo + off + l));
    }
  }

  template <int BN>
  __device__ __forceinline__ void run(const Tile& t, const GemmArgs& a, uint32_t taddr, int r,
                                      bool zero, int chalf, float* stg) const {
    constexpr int NB = BN / 64;          // 32-column blocks handled by this warp
    const int lane = r & 31;
    const long long row = a.mode == 0 ? (long long)t.row_base + t.m0 + r : (long long)t.m0 + r;
    const long long row0 = row - lane;
    const long long goff = a.mode == 0 ? 0 : (long long)t.g * group_stride;
    const bool row_ok = r < t.rows_valid;
    const int rows_ok = max(0, min(32, t.rows_valid - (r - lane)));
    const int sub = lane >> 2, c8 = (lane & 3) * 8;
    const int c_begin = chalf * NB;
    const long long off0 = goff + row0 * ld + (long long)t.n_tile * BN;
    // coalesced path: whole 32-column blocks, 16-byte aligned rows (4 lanes x 16 bytes per row)
    const bool vec_ok = (ld & 7) == 0 && aligned16(P + off0) && aligned16(Mo + off0) && aligned16(Vo + off0);
#pragma unroll 1
    for (int k = 0; k < NB; ++k) {
      const int c = c_begin + k;
      const int col = t.n_tile * BN + c * 32;
      if (col >= a.N) break;
      const int ncols = min(32, a.N - col);
      const long long off = off0 + c * 32;
      const bool fast = vec_ok && ncols == 32;
      // parameter and moments do not depend on the accumulator: issue their loads first
      uint4 b[12];
      if (fast && rows_ok == 32) {
#pragma unroll
        for (int pass = 0; pass < 4; ++pass) {
          const long long o = off + (long long)(pass * 8 + sub) * ld + c8;
          b[pass * 3 + 0] = *reinterpret_cast<const uint4*>(P + o);
          b[pass * 3 + 1] = *reinterpret_cast<const uint4*>(Mo + o);
          b[pass * 3 + 2] = *reinterpret_cast<const uint4*>(Vo + o);
        }
      } else if (fast) {
#pragma unroll
        for (int pass = 0; pass < 4; ++pass) {
          const int rr = pass * 8 + sub;
          if (rr < rows_ok) {
            const long long o = off + (long long)rr * ld + c8;
            b[pass * 3 + 0] = *reinterpret_cast<const uint4*>(P + o);
            b[pass * 3 + 1] = *reinterpret_cast<const uint4*>(Mo + o);
            b[pass * 3 + 2] = *reinterpret_cast<const uint4*>(Vo + o);
          }
        }
      }
      float g[32];
      load_acc(taddr + c * 32, g, zero);
      if (rows_ok == 0) continue;
      if (fast && rows_ok == 32) {
        // all rows valid (the common case): branch-free, so that the 32 independent update chains
        // of the four passes can be interleaved by the scheduler
        stage_put(stg, lane, g);
        float gg[4][8];
#pragma unroll
        for (int pass = 0; pass < 4; ++pass) {
          const int rr = pass * 8 + sub;
          const float4 ga = *reinterpret_cast<const float4*>(stg + rr * kStgLd + c8);
          const float4 gb = *reinterpret_cast<const float4*>(stg + rr * kStgLd + c8 + 4);
          gg[pass][0] = ga.x; gg[pass][1] = ga.y; gg[pass][2] = ga.z; gg[pass][3] = ga.w;
          gg[pass][4] = gb.x; gg[pass][5] = gb.y; gg[pass][6] = gb.z; gg[pass][7] = gb.w;
        }
#pragma unroll
        for (int pass = 0; pass < 4; ++pass) update8(gg[pass], b[pass * 3 + 0], b[pass * 3 + 1], b[pass * 3 + 2]);
#pragma unroll
        for (int pass = 0; pass < 4; ++pass) {
          const long long o = off + (long long)(pass * 8 + sub) * ld + c8;
          *reinterpret_cast<uint4*>(Mo + o) = b[pass * 3 + 1];
          *reinterpret_cast<uint4*>(Vo + o) = b[pass * 3 + 2];
          *reinterpret_cast<uint4*>(P + o) = b[pass * 3 + 0];
        }
        __syncwarp();
      } else if (fast) {
        stage_put(stg, lane, g);
#pragma unroll
        for (int pass = 0; pass < 4; ++pass) {
          const int rr = pass * 8 + sub;
          if (rr < rows_ok) {
            const long long o = off + (long long)rr * ld + c8;
            const float4 ga = *reinterpret_cast<const float4*>(stg + rr * kStgLd + c8);
            const float4 gb = *reinterpret_cast<const float4*>(stg + rr * kStgLd + c8 + 4);
            const float gg[8] = {ga.x, ga.y, ga.z, ga.w, gb.x, gb.y, gb.z, gb.w};
            update8(gg, b[pass * 3 + 0], b[pass * 3 + 1], b[pass * 3 + 2]);
            *reinterpret_cast<uint4*>(Mo + o) = b[pass * 3 + 1];
            *reinterpret_cast<uint4*>(Vo + o) = b[pass * 3 + 2];
            *reinterpret_cast<uint4*>(P + o) = b[pass * 3 + 0];
          }
        }
        __syncwarp();
      } else if (row_ok) {
        const long long o = off + (long long)lane * ld;
        for (int i = 0; i < ncols; ++i) {
          const float gi = g[i] * alpha;
          float wi = __bfloat162float(P[o + i]);
          const float mi = beta1 * __bfloat162float(Mo[o + i]) + (1.f - beta1) * gi;
          const float vi = beta2 * __bfloat162float(Vo[o + i]) + (1.f - beta2) * gi * gi;
          wi -= lr * ((mi * rbc1) / (sqrtf(vi * rbc2) + eps) + weight_decay * wi);
          Mo[o + i] = __float2bfloat16(mi);
          Vo[o + i] = __float2bfloat16(vi);
          P[o + i] = __float2bfloat16(wi);
        }
      }
    }
  }
  __device__ __forceinline__ void tile_done(const Tile&, const GemmArgs&, int) const {}
};

// ----------------------------------------------------------------------------------------
// Epilogue 1: activation x routing probability (forward FC1).  Non-gated: out = act(x) * p.
// Gated (SwiGLU): the tile holds 128 gate columns then 128 up columns; out = silu(g) * u * p.
// Optionally keeps the pre-activation for the backward pass.
// Reference semantics: fluid/moe/forward.py:231-238,299,317 (probability applied between the
// activation and FC2).
// ----------------------------------------------------------------------------------------
struct EpiAct {
  __nv_bfloat16* act_out;
  long long ld_act;
  __nv_bfloat16* pre_out;
  long long ld_pre;
  const float* probs;
  int act_kind;

  template <int BN>
  __device__ __forceinline__ void run(const Tile& t, const GemmArgs& a, uint32_t taddr, int r,
                                      bool zero, int chalf, float* stg) const {
    const int lane = r & 31;
    const long long row = (long long)t.row_base + t.m0 + r;
    const long long row0 = row - lane;
    const bool row_ok = r < t.rows_valid;
    const int rows_ok = max(0, min(32, t.rows_valid - (r - lane)));
    const float p = (row_ok && probs) ? probs[row] : 1.0f;
    if (a.gated) {
      const int c_first = chalf * (BN / 128), c_last = (chalf + 1) * (BN / 128);
      __nv_bfloat16* act0 = act_out + row0 * ld_act;
      __nv_bfloat16* pre0 = pre_out ? pre_out + row0 * ld_pre : nullptr;
      if (rows_ok == 32 && t.n_tile * (BN / 2) + c_last * 32 <= a.N && ((ld_act | ld_pre | a.n_half) & 7) == 0 &&
          aligned16(act0) && aligned16(pre0)) {
        // Whole SwiGLU tile inside the matrix (the common case): the up half goes through the
        // shared-memory stage first and is kept in the coalesced layout (4 lanes x 8 columns per
        // row, 8 rows per pass), the gate half follows, and activation and both pre-activation
        // halves are computed and stored in that layout: two trips through the stage per block
        // instead of one per stored array.
        const int sub = lane >> 2, c8 = (lane & 3) * 8;
        float pr[4];
#pragma unroll
        for (int pass = 0; pass < 4; ++pass) pr[pass] = probs ? probs[row0 + pass * 8 + sub] : 1.0f;
#pragma unroll 1
        for (int c = c_first; c < c_last; ++c) {
          const int col = t.n_tile * (BN / 2) + c * 32;
          float ur[4][8];
          {
            float u[32];
            load_acc(taddr + BN / 2 + c * 32, u, zero);
            stage_put(stg, lane, u);
          }
#pragma unroll
          for (int pass = 0; pass < 4; ++pass) {
            const int rr = pass * 8 + sub;
            const float4 xa = *reinterpret_cast<const float4*>(stg + rr * kStgLd + c8);
            const float4 xb = *reinterpret_cast<const float4*>(stg + rr * kStgLd + c8 + 4);
            ur[pass][0] = xa.x; ur[pass][1] = xa.y; ur[pass][2] = xa.z; ur[pass][3] = xa.w;
            ur[pass][4] = xb.x; ur[pass][5] = xb.y; ur[pass][6] = xb.z; ur[pass][7] = xb.w;
            if (pre0) {
              uint4 q;
              q.x = pack_bf16x2(xa.x, xa.y); q.y = pack_bf16x2(xa.z, xa.w);
              q.z = pack_bf16x2(xb.x, xb.y); q.w = pack_bf16x2(xb.z, xb.w);
              *reinterpret_cast<uint4*>(pre0 + (long long)rr * ld_pre + a.n_half + col + c8) = q;
            }
          }
          {
            float g[32];
            load_acc(taddr + c * 32, g, zero);
            stage_put(stg, lane, g);
          }
#pragma unroll
          for (int pass = 0; pass < 4; ++pass) {
            const int rr = pass * 8 + sub;
            const float4 xa = *reinterpret_cast<const float4*>(stg + rr * kStgLd + c8);
            const float4 xb = *reinterpret_cast<const float4*>(stg + rr * kStgLd + c8 + 4);
            const float gv[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
            if (pre0) {
              uint4 q;
              q.x = pack_bf16x2(xa.x, xa.y); q.y = pack_bf16x2(xa.z, xa.w);
              q.z = pack_bf16x2(xb.x, xb.y); q.w = pack_bf16x2(xb.z, xb.w);
              *reinterpret_cast<uint4*>(pre0 + (long long)rr * ld_pre + col + c8) = q;
            }
            float o[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) o[i] = silu_f(gv[i]) * ur[pass][i] * pr[pass];
            uint4 q;
            q.x = pack_bf16x2(o[0], o[1]); q.y = pack_bf16x2(o[2], o[3]);
            q.z = pack_bf16x2(o[4], o[5]); q.w = pack_bf16x2(o[6], o[7]);
            *reinterpret_cast<uint4*>(act0 + (long long)rr * ld_act + col + c8) = q;
          }
        }
        __syncwarp();
        return;
      }
#pragma unroll 1
      for (int c = c_first; c < c_last; ++c) {
        const int col = t.n_tile * (BN / 2) + c * 32;
        if (col >= a.N) break;
        float g[32], u[32];
        load_acc(taddr + c * 32, g, zero);
        load_acc(taddr + BN / 2 + c * 32, u, zero);
        if (rows_ok == 0) continue;
        const int ncols = min(32, a.N - col);
        if (pre_out) {
          put_block_bf16(stg, lane, g, rows_ok, row_ok, pre_out + row0 * ld_pre + col, ld_pre, ncols);
          put_block_bf16(stg, lane, u, rows_ok, row_ok, pre_out + row0 * ld_pre + a.n_half + col, ld_pre, ncols);
        }
#pragma unroll
        for (int i = 0; i < 32; ++i) g[i] = silu_f(g[i]) * u[i] * p;
        put_block_bf16(stg, lane, g, rows_ok, row_ok, act_out + row0 * ld_act + col, ld_act, ncols);
      }
    } else {
      const int c_first = chalf * (BN / 64), c_last = (chalf + 1) * (BN / 64);
      __nv_bfloat16* act0 = act_out + row0 * ld_act;
      __nv_bfloat16* pre0 = pre_out ? pre_out + row0 * ld_pre : nullptr;
      if (rows_ok == 32 && t.n_tile * BN + c_last * 32 <= a.N && ((ld_act | ld_pre) & 7) == 0 && aligned16(act0) &&
          aligned16(pre0)) {
        // Whole tile inside the matrix: one trip through the stage per block, pre-activation and
        // activation are packed and stored from the coalesced layout.
        const int sub = lane >> 2, c8 = (lane & 3) * 8;
        float pr[4];
#pragma unroll
        for (int pass = 0; pass < 4; ++pass) pr[pass] = probs ? probs[row0 + pass * 8 + sub] : 1.0f;
#pragma unroll 1
        for (int c = c_first; c < c_last; ++c) {
          const int col = t.n_tile * BN + c * 32;
          {
            float v[32];
            load_acc(taddr + c * 32, v, zero);
            stage_put(stg, lane, v);
          }
#pragma unroll
          for (int pass = 0; pass < 4; ++pass) {
            const int rr = pass * 8 + sub;
            const float4 xa = *reinterpret_cast<const float4*>(stg + rr * kStgLd + c8);
            const float4 xb = *reinterpret_cast<const float4*>(stg + rr * kStgLd + c8 + 4);
            const float xv[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
            if (pre0) {
              uint4 q;
              q.x = pack_bf16x2(xa.x, xa.y); q.y = pack_bf16x2(xa.z, xa.w);
              q.z = pack_bf16x2(xb.x, xb.y); q.w = pack_bf16x2(xb.z, xb.w);
              *reinterpret_cast<uint4*>(pre0 + (long long)rr * ld_pre + col + c8) = q;
            }
            float o[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) o[i] = act_f(act_kind, xv[i]) * pr[pass];
            uint4 q;
            q.x = pack_bf16x2(o[0], o[1]); q.y = pack_bf16x2(o[2], o[3]);
            q.z = pack_bf16x2(o[4], o[5]); q.w = pack_bf16x2(o[6], o[7]);
            *reinterpret_cast<uint4*>(act0 + (long long)rr * ld_act + col + c8) = q;
          }
        }
        __syncwarp();
        return;
      }
#pragma unroll 1
      for (int c = c_first; c < c_last; ++c) {
        const int col = t.n_tile * BN + c * 32;
        if (col >= a.N) break;
        float v[32];
        load_acc(taddr + c * 32, v, zero);
        if (rows_ok == 0) continue;
        const int ncols = min(32, a.N - col);
        if (pre_out) put_block_bf16(stg, lane, v, rows_ok, row_ok, pre_out + row0 * ld_pre + col, ld_pre, ncols);
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = act_f(act_kind, v[i]) * p;
        put_block_bf16(stg, lane, v, rows_ok, row_ok, act_out + row0 * ld_act + col, ld_act, ncols);
      }
    }
  }
  __device__ __forceinline__ void tile_done(const Tile&, const GemmArgs&, int) const {}
};

// ----------------------------------------------------------------------------------------
// Epilogue 3: backward of (act x prob), fused after dActW = dY * W2^T.
//   a = act(pre); dprob_partial[row, n_tile, half] = sum_cols(acc * a); dpre = acc * p * act'(pre)
//   gated: a = silu(g) * u; dg = acc * p * u * silu'(g); du = acc * p * silu(g)
// Partial sums per N tile and per column half (two epilogue warps share a row) keep the
// probability gradient deterministic (no atomics): dprobs_partial is [rows, n_tiles, 2].
// Reference math: fluid/moe/backward.py:341-356,1046-1061.
// ----------------------------------------------------------------------------------------
struct EpiDAct {
  const __nv_bfloat16* pre_in;
  long long ld_pre_in;
  __nv_bfloat16* dpre;
  long long ld_dpre;
  const float* probs;
  float* dprobs_partial;  // [rows, n_tiles, 2]
  int n_tiles;
  int act_kind;
  int gated;   // activation is SwiGLU: pre_in / dpre hold [gate | up] halves `n_half` apart
  int n_half;

  static constexpr bool kPrefetch = true;
  // Called one tile ahead: pull this thread's row of the pre-activations (gate and up half of the
  // tile's columns) into L2 while the tensor core still works on the tile.
  template <int BN>
  __device__ __forceinline__ void prefetch(const Tile& t, const GemmArgs& a, int r, int chalf) const {
    if (r >= t.rows_valid) return;
    const int col0 = t.n_tile * BN + chalf * (BN / 2);
    const __nv_bfloat16* src = pre_in + ((long long)t.row_base + t.m0 + r) * ld_pre_in + col0;
#pragma unroll
    for (int l = 0; l < BN / 2; l += 64) {     // 64 bf16 = one 128-byte line
      if (col0 + l >= a.N) break;
      asm volatile("prefetch.global.L2 [%0];" ::"l"(src + l));
      if (gated) asm volatile("prefetch.global.L2 [%0];" ::"l"(src + n_half + l));
    }
  }

  template <int BN>
  __device__ __forceinline__ void run(const Tile& t, const GemmArgs& a, uint32_t taddr, int r,
                                      bool zero, int chalf, float* stg) const {
    const int lane = r & 31;
    const long long row = (long long)t.row_base + t.m0 + r;
    const long long row0 = row - lane;
    const bool row_ok = r < t.rows_valid;
    const int rows_ok = max(0, min(32, t.rows_valid - (r - lane)));
    const float p = (row_ok && probs) ? probs[row] : 1.0f;
    float dp = 0.f;
    const int c_first = chalf * (BN / 64), c_last = (chalf + 1) * (BN / 64);
    const __nv_bfloat16* pre0 = pre_in + row0 * ld_pre_in;
    __nv_bfloat16* dpre0 = dpre + row0 * ld_dpre;
    if (gated && rows_ok == 32 && t.n_tile * BN + c_last * 32 <= a.N && ((ld_pre_in | ld_dpre | n_half) & 7) == 0 &&
        aligned16(pre0) && aligned16(dpre0)) {
      // Whole SwiGLU tile inside the matrix (the common case).  Only the accumulator goes through
      // the shared-memory stage; gate and up pre-activations are read, and their gradients written,
      // in the coalesced layout (4 lanes x 16 bytes per row, 8 rows per pass), and all eight loads
      // of a block are issued before the accumulator is fetched, so their latency overlaps.  The
      // probability gradient is summed per (row, lane quad) and folded to one value per row at the end.
      const int sub = lane >> 2, c8 = (lane & 3) * 8;
      float pr[4], dq[4];
#pragma unroll
      for (int pass = 0; pass < 4; ++pass) {
        pr[pass] = probs ? probs[row0 + pass * 8 + sub] : 1.0f;
        dq[pass] = 0.f;
      }
#pragma unroll 1
      for (int c = c_first; c < c_last; ++c) {
        const int col = t.n_tile * BN + c * 32;
        uint4 rg[4], ru[4];
#pragma unroll
        for (int pass = 0; pass < 4; ++pass) {
          const long long o = (long long)(pass * 8 + sub) * ld_pre_in + col + c8;
          rg[pass] = *reinterpret_cast<const uint4*>(pre0 + o);
          ru[pass] = *reinterpret_cast<const uint4*>(pre0 + o + n_half);
        }
        {
          float v[32];
          load_acc(taddr + c * 32, v, zero);
          stage_put(stg, lane, v);
        }
#pragma unroll
        for (int pass = 0; pass < 4; ++pass) {
          const int rr = pass * 8 + sub;
          const float4 va = *reinterpret_cast<const float4*>(stg + rr * kStgLd + c8);
          const float4 vb = *reinterpret_cast<const float4*>(stg + rr * kStgLd + c8 + 4);
          const float vv[8] = {va.x, va.y, va.z, va.w, vb.x, vb.y, vb.z, vb.w};
          const uint32_t* wg = reinterpret_cast<const uint32_t*>(&rg[pass]);
          const uint32_t* wu = reinterpret_cast<const uint32_t*>(&ru[pass]);
          float og[8], ou[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            // bf16 -> fp32 is a 16-bit shift of the bit pattern
            const uint32_t gw = wg[i >> 1], uw = wu[i >> 1];
            const float gi = __uint_as_float((i & 1) ? (gw & 0xffff0000u) : (gw << 16));
            const float ui = __uint_as_float((i & 1) ? (uw & 0xffff0000u) : (uw << 16));
            const float sg = sigmoid_f(gi);
            const float sl = gi * sg;
            dq[pass] += vv[i] * sl * ui;
            const float da = vv[i] * pr[pass];
            og[i] = da * ui * (sg * (1.0f + gi * (1.0f - sg)));
            ou[i] = da * sl;
          }
          uint4 pg, pu;
          pg.x = pack_bf16x2(og[0], og[1]); pg.y = pack_bf16x2(og[2], og[3]);
          pg.z = pack_bf16x2(og[4], og[5]); pg.w = pack_bf16x2(og[6], og[7]);
          pu.x = pack_bf16x2(ou[0], ou[1]); pu.y = pack_bf16x2(ou[2], ou[3]);
          pu.z = pack_bf16x2(ou[4], ou[5]); pu.w = pack_bf16x2(ou[6], ou[7]);
          const long long o = (long long)rr * ld_dpre + col + c8;
          *reinterpret_cast<uint4*>(dpre0 + o) = pg;
          *reinterpret_cast<uint4*>(dpre0 + o + n_half) = pu;
        }
      }
      __syncwarp();
      // row pass * 8 + sub: sum over its four lanes, then hand every lane the sum of its own row
#pragma unroll
      for (int pass = 0; pass < 4; ++pass) {
        float x = dq[pass];
        x += __shfl_xor_sync(0xffffffffu, x, 1);
        x += __shfl_xor_sync(0xffffffffu, x, 2);
        x = __shfl_sync(0xffffffffu, x, (lane & 7) * 4);
        if ((lane >> 3) == pass) dp = x;
      }
      if (dprobs_partial) dprobs_partial[(row * n_tiles + t.n_tile) * 2 + chalf] = dp;
      return;
    }
    if (!gated && rows_ok == 32 && t.n_tile * BN + c_last * 32 <= a.N && ((ld_pre_in | ld_dpre) & 7) == 0 &&
        aligned16(pre0) && aligned16(dpre0)) {
      // The same for a plain activation (GELU, SiLU): one array in, one out.
      const int sub = lane >> 2, c8 = (lane & 3) * 8;
      float pr[4], dq[4];
#pragma unroll
      for (int pass = 0; pass < 4; ++pass) {
        pr[pass] = probs ? probs[row0 + pass * 8 + sub] : 1.0f;
        dq[pass] = 0.f;
      }
#pragma unroll 1
      for (int c = c_first; c < c_last; ++c) {
        const int col = t.n_tile * BN + c * 32;
        uint4 rx[4];
#pragma unroll
        for (int pass = 0; pass < 4; ++pass)
          rx[pass] = *reinterpret_cast<const uint4*>(pre0 + (long long)(pass * 8 + sub) * ld_pre_in + col + c8);
        {
          float v[32];
          load_acc(taddr + c * 32, v, zero);
          stage_put(stg, lane, v);
        }
#pragma unroll
        for (int pass = 0; pass < 4; ++pass) {
          const int rr = pass * 8 + sub;
          const float4 va = *reinterpret_cast<const float4*>(stg + rr * kStgLd + c8);
          const float4 vb = *reinterpret_cast<const float4*>(stg + rr * kStgLd + c8 + 4);
          const float vv[8] = {va.x, va.y, va.z, va.w, vb.x, vb.y, vb.z, vb.w};
          const uint32_t* wx = reinterpret_cast<const uint32_t*>(&rx[pass]);
          float o[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const uint32_t xw = wx[i >> 1];
            const float xi = __uint_as_float((i & 1) ? (xw & 0xffff0000u) : (xw << 16));
            dq[pass] += vv[i] * act_f(act_kind, xi);
            o[i] = vv[i] * pr[pass] * dact_f(act_kind, xi);
          }
          uint4 q;
          q.x = pack_bf16x2(o[0], o[1]); q.y = pack_bf16x2(o[2], o[3]);
          q.z = pack_bf16x2(o[4], o[5]); q.w = pack_bf16x2(o[6], o[7]);
          *reinterpret_cast<uint4*>(dpre0 + (long long)rr * ld_dpre + col + c8) = q;
        }
      }
      __syncwarp();
#pragma unroll
      for (int pass = 0; pass < 4; ++pass) {
        float x = dq[pass];
        x += __shfl_xor_sync(0xffffffffu, x, 1);
        x += __shfl_xor_sync(0xffffffffu, x, 2);
        x = __shfl_sync(0xffffffffu, x, (lane & 7) * 4);
        if ((lane >> 3) == pass) dp = x;
      }
      if (dprobs_partial) dprobs_partial[(row * n_tiles + t.n_tile) * 2 + chalf] = dp;
      return;
    }
#pragma unroll 1
    for (int c = c_first; c < c_last; ++c) {
      const int col = t.n_tile * BN + c * 32;
      if (col >= a.N) break;
      float v[32];
      load_acc(taddr + c * 32, v, zero);
      if (rows_ok == 0) continue;
      const int ncols = min(32, a.N - col);
      if (gated) {
        float g[32], u[32];
        get_block_bf16(stg, lane, g, rows_ok, row_ok, pre_in + row0 * ld_pre_in + col, ld_pre_in, ncols);
        get_block_bf16(stg, lane, u, rows_ok, row_ok, pre_in + row0 * ld_pre_in + n_half + col, ld_pre_in, ncols);
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float sg = sigmoid_f(g[i]);          // one sigmoid serves silu and its derivative
          const float s = g[i] * sg;
          dp += v[i] * s * u[i];
          const float da = v[i] * p;
          g[i] = da * u[i] * (sg * (1.0f + g[i] * (1.0f - sg)));
          u[i] = da * s;
        }
        put_block_bf16(stg, lane, g, rows_ok, row_ok, dpre + row0 * ld_dpre + col, ld_dpre, ncols);
        put_block_bf16(stg, lane, u, rows_ok, row_ok, dpre + row0 * ld_dpre + n_half + col, ld_dpre, ncols);
      } else {
        float x[32];
        get_block_bf16(stg, lane, x, rows_ok, row_ok, pre_in + row0 * ld_pre_in + col, ld_pre_in, ncols);
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          dp += v[i] * act_f(act_kind, x[i]);
          x[i] = v[i] * p * dact_f(act_kind, x[i]);
        }
        put_block_bf16(stg, lane, x, rows_ok, row_ok, dpre + row0 * ld_dpre + col, ld_dpre, ncols);
      }
    }
    if (row_ok && dprobs_partial) dprobs_partial[(row * n_tiles + t.n_tile) * 2 + chalf] = dp;
  }
  __device__ __forceinline__ void tile_done(const Tile&, const GemmArgs&, int) const {}
};

// ----------------------------------------------------------------------------------------
// Epilogue 2: scatter rows to their owners (FC2 + combine).  Row R of the result is written
// as bf16 to dst_base[dst_rank[R]] + dst_row[R] * ld_dst, which may be another GPU's buffer
// mapped over NVLink (plain 16-byte peer stores, 64 contiguous bytes per row per instruction
// group).  After a tile, each destination's arrival counter grows by the number of rows the
// tile sent it; the owner waits until its counter equals rows_expected * n_tiles * 2 (each of
// the two epilogue warps that share a row reports its half).  Replaces the combine all-to-all
// rounds of fluid/moe/forward.py:903-948.
// ----------------------------------------------------------------------------------------
struct EpiScatter {
  __nv_bfloat16* const* dst_base;
  const int* dst_rank;
  const int* dst_row;
  long long ld_dst;
  int* const* dst_flags;  // per destination rank: pointer to the counter this rank bumps
  int num_ranks;
  // One fp32 per row that rides along (the routing-probability gradient on the way back to the
  // token owner, which the reference sends through a separate small all-to-all,
  // fluid/layer/transformer.py:526-538): stored by the first column tile's first warp group,
  // before the release that publishes the row.
  const float* row_aux;
  float* const* row_aux_dst;

  template <int BN>
  __device__ __forceinline__ void run(const Tile& t, const GemmArgs& a, uint32_t taddr, int r,
                                      bool zero, int chalf, float* stg) const {
    const int lane = r & 31;
    const long long row = (long long)t.row_base + t.m0 + r;
    const bool row_ok = r < t.rows_valid;
    int rank = -1;
    long long drow = 0;
    if (row_ok) {
      rank = dst_rank[row];
      drow = dst_row[row];
    }
    if (row_aux != nullptr && t.n_tile == 0 && chalf == 0 && rank >= 0)
      row_aux_dst[rank][drow] = row_aux[row];
    __nv_bfloat16* base = rank >= 0 ? dst_base[rank] + drow * ld_dst : nullptr;
    const bool fast = (ld_dst & 7) == 0 &&
                      __all_sync(0xffffffffu, base == nullptr || aligned16(base));
#pragma unroll 1
    for (int c = chalf * (BN / 64); c < (chalf + 1) * (BN / 64); ++c) {
      const int col = t.n_tile * BN + c * 32;
      if (col >= a.N) break;
      float v[32];
      load_acc(taddr + c * 32, v, zero);
      const int ncols = min(32, a.N - col);
      if (fast && ncols == 32 && (col & 7) == 0) {
        staged_store_bf16_scatter(stg, lane, v, base ? base + col : nullptr);
      } else if (base != nullptr) {
        store_row_bf16(base + col, v, ncols);
      }
    }
    if (dst_flags != nullptr) __threadfence_system();
  }
  // Called by every epilogue thread after the tile's stores; `r` is the thread's row in the
  // tile.  Each warp aggregates its 32 rows by destination, so no cross-warp barrier is needed.
  __device__ __forceinline__ void tile_done(const Tile& t, const GemmArgs& a, int r) const {
    if (dst_flags == nullptr) return;
    const long long row = (long long)t.row_base + t.m0 + r;
    const int rank = r < t.rows_valid ? dst_rank[row] : -1;
    __syncwarp();
    const unsigned peers = __match_any_sync(0xffffffffu, rank);
    const int leader = __ffs(peers) - 1;
    if ((int)(threadIdx.x & 31) == leader && rank >= 0)
      flag_release_add(dst_flags[rank], __popc(peers));
  }
};

// ----------------------------------------------------------------------------------------
// Epilogue 4: scatter COLUMN blocks to their owners (QKV projection + SP->HP exchange, and
// out-projection input gradient + SP->HP).  Columns [p*cpr, (p+1)*cpr) of every result row
// belong to rank p; they are stored as bf16 into rank p's buffer at row (dst_row_offset + row),
// column (col - p*cpr), leading dimension dst_ld -- the position the all-to-all would have put
// them (fluid/core/comm.py:162-209).  Each warp adds the rows it delivered, once per 32-column
// chunk, to the destination's counter for this source; the owner waits for
// rows * (cpr / 32) per source.
// ----------------------------------------------------------------------------------------
struct EpiColScatter {
  __nv_bfloat16* const* dst_base;
  int cols_per_rank;
  long long dst_ld;
  long long dst_row_offset;
  int* const* dst_flags;

  template <int BN>
  __device__ __forceinline__ void run(const Tile& t, const GemmArgs& a, uint32_t taddr, int r,
                                      bool zero, int chalf, float* stg) const {
    const int lane = r & 31;
    const long long row0 = (long long)t.row_base + t.m0 + (r - lane);
    const bool row_ok = r < t.rows_valid;
    const int rows_ok = max(0, min(32, t.rows_valid - (r - lane)));
    int pend_rank = -1, pend_cnt = 0;
#pragma unroll 1
    for (int c = chalf * (BN / 64); c < (chalf + 1) * (BN / 64); ++c) {
      const int col = t.n_tile * BN + c * 32;
      if (col >= a.N) break;
      float v[32];
      load_acc(taddr + c * 32, v, zero);
      if (rows_ok == 0) continue;
      const int rank = col / cols_per_rank;
      const int cin = col - rank * cols_per_rank;
      __nv_bfloat16* base = dst_base[rank] + (dst_row_offset + row0) * dst_ld + cin;
      put_block_bf16(stg, lane, v, rows_ok, row_ok, base, dst_ld, min(32, a.N - col));
      if (rank != pend_rank) {
        if (pend_cnt > 0 && dst_flags != nullptr) {
          __threadfence_system();
          __syncwarp();
          if (lane == 0) flag_release_add(dst_flags[pend_rank], pend_cnt);
        }
        pend_rank = rank;
        pend_cnt = 0;
      }
      pend_cnt += rows_ok;
    }
    if (pend_cnt > 0 && dst_flags != nullptr) {
      __threadfence_system();
      __syncwarp();
      if (lane == 0) flag_release_add(dst_flags[pend_rank], pend_cnt);
    }
  }
  __device__ __forceinline__ void tile_done(const Tile&, const GemmArgs&, int) const {}
};

// ----------------------------------------------------------------------------------------
// host side
// ----------------------------------------------------------------------------------------
}  // namespace fm
extern "C" void fm_set_error(const char* msg);
namespace fm {
static void set_err(const char* msg) { fm_set_error(msg); }

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  if (fn) return fn;
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) !=
          cudaSuccess ||
      q != cudaDriverEntryPointSuccess)
    return nullptr;
  fn = reinterpret_cast<EncodeTiledFn>(p);
  return fn;
}

// 2-D bf16 tensor map, 128-byte swizzle, box = {64 inner, box_outer}.
static bool make_tmap(CUtensorMap* m, const void* ptr, long long inner, long long outer,
                      long long ld, int box_outer) {
  EncodeTiledFn enc = get_encode();
  if (!enc) {
    set_err("cuTensorMapEncodeTiled unavailable");
    return false;
  }
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) || ((ld * 2) & 15)) {
    set_err("TMA operand must be 16-byte aligned with a 16-byte-multiple row stride");
    return false;
  }
  cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)outer};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides,
                   box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    char buf[256];
    snprintf(buf, sizeof(buf), "cuTensorMapEncodeTiled failed: %d (inner=%lld outer=%lld ld=%lld)",
             (int)r, inner, outer, ld);
    set_err(buf);
    return false;
  }
  return true;
}

// 3-D view of an MN-major operand stored [outer, inner] (inner contiguous, a multiple of 64):
// dims {64, outer, inner / 64}; one box {64, 64 k-rows, nblk} lands as nblk slabs of [64 k][64 mn].
static bool make_tmap_mn3d(CUtensorMap* m, const void* ptr, long long inner, long long outer,
                           long long ld, int nblk) {
  EncodeTiledFn enc = get_encode();
  if (!enc) {
    set_err("cuTensorMapEncodeTiled unavailable");
    return false;
  }
  cuuint64_t dims[3] = {64, (cuuint64_t)outer, (cuuint64_t)(inner / 64)};
  cuuint64_t strides[2] = {(cuuint64_t)ld * 2, 128};
  cuuint32_t box[3] = {64, 64, (cuuint32_t)nblk};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides,
                   box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    char buf[256];
    snprintf(buf, sizeof(buf), "cuTensorMapEncodeTiled (3-D) failed: %d (inner=%lld outer=%lld ld=%lld)",
             (int)r, inner, outer, ld);
    set_err(buf);
    return false;
  }
  return true;
}

static int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  }
  return n;
}

template <bool A_MN, bool B_MN, int BN, class Epi, class Gate>
static int launch_one(const CUtensorMap& ta, const CUtensorMap& tb, const GemmArgs& args,
                      const Epi& epi, const Gate& gate, int grid, cudaStream_t stream) {
  auto kern = gemm_sm100_kernel<A_MN, B_MN, BN, Epi, Gate>;
  constexpr int smem = gemm_smem_bytes<BN>();
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) {
      set_err(cudaGetErrorString(e));
      return (int)e;
    }
    configured = true;
  }
  kern<<<grid, kGemmThreads, smem, stream>>>(ta, tb, args, epi, gate);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_err(cudaGetErrorString(e));
    return (int)e;
  }
  return 0;
}

// Workspace of the dynamic tile order, one per (device, stream): launches on one stream run one
// after another, so they can share claim counters (used in rotation; a launch zeroes the counter
// that comes up half a rotation later) and the log (entries carry the launch's epoch).  A stream
// that is being captured into a graph keeps the static order, because a replay would repeat the
// epoch of the capture.
struct SchedWorkspace {
  int* ctrs = nullptr;
  unsigned long long* log = nullptr;
  size_t log_entries = 0;
  unsigned int epoch = 0;
};
constexpr int kSchedCounters = 64;

static bool sched_dynamic_enabled() {
  static int on = -1;
  if (on < 0) {
    const char* e = getenv("FLUIDMOE_GEMM_DYNAMIC_TILES");
    on = (e == nullptr || e[0] != '0') ? 1 : 0;
  }
  return on == 1;
}

// Fills the scheduler fields of `args` for a launch of `pairs` CTA pairs over at most `tiles`
// tiles; leaves them empty (static order) when the dynamic order is off or cannot be used.
static void sched_prepare(GemmArgs& args, int pairs, long long tiles, cudaStream_t stream) {
  args.sched_ctr = nullptr;
  args.sched_ctr_reset = nullptr;
  args.sched_log = nullptr;
  args.sched_cap = 0;
  args.sched_epoch = 0;
  if (!sched_dynamic_enabled() || tiles <= pairs || tiles > (1ll << 24)) return;
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(stream, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) {
    (void)cudaGetLastError();
    return;
  }
  static std::mutex mu;
  static std::map<std::pair<int, cudaStream_t>, SchedWorkspace> table;
  int dev = 0;
  cudaGetDevice(&dev);
  std::lock_guard<std::mutex> lock(mu);
  SchedWorkspace& ws = table[std::make_pair(dev, stream)];
  if (ws.ctrs == nullptr) {
    if (cudaMalloc(&ws.ctrs, kSchedCounters * sizeof(int)) != cudaSuccess) {
      (void)cudaGetLastError();
      ws.ctrs = nullptr;
      return;
    }
    cudaMemsetAsync(ws.ctrs, 0, kSchedCounters * sizeof(int), stream);
  }
  // A pair can claim every tile but the other pairs' first ones, and one claim past the end.
  const size_t cap_per_pair = (size_t)(tiles + 2);
  const size_t need = cap_per_pair * (size_t)pairs;
  if (need * sizeof(unsigned long long) > ((size_t)64 << 20)) return;   // very many tiles: static order
  if (need > ws.log_entries) {
    // The old log may still be read by a launch in flight on this stream: it is not freed (logs
    // only grow a few times, while the largest problem of a model is met for the first time).
    unsigned long long* fresh = nullptr;
    if (cudaMalloc(&fresh, need * sizeof(unsigned long long)) != cudaSuccess) {
      (void)cudaGetLastError();
      return;
    }
    cudaMemsetAsync(fresh, 0, need * sizeof(unsigned long long), stream);
    ws.log = fresh;
    ws.log_entries = need;
  }
  if (++ws.epoch == 0) ws.epoch = 1;
  args.sched_ctr = ws.ctrs + ws.epoch % kSchedCounters;
  args.sched_ctr_reset = ws.ctrs + (ws.epoch + kSchedCounters / 2) % kSchedCounters;
  args.sched_log = ws.log;
  args.sched_cap = (int)cap_per_pair;
  args.sched_epoch = ws.epoch;
}

template <bool A_MN, bool B_MN, class Epi, class Gate>
static int launch_pair(const CUtensorMap& ta, const CUtensorMap& tb, const GemmArgs& args_in,
                       const Epi& epi, const Gate& gate, int grid, cudaStream_t stream) {
  auto kern = gemm2_sm100_kernel<A_MN, B_MN, Epi, Gate>;
  constexpr int smem = gemm2_smem_bytes();
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) {
      set_err(cudaGetErrorString(e));
      return (int)e;
    }
    configured = true;
  }
  // The kernel is persistent: never launch more pairs than can be resident at once (pairs must
  // sit on two SMs of one GPC, so this can be fewer than SMs / 2).
  static int max_pairs = 0;
  if (max_pairs == 0) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(sm_count() & ~1);
    cfg.blockDim = dim3(kGemmThreads);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) {
      (void)cudaGetLastError();
      n = sm_count() / 2 - 2;
    }
    max_pairs = n;
  }
  grid &= ~1;   // whole CTA pairs
  if (grid > 2 * max_pairs) grid = 2 * max_pairs;
  if (grid < 2) grid = 2;
  GemmArgs args = args_in;
  sched_prepare(args, grid / 2, args_in.sched_cap, stream);   // sched_cap arrives as the tile bound
  kern<<<grid, kGemmThreads, smem, stream>>>(ta, tb, args, epi, gate);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_err(cudaGetErrorString(e));
    return (int)e;
  }
  return 0;
}

template <class Epi, class Gate>
static int dispatch_shape(const FmGemmDesc* d, const CUtensorMap& ta, const CUtensorMap& tb,
                          const GemmArgs& args, const Epi& epi, const Gate& gate, int grid,
                          cudaStream_t s) {
  const bool amn = d->a_mn != 0, bmn = d->b_mn != 0;
  if (d->cta_pair && d->bn == 256) {
    if (!amn && !bmn) return launch_pair<false, false>(ta, tb, args, epi, gate, grid, s);
    if (!amn && bmn) return launch_pair<false, true>(ta, tb, args, epi, gate, grid, s);
    if (amn && bmn) return launch_pair<true, true>(ta, tb, args, epi, gate, grid, s);
  }
  if (d->bn == 256) {
    if (!amn && !bmn) return launch_one<false, false, 256>(ta, tb, args, epi, gate, grid, s);
    if (!amn && bmn) return launch_one<false, true, 256>(ta, tb, args, epi, gate, grid, s);
    if (amn && bmn) return launch_one<true, true, 256>(ta, tb, args, epi, gate, grid, s);
  } else if (d->bn == 128) {
    if (!amn && !bmn) return launch_one<false, false, 128>(ta, tb, args, epi, gate, grid, s);
    if (!amn && bmn) return launch_one<false, true, 128>(ta, tb, args, epi, gate, grid, s);
    if (amn && bmn) return launch_one<true, true, 128>(ta, tb, args, epi, gate, grid, s);
  }
  set_err("unsupported operand-major / tile combination");
  return -2;
}

template <class Epi>
static int dispatch_gate(const FmGemmDesc* d, const CUtensorMap& ta, const CUtensorMap& tb,
                         const GemmArgs& args, const Epi& epi, int grid, cudaStream_t s) {
  if (d->gate_flags != nullptr && d->gate_k_blocks_per_src > 0) {
    GateKSource g{d->gate_flags, d->gate_k_blocks_per_src, d->gate_blocks_per_group,
                  d->gate_expected > 0 ? d->gate_expected : 1};
    return dispatch_shape(d, ta, tb, args, epi, g, grid, s);
  }
  if (d->gate_flags != nullptr) {
    GateRowBlockFlags g{d->gate_flags, d->gate_group_base, d->gate_blocks_per_group,
                        d->gate_expected};
    return dispatch_shape(d, ta, tb, args, epi, g, grid, s);
  }
  return dispatch_shape(d, ta, tb, args, epi, GateNone{}, grid, s);
}

}  // namespace fm


extern "C" int fm_gemm_launch(const FmGemmDesc* d, cudaStream_t stream) {
  using namespace fm;
  if (d->bn != 128 && d->bn != 256) {
    set_err("bn must be 128 or 256");
    return -1;
  }
  if (d->gated && d->bn != 256) {
    set_err("gated tiles need bn == 256");
    return -1;
  }
  if (d->mode == 1 && !(d->a_mn && d->b_mn)) {
    set_err("grouped-K mode needs both operands stored [rows, M] / [rows, N]");
    return -1;
  }
  if (d->gated && d->n_half % 8 != 0) {
    set_err("gated layout needs the up half to start at a multiple of 8 columns");
    return -1;
  }
  if (d->mode == 0 && d->K % 8 != 0) {
    set_err("K must be a multiple of 8");
    return -1;
  }
  if (d->mode == 0 && d->num_groups > 1 && d->K % kBK != 0) {
    set_err("grouped GEMM needs K to be a multiple of 64");
    return -1;
  }
  CUtensorMap ta, tb;
  // One 3-D box per MN-major tile when every tile starts on a 64-element boundary of a
  // 64-multiple inner extent; otherwise 64-wide 2-D boxes.
  const bool a3 = d->a_mn && d->a_inner % 64 == 0 && (d->mode == 1 || d->group_offs == nullptr) &&
                  (d->mode == 1 || d->uniform_rows % 64 == 0);
  const bool b3 = d->b_mn && d->b_inner % 64 == 0 && (!d->gated || d->n_half % 64 == 0);
  const bool mn3d = (!d->a_mn || a3) && (!d->b_mn || b3) && (d->a_mn || d->b_mn) &&
                    ((uintptr_t)d->A % 16 == 0) && ((uintptr_t)d->B % 16 == 0) && d->lda % 8 == 0 &&
                    d->ldb % 8 == 0;
  // The CTA-pair kernel fetches MN-major operands only through 3-D boxes.
  FmGemmDesc dd = *d;
  if (dd.cta_pair && (dd.bn != 256 || ((dd.a_mn || dd.b_mn) && !mn3d) || (dd.mode == 0 && dd.a_mn)))
    dd.cta_pair = 0;
  d = &dd;
  // A: K-major -> box {64 k, 128 rows}; MN-major -> box {64 rows, 64 k}
  if (d->a_mn && mn3d) {
    if (!make_tmap_mn3d(&ta, d->A, d->a_inner, d->a_outer, d->lda, kBM / 64)) return -3;
  } else if (!make_tmap(&ta, d->A, d->a_inner, d->a_outer, d->lda, d->a_mn ? 64 : 128)) {
    return -3;
  }
  // B: K-major -> box {64 k, 128 n}; MN-major -> box {64 n, 64 k}
  if (d->b_mn && mn3d) {
    if (!make_tmap_mn3d(&tb, d->B, d->b_inner, d->b_outer, d->ldb,
                        (d->gated || d->cta_pair) ? d->bn / 128 : d->bn / 64))
      return -3;
  } else if (!make_tmap(&tb, d->B, d->b_inner, d->b_outer, d->ldb, d->b_mn ? 64 : 128)) {
    return -3;
  }

  GemmArgs args;
  memset(&args, 0, sizeof(args));
  args.mode = d->mode;
  args.num_groups = d->num_groups;
  args.M = d->M;
  args.N = d->N;
  args.K = d->K;
  args.uniform_rows = d->uniform_rows;
  args.group_rows = d->group_rows;
  args.group_offs = d->group_offs;
  args.group_b = d->group_b;
  args.b_group_stride = d->b_group_stride;
  args.gated = d->gated;
  args.n_half = d->n_half;
  args.swizzle_m = d->swizzle_m;
  args.mn3d = mn3d ? 1 : 0;
  args.n_rotate = d->n_rotate;
  args.k_rotate = d->k_rotate;
  args.timeout_ns = d->timeout_ns ? d->timeout_ns : 4000000000ull;
  args.status = d->status;
  args.wait_ns = d->wait_ns;

  int grid = sm_count();
  if (d->max_ctas > 0 && d->max_ctas < grid) grid = d->max_ctas;
  // Do not launch more CTAs than tiles when the tile count is known on the host.
  {
    const int npt = d->gated ? d->bn / 2 : d->bn;
    const long long nt = (d->N + npt - 1) / npt;
    const int tm = d->cta_pair ? 2 * kBM : kBM;
    if (d->group_rows == nullptr) {
      const long long mt = d->mode == 0 ? (d->uniform_rows + tm - 1) / tm : (d->M + tm - 1) / tm;
      const long long tiles = nt * mt * d->num_groups * (d->cta_pair ? 2 : 1);
      if (tiles < grid) grid = (int)(tiles > 0 ? tiles : 1);
    }
    // Upper bound of the tile count for the dynamic tile order of the CTA-pair kernel (the launcher
    // replaces it by the log's row length).  With row counts in device memory the rows of A bound it.
    long long bound;
    if (d->mode == 1)
      bound = nt * ((d->M + tm - 1) / tm) * d->num_groups;
    else if (d->group_rows == nullptr)
      bound = nt * ((d->uniform_rows + tm - 1) / tm) * d->num_groups;
    else
      bound = nt * (d->a_outer / tm + d->num_groups);
    args.sched_cap = (int)(bound < (1ll << 30) ? bound : 0);
  }

  switch (d->epi) {
    case FM_EPI_STORE: {
      EpiStore e{d->C, d->ldc, d->c_group_stride, d->out_fp32, d->accumulate,
                 d->alpha == 0.f ? 1.0f : d->alpha};
      return dispatch_gate(d, ta, tb, args, e, grid, stream);
    }
    case FM_EPI_ACT: {
      EpiAct e{reinterpret_cast<__nv_bfloat16*>(d->act_out), d->ld_act,
               reinterpret_cast<__nv_bfloat16*>(d->pre_out), d->ld_pre, d->probs, d->act_kind};
      return dispatch_gate(d, ta, tb, args, e, grid, stream);
    }
    case FM_EPI_DACT: {
      const int nt = (d->N + d->bn - 1) / d->bn;
      EpiDAct e{reinterpret_cast<const __nv_bfloat16*>(d->pre_in), d->ld_pre_in,
                reinterpret_cast<__nv_bfloat16*>(d->C), d->ldc, d->probs, d->dprobs, nt,
                d->act_kind, d->gated, d->n_half};
      args.gated = 0;  // here `gated` describes the activation, not the layout of B
      return dispatch_gate(d, ta, tb, args, e, grid, stream);
    }
    case FM_EPI_SCATTER: {
      EpiScatter e{reinterpret_cast<__nv_bfloat16* const*>(d->dst_base), d->dst_rank, d->dst_row,
                   d->ld_dst, d->dst_flags, d->num_ranks, d->row_aux, d->row_aux_dst};
      return dispatch_gate(d, ta, tb, args, e, grid, stream);
    }
    case FM_EPI_COLSCATTER: {
      if (d->cols_per_rank <= 0 || d->cols_per_rank % 32 != 0) {
        set_err("column scatter needs cols_per_rank to be a positive multiple of 32");
        return -1;
      }
      EpiColScatter e{reinterpret_cast<__nv_bfloat16* const*>(d->dst_base), d->cols_per_rank, d->ld_dst,
                      d->dst_row_offset, d->dst_flags};
      return dispatch_gate(d, ta, tb, args, e, grid, stream);
    }
    case FM_EPI_ADAM: {
      if (d->adam_p == nullptr || d->adam_m == nullptr || d->adam_v == nullptr) {
        set_err("optimizer epilogue needs parameter and moment pointers");
        return -1;
      }
      EpiAdam e{reinterpret_cast<__nv_bfloat16*>(d->adam_p), reinterpret_cast<__nv_bfloat16*>(d->adam_m),
                reinterpret_cast<__nv_bfloat16*>(d->adam_v), d->ldc, d->c_group_stride,
                d->alpha == 0.f ? 1.0f : d->alpha, d->adam_lr, d->adam_beta1, d->adam_beta2, d->adam_eps,
                d->adam_wd, d->adam_rbc1, d->adam_rbc2};
      return dispatch_shape(d, ta, tb, args, e, GateNone{}, grid, stream);
    }
    default:
      set_err("unknown epilogue");
      return -1;
  }
}
