// Causal grouped-query flash attention (forward) on tcgen05 / TMEM, head dim 128.
//
// One CTA owns a 128-row query tile of one head.  Warp 0 streams K and V blocks of 128
// positions through a two-stage shared-memory ring with TMA; warp 1 issues S = Q K^T and
// O_j = P_j V_j with accumulators in TMEM; warps 2-5 (one thread per query row, which is the
// natural TMEM layout: no cross-thread reductions) run the online softmax: they read S from
// TMEM, keep the running max / sum, write P (bf16) into shared memory in the 128-byte-swizzled
// K-major layout the MMA expects, and fold each finished O_j into a register accumulator with
// the usual rescale.  Only the log-sum-exp is kept for the backward pass.
//
// Q, K and V are read in place from the packed projection buffer
// [s, b, G, (q_per_group + 2) * d] (query heads, key head, value head of every KV group), so no
// split / transpose copies are made.  The reference calls PyTorch SDPA or Transformer Engine
// here (fluid/attention/forward.py:280-329).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cstdio>
#include <cstdlib>
#include <type_traits>
#include <vector>
#include <math.h>
#include <stdio.h>

#include "../include/fm_ops.h"
#include "../include/sm100_ptx.cuh"

extern "C" void fm_set_error(const char* msg);

namespace fm {

constexpr int kFaD = 128;
constexpr int kFaBM = 128;   // query rows per CTA
constexpr int kFaBN = 128;   // key/value positions per block
constexpr int kFaThreads = 192;
constexpr int kKernelIdFlashFwd = 20;
constexpr int kTileBytes = 128 * 128 * 2;  // one [128, 128] bf16 tile = two 64-wide K blocks

struct FlashFwdArgs {
  int s, b, G, qpg;
  float scale_log2;      // softmax scale * log2(e)
  __nv_bfloat16* out;    // [s, b, G*qpg, d]
  float* lse;            // [b, G*qpg, s]
  unsigned long long timeout_ns;
  int* status;
  long long* prof;       // developer builds (FM_FLASH_PROFILE): per-CTA cycle counters, else null
  const __nv_bfloat16* qkv;   // packed projection buffer (third-generation kernel reads Q rows itself)
  long long row_stride;       // elements between consecutive sequence positions
  // Optional HP -> SP exchange in the epilogue (batch 1, 128 | rows per rank): every output row is
  // also stored into the `attn_in` buffer of the rank that owns its sequence position, at this
  // rank's head columns, and the owner's arrival counter of the row's 128-row block and of this
  // source is raised by the number of rows written (once per warp and head).
  __nv_bfloat16* const* push_dst;   // [P] peers' attn_in [rows per rank, P * heads * d], or null
  int* const* push_flags;           // [P] peers' counters [P * row_blocks]
  int push_me, push_P, push_sl, push_row_blocks;
};

// Cycle counters of one softmax thread and of the MMA thread, per CTA (developer builds only).
#ifdef FM_FLASH_PROFILE
#define FA_PROF_NOW() clock64()
#define FA_PROF_ADD(acc, t0) acc += clock64() - (t0)
// event trace of CTA 0, key blocks [8, 24): slot (j - 8) * 16 + k behind the per-CTA counters
#define FA_TRACE(a, j, k)                                                             \
  do {                                                                                \
    if ((a).prof != nullptr && blockIdx.x == 0 && (j) >= 8 && (j) < 24)               \
      (a).prof[(long long)gridDim.x * 16 + ((j) - 8) * 16 + (k)] = clock64();         \
  } while (0)
#else
#define FA_PROF_NOW() 0ll
#define FA_PROF_ADD(acc, t0) (void)(t0)
#define FA_TRACE(a, j, k) (void)0
#endif

__global__ void __launch_bounds__(kFaThreads, 1)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tmap, const FlashFwdArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = smem + kTileBytes;          // 2 stages
  uint8_t* sV = smem + 3 * kTileBytes;      // 2 stages
  uint8_t* sP = smem + 5 * kTileBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 6 * kTileBytes);
  uint64_t* q_full = bars;            // [1]
  uint64_t* k_full = bars + 1;        // [2]
  uint64_t* v_full = bars + 3;        // [2]
  uint64_t* k_empty = bars + 5;       // [2]
  uint64_t* v_empty = bars + 7;       // [2]
  uint64_t* s_full = bars + 9;        // [1]
  uint64_t* p_full = bars + 10;       // [1]
  uint64_t* o_full = bars + 11;       // [1]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 12);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nq = (a.s + kFaBM - 1) / kFaBM;
  const int qt = nq - 1 - (int)blockIdx.x;  // longest rows first
  const int h = blockIdx.y, bb = blockIdx.z;
  const int g = h / a.qpg, hi = h % a.qpg;
  const int heads_per_group = a.qpg + 2;
  const int col_q = ((bb * a.G + g) * heads_per_group + hi) * kFaD;
  const int col_k = ((bb * a.G + g) * heads_per_group + a.qpg) * kFaD;
  const int col_v = col_k + kFaD;
  const int q0 = qt * kFaBM;
  const int nblocks = min(qt + 1, (a.s + kFaBN - 1) / kFaBN);  // causal: blocks 0 .. qt
  const uint64_t timeout = a.timeout_ns;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_empty[i], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(p_full, 4);
    mbar_init(o_full, 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 256);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_s = tmem_base;         // S: columns [0, 128)
  const uint32_t tmem_o = tmem_base + 128;   // O_j: columns [128, 256)

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(q_full, kTileBytes);
      tma_load_2d(sQ, &tmap, q_full, col_q, q0);
      tma_load_2d(sQ + kTileBytes / 2, &tmap, q_full, col_q + 64, q0);
      for (int j = 0; j < nblocks; ++j) {
        const int st = j & 1;
        const uint32_t ph = ((j >> 1) & 1) ^ 1;
        if (!mbar_wait(&k_empty[st], ph, timeout, abort_flag)) {
          report_status(a.status, kStatusMbarTimeout, kKernelIdFlashFwd, 100 + st, 0, 0);
          break;
        }
        mbar_expect_tx(&k_full[st], kTileBytes);
        tma_load_2d(sK + st * kTileBytes, &tmap, &k_full[st], col_k, j * kFaBN);
        tma_load_2d(sK + st * kTileBytes + kTileBytes / 2, &tmap, &k_full[st], col_k + 64, j * kFaBN);
        if (!mbar_wait(&v_empty[st], ph, timeout, abort_flag)) {
          report_status(a.status, kStatusMbarTimeout, kKernelIdFlashFwd, 110 + st, 0, 0);
          break;
        }
        mbar_expect_tx(&v_full[st], kTileBytes);
        tma_load_2d(sV + st * kTileBytes, &tmap, &v_full[st], col_v, j * kFaBN);
        tma_load_2d(sV + st * kTileBytes + kTileBytes / 2, &tmap, &v_full[st], col_v + 64, j * kFaBN);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_qk = umma_idesc_bf16(128, 128, false, false);
      constexpr uint32_t idesc_pv = umma_idesc_bf16(128, 128, false, true);
      const uint32_t q_addr = smem_u32(sQ), p_addr = smem_u32(sP);
      bool ok = mbar_wait(q_full, 0, timeout, abort_flag);
      if (!ok) report_status(a.status, kStatusMbarTimeout, kKernelIdFlashFwd, 200, 0, 0);
      for (int j = 0; ok && j < nblocks; ++j) {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        // S_j = Q K_j^T  (the S buffer is free: P_{j-1} was published after S_{j-1} was read)
        if (!mbar_wait(&k_full[st], ph, timeout, abort_flag)) {
          report_status(a.status, kStatusMbarTimeout, kKernelIdFlashFwd, 210 + st, 0, 0);
          break;
        }
        tc_fence_after_sync();
        const uint32_t k_addr = smem_u32(sK + st * kTileBytes);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t off = (kk >> 2) * (kTileBytes / 2) + (kk & 3) * 32;
          umma_bf16(tmem_s, umma_smem_desc(q_addr + off, 0, 1024),
                    umma_smem_desc(k_addr + off, 0, 1024), idesc_qk, kk > 0 ? 1u : 0u);
        }
        umma_commit(&k_empty[st]);
        umma_commit(s_full);
        // O_j = P_j V_j once the softmax warps have published P_j
        if (!mbar_wait(p_full, j & 1, timeout, abort_flag)) {
          report_status(a.status, kStatusMbarTimeout, kKernelIdFlashFwd, 220, 0, 0);
          break;
        }
        if (!mbar_wait(&v_full[st], ph, timeout, abort_flag)) {
          report_status(a.status, kStatusMbarTimeout, kKernelIdFlashFwd, 230 + st, 0, 0);
          break;
        }
        tc_fence_after_sync();
        const uint32_t v_addr = smem_u32(sV + st * kTileBytes);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t poff = (kk >> 2) * (kTileBytes / 2) + (kk & 3) * 32;
          umma_bf16(tmem_o, umma_smem_desc(p_addr + poff, 0, 1024),
                    umma_smem_desc(v_addr + kk * 2048, kTileBytes / 2, 1024), idesc_pv,
                    kk > 0 ? 1u : 0u);
        }
        umma_commit(&v_empty[st]);
        umma_commit(o_full);
      }
    }
  } else {
    // ------------------------------- softmax warps -------------------------------
    const int q = warp & 3;
    const int r = q * 32 + lane;        // row inside the tile == TMEM lane
    const int row = q0 + r;             // query position
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    float o_acc[kFaD];
#pragma unroll
    for (int i = 0; i < kFaD; ++i) o_acc[i] = 0.f;
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    for (int j = 0; j < nblocks; ++j) {
      if (!mbar_wait(s_full, j & 1, timeout, abort_flag)) {
        if (lane == 0) report_status(a.status, kStatusMbarTimeout, kKernelIdFlashFwd, 300, 0, 0);
        ok = false;
        break;
      }
      tc_fence_after_sync();
      if (j > 0) {
        // fold O_{j-1} (its MMAs were issued before S_j's, so they have completed)
        if (!mbar_wait(o_full, (j - 1) & 1, timeout, abort_flag)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
#pragma unroll
        for (int c = 0; c < kFaD / 32; ++c) {
          uint32_t v[32];
          tmem_ld_32x32(tmem_o + lane_addr + c * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o_acc[c * 32 + i] += __uint_as_float(v[i]);
        }
      }
      const bool diag = (j == qt);
      const int kv0 = j * kFaBN;
      // pass 1: row maximum of the scaled scores
      float m_blk = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < kFaBN / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(tmem_s + lane_addr + c * 32, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int col = kv0 + c * 32 + i;
          const bool masked = (diag && col > row) || col >= a.s;
          const float x = masked ? -INFINITY : __uint_as_float(v[i]) * a.scale_log2;
          m_blk = fmaxf(m_blk, x);
        }
      }
      const float m_new = fmaxf(m_run, m_blk);
      const float m_use = m_new == -INFINITY ? 0.f : m_new;
      const float alpha = exp2f(m_run - m_use);   // exp2(-inf) = 0 on the first block
      // pass 2: probabilities -> shared memory (bf16, swizzled K-major), row sum
      float l_blk = 0.f;
#pragma unroll 1
      for (int c = 0; c < kFaBN / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(tmem_s + lane_addr + c * 32, v);
        tmem_ld_wait();
        float p[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int col = kv0 + c * 32 + i;
          const bool masked = (diag && col > row) || col >= a.s;
          p[i] = masked ? 0.f : exp2f(__uint_as_float(v[i]) * a.scale_log2 - m_use);
          l_blk += p[i];
        }
        // columns [c*32, c*32+32) of row r: K block kb = c / 2, 16-byte chunks (c & 1) * 4 + 0..3
        uint8_t* rowp = sP + (c >> 1) * (kTileBytes / 2) + r * 128;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
          const int chunk = ((c & 1) * 4 + w) ^ (r & 7);
          uint4 pk;
          pk.x = pack_bf16x2(p[8 * w + 0], p[8 * w + 1]);
          pk.y = pack_bf16x2(p[8 * w + 2], p[8 * w + 3]);
          pk.z = pack_bf16x2(p[8 * w + 4], p[8 * w + 5]);
          pk.w = pack_bf16x2(p[8 * w + 6], p[8 * w + 7]);
          *reinterpret_cast<uint4*>(rowp + chunk * 16) = pk;
        }
      }
      l_run = l_run * alpha + l_blk;
      m_run = m_new;
#pragma unroll
      for (int i = 0; i < kFaD; ++i) o_acc[i] *= alpha;
      // publish P_j: generic-proxy writes -> async proxy, TMEM reads done
      fence_proxy_async_smem();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    if (ok && nblocks > 0) {
      if (mbar_wait(o_full, (nblocks - 1) & 1, timeout, abort_flag)) {
        tc_fence_after_sync();
#pragma unroll
        for (int c = 0; c < kFaD / 32; ++c) {
          uint32_t v[32];
          tmem_ld_32x32(tmem_o + lane_addr + c * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o_acc[c * 32 + i] += __uint_as_float(v[i]);
        }
        if (row < a.s) {
          const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
          const int hq = a.G * a.qpg;
          __nv_bfloat16* dst = a.out + (((long long)row * a.b + bb) * hq + h) * kFaD;
#pragma unroll
          for (int w = 0; w < kFaD / 8; ++w) {
            uint4 pk;
            pk.x = pack_bf16x2(o_acc[8 * w + 0] * inv, o_acc[8 * w + 1] * inv);
            pk.y = pack_bf16x2(o_acc[8 * w + 2] * inv, o_acc[8 * w + 3] * inv);
            pk.z = pack_bf16x2(o_acc[8 * w + 4] * inv, o_acc[8 * w + 5] * inv);
            pk.w = pack_bf16x2(o_acc[8 * w + 6] * inv, o_acc[8 * w + 7] * inv);
            reinterpret_cast<uint4*>(dst)[w] = pk;
          }
          a.lse[((long long)bb * hq + h) * a.s + row] =
              (m_run + log2f(l_run)) * 0.6931471805599453f;
        }
      }
    }
    tc_fence_before_sync();
  }

  if (*abort_flag) {
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 256);
  }
}

// =========================================================================================
// Second-generation forward: one CTA owns TWO consecutive 128-row query tiles of a head and
// ping-pongs between them.  While the softmax warps of one tile work on their score block, the
// tensor core runs P.V of the other tile and the next Q.K^T, so MMA and softmax overlap.
// The probability block is written back to TMEM over the score block (bf16, two values per
// 32-bit column) and P.V takes its A operand from TMEM, which frees the shared memory that
// staged P before and lets K/V blocks (shared by both tiles) be double buffered.  The output
// accumulates in TMEM across key blocks; it is rescaled only when the running row maximum grows
// by more than 2^8 (otherwise the stale maximum stays in use, which is exact after the final
// division by the row sum).
// =========================================================================================
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// 2^x on the FMA pipe: x = j + f with j = rint(x), f in [-0.5, 0.5]; 2^f by a cubic (relative
// error 7.5e-5, far below bf16 resolution), 2^j by adding j to the exponent field.  The
// special-function unit delivers 16 ex2 per clock and SM, which for head dim 128 is as many
// clocks per key block as the tensor core needs for the two products; moving a share of the
// exponentials here takes the unit off the critical path.
__device__ __forceinline__ float poly_exp2(float x) {
  constexpr float kMagic = 12582912.0f;   // 1.5 * 2^23: adding it leaves rint(x) in the low mantissa bits
  x = fmaxf(x, -126.0f);
  const float t = x + kMagic;
  const float f = x - (t - kMagic);
  float p = fmaf(f, 0.055171649903059006f, 0.2426111251115799f);
  p = fmaf(p, f, 0.6932609677314758f);
  p = fmaf(p, f, 0.9999280571937561f);
  return __int_as_float(__float_as_int(p) + (__float_as_int(t) << 23));
}

__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

constexpr int kFa2Threads = 320;   // TMA warp, MMA warp, 4 + 4 softmax warps
constexpr int kKernelIdFlashFwd2 = 21;
constexpr int kFa2DefaultPoly = 7;    // index into the launcher's table: uniform issue, P handed over in two parts

// kPoly: of every four value pairs, how many take their exponential from poly_exp2x2.
// kUniform: the whole MMA warp walks the issue loop and one elected lane issues, so that the
// compiler can keep descriptors and loop state in the warp's uniform registers.
// kPParts (1, 2 or 4): the softmax hands P over in that many parts of 128 / kPParts keys and the
// k-steps of P.V that read a part are issued as soon as it is there, so that they overlap the
// exponentials of the later parts (the tile's softmax and its two products sit in series).
template <int kPoly, bool kUniform = false, int kPParts = 1>
__global__ void __launch_bounds__(kFa2Threads, 1)
flash_fwd2_kernel(const __grid_constant__ CUtensorMap tmap, const FlashFwdArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;                      // 2 tiles
  uint8_t* sK = smem + 2 * kTileBytes;     // 2 stages
  uint8_t* sV = smem + 4 * kTileBytes;     // 2 stages
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 6 * kTileBytes);
  uint64_t* q_full = bars;           // [2]
  uint64_t* k_full = bars + 2;       // [2]
  uint64_t* v_full = bars + 4;       // [2]
  uint64_t* k_empty = bars + 6;      // [2]
  uint64_t* v_empty = bars + 8;      // [2]
  uint64_t* s_full = bars + 10;      // [2] per tile
  uint64_t* p_full = bars + 12;      // [2]
  uint64_t* o_full = bars + 14;      // [2]
  uint64_t* p_part = bars + 18;      // [2][3] parts 0 .. kPParts-2 of P (the last part is p_full)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nq = (a.s + kFaBM - 1) / kFaBM;
  const int npairs = (nq + 1) / 2;
  // One-dimensional grid ordered by work: every (head, batch) of the longest tile pair comes
  // first, the shortest pairs last, so that the hardware's in-order CTA dispatch is a
  // longest-job-first schedule over the whole launch (a causal tile pair p costs 4p + 3 blocks).
  // Neighbouring CTAs are the query heads of one KV group: they share K/V in L2.
  const int hq_all = a.G * a.qpg;
  const int per_pair = hq_all * a.b;
  const int pair = npairs - 1 - (int)blockIdx.x / per_pair;
  const int rem_lin = (int)blockIdx.x % per_pair;
  const int h = rem_lin % hq_all, bb = rem_lin / hq_all;
  const int g = h / a.qpg, hi = h % a.qpg;
  const int heads_per_group = a.qpg + 2;
  const int col_q = ((bb * a.G + g) * heads_per_group + hi) * kFaD;
  const int col_k = ((bb * a.G + g) * heads_per_group + a.qpg) * kFaD;
  const int col_v = col_k + kFaD;
  const int nkv = (a.s + kFaBN - 1) / kFaBN;
  int nblk[2];
  nblk[0] = min(2 * pair + 1, nkv);
  nblk[1] = (2 * pair + 1 < nq) ? min(2 * pair + 2, nkv) : 0;
  const int nmax = max(nblk[0], nblk[1]);
  const uint64_t timeout = a.timeout_ns;

  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&q_full[i], 1);
      mbar_init(&k_full[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[i], 4);
      for (int c = 0; c < 3; ++c) mbar_init(&p_part[i * 3 + c], 4);
      mbar_init(&o_full[i], 1);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      for (int w = 0; w < 2; ++w) {
        if (nblk[w] == 0) continue;
        const int q0 = (2 * pair + w) * kFaBM;
        mbar_expect_tx(&q_full[w], kTileBytes);
        tma_load_2d(sQ + w * kTileBytes, &tmap, &q_full[w], col_q, q0);
        tma_load_2d(sQ + w * kTileBytes + kTileBytes / 2, &tmap, &q_full[w], col_q + 64, q0);
      }
      for (int j = 0; j < nmax; ++j) {
        const int st = j & 1;
        const uint32_t ph = ((j >> 1) & 1) ^ 1;
        if (!mbar_wait(&k_empty[st], ph, timeout, abort_flag)) {
          report_status(a.status, kStatusMbarTimeout, kKernelIdFlashFwd2, 100 + st, 0, 0);
          break;
        }
        mbar_expect_tx(&k_full[st], kTileBytes);
        tma_load_2d(sK + st * kTileBytes, &tmap, &k_full[st], col_k, j * kFaBN);
        tma_load_2d(sK + st * kTileBytes + kTileBytes / 2, &tmap, &k_full[st], col_k + 64, j * kFaBN);
        if (!mbar_wait(&v_empty[st], ph, timeout, abort_flag)) {
          report_status(a.status, kStatusMbarTimeout, kKernelIdFlashFwd2, 110 + st, 0, 0);
          break;
        }
        mbar_expect_tx(&v_full[st], kTileBytes);
        tma_load_2d(sV + st * kTileBytes, &tmap, &v_full[st], col_v, j * kFaBN);
        tma_load_2d(sV + st * kTileBytes + kTileBytes / 2, &tmap, &v_full[st], col_v + 64, j * kFaBN);
      }
    }
  } else if (warp == 1) {
    if (kUniform || lane == 0) {
      constexpr uint32_t idesc_qk = umma_idesc_bf16(128, 128, false, false);
      constexpr uint32_t idesc_pv = umma_idesc_bf16(128, 128, false, true);
      bool ok = true;
      // Every operand descriptor of the loop, complete, in registers: the issuing thread shares
      // its scheduler with two busy softmax warps and gets an issue slot only every 15 to 20
      // cycles, so each extra instruction per MMA (an address add, a register-pair move) shows
      // up in the tensor pipe's idle time.  The loop below is specialised on the tile and on
      // the K/V stage so that every index into these arrays is a compile-time constant.
      constexpr uint32_t kDescHi = umma_desc_hi(1024);
      uint64_t qd[2][8], kd[2][8], vd[2][8];
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        uint32_t lo[8];
        umma_lo_k_major(smem_u32(sQ + t * kTileBytes), kTileBytes / 2, lo);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) qd[t][kk] = umma_desc_join(lo[kk], kDescHi);
        umma_lo_k_major(smem_u32(sK + t * kTileBytes), kTileBytes / 2, lo);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) kd[t][kk] = umma_desc_join(lo[kk], kDescHi);
        umma_lo_mn_major(smem_u32(sV + t * kTileBytes), kTileBytes / 2, lo);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) vd[t][kk] = umma_desc_join(lo[kk], kDescHi);
      }
      auto issue_qk = [&](auto w_c, auto st_c) {          // S_w = Q_w K(stage)^T
        constexpr int W = decltype(w_c)::value, ST = decltype(st_c)::value;
        const uint32_t d = tmem_base + W * 128;
        if (!kUniform || elect_one()) {
          umma_bf16(d, qd[W][0], kd[ST][0], idesc_qk, 0u);
#pragma unroll
          for (int kk = 1; kk < 8; ++kk) umma_bf16_acc(d, qd[W][kk], kd[ST][kk], idesc_qk);
          umma_commit(&s_full[W]);
        }
        if (kUniform) __syncwarp();
      };
      // k-steps [k0, k1) of O_w (+)= P_w V(stage); the last call (k1 == 8) commits
      auto issue_pv = [&](auto w_c, auto st_c, uint32_t first_acc, int k0, int k1) {
        constexpr int W = decltype(w_c)::value, ST = decltype(st_c)::value;
        const uint32_t d = tmem_base + 256 + W * 128, pa = tmem_base + W * 128;
        if (!kUniform || elect_one()) {
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            if (kk < k0 || kk >= k1) continue;
            if (kk == 0) umma_bf16_ts(d, pa, vd[ST][0], idesc_pv, first_acc);
            else umma_bf16_ts_acc(d, pa + kk * 8, vd[ST][kk], idesc_pv);
          }
          if (k1 == 8) umma_commit(&o_full[W]);
        }
        if (kUniform) __syncwarp();
      };
      auto wait_or_fail = [&](uint64_t* bar, uint32_t parity, int what) {
        if (mbar_wait(bar, parity, timeout, abort_flag)) return true;
        report_status(a.status, kStatusMbarTimeout, kKernelIdFlashFwd2, what, 0, 0);
        return false;
      };
      using I0 = std::integral_constant<int, 0>;
      using I1 = std::integral_constant<int, 1>;
      [[maybe_unused]] long long pm_total = FA_PROF_NOW(), pm_wait_p = 0, pm_wait_kv = 0;
      // prologue: S_w(0) for both tiles
      for (int w = 0; ok && w < 2; ++w)
        if (nblk[w] > 0) ok = wait_or_fail(&q_full[w], 0, 200 + w);
      if (ok && nmax > 0) ok = wait_or_fail(&k_full[0], 0, 210);
      if (ok) {
        tc_fence_after_sync();
        if (nblk[0] > 0) issue_qk(I0{}, I0{});
        if (nblk[1] > 0) issue_qk(I1{}, I0{});
        if (!kUniform || elect_one()) umma_commit(&k_empty[0]);
      }
      // one key block of both tiles, K/V stage ST (compile time)
      auto step = [&](auto st_c, int j) {
        constexpr int ST = decltype(st_c)::value;
        using SN = std::integral_constant<int, ST ^ 1>;
        const uint32_t ph = (j >> 1) & 1;
        [[maybe_unused]] long long t0 = FA_PROF_NOW();
        if (!wait_or_fail(&v_full[ST], ph, 230 + ST)) return false;
        FA_PROF_ADD(pm_wait_kv, t0);
        bool k_next_ready = false;
        auto tile = [&](auto w_c) {
          constexpr int W = decltype(w_c)::value;
          if (j >= nblk[W]) return true;
          t0 = FA_PROF_NOW();
          FA_TRACE(a, j, W * 8 + 0);                    // MMA thread starts waiting for P_w(j)
          constexpr int kStepsPerPart = 8 / kPParts;
#pragma unroll
          for (int part = 0; part + 1 < kPParts; ++part) {
            if (!wait_or_fail(&p_part[W * 3 + part], j & 1, 225 + W)) return false;
            tc_fence_after_sync();
            issue_pv(w_c, st_c, j > 0 ? 1u : 0u, part * kStepsPerPart, (part + 1) * kStepsPerPart);
          }
          if (!wait_or_fail(&p_full[W], j & 1, 220 + W)) return false;
          FA_PROF_ADD(pm_wait_p, t0);
          FA_TRACE(a, j, W * 8 + 1);                    // ... has it
          tc_fence_after_sync();
          issue_pv(w_c, st_c, j > 0 ? 1u : 0u, 8 - kStepsPerPart, 8);
          FA_TRACE(a, j, W * 8 + 2);                    // P.V issued
          if (j + 1 < nblk[W]) {
            if (!k_next_ready) {
              t0 = FA_PROF_NOW();
              if (!wait_or_fail(&k_full[ST ^ 1], ((j + 1) >> 1) & 1, 240)) return false;
              FA_PROF_ADD(pm_wait_kv, t0);
              tc_fence_after_sync();
              k_next_ready = true;
            }
            issue_qk(w_c, SN{});
            FA_TRACE(a, j, W * 8 + 3);                  // Q.K^T of the next block issued
          }
          return true;
        };
        if (!tile(I0{})) return false;
        if (!tile(I1{})) return false;
        if (!kUniform || elect_one()) {
          umma_commit(&v_empty[ST]);
          if (j + 1 < nmax) umma_commit(&k_empty[ST ^ 1]);
        }
        return true;
      };
      for (int j = 0; ok && j < nmax; ++j) ok = (j & 1) ? step(I1{}, j) : step(I0{}, j);
#ifdef FM_FLASH_PROFILE
      if (a.prof != nullptr && lane == 0) {
        long long* pr = a.prof + (long long)blockIdx.x * 16;
        pr[0] = clock64() - pm_total;
        pr[1] = pm_wait_p;
        pr[2] = pm_wait_kv;
        pr[3] = nblk[0] + nblk[1];
      }
#endif
    }
  } else {
    // ------------------------------- softmax warps -------------------------------
    // One thread per query row; the row's 128 scores of a key block stay in registers.
    const int sw = warp - 2;
    const int w = sw >> 2;               // which query tile this warp owns
    const int q = warp & 3;              // TMEM lane quarter
    const int r = q * 32 + lane;
    const int qt = 2 * pair + w;
    const int row = qt * kFaBM + r;
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    const uint32_t t_s = tmem_base + w * 128 + lane_addr;          // S (fp32) / P (packed bf16)
    const uint32_t t_o = tmem_base + 256 + w * 128 + lane_addr;    // O accumulator
    const int nb = nblk[w];
    float m_used = -INFINITY, l_run = 0.f;
    bool ok = true;
    [[maybe_unused]] long long ps_total = FA_PROF_NOW(), ps_wait = 0, ps_max = 0, ps_exp = 0, ps_resc = 0;
    for (int j = 0; j < nb; ++j) {
      [[maybe_unused]] long long t0 = FA_PROF_NOW();
      if (!__all_sync(0xffffffffu, mbar_wait(&s_full[w], j & 1, timeout, abort_flag))) {
        if (lane == 0) report_status(a.status, kStatusMbarTimeout, kKernelIdFlashFwd2, 300 + w, 0, 0);
        ok = false;
        break;
      }
      tc_fence_after_sync();
      FA_PROF_ADD(ps_wait, t0);
      if (lane == 0 && q == 2 % 4) FA_TRACE(a, j, w * 8 + 4);      // softmax has S_w(j)
      t0 = FA_PROF_NOW();
      const int kv0 = j * kFaBN;
      // only the diagonal block and a ragged last block need masking
      const bool diag = (j == qt);
      const bool masked = diag || kv0 + kFaBN > a.s;
      auto mask_chunk = [&](uint32_t* v, int c) {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int col = kv0 + c * 32 + i;
          if ((diag && col > row) || col >= a.s) v[i] = 0xff800000u;   // -inf
        }
      };
      // The whole score row (128 values) is kept in registers: one TMEM read per block.
      uint32_t sv[4][32];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld_32x32(t_s + c * 32, sv[c]);
      tmem_ld_wait();
      if (masked) {
#pragma unroll
        for (int c = 0; c < 4; ++c) mask_chunk(sv[c], c);
      }
      // row maximum: eight independent chains of three-input maxima
      float mx[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) mx[k] = -INFINITY;
#pragma unroll
      for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int i = 0; i < 16; ++i)
          mx[i & 7] = fmax3(mx[i & 7], __uint_as_float(sv[c][2 * i]), __uint_as_float(sv[c][2 * i + 1]));
      const float m_raw = fmaxf(fmax3(mx[0], mx[1], mx[2]), fmax3(fmax3(mx[3], mx[4], mx[5]), mx[6], mx[7]));
      const float m_blk = m_raw * a.scale_log2;   // scale > 0
      FA_PROF_ADD(ps_max, t0);
      if (lane == 0 && q == 2 % 4) FA_TRACE(a, j, w * 8 + 5);      // maximum done
      t0 = FA_PROF_NOW();
      // Lazy rescale: keep the old reference maximum unless the new one is more than 2^8 above it.
      const float m_new = fmaxf(m_used, m_blk);
      const bool first = (j == 0);
      const bool grow = !first && (m_new > m_used + 8.0f);
      if (first) m_used = (m_new == -INFINITY) ? 0.f : m_new;
      if (__any_sync(0xffffffffu, grow)) {
        // O holds the sum of blocks 0..j-1; P.V of block j-1 must have finished before it is touched.
        if (!__all_sync(0xffffffffu, mbar_wait(&o_full[w], (j - 1) & 1, timeout, abort_flag))) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const float f = grow ? exp2f(m_used - m_new) : 1.0f;
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t v[32];
          tmem_ld_32x32(t_o + c * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * f);
          tmem_st_32x32(t_o + c * 32, v);
        }
        tmem_st_wait();
        if (grow) {
          l_run *= f;
          m_used = m_new;
        }
      }
      FA_PROF_ADD(ps_resc, t0);
      t0 = FA_PROF_NOW();
      // Exponentials: of every four values, kPoly take the polynomial on the FMA pipe, the others
      // the special-function unit, so that the two pipes work side by side.  Scalar arithmetic on
      // purpose: the packed two-value instructions only run on one of the two FMA pipes.
      float l_part[8];                            // independent partial row sums
#pragma unroll
      for (int k = 0; k < 8; ++k) l_part[k] = 0.f;
      const float sc = a.scale_log2, neg_m = -m_used;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float x0 = fmaf(__uint_as_float(sv[c][2 * i]), sc, neg_m);
          const float x1 = fmaf(__uint_as_float(sv[c][2 * i + 1]), sc, neg_m);
          float p0, p1;
#ifdef FM_FLASH_PROFILE
          if constexpr (kPoly == 5) {           // timing experiment of developer builds: no exponential
            p0 = x0;
            p1 = x1;
          } else
#endif
          {
            // value 2i of a pair uses the polynomial when (i & 1) * 2 < kPoly, value 2i + 1 when
            // (i & 1) * 2 + 1 < kPoly: kPoly of every four consecutive values
            p0 = ((i & 1) * 2 < kPoly) ? poly_exp2(x0) : fast_exp2(x0);
            p1 = ((i & 1) * 2 + 1 < kPoly) ? poly_exp2(x1) : fast_exp2(x1);
          }
          l_part[i & 7] += p0;
          l_part[(i + 4) & 7] += p1;
          pk[i] = pack_bf16x2(p0, p1);
        }
        // P columns [16c, 16c+16) alias score columns; the scores are already in registers
        tmem_st_32x16(t_s + c * 16, pk);
        if constexpr (kPParts > 1) {
          // chunk c holds 32 keys: part boundaries after chunk 1 (two parts) or after every chunk (four)
          if (c < 3 && (kPParts == 4 || c == 1)) {
            tmem_st_wait();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_part[w * 3 + (kPParts == 4 ? c : 0)]);
          }
        }
      }
      tmem_st_wait();
      l_run += ((l_part[0] + l_part[1]) + (l_part[2] + l_part[3])) + ((l_part[4] + l_part[5]) + (l_part[6] + l_part[7]));
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[w]);
      if (lane == 0 && q == 2 % 4) FA_TRACE(a, j, w * 8 + 6);      // P_w(j) handed over
      FA_PROF_ADD(ps_exp, t0);
    }
#ifdef FM_FLASH_PROFILE
    if (a.prof != nullptr && sw == 0 && lane == 0) {
      long long* pr = a.prof + (long long)blockIdx.x * 16;
      pr[4] = clock64() - ps_total;
      pr[5] = ps_wait;
      pr[6] = 0;
      pr[7] = ps_max;
      pr[8] = ps_resc;
      pr[9] = ps_exp;
      pr[10] = nb;
    }
#endif
    if (ok && nb > 0 && mbar_wait(&o_full[w], (nb - 1) & 1, timeout, abort_flag)) {
      tc_fence_after_sync();
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      const int hq = a.G * a.qpg;
      __nv_bfloat16* dst = a.out + (((long long)row * a.b + bb) * hq + h) * kFaD;
      // HP -> SP in the epilogue: the row also goes to the rank that owns its sequence position
      const int push_p = a.push_dst != nullptr ? row / a.push_sl : 0;
      const int push_i = row - push_p * a.push_sl;
      uint4* push_to = nullptr;
      if (a.push_dst != nullptr && row < a.s)
        push_to = reinterpret_cast<uint4*>(a.push_dst[push_p] + (long long)push_i * a.push_P * hq * kFaD +
                                           ((long long)a.push_me * hq + h) * kFaD);
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(t_o + c * 32, v);
        tmem_ld_wait();
        if (row < a.s) {
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            uint4 o;
            o.x = pack_bf16x2(__uint_as_float(v[8 * u + 0]) * inv, __uint_as_float(v[8 * u + 1]) * inv);
            o.y = pack_bf16x2(__uint_as_float(v[8 * u + 2]) * inv, __uint_as_float(v[8 * u + 3]) * inv);
            o.z = pack_bf16x2(__uint_as_float(v[8 * u + 4]) * inv, __uint_as_float(v[8 * u + 5]) * inv);
            o.w = pack_bf16x2(__uint_as_float(v[8 * u + 6]) * inv, __uint_as_float(v[8 * u + 7]) * inv);
            reinterpret_cast<uint4*>(dst)[c * 4 + u] = o;
            if (push_to != nullptr) push_to[c * 4 + u] = o;
          }
        }
      }
      if (row < a.s)
        a.lse[((long long)bb * hq + h) * a.s + row] = (m_used + log2f(l_run)) * 0.6931471805599453f;
      if (a.push_dst != nullptr) {
        // one release per warp: its 32 rows share the owner and the 128-row block
        const int row0 = row - lane;
        __syncwarp();
        if (lane == 0 && row0 < a.s) {
          __threadfence_system();
          flag_release_add(a.push_flags[push_p] + a.push_me * a.push_row_blocks + push_i / 128, min(32, a.s - row0));
        }
      }
    }
    tc_fence_before_sync();
  }

  if (*abort_flag) {
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

// =========================================================================================
// Third-generation forward.  What the cycle counters and the event trace of the second
// generation showed: the softmax of a tile (about 1900 cycles per key block) sits in series
// with the tile's own two products, because P is written over S and the next Q.K^T can only
// follow P.V.  Here one CTA owns ONE 128-row query tile and P has columns of its own:
//   TMEM columns: O [0,128) | S_0 [128,256) | S_1 [256,384) | P_0 [384,448) | P_1 [448,512)
// Two softmax groups (four warps each, one thread per row) take the even and the odd key
// blocks.  A group reads its score block into registers and releases the buffer at once, so the
// tensor core computes the scores of block j+2 while the group is still busy with the
// exponentials of block j; when it has finished, its next scores are waiting.  The running
// reference maximum of a row is handed from the group of block j to the group of block j+1
// through shared memory and a named barrier right after the maximum pass.  Each group keeps
// its own partial row sum, rescaled whenever it sees a new reference maximum; O is rescaled
// (rarely: only when the maximum grows by more than 2^8) by the group that detects the growth,
// between P.V of block j-1 and P.V of block j.  K/V blocks go through three-stage TMA rings; the
// MMA warp walks its loop as a whole and one elected lane issues.
// =========================================================================================
constexpr int kFa3Threads = 384;   // warps 0-3 / 4-7: the two softmax groups; 8: TMA, 9 / 10: MMA issue, 11 idle
constexpr int kFa3Stages = 3;
constexpr int kKernelIdFlashFwd3 = 23;
constexpr int kFa3DefaultPoly = 0;

__device__ __forceinline__ void named_bar_sync(int id, int count) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}
__device__ __forceinline__ void named_bar_arrive(int id, int count) {
  asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(count) : "memory");
}
// Register re-allocation between warpgroups (four consecutive warps): the producer group gives
// registers back to the pool, the softmax groups take them.
template <int kRegs>
__device__ __forceinline__ void warpgroup_reg_inc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegs));
}
template <int kRegs>
__device__ __forceinline__ void warpgroup_reg_dec() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegs));
}

template <int kPoly>
__global__ void __launch_bounds__(kFa3Threads, 1)
flash_fwd3_kernel(const __grid_constant__ CUtensorMap tmap, const FlashFwdArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;                                        // one tile
  uint8_t* sK = smem + kTileBytes;                           // kFa3Stages tiles
  uint8_t* sV = smem + (1 + kFa3Stages) * kTileBytes;        // kFa3Stages tiles
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (1 + 2 * kFa3Stages) * kTileBytes);
  uint64_t* k_full = bars;                       // [3]
  uint64_t* v_full = bars + kFa3Stages;          // [3]
  uint64_t* k_empty = bars + 2 * kFa3Stages;     // [3]
  uint64_t* v_empty = bars + 3 * kFa3Stages;     // [3]
  uint64_t* s_full = bars + 4 * kFa3Stages;      // [2] per score buffer
  uint64_t* p_full = s_full + 2;                 // [2]
  uint64_t* o_full = s_full + 4;                 // [2] by block parity
  uint64_t* q_full = s_full + 6;                 // [1]
  uint64_t* s_free = s_full + 7;                 // [2] the group has its score block in registers
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(s_full + 9);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* m_pub = reinterpret_cast<float*>(s_full + 10);  // [128] reference maximum handed to the next block
  float* l_x = m_pub + 128;                              // [2][128] partial row sums of the two groups

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nq = (a.s + kFaBM - 1) / kFaBM;
  // One-dimensional grid, longest tiles first (tile t costs t + 1 key blocks); neighbouring CTAs
  // are the query heads of one KV group, which share K/V in L2.
  const int hq_all = a.G * a.qpg;
  const int per_tile = hq_all * a.b;
  const int qt = nq - 1 - (int)blockIdx.x / per_tile;
  const int rem_lin = (int)blockIdx.x % per_tile;
  const int h = rem_lin % hq_all, bb = rem_lin / hq_all;
  const int g_kv = h / a.qpg, hi = h % a.qpg;
  const int heads_per_group = a.qpg + 2;
  const int col_q = ((bb * a.G + g_kv) * heads_per_group + hi) * kFaD;
  const int col_k = ((bb * a.G + g_kv) * heads_per_group + a.qpg) * kFaD;
  const int col_v = col_k + kFaD;
  const int nkv = (a.s + kFaBN - 1) / kFaBN;
  const int nb = min(qt + 1, nkv);
  const uint64_t timeout = a.timeout_ns;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kFa3Stages; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[i], 4);
      mbar_init(&o_full[i], 1);
      mbar_init(&s_free[i], 4);
    }
    mbar_init(q_full, 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap);
  }
  if (warp == 9) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  constexpr uint32_t kColO = 0, kColS = 128, kColP = 384;

  if (warp >= 8) {
  warpgroup_reg_dec<96>();
  if (warp == 8) {
    if (lane == 0) {
      mbar_expect_tx(q_full, kTileBytes);
      tma_load_2d(sQ, &tmap, q_full, col_q, qt * kFaBM);
      tma_load_2d(sQ + kTileBytes / 2, &tmap, q_full, col_q + 64, qt * kFaBM);
      for (int j = 0; j < nb; ++j) {
        const int st = j % kFa3Stages;
        const uint32_t ph = ((j / kFa3Stages) & 1) ^ 1;
        if (!mbar_wait(&k_empty[st], ph, timeout, abort_flag)) {
          report_status(a.status, kStatusMbarTimeout, kKernelIdFlashFwd3, 100 + st, 0, 0);
          break;
        }
        mbar_expect_tx(&k_full[st], kTileBytes);
        tma_load_2d(sK + st * kTileBytes, &tmap, &k_full[st], col_k, j * kFaBN);
        tma_load_2d(sK + st * kTileBytes + kTileBytes / 2, &tmap, &k_full[st], col_k + 64, j * kFaBN);
        if (!mbar_wait(&v_empty[st], ph, timeout, abort_flag)) {
          report_status(a.status, kStatusMbarTimeout, kKernelIdFlashFwd3, 110 + st, 0, 0);
          break;
        }
        mbar_expect_tx(&v_full[st], kTileBytes);
        tma_load_2d(sV + st * kTileBytes, &tmap, &v_full[st], col_v, j * kFaBN);
        tma_load_2d(sV + st * kTileBytes + kTileBytes / 2, &tmap, &v_full[st], col_v + 64, j * kFaBN);
      }
    }
  } else if (warp == 9 || warp == 10) {
    // Two issuing warps on two schedulers: warp 9 issues the score products, warp 10 the P.V
    // products.  The two streams touch different accumulators and are ordered only through the
    // barriers below, and an issuing warp that shares its scheduler with two busy softmax warps
    // needs about 85 cycles per MMA: one warp could not issue the sixteen MMAs of a key block in
    // the 1024 cycles the tensor core needs for them.
    constexpr uint32_t idesc_qk = umma_idesc_bf16(128, 128, false, false);
    constexpr uint32_t idesc_pv = umma_idesc_bf16(128, 128, false, true);
    constexpr uint32_t kTileAdd = kTileBytes >> 4;
    bool ok = true;
    auto wait_or_fail = [&](uint64_t* bar, uint32_t parity, int what) {
      if (__all_sync(0xffffffffu, mbar_wait(bar, parity, timeout, abort_flag))) return true;
      if (lane == 0) report_status(a.status, kStatusMbarTimeout, kKernelIdFlashFwd3, what, 0, 0);
      return false;
    };
    [[maybe_unused]] long long pm_total = FA_PROF_NOW(), pm_wait_p = 0, pm_wait_kv = 0;
    if (warp == 9) {
      uint32_t q_lo[8], k_lo[8];      // low descriptor words of the eight k-steps, stage 0
      umma_lo_k_major(smem_u32(sQ), kTileBytes / 2, q_lo);
      umma_lo_k_major(smem_u32(sK), kTileBytes / 2, k_lo);
      auto issue_qk = [&](int j) {      // S_{j&1} = Q K_j^T
        if (elect_one()) {
          umma8_ss(tmem_base + kColS + (j & 1) * 128, q_lo, 0, k_lo, (j % kFa3Stages) * kTileAdd, idesc_qk, 0u);
          umma_commit(&s_full[j & 1]);
          umma_commit(&k_empty[j % kFa3Stages]);
        }
        __syncwarp();
      };
      ok = wait_or_fail(q_full, 0, 200);
      for (int j = 0; ok && j < nb; ++j) {
        // blocks 0 and 1 find their buffers free; block j >= 2 follows the group of block j - 2,
        // which releases the buffer as soon as it has the scores in registers
        [[maybe_unused]] long long t0 = FA_PROF_NOW();
        if (j >= 2) ok = wait_or_fail(&s_free[j & 1], ((j - 2) >> 1) & 1, 250 + (j & 1));
        if (ok) ok = wait_or_fail(&k_full[j % kFa3Stages], (j / kFa3Stages) & 1, 240);
        FA_PROF_ADD(pm_wait_kv, t0);
        if (!ok) break;
        tc_fence_after_sync();
        issue_qk(j);
      }
    } else {
      uint32_t v_lo[8];
      umma_lo_mn_major(smem_u32(sV), kTileBytes / 2, v_lo);
      auto issue_pv = [&](int j) {      // O += P_{j&1} V_j, A = P from TMEM
        if (elect_one()) {
          umma8_ts(tmem_base + kColO, tmem_base + kColP + (j & 1) * 64, 32, v_lo, (j % kFa3Stages) * kTileAdd,
                   idesc_pv, j > 0 ? 1u : 0u);
          umma_commit(&o_full[j & 1]);
          umma_commit(&v_empty[j % kFa3Stages]);
        }
        __syncwarp();
      };
      for (int j = 0; ok && j < nb; ++j) {
        [[maybe_unused]] long long t1 = FA_PROF_NOW();
        ok = wait_or_fail(&v_full[j % kFa3Stages], (j / kFa3Stages) & 1, 230);
        FA_PROF_ADD(pm_wait_kv, t1);
        t1 = FA_PROF_NOW();
        if (ok) ok = wait_or_fail(&p_full[j & 1], (j >> 1) & 1, 220 + (j & 1));
        FA_PROF_ADD(pm_wait_p, t1);
        if (!ok) break;
        tc_fence_after_sync();
        issue_pv(j);
      }
#ifdef FM_FLASH_PROFILE
      if (a.prof != nullptr && lane == 0) {
        long long* pr = a.prof + (long long)blockIdx.x * 16;
        pr[0] = clock64() - pm_total;
        pr[1] = pm_wait_p;
        pr[2] = pm_wait_kv;
        pr[3] = nb;
      }
#endif
    }
  }
  } else {
    warpgroup_reg_inc<200>();
    // ------------------------------- softmax warps -------------------------------
    const int g = warp >> 2;             // softmax group: blocks j with (j & 1) == g
    const int q = warp & 3;              // TMEM lane quarter
    const int r = q * 32 + lane;
    const int row = qt * kFaBM + r;
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    const uint32_t t_s = tmem_base + kColS + g * 128 + lane_addr;   // this group's score buffer (fp32)
    const uint32_t t_p = tmem_base + kColP + g * 64 + lane_addr;    // this group's P buffer (bf16 pairs)
    const uint32_t t_o = tmem_base + kColO + lane_addr;
    // named barriers: 1 + (block parity) * 4 + q hands the maximum from the group of block j to
    // the group of block j + 1 (32 threads arrive, 32 wait); 9 + q joins both groups at the end
    bool ok = true;
    float m_seen = -INFINITY, l_own = 0.f;
    const float sc = a.scale_log2;
    [[maybe_unused]] long long ps_total = FA_PROF_NOW(), ps_wait = 0, ps_max = 0, ps_bar = 0, ps_exp = 0, ps_resc = 0;
    for (int j = g; j < nb; j += 2) {
      [[maybe_unused]] long long t0 = FA_PROF_NOW();
      // After a failed wait the group keeps walking its blocks (without touching TMEM) so that
      // the other group never waits alone at a named barrier.
      if (ok && !__all_sync(0xffffffffu, mbar_wait(&s_full[g], (j >> 1) & 1, timeout, abort_flag))) {
        if (lane == 0) report_status(a.status, kStatusMbarTimeout, kKernelIdFlashFwd3, 300 + g, 0, 0);
        ok = false;
      }
      if (!ok) {
        if (j > 0) named_bar_sync(1 + ((j - 1) & 1) * 4 + q, 64);
        named_bar_arrive(1 + (j & 1) * 4 + q, 64);
        continue;
      }
      tc_fence_after_sync();
      FA_PROF_ADD(ps_wait, t0);
      t0 = FA_PROF_NOW();
      const int kv0 = j * kFaBN;
      const bool diag = (j == qt);
      uint32_t sv[4][32];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld_32x32(t_s + c * 32, sv[c]);
      tmem_ld_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_free[g]);      // the buffer may take the scores of block j + 2
      if (diag || kv0 + kFaBN > a.s) {
        // only the diagonal block and a ragged last block need masking
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int col = kv0 + c * 32 + i;
            if ((diag && col > row) || col >= a.s) sv[c][i] = 0xff800000u;   // -inf
          }
      }
      float mx[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) mx[k] = -INFINITY;
#pragma unroll
      for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int i = 0; i < 16; ++i)
          mx[i & 7] = fmax3(mx[i & 7], __uint_as_float(sv[c][2 * i]), __uint_as_float(sv[c][2 * i + 1]));
      const float m_blk =
          fmaxf(fmax3(mx[0], mx[1], mx[2]), fmax3(fmax3(mx[3], mx[4], mx[5]), mx[6], mx[7])) * sc;   // scale > 0
      FA_PROF_ADD(ps_max, t0);
      t0 = FA_PROF_NOW();
      // the reference maximum after block j-1, from the other group
      if (j > 0) {
        named_bar_sync(1 + ((j - 1) & 1) * 4 + q, 64);
        const float m_prev = m_pub[r];
        if (m_prev != m_seen) {
          l_own *= exp2f(m_seen - m_prev);    // m_seen = -inf only while l_own = 0: 0 * 0
          m_seen = m_prev;
        }
      }
      FA_PROF_ADD(ps_bar, t0);
      t0 = FA_PROF_NOW();
      // Lazy rescale: keep the reference maximum unless the block's is more than 2^8 above it.
      const float m_new = fmaxf(m_seen, m_blk);
      const bool first = (j == 0);
      const bool grow = !first && (m_new > m_seen + 8.0f);
      const float m_old = m_seen;
      if (first) m_seen = (m_new == -INFINITY) ? 0.f : m_new;
      if (grow) m_seen = m_new;
      m_pub[r] = m_seen;
      named_bar_arrive(1 + (j & 1) * 4 + q, 64);      // the next block's group may go on
      if (__any_sync(0xffffffffu, grow)) {
        // O holds the sum of blocks 0..j-1; P.V of block j-1 must have finished before it is touched.
        if (!__all_sync(0xffffffffu, mbar_wait(&o_full[(j - 1) & 1], ((j - 1) >> 1) & 1, timeout, abort_flag))) {
          ok = false;
          continue;
        }
        tc_fence_after_sync();
        const float f = grow ? exp2f(m_old - m_new) : 1.0f;
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t v[32];
          tmem_ld_32x32(t_o + c * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * f);
          tmem_st_32x32(t_o + c * 32, v);
        }
        tmem_st_wait();
        if (grow) l_own *= f;
      }
      FA_PROF_ADD(ps_resc, t0);
      t0 = FA_PROF_NOW();
      // P.V of block j - 2 read this group's P buffer; it has to be done before P is overwritten
      if (j >= 2 && !__all_sync(0xffffffffu, mbar_wait(&o_full[g], ((j >> 1) - 1) & 1, timeout, abort_flag))) {
        ok = false;
        continue;
      }
      float l_part[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) l_part[k] = 0.f;
      const float neg_m = -m_seen;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float x0 = fmaf(__uint_as_float(sv[c][2 * i]), sc, neg_m);
          const float x1 = fmaf(__uint_as_float(sv[c][2 * i + 1]), sc, neg_m);
          const float p0 = ((i & 1) * 2 < kPoly) ? poly_exp2(x0) : fast_exp2(x0);
          const float p1 = ((i & 1) * 2 + 1 < kPoly) ? poly_exp2(x1) : fast_exp2(x1);
          l_part[i & 7] += p0;
          l_part[(i + 4) & 7] += p1;
          pk[i] = pack_bf16x2(p0, p1);
        }
        tmem_st_32x16(t_p + c * 16, pk);
      }
      tmem_st_wait();
      l_own += ((l_part[0] + l_part[1]) + (l_part[2] + l_part[3])) + ((l_part[4] + l_part[5]) + (l_part[6] + l_part[7]));
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[g]);
      FA_PROF_ADD(ps_exp, t0);
    }
#ifdef FM_FLASH_PROFILE
    if (a.prof != nullptr && warp == 0 && lane == 0) {
      long long* pr = a.prof + (long long)blockIdx.x * 16;
      pr[4] = clock64() - ps_total;
      pr[5] = ps_wait;
      pr[6] = ps_bar;
      pr[7] = ps_max;
      pr[8] = ps_resc;
      pr[9] = ps_exp;
      pr[10] = (nb + 1) / 2;
    }
#endif
    // the group that did not own the last block still has to see its reference maximum
    if (((nb - 1) & 1) != g) {
      named_bar_sync(1 + ((nb - 1) & 1) * 4 + q, 64);
      const float m_last = m_pub[r];
      if (m_last != m_seen) {
        l_own *= exp2f(m_seen - m_last);
        m_seen = m_last;
      }
    }
    l_x[g * 128 + r] = l_own;
    named_bar_sync(9 + q, 64);
    const float l_run = l_x[r] + l_x[128 + r];
    if (ok && mbar_wait(&o_full[(nb - 1) & 1], ((nb - 1) >> 1) & 1, timeout, abort_flag)) {
      tc_fence_after_sync();
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      const int hq = a.G * a.qpg;
      __nv_bfloat16* dst = a.out + (((long long)row * a.b + bb) * hq + h) * kFaD + g * 64;
#pragma unroll 1
      for (int c = 0; c < 2; ++c) {       // this group's half of the head dimension
        uint32_t v[32];
        tmem_ld_32x32(t_o + g * 64 + c * 32, v);
        tmem_ld_wait();
        if (row < a.s) {
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            uint4 o;
            o.x = pack_bf16x2(__uint_as_float(v[8 * u + 0]) * inv, __uint_as_float(v[8 * u + 1]) * inv);
            o.y = pack_bf16x2(__uint_as_float(v[8 * u + 2]) * inv, __uint_as_float(v[8 * u + 3]) * inv);
            o.z = pack_bf16x2(__uint_as_float(v[8 * u + 4]) * inv, __uint_as_float(v[8 * u + 5]) * inv);
            o.w = pack_bf16x2(__uint_as_float(v[8 * u + 6]) * inv, __uint_as_float(v[8 * u + 7]) * inv);
            reinterpret_cast<uint4*>(dst)[c * 4 + u] = o;
          }
        }
      }
      if (row < a.s && g == 0)
        a.lse[((long long)bb * hq + h) * a.s + row] = (m_seen + log2f(l_run)) * 0.6931471805599453f;
    }
    tc_fence_before_sync();
  }

  if (*abort_flag) {
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 9) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

// =========================================================================================
// Backward.  One CTA owns a 128-position key/value block of one KV head and walks every query
// tile (and every query head of the group) that attends to it.  Per step, on tcgen05:
//   S  = Q K^T,  dP = dO V^T                      (accumulators in TMEM)
//   P  = exp2(S * c - lse),  dS = P * (dP - delta) * scale     (one thread per query row)
//   dV += P^T dO,  dK += dS^T Q                   (accumulate in TMEM across all steps)
//   dQ  = dS K                                    (added to an fp32 buffer with vector atomics)
// P and dS are staged once in shared memory in the 128-byte-swizzled layout, which serves both as
// K-major A operand (dS K) and as MN-major A operand (P^T dO, dS^T Q).  dK / dV are written
// straight into the packed [q.. | k | v] gradient buffer, so no concatenation pass is needed
// (the reference concatenates dQ, dK, dV per KV group, fluid/attention/backward.py:284-287).
// =========================================================================================
constexpr int kKernelIdFlashBwd = 22;

struct FlashBwdArgs {
  int s, b, G, qpg;
  float scale, scale_log2;
  const float* lse;      // [b, hq, s]
  const float* delta;    // [b, hq, s]  rowsum(dO * O)
  float* dq_accum;       // [s, b, hq, d] fp32, zero-initialised
  __nv_bfloat16* dqkv;   // packed gradient buffer [s, b, G, (qpg + 2) * d]
  unsigned long long timeout_ns;
  int* status;
  int hsplit;            // CTAs per (K/V block, KV head): each takes qpg / hsplit query heads
  float* dkv_accum;      // [s, b, G, 2, d] fp32, zero-initialised; used when hsplit > 1
};

constexpr int kKernelIdDeltaWait = 17;
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ dout,
                                  float* __restrict__ delta, int s, int b, int hq, const int* wait_flags,
                                  int wait_n, int wait_expected, unsigned long long* wait_ns,
                                  unsigned long long timeout_ns, int* status) {
  // first consumer of the output gradient that peers fill (SP -> HP exchange of the backward pass)
  if (wait_flags != nullptr)
    wait_counters_cta(wait_flags, wait_n, wait_expected, wait_ns, timeout_ns, status, kKernelIdDeltaWait);
  // one warp per (row, batch, head): delta[b, h, row] = sum_d dO * O   (d == 128)
  const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long total = (long long)s * b * hq;
  if (w >= total) return;
  const int lane = threadIdx.x & 31;
  const uint2 o = reinterpret_cast<const uint2*>(out + w * kFaD)[lane];
  const uint2 g = reinterpret_cast<const uint2*>(dout + w * kFaD)[lane];
  const __nv_bfloat162 o0 = *reinterpret_cast<const __nv_bfloat162*>(&o.x);
  const __nv_bfloat162 o1 = *reinterpret_cast<const __nv_bfloat162*>(&o.y);
  const __nv_bfloat162 g0 = *reinterpret_cast<const __nv_bfloat162*>(&g.x);
  const __nv_bfloat162 g1 = *reinterpret_cast<const __nv_bfloat162*>(&g.y);
  float acc = __low2float(o0) * __low2float(g0) + __high2float(o0) * __high2float(g0) +
              __low2float(o1) * __low2float(g1) + __high2float(o1) * __high2float(g1);
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (lane == 0) {
    const long long h = w % hq, bb = (w / hq) % b, row = w / ((long long)hq * b);
    delta[(bb * hq + h) * s + row] = acc;
  }
}

// dq_accum (fp32 [s, b, hq, d]) -> bf16 into the query-head columns of the packed buffer
__global__ void attn_dq_store_kernel(const float* __restrict__ dq, __nv_bfloat16* __restrict__ dqkv,
                                     long long rows /* s*b */, int G, int qpg, float mul) {
  const int hq = G * qpg;
  const long long total = rows * hq * (kFaD / 8);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int v8 = (int)(i % (kFaD / 8));
    const long long rh = i / (kFaD / 8);
    const int h = (int)(rh % hq);
    const long long row = rh / hq;
    const float4 a = reinterpret_cast<const float4*>(dq + rh * kFaD)[v8 * 2];
    const float4 c = reinterpret_cast<const float4*>(dq + rh * kFaD)[v8 * 2 + 1];
    uint4 p;
    p.x = pack_bf16x2(a.x * mul, a.y * mul); p.y = pack_bf16x2(a.z * mul, a.w * mul);
    p.z = pack_bf16x2(c.x * mul, c.y * mul); p.w = pack_bf16x2(c.z * mul, c.w * mul);
    const int g = h / qpg, hi = h % qpg;
    __nv_bfloat16* dst = dqkv + ((row * G + g) * (qpg + 2) + hi) * kFaD;
    reinterpret_cast<uint4*>(dst)[v8] = p;
  }
}

// dkv_accum (fp32 [s*b, G, 2, d]) -> bf16 into the key / value columns of the packed buffer
__global__ void attn_dkv_store_kernel(const float* __restrict__ dkv, __nv_bfloat16* __restrict__ dqkv,
                                      long long rows /* s*b */, int G, int qpg) {
  const long long total = rows * G * 2 * (kFaD / 8);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int v8 = (int)(i % (kFaD / 8));
    const long long rgw = i / (kFaD / 8);          // (row, g, which)
    const int which = (int)(rgw % 2);
    const long long rg = rgw / 2;                  // row * G + g
    const float4 a = reinterpret_cast<const float4*>(dkv + rgw * kFaD)[v8 * 2];
    const float4 c = reinterpret_cast<const float4*>(dkv + rgw * kFaD)[v8 * 2 + 1];
    uint4 p;
    p.x = pack_bf16x2(a.x, a.y); p.y = pack_bf16x2(a.z, a.w);
    p.z = pack_bf16x2(c.x, c.y); p.w = pack_bf16x2(c.z, c.w);
    __nv_bfloat16* dst = dqkv + (rg * (qpg + 2) + qpg + which) * kFaD;
    reinterpret_cast<uint4*>(dst)[v8] = p;
  }
}

__global__ void __launch_bounds__(kFaThreads, 1)
flash_bwd_kernel(const __grid_constant__ CUtensorMap tmap_qkv, const __grid_constant__ CUtensorMap tmap_do,
                 const FlashBwdArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = smem + kTileBytes;
  uint8_t* sQ = smem + 2 * kTileBytes;
  uint8_t* sdO = smem + 3 * kTileBytes;
  uint8_t* sP = smem + 4 * kTileBytes;
  uint8_t* sdS = smem + 5 * kTileBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 6 * kTileBytes);
  uint64_t* kv_full = bars;        // K and V of this block
  uint64_t* qdo_full = bars + 1;   // Q_i and dO_i of the current step
  uint64_t* qdo_empty = bars + 2;  // the step's MMAs have finished reading Q_i / dO_i
  uint64_t* sdp_full = bars + 3;   // S and dP are in TMEM
  uint64_t* pds_full = bars + 4;   // P and dS are in shared memory (4 warps)
  uint64_t* dq_full = bars + 5;    // dQ is in TMEM (and dV, dK updated)
  uint64_t* dq_read = bars + 6;    // dQ has been drained (4 warps)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 7);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int j = blockIdx.x, g = blockIdx.y, bb = blockIdx.z;
  const int nq = (a.s + kFaBM - 1) / kFaBM;
  const int hq = a.G * a.qpg;
  const int hpg = a.qpg + 2;
  const int col_k = ((bb * a.G + g) * hpg + a.qpg) * kFaD;
  const int col_v = col_k + kFaD;
  const int tiles = nq - j;                 // query tiles i = j .. nq-1
  const int nsteps = tiles * a.qpg;
  const uint64_t timeout = a.timeout_ns;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    mbar_init(qdo_full, 1);
    mbar_init(qdo_empty, 1);
    mbar_init(sdp_full, 1);
    mbar_init(pds_full, 4);
    mbar_init(dq_full, 1);
    mbar_init(dq_read, 4);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_qkv);
    tma_prefetch_desc(&tmap_do);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t t_s = tmem_base, t_dp = tmem_base + 128, t_dv = tmem_base + 256, t_dk = tmem_base + 384;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(kv_full, 2 * kTileBytes);
      tma_load_2d(sK, &tmap_qkv, kv_full, col_k, j * kFaBN);
      tma_load_2d(sK + kTileBytes / 2, &tmap_qkv, kv_full, col_k + 64, j * kFaBN);
      tma_load_2d(sV, &tmap_qkv, kv_full, col_v, j * kFaBN);
      tma_load_2d(sV + kTileBytes / 2, &tmap_qkv, kv_full, col_v + 64, j * kFaBN);
      for (int n = 0; n < nsteps; ++n) {
        const int hi = n / tiles, i = j + n % tiles;
        if (!mbar_wait(qdo_empty, (n & 1) ^ 1, timeout, abort_flag)) {
          report_status(a.status, kStatusMbarTimeout, kKernelIdFlashBwd, 100, 0, 0);
          break;
        }
        const int col_q = ((bb * a.G + g) * hpg + hi) * kFaD;
        const int col_do = (bb * hq + g * a.qpg + hi) * kFaD;
        mbar_expect_tx(qdo_full, 2 * kTileBytes);
        tma_load_2d(sQ, &tmap_qkv, qdo_full, col_q, i * kFaBM);
        tma_load_2d(sQ + kTileBytes / 2, &tmap_qkv, qdo_full, col_q + 64, i * kFaBM);
        tma_load_2d(sdO, &tmap_do, qdo_full, col_do, i * kFaBM);
        tma_load_2d(sdO + kTileBytes / 2, &tmap_do, qdo_full, col_do + 64, i * kFaBM);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t id_kk = umma_idesc_bf16(128, 128, false, false);   // A K-major, B K-major
      constexpr uint32_t id_mm = umma_idesc_bf16(128, 128, true, true);     // A MN-major, B MN-major
      constexpr uint32_t id_km = umma_idesc_bf16(128, 128, false, true);    // A K-major, B MN-major
      const uint32_t aK = smem_u32(sK), aV = smem_u32(sV), aQ = smem_u32(sQ), aO = smem_u32(sdO);
      const uint32_t aP = smem_u32(sP), aS = smem_u32(sdS);
      constexpr uint32_t HALF = kTileBytes / 2;
      auto kdesc = [&](uint32_t base, int kk) {   // K-major operand, k-step kk of 8
        return umma_smem_desc(base + (kk >> 2) * HALF + (kk & 3) * 32, 0, 1024);
      };
      auto mdesc = [&](uint32_t base, int kk) {   // MN-major operand ([128 k rows][64] slabs)
        return umma_smem_desc(base + kk * 2048, HALF, 1024);
      };
      bool ok = mbar_wait(kv_full, 0, timeout, abort_flag);
      if (!ok) report_status(a.status, kStatusMbarTimeout, kKernelIdFlashBwd, 200, 0, 0);
      for (int n = 0; ok && n < nsteps; ++n) {
        const uint32_t par = n & 1;
        if (!mbar_wait(qdo_full, par, timeout, abort_flag) ||
            !mbar_wait(dq_read, par ^ 1, timeout, abort_flag)) {   // S columns (= dQ) are free again
          report_status(a.status, kStatusMbarTimeout, kKernelIdFlashBwd, 210, 0, 0);
          break;
        }
        tc_fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) umma_bf16(t_s, kdesc(aQ, kk), kdesc(aK, kk), id_kk, kk > 0);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) umma_bf16(t_dp, kdesc(aO, kk), kdesc(aV, kk), id_kk, kk > 0);
        umma_commit(sdp_full);
        if (!mbar_wait(pds_full, par, timeout, abort_flag)) {
          report_status(a.status, kStatusMbarTimeout, kKernelIdFlashBwd, 220, 0, 0);
          break;
        }
        tc_fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) umma_bf16(t_dv, mdesc(aP, kk), mdesc(aO, kk), id_mm, (n > 0 || kk > 0));
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) umma_bf16(t_dk, mdesc(aS, kk), mdesc(aQ, kk), id_mm, (n > 0 || kk > 0));
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) umma_bf16(t_s, kdesc(aS, kk), mdesc(aK, kk), id_km, kk > 0);
        umma_commit(qdo_empty);
        umma_commit(dq_full);
      }
    }
  } else {
    const int q = warp & 3;
    const int r = q * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    bool ok = true;
    for (int n = 0; n < nsteps; ++n) {
      const uint32_t par = n & 1;
      const int hi = n / tiles, i = j + n % tiles;
      const int h = g * a.qpg + hi;
      const int row = i * kFaBM + r;
      const bool row_ok = row < a.s;
      const float lse2 = row_ok ? a.lse[((long long)bb * hq + h) * a.s + row] * 1.4426950408889634f : 0.f;
      const float dl = row_ok ? a.delta[((long long)bb * hq + h) * a.s + row] : 0.f;
      if (!mbar_wait(sdp_full, par, timeout, abort_flag)) {
        if (lane == 0) report_status(a.status, kStatusMbarTimeout, kKernelIdFlashBwd, 300, 0, 0);
        ok = false;
        break;
      }
      tc_fence_after_sync();
      const bool diag = (i == j);
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t sv[32], dv[32];
        tmem_ld_32x32(t_s + lane_addr + c * 32, sv);
        tmem_ld_32x32(t_dp + lane_addr + c * 32, dv);
        tmem_ld_wait();
        uint8_t* prow = sP + (c >> 1) * (kTileBytes / 2) + r * 128;
        uint8_t* drow = sdS + (c >> 1) * (kTileBytes / 2) + r * 128;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
          float p[8], ds[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const int col = j * kFaBN + c * 32 + w * 8 + e;
            const bool masked = !row_ok || (diag && col > row) || col >= a.s;
            p[e] = masked ? 0.f : exp2f(__uint_as_float(sv[w * 8 + e]) * a.scale_log2 - lse2);
            ds[e] = p[e] * (__uint_as_float(dv[w * 8 + e]) - dl) * a.scale;
          }
          const int chunk = ((c & 1) * 4 + w) ^ (r & 7);
          uint4 pp, dd;
          pp.x = pack_bf16x2(p[0], p[1]); pp.y = pack_bf16x2(p[2], p[3]);
          pp.z = pack_bf16x2(p[4], p[5]); pp.w = pack_bf16x2(p[6], p[7]);
          dd.x = pack_bf16x2(ds[0], ds[1]); dd.y = pack_bf16x2(ds[2], ds[3]);
          dd.z = pack_bf16x2(ds[4], ds[5]); dd.w = pack_bf16x2(ds[6], ds[7]);
          *reinterpret_cast<uint4*>(prow + chunk * 16) = pp;
          *reinterpret_cast<uint4*>(drow + chunk * 16) = dd;
        }
      }
      fence_proxy_async_smem();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(pds_full);
      // drain dQ of this step
      if (!mbar_wait(dq_full, par, timeout, abort_flag)) {
        if (lane == 0) report_status(a.status, kStatusMbarTimeout, kKernelIdFlashBwd, 310, 0, 0);
        ok = false;
        break;
      }
      tc_fence_after_sync();
      float* dq_row = a.dq_accum + (((long long)row * a.b + bb) * hq + h) * kFaD;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(t_s + lane_addr + c * 32, v);
        tmem_ld_wait();
        if (row_ok) {
#pragma unroll
          for (int u = 0; u < 8; ++u)
            red_add_v4_f32(dq_row + c * 32 + 4 * u, __uint_as_float(v[4 * u]), __uint_as_float(v[4 * u + 1]),
                           __uint_as_float(v[4 * u + 2]), __uint_as_float(v[4 * u + 3]));
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(dq_read);
    }
    if (ok && nsteps > 0) {
      // dK / dV of this block are complete once the last step's MMAs have finished (dq_full).
      const int kvrow = j * kFaBN + r;
      __nv_bfloat16* dk_dst = a.dqkv + (((long long)kvrow * a.b + bb) * a.G + g) * hpg * kFaD + a.qpg * kFaD;
      __nv_bfloat16* dv_dst = dk_dst + kFaD;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t vk[32], vv[32];
        tmem_ld_32x32(t_dk + lane_addr + c * 32, vk);
        tmem_ld_32x32(t_dv + lane_addr + c * 32, vv);
        tmem_ld_wait();
        if (kvrow < a.s) {
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            uint4 k4, v4;
            k4.x = pack_bf16x2(__uint_as_float(vk[8 * u]), __uint_as_float(vk[8 * u + 1]));
            k4.y = pack_bf16x2(__uint_as_float(vk[8 * u + 2]), __uint_as_float(vk[8 * u + 3]));
            k4.z = pack_bf16x2(__uint_as_float(vk[8 * u + 4]), __uint_as_float(vk[8 * u + 5]));
            k4.w = pack_bf16x2(__uint_as_float(vk[8 * u + 6]), __uint_as_float(vk[8 * u + 7]));
            v4.x = pack_bf16x2(__uint_as_float(vv[8 * u]), __uint_as_float(vv[8 * u + 1]));
            v4.y = pack_bf16x2(__uint_as_float(vv[8 * u + 2]), __uint_as_float(vv[8 * u + 3]));
            v4.z = pack_bf16x2(__uint_as_float(vv[8 * u + 4]), __uint_as_float(vv[8 * u + 5]));
            v4.w = pack_bf16x2(__uint_as_float(vv[8 * u + 6]), __uint_as_float(vv[8 * u + 7]));
            reinterpret_cast<uint4*>(dk_dst)[c * 4 + u] = k4;
            reinterpret_cast<uint4*>(dv_dst)[c * 4 + u] = v4;
          }
        }
      }
    }
    tc_fence_before_sync();
  }

  if (*abort_flag) {
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}


// =========================================================================================
// Second-generation backward: same ownership (one CTA per 128-position K/V block and KV head)
// but in the transposed orientation, which lets the five MMAs of a step overlap with the
// element-wise work of the neighbouring steps:
//   S^T  = K Q^T,  dP^T = V dO^T       (key/value position on the TMEM lanes)
//   P^T  = exp2(S^T c - lse[q])          written back to TMEM over S^T (bf16), A operand of
//   dV  += P^T dO                        straight from TMEM
//   dS^T = P^T (dP^T - delta[q])         staged once in swizzled shared memory: K-major A of
//   dK  += dS^T Q                        and MN-major A of
//   dQ   = dS K                          whose accumulator re-uses the dP^T columns
// Q tiles are double buffered and S^T of step n+1 is issued before the tensor core waits for dS^T
// of step n.  Eight softmax warps (two per TMEM lane quarter, 64 query positions each) keep two
// warps per scheduler busy; four more warps drain dQ: TMEM -> swizzled shared-memory boxes ->
// TMA reduce-add into the fp32 dQ buffer (whole 128-byte lines instead of per-thread atomics).
// TMEM: S^T/P^T, dP^T/dQ, dV, dK = 512 columns.  The softmax scale is applied once at the end
// (to dK here, to dQ in the store kernel).
// =========================================================================================
constexpr int kFaB2Threads = 480;   // TMA warp, MMA warp A, 8 softmax warps, 4 dQ-drain warps, MMA warp B
constexpr int kKernelIdFlashBwd2 = 23;
constexpr int kFaB2StageBytes = 4 * 2 * 4096;   // per drain warp: two [32 rows][32 fp32] boxes
constexpr int kFaB2Smem = 6 * kTileBytes + kFaB2StageBytes + 2 * 2 * 128 * 4 + 256;

__global__ void __launch_bounds__(kFaB2Threads, 1)
flash_bwd2_kernel(const __grid_constant__ CUtensorMap tmap_qkv, const __grid_constant__ CUtensorMap tmap_do,
                  const __grid_constant__ CUtensorMap tmap_dq, const FlashBwdArgs a) {
  extern __shared__ __align__(1024) uint8_t smem_b2[];
  uint8_t* smem = smem_b2;
  if ((smem_u32(smem) & 1023u) != 0) {   // the swizzled tiles need a 1024-byte aligned base
    if (threadIdx.x == 0) report_status(a.status, kStatusMbarTimeout, kKernelIdFlashBwd2, 1, 0, 0);
    return;
  }
  uint8_t* sK = smem;
  uint8_t* sV = smem + kTileBytes;
  uint8_t* sQ = smem + 2 * kTileBytes;     // 2 stages
  uint8_t* sdO = smem + 4 * kTileBytes;    // 1 stage
  uint8_t* sdS = smem + 5 * kTileBytes;
  uint8_t* sStage = smem + 6 * kTileBytes; // dQ boxes on their way to the TMA reduction
  float* s_lse = reinterpret_cast<float*>(sStage + kFaB2StageBytes);   // [2][128]  lse * log2(e)
  float* s_dl = s_lse + 256;                                           // [2][128]  delta
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_dl + 256);
  uint64_t* kv_full = bars;
  uint64_t* q_full = bars + 1;      // [2]
  uint64_t* q_empty = bars + 3;     // [2]
  uint64_t* do_full = bars + 5;
  uint64_t* do_empty = bars + 6;
  uint64_t* s_full = bars + 7;      // S^T(n) is in TMEM
  uint64_t* p_full = bars + 8;      // P^T(n) is in TMEM (8 warps)
  uint64_t* dp_full = bars + 9;     // dP^T(n) is in TMEM
  uint64_t* ds_full = bars + 10;    // dS^T(n) is in shared memory (8 warps)
  uint64_t* dq_full = bars + 11;    // dQ(n) is in TMEM
  uint64_t* dq_read = bars + 12;    // dQ(n) has left TMEM (4 warps)
  uint64_t* done_full = bars + 13;  // every MMA of this CTA has finished
  uint64_t* stats_full = bars + 14; // [2] lse / delta of a step are in shared memory (128 threads)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // One-dimensional grid, longest job first over the whole launch: K/V block j (tiles = nq - j
  // query tiles to walk) of every (KV head, head split, batch) before block j + 1 of any.
  const int ny = a.G * a.hsplit;
  const int j = (int)blockIdx.x / (ny * a.b);
  const int y_lin = (int)blockIdx.x % ny, bb = ((int)blockIdx.x / ny) % a.b;
  const int g = y_lin / a.hsplit;
  const int heads_here = a.qpg / a.hsplit;                      // query heads of this CTA
  const int head0 = (y_lin % a.hsplit) * heads_here;             // first of them within the group
  const int nq = (a.s + kFaBM - 1) / kFaBM;
  const int hq = a.G * a.qpg;
  const int hpg = a.qpg + 2;
  const int col_k = ((bb * a.G + g) * hpg + a.qpg) * kFaD;
  const int col_v = col_k + kFaD;
  const int tiles = nq - j;                 // query tiles i = j .. nq-1
  const int nsteps = tiles * heads_here;
  const uint64_t timeout = a.timeout_ns;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&q_full[i], 1);
      mbar_init(&q_empty[i], 1);
      mbar_init(&stats_full[i], 128);
    }
    mbar_init(do_full, 1);
    mbar_init(do_empty, 2);       // dV (issuing warp A) and dP^T (issuing warp B) have read dO
    mbar_init(s_full, 1);
    mbar_init(p_full, 8);
    mbar_init(dp_full, 1);
    mbar_init(ds_full, 8);
    mbar_init(dq_full, 1);
    mbar_init(dq_read, 4);
    mbar_init(done_full, 2);      // both issuing warps
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_qkv);
    tma_prefetch_desc(&tmap_do);
    tma_prefetch_desc(&tmap_dq);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t t_s = tmem_base, t_dp = tmem_base + 128, t_dv = tmem_base + 256, t_dk = tmem_base + 384;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(kv_full, 2 * kTileBytes);
      tma_load_2d(sK, &tmap_qkv, kv_full, col_k, j * kFaBN);
      tma_load_2d(sK + kTileBytes / 2, &tmap_qkv, kv_full, col_k + 64, j * kFaBN);
      tma_load_2d(sV, &tmap_qkv, kv_full, col_v, j * kFaBN);
      tma_load_2d(sV + kTileBytes / 2, &tmap_qkv, kv_full, col_v + 64, j * kFaBN);
      for (int n = 0; n < nsteps; ++n) {
        const int st = n & 1;
        const int hi = head0 + n / tiles, i = j + n % tiles;
        if (!mbar_wait(&q_empty[st], ((n >> 1) & 1) ^ 1, timeout, abort_flag)) {
          report_status(a.status, kStatusMbarTimeout, kKernelIdFlashBwd2, 100 + st, 0, 0);
          break;
        }
        const int col_q = ((bb * a.G + g) * hpg + hi) * kFaD;
        uint8_t* q_dst = sQ + st * kTileBytes;
        mbar_expect_tx(&q_full[st], kTileBytes);
        tma_load_2d(q_dst, &tmap_qkv, &q_full[st], col_q, i * kFaBM);
        tma_load_2d(q_dst + kTileBytes / 2, &tmap_qkv, &q_full[st], col_q + 64, i * kFaBM);
        if (!mbar_wait(do_empty, (n & 1) ^ 1, timeout, abort_flag)) {   // dV(n-1) has read dO(n-1)
          report_status(a.status, kStatusMbarTimeout, kKernelIdFlashBwd2, 110, 0, 0);
          break;
        }
        const int col_do = (bb * hq + g * a.qpg + hi) * kFaD;
        mbar_expect_tx(do_full, kTileBytes);
        tma_load_2d(sdO, &tmap_do, do_full, col_do, i * kFaBM);
        tma_load_2d(sdO + kTileBytes / 2, &tmap_do, do_full, col_do + 64, i * kFaBM);
      }
    }
  } else if (warp == 1 || warp == 14) {
    // Two issuing warps on two schedulers, each walking its loop as a whole with one elected lane
    // issuing (uniform control flow keeps descriptors and loop state in uniform registers):
    //   warp 1:  S^T(n) = K Q^T and dV += P^T dO       (P^T sits over S^T, so the two stay in order)
    //   warp 14: dP^T(n) = V dO^T, dQ = dS K, dK += dS^T Q   (dQ sits over dP^T, likewise)
    // An issuing warp shares its scheduler with busy softmax warps and needs about 85 cycles per
    // MMA; one warp could not issue the forty MMAs of a step in the 2560 cycles the tensor core
    // needs for them.  The two streams are ordered against each other only through barriers.
    constexpr uint32_t id_kk = umma_idesc_bf16(128, 128, false, false);   // A K-major, B K-major
    constexpr uint32_t id_mm = umma_idesc_bf16(128, 128, true, true);     // A MN-major, B MN-major
    constexpr uint32_t id_km = umma_idesc_bf16(128, 128, false, true);    // A K-major / TMEM, B MN-major
    constexpr uint32_t HALF = kTileBytes / 2;
    constexpr uint32_t kTileAdd = kTileBytes >> 4;
    auto wait_or_fail = [&](uint64_t* bar, uint32_t parity, int what) {
      if (__all_sync(0xffffffffu, mbar_wait(bar, parity, timeout, abort_flag))) return true;
      if (lane == 0) report_status(a.status, kStatusMbarTimeout, kKernelIdFlashBwd2, what, 0, 0);
      return false;
    };
    bool ok = wait_or_fail(kv_full, 0, 200);
    if (warp == 1) {
      // low descriptor words of the eight k-steps (K-major: the tile's rows are the M / N index;
      // MN-major: the tile's rows are the k index)
      uint32_t k_km[8], q_km[8], o_mn[8];
      umma_lo_k_major(smem_u32(sK), HALF, k_km);
      umma_lo_k_major(smem_u32(sQ), HALF, q_km);      // stage 0; stage 1 is one tile further
      umma_lo_mn_major(smem_u32(sdO), HALF, o_mn);
      auto issue_s = [&](int n) {     // S^T(n) = K Q(n)^T
        if (elect_one()) {
          umma8_ss(t_s, k_km, 0, q_km, (n & 1) * kTileAdd, id_kk, 0u);
          umma_commit(s_full);
        }
        __syncwarp();
      };
      if (ok && nsteps > 0) ok = wait_or_fail(&q_full[0], 0, 201);
      if (ok && nsteps > 0) {
        tc_fence_after_sync();
        issue_s(0);
      }
      for (int n = 0; ok && n < nsteps; ++n) {
        if (!(ok = wait_or_fail(p_full, n & 1, 210))) break;
        tc_fence_after_sync();
        // dV += P^T dO, A from TMEM: query positions 0-63 sit in columns [0, 32) of the S^T block,
        // positions 64-127 in columns [64, 96) (each softmax warp writes over its own scores)
        if (elect_one()) {
          umma8_ts(t_dv, t_s, 64, o_mn, 0, id_km, n > 0 ? 1u : 0u);
          umma_commit(do_empty);
        }
        __syncwarp();
        if (n + 1 < nsteps) {
          if (!(ok = wait_or_fail(&q_full[(n + 1) & 1], ((n + 1) >> 1) & 1, 220))) break;
          tc_fence_after_sync();
          issue_s(n + 1);
        }
      }
    } else {
      uint32_t v_km[8], o_km[8], s_km[8], k_mn[8], q_mn[8], s_mn[8];
      umma_lo_k_major(smem_u32(sV), HALF, v_km);
      umma_lo_k_major(smem_u32(sdO), HALF, o_km);
      umma_lo_k_major(smem_u32(sdS), HALF, s_km);
      umma_lo_mn_major(smem_u32(sK), HALF, k_mn);
      umma_lo_mn_major(smem_u32(sQ), HALF, q_mn);     // stage 0; stage 1 is one tile further
      umma_lo_mn_major(smem_u32(sdS), HALF, s_mn);
      auto issue_dp = [&]() {         // dP^T(n) = V dO(n)^T
        if (elect_one()) {
          umma8_ss(t_dp, v_km, 0, o_km, 0, id_kk, 0u);
          umma_commit(dp_full);
          umma_commit(do_empty);
        }
        __syncwarp();
      };
      if (ok && nsteps > 0) ok = wait_or_fail(do_full, 0, 202);
      if (ok && nsteps > 0) {
        tc_fence_after_sync();
        issue_dp();
      }
      for (int n = 0; ok && n < nsteps; ++n) {
        const uint32_t par = n & 1;
        if (!(ok = wait_or_fail(ds_full, par, 230))) break;
        tc_fence_after_sync();
        // dQ first: its drain (and then dP^T of the next step, which re-uses the columns) is on the
        // critical path, dK is not
        if (elect_one()) {
          umma8_ss(t_dp, s_mn, 0, k_mn, 0, id_mm, 0u);
          umma_commit(dq_full);
          umma8_ss(t_dk, s_km, 0, q_mn, (n & 1) * kTileAdd, id_km, n > 0 ? 1u : 0u);
          umma_commit(&q_empty[n & 1]);
        }
        __syncwarp();
        if (n + 1 < nsteps) {
          if (!(ok = wait_or_fail(do_full, par ^ 1, 235))) break;
          if (!(ok = wait_or_fail(dq_read, par, 240))) break;
          tc_fence_after_sync();
          issue_dp();
        }
      }
    }
    if (ok && elect_one()) umma_commit(done_full);
    __syncwarp();
  } else if (warp < 10) {
    // ---- softmax warps: thread (r, hf) owns key/value position j*128 + r and query positions
    //      [hf*64, hf*64 + 64) of the step's tile ----
    const int q = warp & 3;
    const int hf = (warp - 2) >> 2;
    const int r = q * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    const uint32_t t_s_mine = t_s + lane_addr + hf * 64;     // my 64 score columns; P^T goes to the first 32
    const uint32_t t_dp_mine = t_dp + lane_addr + hf * 64;
    bool ok = true;
    int tile_in_head = 0;
    for (int n = 0; n < nsteps; ++n) {
      const uint32_t par = n & 1;
      const int st = n & 1;
      const bool diag = tile_in_head == 0;     // first query tile of a head = the diagonal block
      if (++tile_in_head == tiles) tile_in_head = 0;
      if (!mbar_wait(&stats_full[st], (n >> 1) & 1, timeout, abort_flag) ||
          !mbar_wait(s_full, par, timeout, abort_flag)) {
        if (lane == 0) report_status(a.status, kStatusMbarTimeout, kKernelIdFlashBwd2, 300, 0, 0);
        ok = false;
        break;
      }
      tc_fence_after_sync();
      uint32_t pk[32];    // my 64 P^T values, bf16 pairs along the query positions
      {
        uint32_t sv[2][32];
        tmem_ld_32x32(t_s_mine, sv[0]);
        tmem_ld_32x32(t_s_mine + 32, sv[1]);
        tmem_ld_wait();
        const float4* l4 = reinterpret_cast<const float4*>(s_lse + st * 128 + hf * 64);
#pragma unroll
        for (int c = 0; c < 2; ++c) {
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const float4 l = l4[c * 8 + u];
            float p0 = fast_exp2(fmaf(__uint_as_float(sv[c][4 * u + 0]), a.scale_log2, -l.x));
            float p1 = fast_exp2(fmaf(__uint_as_float(sv[c][4 * u + 1]), a.scale_log2, -l.y));
            float p2 = fast_exp2(fmaf(__uint_as_float(sv[c][4 * u + 2]), a.scale_log2, -l.z));
            float p3 = fast_exp2(fmaf(__uint_as_float(sv[c][4 * u + 3]), a.scale_log2, -l.w));
            if (diag) {   // causal: key position r may not exceed the query position
              const int col = hf * 64 + c * 32 + 4 * u;
              p0 = (r > col + 0) ? 0.f : p0;
              p1 = (r > col + 1) ? 0.f : p1;
              p2 = (r > col + 2) ? 0.f : p2;
              p3 = (r > col + 3) ? 0.f : p3;
            }
            pk[c * 16 + 2 * u] = pack_bf16x2(p0, p1);
            pk[c * 16 + 2 * u + 1] = pack_bf16x2(p2, p3);
          }
        }
      }
      tmem_st_32x32(t_s_mine, pk);
      tmem_st_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);

      if (!mbar_wait(dp_full, par, timeout, abort_flag)) {
        if (lane == 0) report_status(a.status, kStatusMbarTimeout, kKernelIdFlashBwd2, 310, 0, 0);
        ok = false;
        break;
      }
      tc_fence_after_sync();
      {
        uint32_t dv[2][32];
        tmem_ld_32x32(t_dp_mine, dv[0]);
        tmem_ld_32x32(t_dp_mine + 32, dv[1]);
        tmem_ld_wait();
        const float4* d4 = reinterpret_cast<const float4*>(s_dl + st * 128 + hf * 64);
        uint8_t* drow = sdS + hf * (kTileBytes / 2) + r * 128;
#pragma unroll
        for (int w = 0; w < 8; ++w) {     // 8 query positions = one 16-byte chunk
          const int c = w >> 2, e0 = (w & 3) * 8;
          const float4 da = d4[w * 2], db = d4[w * 2 + 1];
          const float dl[8] = {da.x, da.y, da.z, da.w, db.x, db.y, db.z, db.w};
          uint32_t o[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const __nv_bfloat162 pp = *reinterpret_cast<const __nv_bfloat162*>(&pk[w * 4 + e]);
            const float d0 = __low2float(pp) * (__uint_as_float(dv[c][e0 + 2 * e]) - dl[2 * e]);
            const float d1 = __high2float(pp) * (__uint_as_float(dv[c][e0 + 2 * e + 1]) - dl[2 * e + 1]);
            o[e] = pack_bf16x2(d0, d1);
          }
          const int chunk = w ^ (r & 7);
          *reinterpret_cast<uint4*>(drow + chunk * 16) = make_uint4(o[0], o[1], o[2], o[3]);
        }
      }
      fence_proxy_async_smem();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(ds_full);
    }
    if (ok && nsteps > 0 && mbar_wait(done_full, 0, timeout, abort_flag)) {
      // dK / dV of this block: each warp converts its 64 columns
      tc_fence_after_sync();
      const int kvrow = j * kFaBN + r;
      __nv_bfloat16* dk_dst = a.dqkv + (((long long)kvrow * a.b + bb) * a.G + g) * hpg * kFaD + a.qpg * kFaD;
      __nv_bfloat16* dv_dst = dk_dst + kFaD;
#pragma unroll 1
      for (int c = hf * 2; c < hf * 2 + 2; ++c) {
        uint32_t vk[32], vv[32];
        tmem_ld_32x32(t_dk + lane_addr + c * 32, vk);
        tmem_ld_32x32(t_dv + lane_addr + c * 32, vv);
        tmem_ld_wait();
        if (kvrow < a.s && a.hsplit > 1) {
          // several CTAs share this K/V block: add into the fp32 accumulators
          float* acc = a.dkv_accum + ((((long long)kvrow * a.b + bb) * a.G + g) * 2) * kFaD + c * 32;
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            red_add_v4_f32(acc + 4 * u, __uint_as_float(vk[4 * u]) * a.scale, __uint_as_float(vk[4 * u + 1]) * a.scale,
                           __uint_as_float(vk[4 * u + 2]) * a.scale, __uint_as_float(vk[4 * u + 3]) * a.scale);
            red_add_v4_f32(acc + kFaD + 4 * u, __uint_as_float(vv[4 * u]), __uint_as_float(vv[4 * u + 1]),
                           __uint_as_float(vv[4 * u + 2]), __uint_as_float(vv[4 * u + 3]));
          }
        } else if (kvrow < a.s) {
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            uint4 k4, v4;
            k4.x = pack_bf16x2(__uint_as_float(vk[8 * u]) * a.scale, __uint_as_float(vk[8 * u + 1]) * a.scale);
            k4.y = pack_bf16x2(__uint_as_float(vk[8 * u + 2]) * a.scale, __uint_as_float(vk[8 * u + 3]) * a.scale);
            k4.z = pack_bf16x2(__uint_as_float(vk[8 * u + 4]) * a.scale, __uint_as_float(vk[8 * u + 5]) * a.scale);
            k4.w = pack_bf16x2(__uint_as_float(vk[8 * u + 6]) * a.scale, __uint_as_float(vk[8 * u + 7]) * a.scale);
            v4.x = pack_bf16x2(__uint_as_float(vv[8 * u]), __uint_as_float(vv[8 * u + 1]));
            v4.y = pack_bf16x2(__uint_as_float(vv[8 * u + 2]), __uint_as_float(vv[8 * u + 3]));
            v4.z = pack_bf16x2(__uint_as_float(vv[8 * u + 4]), __uint_as_float(vv[8 * u + 5]));
            v4.w = pack_bf16x2(__uint_as_float(vv[8 * u + 6]), __uint_as_float(vv[8 * u + 7]));
            reinterpret_cast<uint4*>(dk_dst)[c * 4 + u] = k4;
            reinterpret_cast<uint4*>(dv_dst)[c * 4 + u] = v4;
          }
        }
      }
    }
    tc_fence_before_sync();
  } else if (warp < 14) {
    // ---- dQ drain warps: warp `q` owns query rows [32q, 32q + 32) of the step's tile and moves them
    //      in two halves of 64 columns: TMEM -> registers -> two swizzled [32 rows][32 fp32] boxes in
    //      shared memory -> TMA reduce-add into the fp32 dQ buffer. ----
    const int q = warp & 3;
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    uint8_t* my_stage = sStage + q * 8192;
    // These warps also fetch the per-row statistics (log-sum-exp, delta) of the query tiles for the
    // softmax warps: one row per thread, loaded two steps ahead, published one step ahead.
    const int r = q * 32 + lane;
    int ld_tile = 0, ld_head = head0;          // (tile, head) of the next step to load
    auto load_stats = [&](float& l2, float& dl) {
      const int row = (j + ld_tile) * kFaBM + r;
      const long long off = ((long long)bb * hq + g * a.qpg + ld_head) * a.s + row;
      const bool row_ok = row < a.s;
      // rows past the end get lse = +inf, which turns their probabilities into exact zeros
      l2 = row_ok ? a.lse[off] : INFINITY;
      dl = row_ok ? a.delta[off] : 0.f;
      if (++ld_tile == tiles) {
        ld_tile = 0;
        ++ld_head;
      }
    };
    float nl2 = 0.f, ndl = 0.f;
    if (nsteps > 0) {
      load_stats(nl2, ndl);
      s_lse[r] = nl2 * 1.4426950408889634f;
      s_dl[r] = ndl;
      mbar_arrive(&stats_full[0]);
      if (nsteps > 1) load_stats(nl2, ndl);     // statistics of step 1, published at the top of step 0
    }
    int cur_tile = 0, cur_head = head0;
    for (int n = 0; n < nsteps; ++n) {
      // stage (n+1)&1 was last read in step n-1, which every softmax warp left before dQ(n-1) existed
      if (n + 1 < nsteps) {
        s_lse[((n + 1) & 1) * 128 + r] = nl2 * 1.4426950408889634f;
        s_dl[((n + 1) & 1) * 128 + r] = ndl;
        mbar_arrive(&stats_full[(n + 1) & 1]);
        if (n + 2 < nsteps) load_stats(nl2, ndl);
      }
      const int hi = cur_head, i = j + cur_tile;
      if (++cur_tile == tiles) {
        cur_tile = 0;
        ++cur_head;
      }
      const int h = g * a.qpg + hi;
      const int row0 = i * kFaBM + q * 32;       // first query row of my box
      if (!mbar_wait(dq_full, n & 1, timeout, abort_flag)) {
        if (lane == 0) report_status(a.status, kStatusMbarTimeout, kKernelIdFlashBwd2, 400, 0, 0);
        break;
      }
      tc_fence_after_sync();
      // Two halves of 64 columns: both boxes of the first half are filled and the second half is
      // already in registers when the TMEM columns are released to the tensor core.
      uint32_t va[2][32];
      tmem_ld_32x32(t_dp + lane_addr, va[0]);
      tmem_ld_32x32(t_dp + lane_addr + 32, va[1]);
      if (lane == 0) bulk_wait_group_read<0>();   // both boxes of the previous step have been read
      tmem_ld_wait();
      __syncwarp();
      auto put_box = [&](int slot, const uint32_t* v) {
        uint8_t* brow = my_stage + slot * 4096 + lane * 128;
#pragma unroll
        for (int c = 0; c < 8; ++c)
          *reinterpret_cast<uint4*>(brow + ((c ^ (lane & 7)) * 16)) =
              make_uint4(v[4 * c], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]);
      };
      auto reduce_boxes = [&](int first_col) {
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          if (row0 < a.s) {
            tma_reduce_add_2d(&tmap_dq, my_stage, ((bb * hq + h) * kFaD) + first_col, row0);
            tma_reduce_add_2d(&tmap_dq, my_stage + 4096, ((bb * hq + h) * kFaD) + first_col + 32, row0);
          }
          bulk_commit_group();
        }
      };
      put_box(0, va[0]);
      put_box(1, va[1]);
      tmem_ld_32x32(t_dp + lane_addr + 64, va[0]);
      tmem_ld_32x32(t_dp + lane_addr + 96, va[1]);
      reduce_boxes(0);
      tmem_ld_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(dq_read);          // every value has left TMEM
        bulk_wait_group_read<0>();     // the first half's boxes have been read
      }
      __syncwarp();
      put_box(0, va[0]);
      put_box(1, va[1]);
      reduce_boxes(64);
    }
    if (lane == 0) bulk_wait_group<0>();    // all reductions have been performed
    tc_fence_before_sync();
  }

  if (*abort_flag) {
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace fm

typedef CUresult (*EncodeTiledFn2)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

extern "C" int fm_flash_attn_fwd(const void* qkv, void* out, float* lse, int s, int b, int G, int qpg, int d,
                                 float scale, unsigned long long timeout_ns, int* status, int version,
                                 cudaStream_t stream) {
  return fm_flash_attn_fwd_push(qkv, out, lse, s, b, G, qpg, d, scale, timeout_ns, status, version, nullptr, nullptr,
                                0, 1, 0, 0, stream);
}

extern "C" int fm_flash_attn_fwd_push(const void* qkv, void* out, float* lse, int s, int b, int G, int qpg, int d,
                                      float scale, unsigned long long timeout_ns, int* status, int version,
                                      void* const* push_dst, int* const* push_flags, int push_me, int push_P,
                                      int push_sl, int push_row_blocks, cudaStream_t stream) {
  if (push_dst != nullptr && (version != 2 || b != 1 || push_sl <= 0 || push_sl % 128 != 0 || push_P * push_sl != s)) {
    fm_set_error("flash_attn_fwd: the epilogue exchange needs the default kernel, batch 1 and 128 | rows per rank");
    return -1;
  }
  if (d != fm::kFaD) {
    fm_set_error("flash_attn_fwd: head_dim must be 128");
    return -1;
  }
  static EncodeTiledFn2 enc = nullptr;
  if (!enc) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess) {
      fm_set_error("cuTensorMapEncodeTiled unavailable");
      return -2;
    }
    enc = reinterpret_cast<EncodeTiledFn2>(p);
  }
  const long long cols = (long long)b * G * (qpg + 2) * d;
  if ((reinterpret_cast<uintptr_t>(qkv) & 15) != 0) {
    fm_set_error("flash_attn_fwd: qkv must be 16-byte aligned");
    return -1;
  }
  CUtensorMap tmap;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)s};
  cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
  cuuint32_t box[2] = {64, 128};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(&tmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(qkv), dims, strides,
                   box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    fm_set_error("flash_attn_fwd: cuTensorMapEncodeTiled failed");
    return -3;
  }
  constexpr int smem = 6 * fm::kTileBytes + 1024 + 256;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(fm::flash_fwd_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) {
      fm_set_error(cudaGetErrorString(e));
      return (int)e;
    }
    configured = true;
  }
  fm::FlashFwdArgs a;
  a.s = s; a.b = b; a.G = G; a.qpg = qpg;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.out = reinterpret_cast<__nv_bfloat16*>(out);
  a.lse = lse;
  a.timeout_ns = timeout_ns ? timeout_ns : 4000000000ull;
  a.status = status;
  a.prof = nullptr;
  constexpr int kMaxFwd2Version = 28;
  a.qkv = reinterpret_cast<const __nv_bfloat16*>(qkv);
  a.row_stride = cols;
  a.push_dst = reinterpret_cast<__nv_bfloat16* const*>(push_dst);
  a.push_flags = push_flags;
  a.push_me = push_me; a.push_P = push_P; a.push_sl = push_sl; a.push_row_blocks = push_row_blocks;
  if (version == 3 || (version >= 30 && version <= 34)) {
    using Fwd3Fn = void (*)(const CUtensorMap, const fm::FlashFwdArgs);
    // 30: special-function exponentials only; 32: two of every four values on the FMA pipe
    static const Fwd3Fn kFwd3[5] = {fm::flash_fwd3_kernel<0>, fm::flash_fwd3_kernel<0>, fm::flash_fwd3_kernel<2>,
                                    fm::flash_fwd3_kernel<2>, fm::flash_fwd3_kernel<2>};
    const int variant = version == 3 ? fm::kFa3DefaultPoly : version - 30;
    constexpr int smem3 = (1 + 2 * fm::kFa3Stages) * fm::kTileBytes + 1024 + 2048;
    static bool configured3[5] = {false, false, false, false, false};
    if (!configured3[variant]) {
      cudaError_t e3 = cudaFuncSetAttribute(kFwd3[variant], cudaFuncAttributeMaxDynamicSharedMemorySize, smem3);
      if (e3 != cudaSuccess) {
        fm_set_error(cudaGetErrorString(e3));
        return (int)e3;
      }
      configured3[variant] = true;
    }
    const int nq3 = (s + fm::kFaBM - 1) / fm::kFaBM;
    dim3 grid3((unsigned)(nq3 * G * qpg * b), 1, 1);
#ifdef FM_FLASH_PROFILE
    static long long* prof3_dev = nullptr;
    const size_t prof3_n = (size_t)grid3.x * 16;
    if (getenv("FLUIDMOE_FLASH_PROFILE") != nullptr) {
      cudaFree(prof3_dev);
      cudaMalloc(&prof3_dev, prof3_n * sizeof(long long));
      cudaMemset(prof3_dev, 0, prof3_n * sizeof(long long));
      a.prof = prof3_dev;
    }
#endif
    kFwd3[variant]<<<grid3, fm::kFa3Threads, smem3, stream>>>(tmap, a);
#ifdef FM_FLASH_PROFILE
    if (a.prof != nullptr) {
      cudaStreamSynchronize(stream);
      std::vector<long long> hp(prof3_n);
      cudaMemcpy(hp.data(), prof3_dev, prof3_n * sizeof(long long), cudaMemcpyDeviceToHost);
      double sum[16] = {0};
      for (size_t c = 0; c < grid3.x; ++c)
        for (int k = 0; k < 16; ++k) sum[k] += (double)hp[c * 16 + k];
      const double mb = sum[3] > 0 ? sum[3] : 1, sb = sum[10] > 0 ? sum[10] : 1;
      fprintf(stderr,
              "[flash_fwd3 profile v%d] cycles: mma thread per block %.0f (wait P %.0f, wait K/V %.0f) | softmax "
              "thread per own block %.0f: wait S %.0f, max pass %.0f, wait other group %.0f, rescale %.0f, exp pass %.0f\n",
              version, sum[0] / mb, sum[1] / mb, sum[2] / mb, sum[4] / sb, sum[5] / sb, sum[7] / sb, sum[6] / sb,
              sum[8] / sb, sum[9] / sb);
    }
#endif
  } else if (version == 2 || (version >= 20 && version <= kMaxFwd2Version)) {
    // versions 20..24 pick the share of polynomial exponentials (0..4 of every 4 pairs)
    using Fwd2Fn = void (*)(const CUtensorMap, const fm::FlashFwdArgs);
    // 20: one issuing lane, special-function exponentials; 22: two of every four exponentials on the FMA
    // pipe; 25: developer timing experiment; 26: the whole MMA warp
    // walks the issue loop (uniform issue); 27 / 28: 26 with P handed over in two / four parts
    static const Fwd2Fn kFwd2[9] = {fm::flash_fwd2_kernel<0>, fm::flash_fwd2_kernel<0>, fm::flash_fwd2_kernel<2>,
                                    fm::flash_fwd2_kernel<2>, fm::flash_fwd2_kernel<2>,
#ifdef FM_FLASH_PROFILE
                                    fm::flash_fwd2_kernel<5>,
#else
                                    fm::flash_fwd2_kernel<0>,
#endif
                                    fm::flash_fwd2_kernel<0, true>, fm::flash_fwd2_kernel<0, true, 2>,
                                    fm::flash_fwd2_kernel<0, true, 4>};
    const int variant = version == 2 ? fm::kFa2DefaultPoly : version - 20;
    constexpr int smem2 = smem;
    static bool configured2[9] = {false, false, false, false, false, false, false, false, false};
    if (!configured2[variant]) {
      cudaError_t e2 = cudaFuncSetAttribute(kFwd2[variant], cudaFuncAttributeMaxDynamicSharedMemorySize, smem2);
      if (e2 != cudaSuccess) {
        fm_set_error(cudaGetErrorString(e2));
        return (int)e2;
      }
      configured2[variant] = true;
    }
    const int nq = (s + fm::kFaBM - 1) / fm::kFaBM;
    dim3 grid2((unsigned)(((nq + 1) / 2) * G * qpg * b), 1, 1);
#ifdef FM_FLASH_PROFILE
    // developer build: synchronous launch, then the per-CTA counters averaged over the CTAs
    static long long* prof_dev = nullptr;
    const size_t prof_n = (size_t)grid2.x * 16 + 16 * 16;
    if (getenv("FLUIDMOE_FLASH_PROFILE") != nullptr) {
      cudaFree(prof_dev);
      cudaMalloc(&prof_dev, prof_n * sizeof(long long));
      cudaMemset(prof_dev, 0, prof_n * sizeof(long long));
      a.prof = prof_dev;
    }
#endif
    kFwd2[variant]<<<grid2, fm::kFa2Threads, smem2, stream>>>(tmap, a);
#ifdef FM_FLASH_PROFILE
    if (a.prof != nullptr) {
      cudaStreamSynchronize(stream);
      std::vector<long long> hp(prof_n);
      cudaMemcpy(hp.data(), prof_dev, prof_n * sizeof(long long), cudaMemcpyDeviceToHost);
      double sum[16] = {0};
      for (size_t c = 0; c < grid2.x; ++c)
        for (int k = 0; k < 16; ++k) sum[k] += (double)hp[c * 16 + k];
      const double mb = sum[3] > 0 ? sum[3] : 1, sb = sum[10] > 0 ? sum[10] : 1;
      {
        const long long* tr = hp.data() + (size_t)grid2.x * 16;
        const long long base = tr[0];
        const char* ev[8] = {"mma:waitP", "mma:gotP", "mma:PVissued", "mma:QKissued", "smx:gotS", "smx:max", "smx:Pdone", ""};
        for (int jj = 0; jj < 6; ++jj)
          for (int w = 0; w < 2; ++w) {
            fprintf(stderr, "  trace block %d tile %d:", jj + 8, w);
            for (int e = 0; e < 7; ++e) fprintf(stderr, " %s=%lld", ev[e], tr[jj * 16 + w * 8 + e] - base);
            fprintf(stderr, "\n");
          }
      }
      fprintf(stderr,
              "[flash_fwd2 profile v%d] per tile-block, cycles: mma thread total %.0f (wait P %.0f, wait K/V %.0f) | "
              "softmax thread total %.0f: wait S %.0f, (unused %.0f), max pass %.0f, rescale %.0f, exp pass %.0f\n",
              version, sum[0] / mb, sum[1] / mb, sum[2] / mb, sum[4] / sb, sum[5] / sb, sum[6] / sb, sum[7] / sb,
              sum[8] / sb, sum[9] / sb);
    }
#endif
  } else {
    dim3 grid((s + fm::kFaBM - 1) / fm::kFaBM, G * qpg, b);
    fm::flash_fwd_kernel<<<grid, fm::kFaThreads, smem, stream>>>(tmap, a);
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    fm_set_error(cudaGetErrorString(e));
    return (int)e;
  }
  return 0;
}

static bool make_rows_tmap_impl(CUtensorMap* m, const void* ptr, long long cols, long long rows, bool f32);
static bool make_rows_tmap(CUtensorMap* m, const void* ptr, long long cols, long long rows) {
  return make_rows_tmap_impl(m, ptr, cols, rows, false);
}
// fp32 [rows, cols] tensor, boxes of [32 rows][32 columns] (128 bytes per row, 128-byte swizzle)
static bool make_f32_box_tmap(CUtensorMap* m, const void* ptr, long long cols, long long rows) {
  return make_rows_tmap_impl(m, ptr, cols, rows, true);
}
static bool make_rows_tmap_impl(CUtensorMap* m, const void* ptr, long long cols, long long rows, bool f32) {
  static EncodeTiledFn2 enc = nullptr;
  if (!enc) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return false;
    enc = reinterpret_cast<EncodeTiledFn2>(p);
  }
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)cols * (f32 ? 4 : 2)};
  cuuint32_t box[2] = {f32 ? 32u : 64u, f32 ? 32u : 128u};
  cuuint32_t estr[2] = {1, 1};
  return enc(m, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
             const_cast<void*>(ptr), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

extern "C" int fm_flash_attn_bwd(const void* qkv, const void* out, const void* dout, const float* lse,
                                 float* delta, float* dq_accum, void* dqkv, int s, int b, int G, int qpg,
                                 int d, float scale, unsigned long long timeout_ns, int* status,
                                 int version, float* dkv_accum, int hsplit, cudaStream_t stream) {
  return fm_flash_attn_bwd_gated(qkv, out, dout, lse, delta, dq_accum, dqkv, s, b, G, qpg, d, scale, timeout_ns,
                                 status, version, dkv_accum, hsplit, nullptr, 0, 0, nullptr, stream);
}

extern "C" int fm_flash_attn_bwd_gated(const void* qkv, const void* out, const void* dout, const float* lse,
                                       float* delta, float* dq_accum, void* dqkv, int s, int b, int G, int qpg,
                                       int d, float scale, unsigned long long timeout_ns, int* status,
                                       int version, float* dkv_accum, int hsplit, const int* wait_flags,
                                       int wait_n, int wait_expected, unsigned long long* wait_ns,
                                       cudaStream_t stream) {
  if (wait_n > 256) {
    fm_set_error("flash_attn_bwd: at most 256 sources");
    return -1;
  }
  if (d != fm::kFaD) {
    fm_set_error("flash_attn_bwd: head_dim must be 128");
    return -1;
  }
  const int hq = G * qpg;
  if ((reinterpret_cast<uintptr_t>(qkv) & 15) || (reinterpret_cast<uintptr_t>(dout) & 15) ||
      (reinterpret_cast<uintptr_t>(dq_accum) & 15) || (reinterpret_cast<uintptr_t>(dqkv) & 15)) {
    fm_set_error("flash_attn_bwd: buffers must be 16-byte aligned");
    return -1;
  }
  CUtensorMap tq, tdo;
  if (!make_rows_tmap(&tq, qkv, (long long)b * G * (qpg + 2) * d, s) ||
      !make_rows_tmap(&tdo, dout, (long long)b * hq * d, s)) {
    fm_set_error("flash_attn_bwd: cuTensorMapEncodeTiled failed");
    return -3;
  }
  const long long nrows = (long long)s * b * hq;
  fm::attn_delta_kernel<<<(unsigned)((nrows + 7) / 8), 256, 0, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(out), reinterpret_cast<const __nv_bfloat16*>(dout), delta, s, b, hq,
      wait_flags, wait_n, wait_expected, wait_ns, timeout_ns ? timeout_ns : 4000000000ull, status);
  constexpr int smem = 6 * fm::kTileBytes + 1024 + 256;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(fm::flash_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) {
      fm_set_error(cudaGetErrorString(e));
      return (int)e;
    }
    configured = true;
  }
  fm::FlashBwdArgs a;
  a.s = s; a.b = b; a.G = G; a.qpg = qpg;
  a.scale = scale;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.lse = lse;
  a.delta = delta;
  a.dq_accum = dq_accum;
  a.dqkv = reinterpret_cast<__nv_bfloat16*>(dqkv);
  a.timeout_ns = timeout_ns ? timeout_ns : 4000000000ull;
  a.status = status;
  a.hsplit = 1;
  a.dkv_accum = nullptr;
  dim3 grid((s + fm::kFaBN - 1) / fm::kFaBN, G, b);
  if (version == 2) {
    static bool configured2 = false;
    if (!configured2) {
      cudaError_t e2 = cudaFuncSetAttribute(fm::flash_bwd2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            fm::kFaB2Smem);
      if (e2 != cudaSuccess) {
        fm_set_error(cudaGetErrorString(e2));
        return (int)e2;
      }
      configured2 = true;
    }
    CUtensorMap tdq;
    if (!make_f32_box_tmap(&tdq, dq_accum, (long long)b * hq * d, s)) {
      fm_set_error("flash_attn_bwd: cuTensorMapEncodeTiled failed (dQ)");
      return -3;
    }
    if (hsplit > 1 && dkv_accum != nullptr && qpg % hsplit == 0 &&
        (reinterpret_cast<uintptr_t>(dkv_accum) & 15) == 0) {
      a.hsplit = hsplit;
      a.dkv_accum = dkv_accum;
      grid.y = G * hsplit;
    }
    dim3 grid_lin(grid.x * grid.y * grid.z, 1, 1);
    fm::flash_bwd2_kernel<<<grid_lin, fm::kFaB2Threads, fm::kFaB2Smem, stream>>>(tq, tdo, tdq, a);
    fm::attn_dq_store_kernel<<<148 * 8, 256, 0, stream>>>(dq_accum, a.dqkv, (long long)s * b, G, qpg, scale);
    if (a.hsplit > 1)
      fm::attn_dkv_store_kernel<<<148 * 4, 256, 0, stream>>>(dkv_accum, a.dqkv, (long long)s * b, G, qpg);
  } else {
    fm::flash_bwd_kernel<<<grid, fm::kFaThreads, smem, stream>>>(tq, tdo, a);
    fm::attn_dq_store_kernel<<<148 * 8, 256, 0, stream>>>(dq_accum, a.dqkv, (long long)s * b, G, qpg, 1.0f);
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    fm_set_error(cudaGetErrorString(e));
    return (int)e;
  }
  return 0;
}
