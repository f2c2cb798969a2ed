// Persistent, warp-specialised tcgen05 GEMM for sm_100a.
//
// One CTA (or a CTA pair sharing a 256 x BN tile through tcgen05.mma.cta_group::2) per SM walks a
// list of output tiles: a static one for the single CTA, one claimed tile by tile from a counter for
// the CTA pair (`TileOrder`), so that pairs which start late, because a collective kernel holds
// their SMs, do fewer tiles instead of making the whole GEMM late.  Warp 0 feeds a shared-memory ring (5 stages for the CTA pair, 4 or 3
// for a single CTA) with TMA tiled loads
// (128-byte swizzle), warp 1 issues tcgen05.mma with the accumulator in TMEM (two accumulators, so
// the epilogue of tile i overlaps the main loop of tile i+1), warps 2-9 (two per TMEM lane quarter,
// each half of the columns) drain TMEM with tcgen05.ld and run a pluggable epilogue.  A pluggable
// gate lets the producer wait (bounded) for a flag before it touches the rows of a tile, which is
// how arriving peer data is consumed tile by tile.
//
// Two problem shapes share the kernel:
//   mode 0 (grouped-M): C[rows_g, N] = A[rows_g, K] * B_g, groups partition the rows of A;
//                       one group == an ordinary dense GEMM.
//   mode 1 (grouped-K): C_g[M, N] (+)= A[rows_g, M]^T * B[rows_g, N]; the weight-gradient
//                       shape, where the contraction runs over the rows of group g.
// Operand majors are template parameters: A and B may each be K-major or MN-major; MN-major
// tiles are loaded as 64-element-wide boxes and described to the MMA through LBO/SBO.
//
// This is the counterpart of the reference's grouped GEMM helpers, which call cuBLAS or an
// external CUTLASS grouped GEMM (fluid/moe/forward.py:217-352, fluid/moe/backward.py:400-480).
#pragma once
#include "../include/sm100_ptx.cuh"

namespace fm {

constexpr int kBM = 128;
constexpr int kBK = 64;
constexpr int kStages = 4;                 // BN = 128; the 256-wide single-CTA tile uses 3
constexpr int kEpiStageFloats = 32 * 36;   // per epilogue warp: 32 rows x 32 columns, padded rows
constexpr int kEpiWarps = 8;    // two warps per TMEM lane quarter, each takes half the columns
constexpr int kGemmThreads = 64 + 32 * kEpiWarps;
constexpr int kKernelIdGemm = 1;
constexpr int kKernelIdGemm2 = 2;

struct GemmArgs {
  int mode;          // 0 grouped-M, 1 grouped-K
  int num_groups;
  int M;             // mode 0: rows of A when group_rows == nullptr and num_groups == 1
                     // mode 1: output rows (columns of A)
  int N;             // output columns produced per tile row (gated: activation columns)
  int K;             // mode 0: contraction length; mode 1: unused
  int uniform_rows;  // rows per group when group_rows == nullptr
  const int* group_rows;  // device, [num_groups], may be nullptr
  const int* group_offs;  // device, [num_groups] row offset of each group in A (and C)
  const int* group_b;     // device, [num_groups]: which B matrix a group uses (nullptr: g)
  int b_group_stride;     // mode 0: rows of the flattened 2-D B between groups
  int gated;              // B holds [gate | up] column halves, tile = 128 gate + 128 up
  int n_half;             // column offset of the `up` half inside B
  int swizzle_m;          // m-tiles per rasterisation super-row (L2 reuse)
  int mn3d;               // MN-major operands are fetched with one 3-D box per tile
  int n_rotate;           // tiles visit N starting at this tile index (destination round-robin)
  int k_rotate;           // the K loop starts at this 64-wide block (local source first)
  unsigned long long timeout_ns;
  int* status;
  // Optional device counter (nullptr = off): nanoseconds the producers of all CTAs spent
  // waiting in a gate for rows that had not arrived yet.  Divided by the number of CTAs it
  // bounds the communication time this kernel could not hide.
  unsigned long long* wait_ns;
  // Dynamic tile order of the CTA-pair kernel (nullptr = every pair walks tiles pair, pair + pairs,
  // ...).  `sched_ctr` is this launch's claim counter (zero at launch), `sched_ctr_reset` a counter
  // that no launch in flight uses and that this launch zeroes for a later one, `sched_log` holds
  // `sched_cap` entries per pair: entry j = (sched_epoch << 32 | tile) is the j-th tile of the pair.
  int* sched_ctr;
  int* sched_ctr_reset;
  unsigned long long* sched_log;
  int sched_cap;
  unsigned int sched_epoch;
};

struct Tile {
  int g;           // group
  int m0;          // mode 0: row offset inside the group; mode 1: offset in output rows
  int n_tile;      // tile index along N
  int rows_valid;  // rows of this tile that exist (<= 128)
  int row_base;    // first row of group g in A
  int nk;          // number of 64-wide K blocks
  int rows_g;      // rows in the group
};

template <int BN, int TM = kBM>
struct TileWalker {
  const GemmArgs& a;
  int g = 0;
  int base = 0;  // tiles before group g
  int nt, mt_fixed;
  __device__ TileWalker(const GemmArgs& args) : a(args) {
    const int n_per_tile = a.gated ? BN / 2 : BN;
    nt = (a.N + n_per_tile - 1) / n_per_tile;
    mt_fixed = (a.M + TM - 1) / TM;
  }
  __device__ __forceinline__ int rows_of(int gi) const {
    return a.group_rows ? a.group_rows[gi] : a.uniform_rows;
  }
  __device__ __forceinline__ int off_of(int gi) const {
    return a.group_offs ? a.group_offs[gi] : gi * a.uniform_rows;
  }
  __device__ __forceinline__ int mtiles_of(int gi) const {
    return a.mode == 0 ? (rows_of(gi) + TM - 1) / TM : mt_fixed;
  }
  // t must not decrease between calls.
  __device__ bool get(int t, Tile& out) {
    while (g < a.num_groups) {
      const int mt = mtiles_of(g);
      const int cnt = mt * nt;
      if (t < base + cnt) {
        const int l = t - base;
        const int sw = a.swizzle_m > 0 ? a.swizzle_m : 8;
        const int per_super = sw * nt;
        const int super = l / per_super;
        const int first_m = super * sw;
        const int gsz = min(sw, mt - first_m);
        const int in_super = l - super * per_super;
        const int m_tile = first_m + in_super % gsz;
        out.n_tile = (in_super / gsz + a.n_rotate) % nt;
        out.g = g;
        out.m0 = m_tile * TM;
        out.rows_g = rows_of(g);
        out.row_base = off_of(g);
        if (a.mode == 0) {
          out.rows_valid = min(TM, out.rows_g - out.m0);
          out.nk = (a.K + kBK - 1) / kBK;
        } else {
          out.rows_valid = min(TM, a.M - out.m0);
          out.nk = (out.rows_g + kBK - 1) / kBK;
        }
        return true;
      }
      base += cnt;
      ++g;
    }
    return false;
  }
};

// Which tile a CTA pair computes j-th.  Static order: pair, pair + pairs, ...  Dynamic order: the
// first tile is the static one, every further tile is claimed from a counter in global memory by
// the leader CTA's producer lane, which writes it into the pair's row of a log in global memory; the
// other roles of both CTAs (peer producer, MMA warp, epilogue warps) read the log.  An entry is one
// 64-bit word (launch epoch << 32 | tile), so a reader needs no ordering beyond the load itself, and
// entries of earlier launches never match.  A persistent kernel with a static order finishes as
// late as its slowest pair: when a collective kernel on another stream holds a few SMs, the pairs
// that could not start until it left still had their full share of tiles to do, and the GEMM took
// its own time plus the collective's.  With claimed tiles the late pairs simply do fewer.
struct TileOrder {
  unsigned long long* row;
  int* ctr;
  unsigned int epoch;
  int cap, pair_id, num_pairs;
  __device__ TileOrder(const GemmArgs& a, int pair, int pairs)
      : row(a.sched_log ? a.sched_log + (size_t)pair * a.sched_cap : nullptr), ctr(a.sched_ctr),
        epoch(a.sched_epoch), cap(a.sched_cap), pair_id(pair), num_pairs(pairs) {}
  __device__ __forceinline__ bool dynamic() const { return row != nullptr; }
  __device__ __forceinline__ int claim() const { return num_pairs + atomicAdd(ctr, 1); }
  __device__ __forceinline__ bool publish(int j, int tile, int* status, volatile int* abort_flag) const {
    if (j >= cap) {   // the host sized the log for every tile of the problem: cannot happen
      report_status(status, kStatusBadArgs, kKernelIdGemm2, 900, cap, j);
      *abort_flag = 1;
      return false;
    }
    const unsigned long long v = ((unsigned long long)epoch << 32) | (unsigned int)tile;
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(row + j), "l"(v) : "memory");
    return true;
  }
  // Raw entry j (issue early, decode late: the load's latency hides behind other work).
  __device__ __forceinline__ unsigned long long peek(int j) const {
    unsigned long long v = 0;
    if (j < cap) asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(row + j) : "memory");
    return v;
  }
  __device__ __forceinline__ bool valid(unsigned long long v) const { return (unsigned int)(v >> 32) == epoch; }
  // Tile j of this pair; -1 when the wait was given up (bounded like every other wait).
  __device__ __forceinline__ int get(int j, unsigned long long seen, unsigned long long timeout_ns, int* status,
                                     volatile int* abort_flag) const {
    if (!dynamic()) return pair_id + j * num_pairs;
    if (valid(seen)) return (int)(unsigned int)seen;
    if (j >= cap) return -1;
    const uint64_t t0 = global_timer_ns();
    while (true) {
      const unsigned long long v = peek(j);
      if (valid(v)) return (int)(unsigned int)v;
      if (*abort_flag) return -1;
      if (global_timer_ns() - t0 > timeout_ns) {
        report_status(status, kStatusFlagTimeout, kKernelIdGemm2, 901, j, (int)(v >> 32));
        *abort_flag = 1;
        return -1;
      }
      __nanosleep(100);
    }
  }
};

// An epilogue may declare `static constexpr bool kPrefetch = true` and a member
// `prefetch<BN>(tile, args, row, chalf)`; the epilogue warps then call it one tile ahead, before
// they wait for the current accumulator, so that operands the epilogue reads are already in L2.
template <class E, class = void>
struct EpiHasPrefetch { static constexpr bool value = false; };
template <class E>
struct EpiHasPrefetch<E, decltype((void)E::kPrefetch)> { static constexpr bool value = true; };

// No gating: every tile is ready when the kernel starts.
struct GateNone {
  __device__ __forceinline__ bool wait(const Tile&, const GemmArgs&, volatile int*) const {
    return true;
  }
  __device__ __forceinline__ bool wait_k(const Tile&, int, bool, const GemmArgs&, volatile int*) const {
    return true;
  }
};

// Per-row-block flags: rows [128*i, 128*i+128) of group g are ready once
// flags[flag_base(g) + i] >= (rows in the block) * expected.  Flags live in this GPU's memory and are bumped by the
// producer (possibly on another GPU) with a system-scope release after its stores.
struct GateRowBlockFlags {
  const int* flags;
  const int* group_flag_base;  // [num_groups] or nullptr (then g * blocks_per_group)
  int blocks_per_group;
  int expected;
  __device__ __forceinline__ bool wait(const Tile& t, const GemmArgs& a,
                                       volatile int* abort_flag) const {
    const int idx = (group_flag_base ? group_flag_base[t.g] : t.g * blocks_per_group) +
                    t.m0 / kBM;
    int observed = 0;
    // One arrival per row: a block is ready when as many rows arrived as it holds.
    const int want = t.rows_valid * expected;
    const uint64_t t0 = a.wait_ns ? global_timer_ns() : 0;
    const bool ok = flag_wait_ge(flags + idx, want, a.timeout_ns, abort_flag, &observed);
    if (a.wait_ns) atomicAdd(a.wait_ns, (unsigned long long)(global_timer_ns() - t0));
    if (ok) return true;
    report_status(a.status, kStatusFlagTimeout, kKernelIdGemm, idx, want, observed);
    return false;
  }
  __device__ __forceinline__ bool wait_k(const Tile&, int, bool, const GemmArgs&, volatile int*) const {
    return true;
  }
};

// Gating along K: the contraction dimension is a concatenation of column blocks that arrive from
// different source ranks (`kblocks_per_src` 64-wide blocks each).  Before the producer loads the
// first K block of a source for a row block it waits until that source has delivered all rows of
// the block: flags[src * row_blocks + row_block] >= rows in the block.  Used by the output
// projection after the HP->SP exchange and by the QKV input gradient.
struct GateKSource {
  const int* flags;
  int kblocks_per_src;
  int row_blocks;      // 128-row blocks per source
  int units_per_row;   // arrivals counted per row (1: whole rows; h: a row arrives head by head)
  __device__ __forceinline__ bool wait(const Tile&, const GemmArgs&, volatile int*) const {
    return true;
  }
  __device__ __forceinline__ bool wait_k(const Tile& t, int kb, bool first, const GemmArgs& a,
                                         volatile int* abort_flag) const {
    if (!first && kb % kblocks_per_src != 0) return true;
    const int src = kb / kblocks_per_src;
    const int idx = src * row_blocks + (t.row_base + t.m0) / kBM;
    int observed = 0;
    const uint64_t t0 = a.wait_ns ? global_timer_ns() : 0;
    const int want = t.rows_valid * units_per_row;
    const bool ok = flag_wait_ge(flags + idx, want, a.timeout_ns, abort_flag, &observed);
    if (a.wait_ns) atomicAdd(a.wait_ns, (unsigned long long)(global_timer_ns() - t0));
    if (ok) return true;
    report_status(a.status, kStatusFlagTimeout, kKernelIdGemm, 10000 + idx, want, observed);
    return false;
  }
};

template <int BN>
constexpr int gemm_stages() {
  return BN == 256 ? 3 : 4;
}
template <int BN>
constexpr int gemm_smem_bytes() {
  return gemm_stages<BN>() * (kBM * kBK * 2 + BN * kBK * 2) + kEpiWarps * kEpiStageFloats * 4 +
         1024 /*align*/ + 256 /*barriers*/;
}

template <bool A_MN, bool B_MN, int BN, class Epi, class Gate>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_sm100_kernel(const __grid_constant__ CUtensorMap tma_a,
                  const __grid_constant__ CUtensorMap tma_b, const GemmArgs args, const Epi epi,
                  const Gate gate) {
  extern __shared__ uint8_t smem_raw[];
  constexpr int A_BYTES = kBM * kBK * 2;
  constexpr int B_BYTES = BN * kBK * 2;
  constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr int NSTAGE = gemm_stages<BN>();
  constexpr uint32_t TMEM_COLS = 2 * BN;  // 256 or 512: powers of two
  static_assert(BN == 128 || BN == 256, "BN must be 128 or 256");

  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* epi_stage = reinterpret_cast<float*>(smem + NSTAGE * STAGE_BYTES);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + NSTAGE * STAGE_BYTES + kEpiWarps * kEpiStageFloats * 4);
  uint64_t* full = bars;                      // [NSTAGE]
  uint64_t* empty = bars + NSTAGE;           // [NSTAGE]
  uint64_t* tfull = bars + 2 * NSTAGE;       // [2]
  uint64_t* tempty = bars + 2 * NSTAGE + 2;  // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * NSTAGE + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < NSTAGE; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tfull[i], 1);
      mbar_init(&tempty[i], kEpiWarps);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tma_a);
    tma_prefetch_desc(&tma_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint64_t timeout = args.timeout_ns;

  if (warp == 0) {
    // ------------------------------- TMA producer -------------------------------
    if (lane == 0) {
      TileWalker<BN> walker(args);
      Tile t;
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int ti = blockIdx.x; ok && walker.get(ti, t); ti += gridDim.x) {
        if (!gate.wait(t, args, abort_flag)) break;
        for (int kb = 0; kb < t.nk; ++kb) {
          const int kbe = args.k_rotate ? (kb + args.k_rotate) % t.nk : kb;
          if (!gate.wait_k(t, kbe, kb == 0, args, abort_flag)) {
            ok = false;
            break;
          }
          if (!mbar_wait(&empty[stage], phase ^ 1, timeout, abort_flag)) {
            report_status(args.status, kStatusMbarTimeout, kKernelIdGemm, 100 + stage, 0, 0);
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * STAGE_BYTES;
          uint8_t* sb = sa + A_BYTES;
          mbar_expect_tx(&full[stage], STAGE_BYTES);
          const int k0 = kbe * kBK;
          // ---- A ----
          if (args.mode == 0) {
            if constexpr (!A_MN) {
              tma_load_2d(sa, &tma_a, &full[stage], k0, t.row_base + t.m0);
            } else {
              // A stored [K, rows]: 64-row-wide boxes along the M index.
              if (args.mn3d) {
                tma_load_3d(sa, &tma_a, &full[stage], 0, k0, (t.row_base + t.m0) / 64);
              } else {
#pragma unroll
                for (int j = 0; j < kBM / 64; ++j)
                  tma_load_2d(sa + j * (64 * kBK * 2), &tma_a, &full[stage],
                              t.row_base + t.m0 + 64 * j, k0);
              }
            }
          } else {
            // grouped-K: A is [rows_total, M], contraction over rows of the group.
            if (args.mn3d) {
              tma_load_3d(sa, &tma_a, &full[stage], 0, t.row_base + k0, t.m0 / 64);
            } else {
#pragma unroll
              for (int j = 0; j < kBM / 64; ++j)
                tma_load_2d(sa + j * (64 * kBK * 2), &tma_a, &full[stage], t.m0 + 64 * j,
                            t.row_base + k0);
            }
          }
          // ---- B ----
          if (args.mode == 0) {
            const int brow = (args.group_b ? args.group_b[t.g] : t.g) * args.b_group_stride;
            if constexpr (!B_MN) {
              // B flattened [G * Nb, K]; 128-row boxes.
#pragma unroll
              for (int j = 0; j < BN / 128; ++j) {
                int n;
                if (args.gated)
                  n = (j < BN / 256 ? 0 : args.n_half) + t.n_tile * (BN / 2) +
                      128 * (j % (BN / 256 > 0 ? BN / 256 : 1));
                else
                  n = t.n_tile * BN + 128 * j;
                tma_load_2d(sb + j * (128 * kBK * 2), &tma_b, &full[stage], k0, brow + n);
              }
            } else {
              // B flattened [G * K, Nb]; 64-column boxes.
              if (args.mn3d) {
                if (args.gated) {
                  const int n = t.n_tile * (BN / 2);
                  tma_load_3d(sb, &tma_b, &full[stage], 0, brow + k0, n / 64);
                  tma_load_3d(sb + (BN / 2) * kBK * 2, &tma_b, &full[stage], 0, brow + k0,
                              (args.n_half + n) / 64);
                } else {
                  tma_load_3d(sb, &tma_b, &full[stage], 0, brow + k0, t.n_tile * BN / 64);
                }
              } else {
#pragma unroll
                for (int j = 0; j < BN / 64; ++j) {
                  int n;
                  if (args.gated)
                    n = (j < BN / 128 ? 0 : args.n_half) + t.n_tile * (BN / 2) +
                        64 * (j % (BN / 128));
                  else
                    n = t.n_tile * BN + 64 * j;
                  tma_load_2d(sb + j * (64 * kBK * 2), &tma_b, &full[stage], n, brow + k0);
                }
              }
            }
          } else {
            if (args.mn3d) {
              tma_load_3d(sb, &tma_b, &full[stage], 0, t.row_base + k0, t.n_tile * BN / 64);
            } else {
#pragma unroll
              for (int j = 0; j < BN / 64; ++j)
                tma_load_2d(sb + j * (64 * kBK * 2), &tma_b, &full[stage], t.n_tile * BN + 64 * j,
                            t.row_base + k0);
            }
          }
          if (++stage == NSTAGE) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer -------------------------------
    if (lane == 0) {
      constexpr bool A_IS_MN = A_MN;  // in mode 1 the launcher instantiates A_MN = true
      constexpr uint32_t idesc = umma_idesc_bf16(kBM, BN, A_IS_MN, B_MN);
      TileWalker<BN> walker(args);
      Tile t;
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int ti = blockIdx.x; ok && walker.get(ti, t); ti += gridDim.x) {
        if (!mbar_wait(&tempty[acc], acc_phase ^ 1, timeout, abort_flag)) {
          report_status(args.status, kStatusMbarTimeout, kKernelIdGemm, 200 + acc, 0, 0);
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < t.nk; ++kb) {
          if (!mbar_wait(&full[stage], phase, timeout, abort_flag)) {
            report_status(args.status, kStatusMbarTimeout, kKernelIdGemm, 300 + stage, 0, 0);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t sb = sa + A_BYTES;
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k) {
            uint64_t da, db;
            if constexpr (!A_IS_MN)
              da = umma_smem_desc(sa + k * 32, 0, 1024);
            else
              da = umma_smem_desc(sa + k * 2048, 64 * kBK * 2, 1024);
            if constexpr (!B_MN)
              db = umma_smem_desc(sb + k * 32, 0, 1024);
            else
              db = umma_smem_desc(sb + k * 2048, 64 * kBK * 2, 1024);
            umma_bf16(d_tmem, da, db, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&empty[stage]);  // frees the stage once these MMAs have read it
          if (++stage == NSTAGE) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        umma_commit(&tfull[acc]);
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1;
        }
      }
    }
  } else {
    // ------------------------------- epilogue (8 warps) -------------------------------
    const int q = warp & 3;             // TMEM lane quarter this warp may read
    const int chalf = (warp - 2) >> 2;  // which half of the tile's columns this warp drains
    TileWalker<BN> walker(args);
    TileWalker<BN> peek(args);
    Tile t;
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int ti = blockIdx.x; walker.get(ti, t); ti += gridDim.x) {
      if constexpr (EpiHasPrefetch<Epi>::value) {
        Tile nx;
        if (ti == (int)blockIdx.x) epi.template prefetch<BN>(t, args, q * 32 + lane, chalf);
        if (peek.get(ti + gridDim.x, nx)) epi.template prefetch<BN>(nx, args, q * 32 + lane, chalf);
      }
      if (!mbar_wait(&tfull[acc], acc_phase, timeout, abort_flag)) {
        if (lane == 0)
          report_status(args.status, kStatusMbarTimeout, kKernelIdGemm, 400 + acc, 0, 0);
        break;
      }
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN;
      epi.template run<BN>(t, args, taddr, q * 32 + lane, t.nk == 0, chalf,
                           epi_stage + (warp - 2) * kEpiStageFloats);
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[acc]);
      epi.tile_done(t, args, q * 32 + lane);
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
  }

  if (*abort_flag) {
    // Give copies that are still in flight time to land before the CTA's shared memory is
    // handed back (they complete within microseconds; this path is the error path only).
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// =========================================================================================
// CTA-pair variant: two CTAs of a cluster compute one 256 x 256 tile with
// tcgen05.mma.cta_group::2.  Each CTA loads its own 128 rows of A and its own 128 columns of
// B (no multicast), so every MMA reads half the shared-memory bytes per CTA that the
// single-CTA kernel reads, and five pipeline stages fit beside the epilogue staging area.  CTA 0 of the pair issues the MMAs;
// completion is broadcast to both CTAs' barriers with tcgen05.commit (multicast of the
// *arrival*, not of a load).  Each CTA drains its own 128 accumulator rows from its own TMEM.
// =========================================================================================
constexpr int kStages2 = 5;

constexpr int gemm2_smem_bytes() {
  return kStages2 * (kBM * kBK * 2 + 128 * kBK * 2) + kEpiWarps * kEpiStageFloats * 4 + 1024 + 256;
}

template <bool A_MN, bool B_MN, class Epi, class Gate>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
gemm2_sm100_kernel(const __grid_constant__ CUtensorMap tma_a,
                   const __grid_constant__ CUtensorMap tma_b, const GemmArgs args, const Epi epi,
                   const Gate gate) {
  constexpr int BN = 256;
  extern __shared__ uint8_t smem_raw[];
  constexpr int A_BYTES = kBM * kBK * 2;          // 128 rows of A
  constexpr int B_BYTES = 128 * kBK * 2;          // this CTA's 128 columns of B
  constexpr int STAGE_BYTES = A_BYTES + B_BYTES;  // per CTA
  constexpr uint32_t TMEM_COLS = 2 * BN;

  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* epi_stage = reinterpret_cast<float*>(smem + kStages2 * STAGE_BYTES);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages2 * STAGE_BYTES + kEpiWarps * kEpiStageFloats * 4);
  uint64_t* full = bars;                        // [kStages2]  used in the leader CTA
  uint64_t* empty = bars + kStages2;            // [kStages2]  one per CTA
  uint64_t* tfull = bars + 2 * kStages2;        // [2]         one per CTA
  uint64_t* tempty = bars + 2 * kStages2 + 2;   // [2]         used in the leader CTA
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages2 + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta_rank = cluster_ctarank();
  const bool leader = cta_rank == 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages2; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tfull[i], 1);
      mbar_init(&tempty[i], 2 * kEpiWarps);   // epilogue warps of both CTAs
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tma_a);
    tma_prefetch_desc(&tma_b);
  }
  __syncthreads();
  cluster_sync_all();   // both CTAs' barriers exist before anyone signals across the pair
  if (warp == 1) {
    tmem_alloc2(tmem_slot, TMEM_COLS);
    tmem_relinquish2();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint64_t timeout = args.timeout_ns;
  const int pair_id = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  if (warp == 0) {
    // ------------------------------- TMA producer (both CTAs) -------------------------------
    if (lane == 0) {
      TileWalker<BN, 2 * kBM> walker(args);
      const TileOrder order(args, pair_id, num_pairs);
      const bool claimer = order.dynamic() && leader;
      if (claimer && pair_id == 0 && args.sched_ctr_reset != nullptr) *args.sched_ctr_reset = 0;
      Tile t;
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int ti = pair_id;
      for (int j = 0; ok && ti >= 0 && walker.get(ti, t); ++j) {
        // The claim of the next tile is issued here and written to the log after the first block's
        // loads, so the counter's round trip hides behind them; every reader finds the entry a
        // whole tile before it needs it.
        int claimed = 0;
        bool published = !claimer;
        if (claimer) claimed = order.claim();
        Tile mine = t;                       // this CTA's 128 rows of the pair tile
        mine.m0 = t.m0 + (int)cta_rank * kBM;
        mine.rows_valid = max(0, min(kBM, t.rows_valid - (int)cta_rank * kBM));
        if (mine.rows_valid > 0 && !gate.wait(mine, args, abort_flag)) break;
        if (t.nk == 0 && !published) {
          ok = order.publish(j + 1, claimed, args.status, abort_flag);
          published = true;
        }
        for (int kb = 0; kb < t.nk; ++kb) {
          const int kbe = args.k_rotate ? (kb + args.k_rotate) % t.nk : kb;
          if (mine.rows_valid > 0 && !gate.wait_k(mine, kbe, kb == 0, args, abort_flag)) {
            ok = false;
            break;
          }
          if (!mbar_wait(&empty[stage], phase ^ 1, timeout, abort_flag)) {
            report_status(args.status, kStatusMbarTimeout, kKernelIdGemm2, 100 + stage, 0, 0);
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * STAGE_BYTES;
          uint8_t* sb = sa + A_BYTES;
          if (leader) mbar_expect_tx(&full[stage], 2 * STAGE_BYTES);
          const int k0 = kbe * kBK;
          // ---- A: this CTA's 128 rows ----
          if (args.mode == 0) {
            tma2_load_2d(sa, &tma_a, &full[stage], k0, t.row_base + mine.m0);
          } else {
            tma2_load_3d(sa, &tma_a, &full[stage], 0, t.row_base + k0, mine.m0 / 64);
          }
          // ---- B: this CTA's 128 columns ----
          int n;
          if (args.gated)
            n = (cta_rank == 0 ? 0 : args.n_half) + t.n_tile * 128;
          else
            n = t.n_tile * BN + (int)cta_rank * 128;
          if (args.mode == 0) {
            const int brow = (args.group_b ? args.group_b[t.g] : t.g) * args.b_group_stride;
            if constexpr (!B_MN)
              tma2_load_2d(sb, &tma_b, &full[stage], k0, brow + n);
            else
              tma2_load_3d(sb, &tma_b, &full[stage], 0, brow + k0, n / 64);
          } else {
            tma2_load_3d(sb, &tma_b, &full[stage], 0, t.row_base + k0, n / 64);
          }
          if (++stage == kStages2) {
            stage = 0;
            phase ^= 1;
          }
          if (!published) {
            ok = order.publish(j + 1, claimed, args.status, abort_flag);
            published = true;
          }
        }
        if (!ok) break;
        ti = claimer ? claimed : order.get(j + 1, 0ull, timeout, args.status, abort_flag);
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer (leader CTA only) -------------------------------
    // The whole warp walks the loop and one elected lane issues: with uniform control flow the
    // compiler keeps loop state and descriptors in the warp's uniform registers, and the issuing
    // warp, which shares its scheduler with busy epilogue warps, spends fewer issue slots per MMA.
    // The low descriptor words of the k-steps of stage 0 are computed once; a stage adds its
    // byte offset / 16 and the constant high word is joined on.
    if (leader) {
      constexpr uint32_t idesc = umma_idesc_bf16(2 * kBM, BN, A_MN, B_MN);
      constexpr int kSteps = kBK / 16;
      constexpr uint32_t kDescHi = umma_desc_hi(1024);
      constexpr uint32_t kStageAdd = STAGE_BYTES >> 4;
      uint32_t a_lo[kSteps], b_lo[kSteps];
      {
        const uint32_t sa0 = smem_u32(smem), sb0 = sa0 + A_BYTES;
#pragma unroll
        for (int k = 0; k < kSteps; ++k) {
          a_lo[k] = A_MN ? umma_desc_lo(sa0 + k * 2048, 64 * kBK * 2) : umma_desc_lo(sa0 + k * 32, 0);
          b_lo[k] = B_MN ? umma_desc_lo(sb0 + k * 2048, 64 * kBK * 2) : umma_desc_lo(sb0 + k * 32, 0);
        }
      }
      auto wait_all = [&](uint64_t* bar, uint32_t parity) {
        return __all_sync(0xffffffffu, mbar_wait(bar, parity, timeout, abort_flag)) != 0;
      };
      TileWalker<BN, 2 * kBM> walker(args);
      const TileOrder order(args, pair_id, num_pairs);
      Tile t;
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      int ti = pair_id;
      for (int j = 0; ok && ti >= 0 && walker.get(ti, t); ++j) {
        unsigned long long seen = 0;   // log entry of the next tile, fetched during the last k block
        if (!wait_all(&tempty[acc], acc_phase ^ 1)) {
          if (lane == 0) report_status(args.status, kStatusMbarTimeout, kKernelIdGemm2, 200 + acc, 0, 0);
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < t.nk; ++kb) {
          if (order.dynamic() && kb == t.nk - 1) seen = order.peek(j + 1);
          if (!wait_all(&full[stage], phase)) {
            if (lane == 0) report_status(args.status, kStatusMbarTimeout, kKernelIdGemm2, 300 + stage, 0, 0);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          if (elect_one()) {
            const uint32_t sadd = stage * kStageAdd;
            umma2_bf16(d_tmem, umma_desc_join(a_lo[0] + sadd, kDescHi), umma_desc_join(b_lo[0] + sadd, kDescHi), idesc,
                       kb > 0 ? 1u : 0u);
#pragma unroll
            for (int k = 1; k < kSteps; ++k)
              umma2_bf16_acc(d_tmem, umma_desc_join(a_lo[k] + sadd, kDescHi), umma_desc_join(b_lo[k] + sadd, kDescHi),
                             idesc);
            umma2_commit_mc(&empty[stage], 3);   // frees the stage in both CTAs
          }
          __syncwarp();
          if (++stage == kStages2) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        if (elect_one()) umma2_commit_mc(&tfull[acc], 3);
        __syncwarp();
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1;
        }
        // every lane reads the same entry, so the tile index stays uniform across the warp
        ti = order.get(j + 1, seen, timeout, args.status, abort_flag);
        ti = __shfl_sync(0xffffffffu, ti, 0);
      }
    }
  } else {
    // ------------------------------- epilogue (8 warps per CTA) -------------------------------
    const int q = warp & 3;
    const int chalf = (warp - 2) >> 2;
    TileWalker<BN, 2 * kBM> walker(args);
    TileWalker<BN, 2 * kBM> peek(args);
    const TileOrder order(args, pair_id, num_pairs);
    Tile t;
    int acc = 0;
    uint32_t acc_phase = 0;
    int ti = pair_id;
    for (int j = 0; ti >= 0 && walker.get(ti, t); ++j) {
      Tile mine = t;
      mine.m0 = t.m0 + (int)cta_rank * kBM;
      mine.rows_valid = max(0, min(kBM, t.rows_valid - (int)cta_rank * kBM));
      // The producer wrote the next tile's log entry while it loaded this tile, which the epilogue
      // reaches at least one main loop later.
      unsigned long long seen = 0;
      if (order.dynamic()) {
        if (lane == 0) seen = order.peek(j + 1);
        seen = __shfl_sync(0xffffffffu, seen, 0);
      }
      if constexpr (EpiHasPrefetch<Epi>::value) {
        Tile nx;
        if (j == 0) epi.template prefetch<BN>(mine, args, q * 32 + lane, chalf);
        const int tn = order.dynamic() ? (order.valid(seen) ? (int)(unsigned int)seen : -1) : ti + num_pairs;
        if (tn >= 0 && peek.get(tn, nx)) {
          nx.rows_valid = max(0, min(kBM, nx.rows_valid - (int)cta_rank * kBM));
          nx.m0 += (int)cta_rank * kBM;
          epi.template prefetch<BN>(nx, args, q * 32 + lane, chalf);
        }
      }
      if (!mbar_wait(&tfull[acc], acc_phase, timeout, abort_flag)) {
        if (lane == 0)
          report_status(args.status, kStatusMbarTimeout, kKernelIdGemm2, 400 + acc, 0, 0);
        break;
      }
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN;
      epi.template run<BN>(mine, args, taddr, q * 32 + lane, t.nk == 0, chalf,
                           epi_stage + (warp - 2) * kEpiStageFloats);
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        if (leader)
          mbar_arrive(&tempty[acc]);
        else
          mbar_arrive_remote(map_to_cta(smem_u32(&tempty[acc]), 0));
      }
      epi.tile_done(mine, args, q * 32 + lane);
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1;
      }
      if (lane == 0) ti = order.get(j + 1, seen, timeout, args.status, abort_flag);
      ti = __shfl_sync(0xffffffffu, ti, 0);
    }
  }

  if (*abort_flag) {
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();   // the peer may still signal this CTA's barriers until here
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc2(tmem_base, TMEM_COLS);
  }
}

}  // namespace fm
