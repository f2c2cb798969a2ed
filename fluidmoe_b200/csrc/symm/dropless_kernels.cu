// Dropless (variable-split) expert-parallel exchange, device-initiated, without a host read.
//
// Every rank routes its T tokens to k of E experts and keeps every pair, so how many rows travel
// between two ranks is only known on the device.  Three kernels replace the host-side planning of
// an all-to-all-v (the reference's README-era API carried input_splits / output_splits on the
// host, README:62-67; its layer avoids every host sync on the hot path,
// fluid/moe/forward.py:153-158,437-441, which this path keeps):
//
//   dropless_plan_kernel     every rank stores its per-expert counts into every peer's [P, E]
//                            table (peer stores + release flag), waits (bounded) for all P rows and
//                            derives, identically on every rank: the 128-aligned row range of each
//                            local expert in the owner's expert-major buffer, where the rows of
//                            each source start inside it, and how many rows come back from whom;
//   dropless_rowmap_kernel   per expert-major row: the rank and the permuted-order row it returns to
//                            (what the FC2 / FC1-dX scatter epilogues take);
//   dropless_dispatch_kernel gathers every routed row and stores it into its owner's buffer with
//                            16-byte peer stores, then bumps the arrival counter of the 128-row
//                            block, which the gated grouped GEMM polls.
//
// Buffers are sized for the worst case by the caller; a plan that would not fit is refused by all
// ranks alike (nothing is sent, a status record is written).
#include <stdio.h>

#include "../include/fm_symm.h"
#include "../include/sm100_ptx.cuh"

extern "C" void fm_set_error(const char* msg);

namespace fm {

constexpr int kKernelIdDroplessPlan = 14;
constexpr int kMaxPlanEntries = 8192;   // P * E ints of shared memory

__device__ __forceinline__ int align128(int v) { return (v + 127) & ~127; }

// One CTA.  `table_ptrs[p]` is rank p's table int[2][P][E] (double buffered by epoch parity),
// `flag_ptrs[p]` rank p's int[P] arrival words.
__global__ void __launch_bounds__(1024, 1)
dropless_plan_kernel(const int* __restrict__ counts, int* const* __restrict__ table_ptrs,
                     int* const* __restrict__ flag_ptrs, int epoch, int P, int me, int E, int nle,
                     int expected_mult, int max_rows, FmDroplessPlan out,
                     unsigned long long timeout_ns, int* status) {
  __shared__ int C[kMaxPlanEntries];      // C[r * E + e]: pairs rank r routes to global expert e
  __shared__ int padded[1024];            // padded rows of global expert e in its owner's buffer
  __shared__ int ok_flag;
  const int t = threadIdx.x;
  const int par = epoch & 1;
  if (t == 0) ok_flag = 1;
  // 1. publish my row in every rank's table
  for (int i = t; i < P * E; i += blockDim.x) {
    const int p = i / E, e = i % E;
    table_ptrs[p][(par * P + me) * E + e] = counts[e];
  }
  __threadfence_system();
  __syncthreads();
  if (t < P) flag_release_store(flag_ptrs[t] + me, epoch);
  // 2. wait for everybody's row
  if (t < P) {
    int observed = 0;
    if (!flag_wait_ge(flag_ptrs[me] + t, epoch, timeout_ns, nullptr, &observed)) {
      report_status(status, kStatusFlagTimeout, kKernelIdDroplessPlan, t, epoch, observed);
      ok_flag = 0;
    }
  }
  __syncthreads();
  const volatile int* mine = table_ptrs[me] + par * P * E;
  for (int i = t; i < P * E; i += blockDim.x) C[i] = ok_flag ? mine[i] : 0;
  __syncthreads();
  // 3. rows of every global expert, padded to whole 128-row blocks
  for (int e = t; e < E; e += blockDim.x) {
    int n = 0;
    for (int r = 0; r < P; ++r) n += C[r * E + e];
    padded[e] = align128(n);
  }
  __syncthreads();
  // the plan must fit in every owner's buffer; all ranks evaluate the same numbers
  if (t == 0) {
    int worst = 0;
    for (int p = 0; p < P; ++p) {
      int tot = 0;
      for (int j = 0; j < nle; ++j) tot += padded[p * nle + j];
      worst = max(worst, tot);
    }
    if (worst > max_rows) {
      report_status(status, kStatusFlagTimeout, kKernelIdDroplessPlan, 1000, max_rows, worst);
      ok_flag = 0;
    }
  }
  __syncthreads();
  if (!ok_flag) {
    for (int i = t; i < P * E; i += blockDim.x) C[i] = 0;
    for (int e = t; e < E; e += blockDim.x) padded[e] = 0;
    __syncthreads();
  }
  // 4. outputs
  for (int i = t; i < P * E; i += blockDim.x) out.counts_all[i] = C[i];
  for (int e = t; e < E; e += blockDim.x) {
    const int p = e / nle, j = e % nle;
    int off = 0;
    for (int jj = 0; jj < j; ++jj) off += padded[p * nle + jj];
    int before_me = 0;
    for (int r = 0; r < me; ++r) before_me += C[r * E + e];
    out.dst_base[e] = off + before_me;
    int s = 0;
    for (int ee = 0; ee < e; ++ee) s += C[me * E + ee];
    out.slot_start[e] = s;
    if (e == E - 1) out.slot_start[E] = s + C[me * E + e];
    if (p == me) {
      int n = 0;
      for (int r = 0; r < P; ++r) n += C[r * E + e];
      out.group_rows[j] = n;
      out.group_offs[j] = off;
      out.group_flag_base[j] = off / 128;
      if (j == nle - 1) out.totals[0] = off + padded[e];
    }
  }
  for (int i = t; i < P * nle; i += blockDim.x) {
    const int r = i / nle, j = i % nle;
    int b = 0;
    for (int rr = 0; rr < r; ++rr) b += C[rr * E + me * nle + j];
    out.before[i] = b;
  }
  for (int i = t; i < P * E; i += blockDim.x) {
    const int r = i / E, e = i % E;
    int s = 0;
    for (int ee = 0; ee < e; ++ee) s += C[r * E + ee];
    out.src_prefix[i] = s;
  }
  if (t < P) {
    int n = 0;
    for (int j = 0; j < nle; ++j) n += C[me * E + t * nle + j];
    out.recv_expected[t] = n * expected_mult;
  }
  if (t == 0) out.totals[1] = ok_flag ? 0 : 1;
}

// grid = P * nle blocks; block (r, j) fills the rows of local expert j that come from source r.
__global__ void dropless_rowmap_kernel(FmDroplessPlan pl, int P, int me, int E, int nle,
                                       int* __restrict__ row_dst_rank, int* __restrict__ row_dst_row) {
  const int r = blockIdx.x / nle, j = blockIdx.x % nle;
  const int e = me * nle + j;
  const int n = pl.counts_all[r * E + e];
  const int start = pl.group_offs[j] + pl.before[r * nle + j];
  const int src0 = pl.src_prefix[r * E + e];
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    row_dst_rank[start + i] = r;
    row_dst_row[start + i] = src0 + i;
  }
  if (r == P - 1) {   // rows that only pad the expert's run to a whole block go nowhere
    const int end = pl.group_offs[j] + pl.group_rows[j];
    const int pad_end = pl.group_offs[j] + align128(pl.group_rows[j]);
    for (int i = end + threadIdx.x; i < pad_end; i += blockDim.x) {
      row_dst_rank[i] = -1;
      row_dst_row[i] = 0;
    }
  }
}

// Sender side.  Slot s of my permuted order (pairs sorted by global expert, `total_slots` = T * k
// of them) is the row x[sorted_idx[s]]; the expert of a slot is found by bisection in `slot_start`.
// The row goes to rank e / nle at absolute row dst_base[e] + (s - slot_start[e]) of its expert-major
// buffer, its probability (if any) into the matching fp32 slot, and the arrival counter of that
// 128-row block grows by one per row.  One warp per row, 16-byte accesses; the system-scope fence
// and the counter update are issued once per run of rows that share a counter.  Slots are visited
// starting with the experts of my right-hand neighbour, the local ones last.
__global__ void dropless_dispatch_kernel(const __nv_bfloat16* __restrict__ x,
                                         const long long* __restrict__ sorted_idx,
                                         const float* __restrict__ probs, FmDroplessPlan pl,
                                         __nv_bfloat16* const* __restrict__ dst_tokens,
                                         float* const* __restrict__ dst_probs,
                                         int* const* __restrict__ dst_flags, long long total_slots,
                                         int H, int E, int nle, int P, int me) {
  const int nvec = H / 8;
  const int lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  constexpr int kRowsPerFence = 8;
  const long long live = pl.slot_start[E];              // 0 when the plan was refused
  const long long nchunks = (live + kRowsPerFence - 1) / kRowsPerFence;
  const long long rot = pl.slot_start[((me + 1) % P) * nle];
  for (long long c = (long long)blockIdx.x * warps_per_block + (threadIdx.x >> 5); c < nchunks;
       c += (long long)gridDim.x * warps_per_block) {
    int* pending_flag = nullptr;
    int pending = 0;
    const long long s_end = min(live, (c + 1) * kRowsPerFence);
    for (long long sv = c * kRowsPerFence; sv < s_end; ++sv) {
      long long s = sv + rot;
      if (s >= live) s -= live;
      int lo = 0, hi = E;                                // largest e with slot_start[e] <= s
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (pl.slot_start[mid] <= s) lo = mid; else hi = mid;
      }
      const int e = lo, p = e / nle;
      const long long drow = (long long)pl.dst_base[e] + (s - pl.slot_start[e]);
      int* flag = dst_flags[p] + (int)(drow >> 7);
      if (flag != pending_flag && pending > 0) {
        __syncwarp();
        if (lane == 0) {
          __threadfence_system();
          flag_release_add(pending_flag, pending);
        }
        pending = 0;
      }
      pending_flag = flag;
      const long long tok = sorted_idx[s];
      const uint4* src = reinterpret_cast<const uint4*>(x + tok * H);
      uint4* dst = reinterpret_cast<uint4*>(dst_tokens[p] + drow * H);
      for (int v = lane; v < nvec; v += 32) dst[v] = src[v];
      if (lane == 0 && probs != nullptr) dst_probs[p][drow] = probs[s];
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
  (void)total_slots;
}

// Zero the rows that pad every group to a whole 128-row block: rows [offs + rows, offs +
// align128(rows)) of a row-major buffer with `row_bytes` bytes per row (a multiple of 16).  The
// weight-gradient GEMMs contract over whole 64-row blocks, so what lies there must be zero.
__global__ void zero_group_padding_kernel(uint8_t* __restrict__ buf, long long row_bytes,
                                          const int* __restrict__ group_rows,
                                          const int* __restrict__ group_offs) {
  const int g = blockIdx.x;
  const long long first = (long long)group_offs[g] + group_rows[g];
  const long long last = (long long)group_offs[g] + align128(group_rows[g]);
  uint4* p = reinterpret_cast<uint4*>(buf + first * row_bytes);
  const long long n = (last - first) * row_bytes / 16;
  const uint4 z = make_uint4(0, 0, 0, 0);
  for (long long i = (long long)blockIdx.y * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.y * blockDim.x)
    p[i] = z;
}

}  // namespace fm

static int dl_check(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    char msg[256];
    snprintf(msg, sizeof(msg), "%s: %s", what, cudaGetErrorString(e));
    fm_set_error(msg);
    return (int)e;
  }
  return 0;
}

extern "C" int fm_dropless_plan(const int* counts, int* const* table_ptrs, int* const* flag_ptrs, int epoch,
                                int P, int me, int E, int nle, int expected_mult, int max_rows,
                                const FmDroplessPlan* out, int* row_dst_rank, int* row_dst_row,
                                unsigned long long timeout_ns, int* status, cudaStream_t stream) {
  if (P * E > fm::kMaxPlanEntries || E > 1024 || P > 1024 || E != P * nle) {
    fm_set_error("dropless_plan: needs ranks * experts <= 8192, experts <= 1024 and experts == ranks * local experts");
    return -1;
  }
  fm::dropless_plan_kernel<<<1, 1024, 0, stream>>>(counts, table_ptrs, flag_ptrs, epoch, P, me, E, nle,
                                                  expected_mult, max_rows, *out,
                                                  timeout_ns ? timeout_ns : 4000000000ull, status);
  int rc = dl_check("dropless_plan");
  if (rc) return rc;
  fm::dropless_rowmap_kernel<<<P * nle, 256, 0, stream>>>(*out, P, me, E, nle, row_dst_rank, row_dst_row);
  return dl_check("dropless_rowmap");
}

extern "C" int fm_dropless_dispatch(const void* x, const long long* sorted_idx, const float* probs,
                                    const FmDroplessPlan* pl, void* const* dst_tokens, float* const* dst_probs,
                                    int* const* dst_flags, long long total_slots, int H, int E, int nle, int P,
                                    int me, int num_ctas, cudaStream_t stream) {
  if (H % 8 != 0) {
    fm_set_error("dropless_dispatch: H must be a multiple of 8");
    return -1;
  }
  if (num_ctas <= 0) num_ctas = 148 * 2;
  fm::dropless_dispatch_kernel<<<num_ctas, 256, 0, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), sorted_idx, probs, *pl,
      reinterpret_cast<__nv_bfloat16* const*>(dst_tokens), dst_probs, dst_flags, total_slots, H, E, nle, P, me);
  return dl_check("dropless_dispatch");
}

extern "C" int fm_zero_group_padding(void* buf, long long row_bytes, const int* group_rows, const int* group_offs,
                                     int num_groups, cudaStream_t stream) {
  if (row_bytes % 16 != 0 || (reinterpret_cast<uintptr_t>(buf) & 15)) {
    fm_set_error("zero_group_padding: rows must be 16-byte multiples and the buffer 16-byte aligned");
    return -1;
  }
  dim3 grid(num_groups, 8);
  fm::zero_group_padding_kernel<<<grid, 256, 0, stream>>>(reinterpret_cast<uint8_t*>(buf), row_bytes,
                                                         group_rows, group_offs);
  return dl_check("zero_group_padding");
}
