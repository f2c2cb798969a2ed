// C ABI of the native library.  Everything here is plain C so that the same entry points can
// be reached from the torch bindings, from ctypes, or from another runtime.
#pragma once
#include <stdint.h>
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

enum FmEpilogue {
  FM_EPI_STORE = 0,    // C = alpha * acc (+ C), bf16 or fp32
  FM_EPI_ACT = 1,      // act(acc) * prob[row] -> bf16 (GELU / SiLU / SwiGLU), optional pre-act copy
  FM_EPI_SCATTER = 2,  // row r of the result goes to dst_base[dst_rank[r]] + dst_row[r] * ld
  FM_EPI_DACT = 3,     // backward of act * prob fused after the FC2 input-gradient GEMM
  FM_EPI_COLSCATTER = 4,  // column block p of the result goes to rank p's buffer
  FM_EPI_ADAM = 5,        // the result is a weight gradient: apply AdamW to the parameter tile in place
};
enum FmAct { FM_ACT_GELU = 0, FM_ACT_SILU = 1, FM_ACT_NONE = 2 };

typedef struct FmGemmDesc {
  // ---- operands (bf16) ----
  const void* A;
  const void* B;
  int a_mn;  // 0: A stored [rows, K] (K contiguous); 1: stored [K, rows] (rows contiguous)
  int b_mn;  // 0: B stored [N, K] (K contiguous); 1: stored [K, N] (N contiguous)
  long long a_inner, a_outer, lda;  // extents / row stride (elements) of A's 2-D storage
  long long b_inner, b_outer, ldb;  // same for B (groups flattened into the outer extent)
  // ---- problem ----
  int mode;  // 0 grouped-M (dense when num_groups == 1), 1 grouped-K (weight gradient)
  int num_groups;
  int M, N, K;
  int uniform_rows;
  const int* group_rows;
  const int* group_offs;
  const int* group_b;  // which B matrix each group multiplies with (null: group index)
  int b_group_stride;
  int gated;
  int n_half;
  int bn;  // 128 or 256
  int swizzle_m;
  int cta_pair;  // 1: two CTAs share a 256 x 256 tile (tcgen05 cta_group::2) when the shape allows
  // ---- epilogue ----
  int epi;
  void* C;
  long long ldc;
  long long c_group_stride;
  int out_fp32;
  int accumulate;
  float alpha;
  // FM_EPI_ACT
  void* act_out;
  long long ld_act;
  void* pre_out;
  long long ld_pre;
  const float* probs;
  int act_kind;
  // FM_EPI_DACT (inputs: saved pre-activation, probs; outputs: dpre, dprobs (atomic fp32))
  const void* pre_in;
  long long ld_pre_in;
  float* dprobs;
  // FM_EPI_SCATTER
  void* const* dst_base;   // device array [num_ranks] of destination base pointers (bf16)
  const int* dst_rank;     // device [rows] destination rank of each row, -1 = drop
  const int* dst_row;      // device [rows] destination row
  long long ld_dst;
  int* const* dst_flags;   // device array [num_ranks]: counter this rank bumps on each peer (may be null)
  int num_ranks;
  const float* row_aux;       // optional: one fp32 per source row that travels with the row ...
  float* const* row_aux_dst;  // ... into row_aux_dst[dst_rank[r]][dst_row[r]] (device array [num_ranks])
  // FM_EPI_COLSCATTER (also uses dst_base, ld_dst, dst_flags)
  int cols_per_rank;
  long long dst_row_offset;
  // FM_EPI_ADAM (bf16 parameter and moments laid out like C: ldc, c_group_stride; alpha scales the gradient)
  void* adam_p;
  void* adam_m;
  void* adam_v;
  float adam_lr, adam_beta1, adam_beta2, adam_eps, adam_wd, adam_rbc1, adam_rbc2;
  // ---- gate (producer waits until flags[...] >= expected before loading a row block) ----
  const int* gate_flags;
  const int* gate_group_base;
  int gate_blocks_per_group;
  int gate_expected;
  int gate_k_blocks_per_src;  // > 0: gate along K by source rank (gate_blocks_per_group = row blocks per source)
  int n_rotate;               // first N tile to visit
  int k_rotate;               // first K block to visit
  // ---- launch ----
  int max_ctas;  // 0 = one per SM
  unsigned long long timeout_ns;
  int* status;   // device int32[8], may be null
  unsigned long long* wait_ns;  // optional device counter: time producers spent waiting in a gate
} FmGemmDesc;

// Returns 0 on success, a cudaError_t / negative code otherwise.  Never allocates.
int fm_gemm_launch(const FmGemmDesc* d, cudaStream_t stream);
const char* fm_last_error(void);

#ifdef __cplusplus
}
#endif
