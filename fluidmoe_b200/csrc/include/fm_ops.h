// C ABI of the element-wise / reduction kernels (csrc/ops/elementwise.cu) and of the attention
// kernels (csrc/ops/flash_attn.cu).  Pointers are device pointers; bf16 unless stated.
#pragma once
#include <stdint.h>
#include <cuda_runtime.h>
#ifdef __cplusplus
extern "C" {
#endif

// kind: 0 LayerNorm, 1 RMSNorm.  mean may be null for RMSNorm, b may be null.
int fm_norm_fwd(const void* x, const void* w, const void* b, void* y, float* mean, float* rstd,
                int T, int H, float eps, int kind, cudaStream_t s);
// Number of CTAs (= rows of the partial buffer [blocks, 2, H] fp32) the backward uses for T rows.
int fm_norm_bwd_blocks(int T);
int fm_norm_bwd(const void* dy, const void* x, const void* w, const float* mean, const float* rstd,
                const void* res_grad, void* dx, float* partial, float* dw, float* db, int T, int H,
                int kind, cudaStream_t s);
// `freqs`: (cos, sin) pairs of the rotation angles, fp32 [positions][rot][2].
int fm_rope_packed(void* t, const float* freqs, long long rows, int heads_per_row, int rope_heads,
                   int d, int rot, int rows_per_pos, int backward, cudaStream_t s);
// The same, preceded by a bounded wait on `wait_n` per-source arrival counters (>= wait_expected):
// RoPE is the first consumer of the projection buffer that peers fill.
int fm_rope_packed_gated(void* t, const float* freqs, long long rows, int heads_per_row, int rope_heads, int d,
                         int rot, int rows_per_pos, int backward, const int* wait_flags, int wait_n,
                         int wait_expected, unsigned long long* wait_ns, unsigned long long timeout_ns,
                         int* status, cudaStream_t s);
// dlogits [T, E] fp32 from the slot-probability gradients (softmax-over-top-k backward, optional
// load-balancing term aux_coef * tpe[e] and z-loss term z_coef * lse * softmax); tpe / logits may be null.
int fm_router_bwd(const float* dprobs_slots, const int* slot_of_token, const long long* top_idx,
                  const float* top_probs, const float* logits, const float* tpe, float aux_coef, float z_coef,
                  int T, int k, int E, float* dlogits, cudaStream_t s);
int fm_topk_softmax(const float* logits, long long* idx, float* probs, int T, int E, int k,
                    cudaStream_t s);
int fm_gather_rows(const void* x, const long long* idx, void* out, long long rows, int H,
                   cudaStream_t s);
int fm_unpermute_reduce(const void* rows, const int* slot, const void* residual, void* out, int T,
                        int k, int H, cudaStream_t s);
// The same, preceded by a bounded wait on `wait_n` per-source arrival counters (>= wait_expected).
int fm_unpermute_reduce_gated(const void* rows, const int* slot, const void* residual, void* out, int T, int k,
                              int H, const int* wait_flags, int wait_n, int wait_expected,
                              unsigned long long* wait_ns, unsigned long long timeout_ns, int* status,
                              cudaStream_t s);
// Moments are fp32, or bf16 when state_bf16 != 0.
// Adam for bf16 parameter / bf16 moments / fp32 gradient with small CTAs (128 threads, <= 80 registers)
// that fit on an SM beside a resident tensor-core kernel; meant for a side stream.
int fm_adam_background(void* p, const float* g, void* m, void* v, long long n, float lr, float beta1,
                       float beta2, float eps, float weight_decay, int step, float grad_scale, int num_ctas,
                       cudaStream_t s);
int fm_adam(void* p, float* master, float* g, void* m, void* v, long long n, float lr, float beta1,
            float beta2, float eps, float weight_decay, int step, float grad_scale, int zero_grad,
            int state_bf16, cudaStream_t s);

// Attention backward on the packed layout.  out / dout: [s, b, G*qpg, d] bf16; lse: [b, G*qpg, s];
// delta: fp32 scratch [b, G*qpg, s]; dq_accum: fp32 scratch [s, b, G*qpg, d], zeroed by the caller;
// dqkv: packed gradient [s, b, G, (qpg + 2) * d] bf16 (every element is written).
int fm_flash_attn_bwd(const void* qkv, const void* out, const void* dout, const float* lse, float* delta,
                      float* dq_accum, void* dqkv, int s, int b, int G, int qpg, int d, float scale,
                      unsigned long long timeout_ns, int* status, int version, float* dkv_accum, int hsplit,
                      cudaStream_t stream);
// The same, with the first kernel of the backward (the delta pass, the first reader of `dout`)
// preceded by a bounded wait on `wait_n` per-source arrival counters (>= wait_expected).
int fm_flash_attn_bwd_gated(const void* qkv, const void* out, const void* dout, const float* lse, float* delta,
                            float* dq_accum, void* dqkv, int s, int b, int G, int qpg, int d, float scale,
                            unsigned long long timeout_ns, int* status, int version, float* dkv_accum, int hsplit,
                            const int* wait_flags, int wait_n, int wait_expected, unsigned long long* wait_ns,
                            cudaStream_t stream);

// Cross-entropy forward + backward in place: loss_out[row] = lse - logit[label]; logits are
// overwritten with (softmax - onehot) * grad_scale (rows with a negative label get zeros).
int fm_cross_entropy(void* logits, const long long* labels, float* loss_out, int T, int V,
                     float grad_scale, cudaStream_t s);

// Padded-capacity routing plan (see moe_plan_kernel).  Outputs: sorted_indices [E*cap] int64,
// slot_probs [E*cap] fp32, slot_of_token [T,k] int32, routed_per_expert [E] int32.
int fm_moe_plan(const long long* top_idx, const float* top_probs, int T, int k, int E, int cap,
                long long* sorted_indices, float* slot_probs, int* slot_of_token,
                int* routed_per_expert, cudaStream_t s);

// Causal GQA flash attention forward on the packed projection buffer
// qkv [s, b, G, (qpg + 2) * d] (d == 128): out [s, b, G*qpg, d] bf16, lse [b, G*qpg, s] fp32.
// version 1: one query tile per CTA, P staged in shared memory; 2: two tiles ping-pong, P in TMEM.
int fm_flash_attn_fwd(const void* qkv, void* out, float* lse, int s, int b, int G, int qpg, int d,
                      float scale, unsigned long long timeout_ns, int* status, int version,
                      cudaStream_t stream);
// The same with the HP -> SP exchange in the epilogue: every output row is also stored into
// push_dst[owner] ([rows per rank, push_P * heads * d], this rank's head columns) and
// push_flags[owner][push_me * push_row_blocks + block] is raised by the rows written (batch 1,
// 128 | push_sl, default kernel only).  push_dst == null: no exchange.
int fm_flash_attn_fwd_push(const void* qkv, void* out, float* lse, int s, int b, int G, int qpg, int d,
                           float scale, unsigned long long timeout_ns, int* status, int version,
                           void* const* push_dst, int* const* push_flags, int push_me, int push_P,
                           int push_sl, int push_row_blocks, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
