// pybind11 bindings of the element-wise kernels.
#include <pybind11/pybind11.h>

#include <stdexcept>
#include <string>

#include "include/fm_api.h"
#include "include/fm_ops.h"

namespace py = pybind11;
using u = uintptr_t;

static void chk(int rc, const char* what) {
  if (rc != 0) throw std::runtime_error(std::string(what) + ": " + fm_last_error());
}
template <class P>
static P p(u v) {
  return reinterpret_cast<P>(v);
}
static cudaStream_t st(u v) { return reinterpret_cast<cudaStream_t>(v); }

void bind_ops(py::module_& m) {
  m.def("norm_fwd", [](u x, u w, u b, u y, u mean, u rstd, int T, int H, float eps, int kind, u s) {
    chk(fm_norm_fwd(p<const void*>(x), p<const void*>(w), p<const void*>(b), p<void*>(y),
                    p<float*>(mean), p<float*>(rstd), T, H, eps, kind, st(s)), "norm_fwd");
  });
  m.def("norm_bwd_blocks", &fm_norm_bwd_blocks);
  m.def("norm_bwd", [](u dy, u x, u w, u mean, u rstd, u res, u dx, u partial, u dw, u db, int T,
                       int H, int kind, u s) {
    chk(fm_norm_bwd(p<const void*>(dy), p<const void*>(x), p<const void*>(w), p<const float*>(mean),
                    p<const float*>(rstd), p<const void*>(res), p<void*>(dx), p<float*>(partial),
                    p<float*>(dw), p<float*>(db), T, H, kind, st(s)), "norm_bwd");
  });
  m.def("rope_packed_gated", [](u t, u freqs, long long rows, int hpr, int rope_heads, int d, int rot,
                                int rows_per_pos, int backward, u flags, int n, int expected, u wait_ns,
                                unsigned long long timeout_ns, u status, u s) {
    chk(fm_rope_packed_gated(p<void*>(t), p<const float*>(freqs), rows, hpr, rope_heads, d, rot, rows_per_pos,
                             backward, p<const int*>(flags), n, expected, p<unsigned long long*>(wait_ns),
                             timeout_ns, p<int*>(status), st(s)), "rope_packed_gated");
  });
  m.def("rope_packed", [](u t, u freqs, long long rows, int hpr, int rope_heads, int d, int rot,
                          int rows_per_pos, int backward, u s) {
    chk(fm_rope_packed(p<void*>(t), p<const float*>(freqs), rows, hpr, rope_heads, d, rot,
                       rows_per_pos, backward, st(s)), "rope_packed");
  });
  m.def("topk_softmax", [](u logits, u idx, u probs, int T, int E, int k, u s) {
    chk(fm_topk_softmax(p<const float*>(logits), p<long long*>(idx), p<float*>(probs), T, E, k, st(s)),
        "topk_softmax");
  });
  m.def("gather_rows", [](u x, u idx, u out, long long rows, int H, u s) {
    chk(fm_gather_rows(p<const void*>(x), p<const long long*>(idx), p<void*>(out), rows, H, st(s)),
        "gather_rows");
  });
  m.def("unpermute_reduce_gated", [](u rows, u slot, u res, u out, int T, int k, int H, u flags, int n, int expected,
                                     u wait_ns, unsigned long long timeout_ns, u status, u s) {
    chk(fm_unpermute_reduce_gated(p<const void*>(rows), p<const int*>(slot), p<const void*>(res), p<void*>(out), T, k,
                                  H, p<const int*>(flags), n, expected, p<unsigned long long*>(wait_ns), timeout_ns,
                                  p<int*>(status), st(s)), "unpermute_reduce_gated");
  });
  m.def("unpermute_reduce", [](u rows, u slot, u res, u out, int T, int k, int H, u s) {
    chk(fm_unpermute_reduce(p<const void*>(rows), p<const int*>(slot), p<const void*>(res),
                            p<void*>(out), T, k, H, st(s)), "unpermute_reduce");
  });
  m.def("moe_plan", [](u ti, u tp, int T, int k, int E, int cap, u si, u sp, u sot, u rpe, u s) {
    chk(fm_moe_plan(p<const long long*>(ti), p<const float*>(tp), T, k, E, cap, p<long long*>(si),
                    p<float*>(sp), p<int*>(sot), p<int*>(rpe), st(s)), "moe_plan");
  });
  m.def("flash_attn_fwd", [](u qkv, u out, u lse, int s_, int b, int G, int qpg, int d, float scale,
                             unsigned long long timeout_ns, u status, int version, u s) {
    chk(fm_flash_attn_fwd(p<const void*>(qkv), p<void*>(out), p<float*>(lse), s_, b, G, qpg, d, scale,
                          timeout_ns, p<int*>(status), version, st(s)), "flash_attn_fwd");
  });
  m.def("flash_attn_fwd_push", [](u qkv, u out, u lse, int s_, int b, int G, int qpg, int d, float scale,
                                  unsigned long long timeout_ns, u status, int version, u push_dst, u push_flags,
                                  int me, int P, int sl, int row_blocks, u s) {
    chk(fm_flash_attn_fwd_push(p<const void*>(qkv), p<void*>(out), p<float*>(lse), s_, b, G, qpg, d, scale,
                               timeout_ns, p<int*>(status), version, p<void* const*>(push_dst),
                               p<int* const*>(push_flags), me, P, sl, row_blocks, st(s)), "flash_attn_fwd_push");
  });
  m.def("cross_entropy", [](u logits, u labels, u loss, int T, int V, float scale, u s) {
    chk(fm_cross_entropy(p<void*>(logits), p<const long long*>(labels), p<float*>(loss), T, V, scale, st(s)),
        "cross_entropy");
  });
  m.def("flash_attn_bwd_gated", [](u qkv, u out, u dout, u lse, u delta, u dq, u dqkv, int s_, int b, int G, int qpg,
                                   int d, float scale, unsigned long long timeout_ns, u status, int version, u dkv,
                                   int hsplit, u flags, int n, int expected, u wait_ns, u s) {
    chk(fm_flash_attn_bwd_gated(p<const void*>(qkv), p<const void*>(out), p<const void*>(dout), p<const float*>(lse),
                                p<float*>(delta), p<float*>(dq), p<void*>(dqkv), s_, b, G, qpg, d, scale, timeout_ns,
                                p<int*>(status), version, p<float*>(dkv), hsplit, p<const int*>(flags), n, expected,
                                p<unsigned long long*>(wait_ns), st(s)), "flash_attn_bwd_gated");
  });
  m.def("flash_attn_bwd", [](u qkv, u out, u dout, u lse, u delta, u dq, u dqkv, int s_, int b, int G, int qpg,
                             int d, float scale, unsigned long long timeout_ns, u status, int version, u dkv, int hsplit, u s) {
    chk(fm_flash_attn_bwd(p<const void*>(qkv), p<const void*>(out), p<const void*>(dout), p<const float*>(lse),
                          p<float*>(delta), p<float*>(dq), p<void*>(dqkv), s_, b, G, qpg, d, scale, timeout_ns,
                          p<int*>(status), version, p<float*>(dkv), hsplit, st(s)), "flash_attn_bwd");
  });
  m.def("router_bwd", [](u dprobs, u slot_of_token, u top_idx, u top_probs, u logits, u tpe, float aux_coef,
                         float z_coef, int T, int k, int E, u dlogits, u s) {
    chk(fm_router_bwd(p<const float*>(dprobs), p<const int*>(slot_of_token), p<const long long*>(top_idx),
                      p<const float*>(top_probs), p<const float*>(logits), p<const float*>(tpe), aux_coef, z_coef,
                      T, k, E, p<float*>(dlogits), st(s)), "router_bwd");
  });
  m.def("adam_background", [](u prm, u g, u mm, u v, long long n, float lr, float b1, float b2, float eps,
                              float wd, int step, float grad_scale, int ctas, u s) {
    chk(fm_adam_background(p<void*>(prm), p<const float*>(g), p<void*>(mm), p<void*>(v), n, lr, b1, b2, eps, wd,
                           step, grad_scale, ctas, st(s)), "adam_background");
  });
  m.def("adam", [](u prm, u master, u g, u mm, u v, long long n, float lr, float b1, float b2,
                   float eps, float wd, int step, float grad_scale, int zero_grad, int state_bf16, u s) {
    chk(fm_adam(p<void*>(prm), p<float*>(master), p<float*>(g), p<void*>(mm), p<void*>(v), n, lr,
                b1, b2, eps, wd, step, grad_scale, zero_grad, state_bf16, st(s)), "adam");
  });
}
