// Python bindings of the native library (pybind11, no dependency on libtorch: tensors cross
// the boundary as raw device pointers, streams as integer handles, so nothing here allocates).
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <stdexcept>
#include <string>

#include "include/fm_api.h"
#include "include/fm_ops.h"
#include "include/fm_symm.h"

namespace py = pybind11;

template <class T>
static T get(const py::dict& d, const char* key, T def) {
  if (!d.contains(key)) return def;
  py::object o = d[key];
  if (o.is_none()) return def;
  return o.cast<T>();
}
template <class P>
static P ptr(const py::dict& d, const char* key) {
  return reinterpret_cast<P>(get<uintptr_t>(d, key, 0));
}

static void check(int rc, const char* what) {
  if (rc != 0) throw std::runtime_error(std::string(what) + ": " + fm_last_error());
}

static void gemm_launch(const py::dict& d, uintptr_t stream) {
  FmGemmDesc g{};
  g.A = ptr<const void*>(d, "A");
  g.B = ptr<const void*>(d, "B");
  g.a_mn = get<int>(d, "a_mn", 0);
  g.b_mn = get<int>(d, "b_mn", 0);
  g.a_inner = get<long long>(d, "a_inner", 0);
  g.a_outer = get<long long>(d, "a_outer", 0);
  g.lda = get<long long>(d, "lda", 0);
  g.b_inner = get<long long>(d, "b_inner", 0);
  g.b_outer = get<long long>(d, "b_outer", 0);
  g.ldb = get<long long>(d, "ldb", 0);
  g.mode = get<int>(d, "mode", 0);
  g.num_groups = get<int>(d, "num_groups", 1);
  g.M = get<int>(d, "M", 0);
  g.N = get<int>(d, "N", 0);
  g.K = get<int>(d, "K", 0);
  g.uniform_rows = get<int>(d, "uniform_rows", 0);
  g.group_rows = ptr<const int*>(d, "group_rows");
  g.group_offs = ptr<const int*>(d, "group_offs");
  g.group_b = ptr<const int*>(d, "group_b");
  g.b_group_stride = get<int>(d, "b_group_stride", 0);
  g.gated = get<int>(d, "gated", 0);
  g.n_half = get<int>(d, "n_half", 0);
  g.bn = get<int>(d, "bn", 256);
  g.swizzle_m = get<int>(d, "swizzle_m", 0);
  g.cta_pair = get<int>(d, "cta_pair", 0);
  g.epi = get<int>(d, "epi", 0);
  g.C = ptr<void*>(d, "C");
  g.ldc = get<long long>(d, "ldc", 0);
  g.c_group_stride = get<long long>(d, "c_group_stride", 0);
  g.out_fp32 = get<int>(d, "out_fp32", 0);
  g.accumulate = get<int>(d, "accumulate", 0);
  g.alpha = get<float>(d, "alpha", 1.0f);
  g.act_out = ptr<void*>(d, "act_out");
  g.ld_act = get<long long>(d, "ld_act", 0);
  g.pre_out = ptr<void*>(d, "pre_out");
  g.ld_pre = get<long long>(d, "ld_pre", 0);
  g.probs = ptr<const float*>(d, "probs");
  g.act_kind = get<int>(d, "act_kind", 0);
  g.pre_in = ptr<const void*>(d, "pre_in");
  g.ld_pre_in = get<long long>(d, "ld_pre_in", 0);
  g.dprobs = ptr<float*>(d, "dprobs");
  g.dst_base = ptr<void* const*>(d, "dst_base");
  g.dst_rank = ptr<const int*>(d, "dst_rank");
  g.dst_row = ptr<const int*>(d, "dst_row");
  g.ld_dst = get<long long>(d, "ld_dst", 0);
  g.dst_flags = ptr<int* const*>(d, "dst_flags");
  g.num_ranks = get<int>(d, "num_ranks", 1);
  g.row_aux = ptr<const float*>(d, "row_aux");
  g.row_aux_dst = ptr<float* const*>(d, "row_aux_dst");
  g.gate_flags = ptr<const int*>(d, "gate_flags");
  g.gate_group_base = ptr<const int*>(d, "gate_group_base");
  g.gate_blocks_per_group = get<int>(d, "gate_blocks_per_group", 0);
  g.gate_expected = get<int>(d, "gate_expected", 0);
  g.gate_k_blocks_per_src = get<int>(d, "gate_k_blocks_per_src", 0);
  g.n_rotate = get<int>(d, "n_rotate", 0);
  g.k_rotate = get<int>(d, "k_rotate", 0);
  g.cols_per_rank = get<int>(d, "cols_per_rank", 0);
  g.dst_row_offset = get<long long>(d, "dst_row_offset", 0);
  g.adam_p = ptr<void*>(d, "adam_p");
  g.adam_m = ptr<void*>(d, "adam_m");
  g.adam_v = ptr<void*>(d, "adam_v");
  g.adam_lr = get<float>(d, "adam_lr", 0.f);
  g.adam_beta1 = get<float>(d, "adam_beta1", 0.f);
  g.adam_beta2 = get<float>(d, "adam_beta2", 0.f);
  g.adam_eps = get<float>(d, "adam_eps", 0.f);
  g.adam_wd = get<float>(d, "adam_wd", 0.f);
  g.adam_rbc1 = get<float>(d, "adam_rbc1", 1.f);
  g.adam_rbc2 = get<float>(d, "adam_rbc2", 1.f);
  g.max_ctas = get<int>(d, "max_ctas", 0);
  g.timeout_ns = get<unsigned long long>(d, "timeout_ns", 0ull);
  g.wait_ns = ptr<unsigned long long*>(d, "wait_ns");
  g.status = ptr<int*>(d, "status");
  check(fm_gemm_launch(&g, reinterpret_cast<cudaStream_t>(stream)), "fm_gemm_launch");
}

void bind_ops(py::module_& m);   // ops_bindings.cpp
void bind_symm(py::module_& m);  // symm_bindings.cpp

PYBIND11_MODULE(_C, m) {
  m.doc() = "fluidmoe_b200 native kernels (sm_100a)";
  m.def("gemm_launch", &gemm_launch, py::arg("desc"), py::arg("stream"));
  m.def("last_error", []() { return std::string(fm_last_error()); });
  m.attr("EPI_STORE") = (int)FM_EPI_STORE;
  m.attr("EPI_ACT") = (int)FM_EPI_ACT;
  m.attr("EPI_SCATTER") = (int)FM_EPI_SCATTER;
  m.attr("EPI_DACT") = (int)FM_EPI_DACT;
  m.attr("EPI_COLSCATTER") = (int)FM_EPI_COLSCATTER;
  m.attr("EPI_ADAM") = (int)FM_EPI_ADAM;
  m.attr("ACT_GELU") = (int)FM_ACT_GELU;
  m.attr("ACT_SILU") = (int)FM_ACT_SILU;
  m.attr("ACT_NONE") = (int)FM_ACT_NONE;
  bind_ops(m);
  bind_symm(m);
}
