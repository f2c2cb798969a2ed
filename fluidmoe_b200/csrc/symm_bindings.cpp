// pybind11 bindings of the symmetric-memory runtime.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <stdexcept>
#include <string>
#include <vector>

#include "include/fm_api.h"
#include "include/fm_symm.h"

namespace py = pybind11;

static void chk(int rc, const char* what) {
  if (rc != 0) throw std::runtime_error(std::string(what) + ": " + fm_last_error());
}
template <class P>
static P as_ptr(uintptr_t v) {
  return reinterpret_cast<P>(v);
}

static FmDroplessPlan plan_from(const std::vector<uintptr_t>& v) {
  if (v.size() != 10) throw std::runtime_error("dropless plan needs 10 device pointers");
  FmDroplessPlan p;
  p.counts_all = as_ptr<int*>(v[0]);
  p.group_rows = as_ptr<int*>(v[1]);
  p.group_offs = as_ptr<int*>(v[2]);
  p.group_flag_base = as_ptr<int*>(v[3]);
  p.dst_base = as_ptr<int*>(v[4]);
  p.slot_start = as_ptr<int*>(v[5]);
  p.before = as_ptr<int*>(v[6]);
  p.src_prefix = as_ptr<int*>(v[7]);
  p.recv_expected = as_ptr<int*>(v[8]);
  p.totals = as_ptr<int*>(v[9]);
  return p;
}

void bind_symm(py::module_& m) {
  m.def("dropless_plan", [](uintptr_t counts, uintptr_t table_ptrs, uintptr_t flag_ptrs, int epoch, int P, int me,
                            int E, int nle, int mult, int max_rows, const std::vector<uintptr_t>& plan,
                            uintptr_t row_rank, uintptr_t row_row, unsigned long long timeout_ns, uintptr_t status,
                            uintptr_t stream) {
    FmDroplessPlan pl = plan_from(plan);
    chk(fm_dropless_plan(as_ptr<const int*>(counts), as_ptr<int* const*>(table_ptrs), as_ptr<int* const*>(flag_ptrs),
                         epoch, P, me, E, nle, mult, max_rows, &pl, as_ptr<int*>(row_rank), as_ptr<int*>(row_row),
                         timeout_ns, as_ptr<int*>(status), as_ptr<cudaStream_t>(stream)),
        "dropless_plan");
  });
  m.def("dropless_dispatch", [](uintptr_t x, uintptr_t sorted_idx, uintptr_t probs, const std::vector<uintptr_t>& plan,
                                uintptr_t dst_tokens, uintptr_t dst_probs, uintptr_t dst_flags, long long total_slots,
                                int H, int E, int nle, int P, int me, int ctas, uintptr_t stream) {
    FmDroplessPlan pl = plan_from(plan);
    chk(fm_dropless_dispatch(as_ptr<const void*>(x), as_ptr<const long long*>(sorted_idx), as_ptr<const float*>(probs),
                             &pl, as_ptr<void* const*>(dst_tokens), as_ptr<float* const*>(dst_probs),
                             as_ptr<int* const*>(dst_flags), total_slots, H, E, nle, P, me, ctas,
                             as_ptr<cudaStream_t>(stream)),
        "dropless_dispatch");
  });
  m.def("zero_group_padding", [](uintptr_t buf, long long row_bytes, uintptr_t rows, uintptr_t offs, int n,
                                 uintptr_t stream) {
    chk(fm_zero_group_padding(as_ptr<void*>(buf), row_bytes, as_ptr<const int*>(rows), as_ptr<const int*>(offs), n,
                              as_ptr<cudaStream_t>(stream)),
        "zero_group_padding");
  });
  m.def("symm_alloc", [](size_t bytes) {
    void* p = nullptr;
    unsigned char h[FM_IPC_HANDLE_BYTES];
    chk(fm_symm_alloc(bytes, &p, h), "symm_alloc");
    return py::make_tuple(reinterpret_cast<uintptr_t>(p),
                          py::bytes(reinterpret_cast<const char*>(h), FM_IPC_HANDLE_BYTES));
  });
  m.def("symm_open", [](const std::string& handle) {
    if (handle.size() != FM_IPC_HANDLE_BYTES) throw std::runtime_error("bad IPC handle size");
    void* p = nullptr;
    chk(fm_symm_open(reinterpret_cast<const unsigned char*>(handle.data()), &p), "symm_open");
    return reinterpret_cast<uintptr_t>(p);
  });
  m.def("symm_close", [](uintptr_t p) { chk(fm_symm_close(as_ptr<void*>(p)), "symm_close"); });
  m.def("symm_free", [](uintptr_t p) { chk(fm_symm_free(as_ptr<void*>(p)), "symm_free"); });
  m.def("can_access_peer", &fm_symm_can_access_peer);
  m.def("symm_barrier", [](uintptr_t flag_ptrs, int rank, int n, int epoch,
                           unsigned long long timeout_ns, uintptr_t status, uintptr_t stream) {
    chk(fm_symm_barrier(as_ptr<int* const*>(flag_ptrs), rank, n, epoch, timeout_ns,
                        as_ptr<int*>(status), as_ptr<cudaStream_t>(stream)),
        "symm_barrier");
  });
  m.def("a2a_push", [](uintptr_t send, uintptr_t send_offs, uintptr_t send_bytes,
                       uintptr_t recv_ptrs, uintptr_t dst_offs, uintptr_t flag_ptrs,
                       uintptr_t counters, int rank, int n, int epoch, int ctas, uintptr_t stream) {
    chk(fm_a2a_push(as_ptr<const void*>(send), as_ptr<const long long*>(send_offs),
                    as_ptr<const long long*>(send_bytes), as_ptr<void* const*>(recv_ptrs),
                    as_ptr<const long long*>(dst_offs), as_ptr<int* const*>(flag_ptrs),
                    as_ptr<int*>(counters), rank, n, epoch, ctas, as_ptr<cudaStream_t>(stream)),
        "a2a_push");
  });
  m.def("permute_dispatch", [](uintptr_t x, uintptr_t idx, uintptr_t probs, uintptr_t dst_tokens,
                               uintptr_t dst_probs, uintptr_t dst_flags, long long total, int H, int cap,
                               int nle, int P, int me, int bpg, int ctas, uintptr_t stream) {
    chk(fm_permute_dispatch(as_ptr<const void*>(x), as_ptr<const long long*>(idx),
                            as_ptr<const float*>(probs), as_ptr<void* const*>(dst_tokens),
                            as_ptr<float* const*>(dst_probs), as_ptr<int* const*>(dst_flags), total, H,
                            cap, nle, P, me, bpg, ctas, as_ptr<cudaStream_t>(stream)),
        "permute_dispatch");
  });
  m.def("rows_push", [](uintptr_t src, uintptr_t dst_base, uintptr_t dst_flags, long long rows_blk, int W,
                        int P, int me, int row_blocks, int ctas, uintptr_t stream) {
    chk(fm_rows_push(as_ptr<const void*>(src), as_ptr<void* const*>(dst_base), as_ptr<int* const*>(dst_flags),
                     rows_blk, W, P, me, row_blocks, ctas, as_ptr<cudaStream_t>(stream)),
        "rows_push");
  });
  m.def("a2a_wait", [](uintptr_t flags, int rank, int n, int epoch, unsigned long long timeout_ns,
                       uintptr_t status, uintptr_t stream) {
    chk(fm_a2a_wait(as_ptr<const int*>(flags), rank, n, epoch, timeout_ns, as_ptr<int*>(status),
                    as_ptr<cudaStream_t>(stream)),
        "a2a_wait");
  });
  m.def("a2a_wait_counts", [](uintptr_t flags, int n, int epoch, uintptr_t expected, uintptr_t wait_ns,
                              unsigned long long timeout_ns, uintptr_t status, uintptr_t stream) {
    chk(fm_a2a_wait_counts(as_ptr<const int*>(flags), n, epoch, as_ptr<const int*>(expected),
                           as_ptr<unsigned long long*>(wait_ns), timeout_ns, as_ptr<int*>(status),
                           as_ptr<cudaStream_t>(stream)),
        "a2a_wait_counts");
  });
  m.def("put_signal", [](uintptr_t src, long long bytes, uintptr_t dst, uintptr_t flag, int value,
                         int ctas, uintptr_t counter, uintptr_t stream) {
    chk(fm_put_signal(as_ptr<const void*>(src), bytes, as_ptr<void*>(dst), as_ptr<int*>(flag), value,
                      ctas, as_ptr<int*>(counter), as_ptr<cudaStream_t>(stream)),
        "put_signal");
  });
  m.def("wait_flag", [](uintptr_t flag, int expected, unsigned long long timeout_ns,
                        uintptr_t status, uintptr_t stream) {
    chk(fm_wait_flag(as_ptr<const int*>(flag), expected, timeout_ns, as_ptr<int*>(status),
                     as_ptr<cudaStream_t>(stream)),
        "wait_flag");
  });
  m.def("allreduce_p2p_slice", [](uintptr_t bufs, long long elem_offset, long long count, int fp32, float scale,
                                  uintptr_t flags, int rank, int n, int epoch, int ctas,
                                  unsigned long long timeout_ns, uintptr_t status, uintptr_t stream) {
    chk(fm_allreduce_p2p_slice(as_ptr<void* const*>(bufs), elem_offset, count, fp32, scale,
                               as_ptr<int* const*>(flags), rank, n, epoch, ctas, timeout_ns,
                               as_ptr<int*>(status), as_ptr<cudaStream_t>(stream)),
        "allreduce_p2p_slice");
  });
  m.def("allreduce_p2p", [](uintptr_t bufs, long long count, int fp32, float scale,
                            uintptr_t flag_ptrs, int rank, int n, int epoch, int ctas,
                            unsigned long long timeout_ns, uintptr_t status, uintptr_t stream) {
    chk(fm_allreduce_p2p(as_ptr<void* const*>(bufs), count, fp32, scale,
                         as_ptr<int* const*>(flag_ptrs), rank, n, epoch, ctas, timeout_ns,
                         as_ptr<int*>(status), as_ptr<cudaStream_t>(stream)),
        "allreduce_p2p");
  });
  m.def("allreduce_nvls", [](uintptr_t mc, long long count, float scale, uintptr_t flag_ptrs, int rank, int n,
                             int epoch, int ctas, unsigned long long timeout_ns, uintptr_t status,
                             uintptr_t stream) {
    chk(fm_allreduce_nvls(as_ptr<float*>(mc), count, scale, as_ptr<int* const*>(flag_ptrs), rank, n, epoch,
                          ctas, timeout_ns, as_ptr<int*>(status), as_ptr<cudaStream_t>(stream)),
        "allreduce_nvls");
  });
}
