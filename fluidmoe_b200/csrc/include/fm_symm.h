// C ABI of the symmetric-memory runtime: slabs of device memory that every rank of a group can
// address directly over NVLink, plus the device-initiated primitives built on them (barrier,
// all-to-all, all-reduce).  It takes the place of the reference's NVSHMEM host wrapper
// (fluid/csrc/nvshmem_ops.cpp): same contract (collective alloc / free, non-owning views,
// stream-ordered put + signal, bounded waits) but the transfers are issued by kernels, not by
// the host.
#pragma once
#include <stdint.h>
#include <cuda_runtime.h>
#ifdef __cplusplus
extern "C" {
#endif

#define FM_IPC_HANDLE_BYTES 64

// ---- slab management (host) ----
// Allocate `bytes` of device memory on the current device and export an IPC handle for it.
int fm_symm_alloc(size_t bytes, void** ptr, unsigned char handle[FM_IPC_HANDLE_BYTES]);
// Map a peer's slab into this process; enables peer access lazily.
int fm_symm_open(const unsigned char handle[FM_IPC_HANDLE_BYTES], void** peer_ptr);
int fm_symm_close(void* peer_ptr);
int fm_symm_free(void* ptr);
int fm_symm_can_access_peer(int dev, int peer_dev);

// ---- device-initiated primitives ----
// Barrier across `nranks` ranks.  flag_ptrs[p] = address of rank p's int32[nranks] barrier
// words (in its slab); every rank passes the same epoch, which grows by one per barrier.
int fm_symm_barrier(int* const* flag_ptrs_dev, int my_rank, int nranks, int epoch,
                    unsigned long long timeout_ns, int* status, cudaStream_t stream);

// All-to-all push: slice p of `send` (send_offs[p] .. +send_bytes[p], 16-byte multiples) is
// stored into rank p's receive buffer at recv_ptrs[p] + dst_offs[p]; afterwards rank p's
// arrival word flag_ptrs[p][my_rank] is set to `epoch` with a system-scope release.
// All index arrays are device arrays of length nranks.
int fm_a2a_push(const void* send, const long long* send_offs, const long long* send_bytes,
                void* const* recv_ptrs, const long long* dst_offs, int* const* flag_ptrs,
                int* local_counters, int my_rank, int nranks, int epoch, int num_ctas,
                cudaStream_t stream);
// Fused permute + dispatch (see permute_dispatch_kernel).  dst_* are device tables indexed by
// destination rank; probs may be null (then no probabilities are sent).
int fm_permute_dispatch(const void* x, const long long* sorted_idx, const float* probs,
                        void* const* dst_tokens, float* const* dst_probs, int* const* dst_flags,
                        long long total_slots, int H, int cap, int nle, int P, int me,
                        int blocks_per_group, int num_ctas, cudaStream_t stream);
// HP->SP push (see rows_push_kernel).
int fm_rows_push(const void* src, void* const* dst_base, int* const* dst_flags, long long rows_blk,
                 int W, int P, int me, int row_blocks, int num_ctas, cudaStream_t stream);
// Wait (bounded) until every peer's arrival word in `my_flags` reached `epoch`.
int fm_a2a_wait(const int* my_flags, int my_rank, int nranks, int epoch,
                unsigned long long timeout_ns, int* status, cudaStream_t stream);
// Same, with per-source thresholds read from device memory (`expected[p]`, may be null: then
// `epoch`) and an optional device counter that accumulates the nanoseconds waited.
int fm_a2a_wait_counts(const int* my_flags, int nranks, int epoch, const int* expected,
                       unsigned long long* wait_ns, unsigned long long timeout_ns, int* status,
                       cudaStream_t stream);

// ---- dropless (variable-split) expert exchange: see symm/dropless_kernels.cu ----
// Device arrays the plan kernel fills (all int32, owned by the caller).
typedef struct {
  int* counts_all;       // [P * E]   pairs rank r routes to global expert e
  int* group_rows;       // [nle]     rows of every local expert (all sources)
  int* group_offs;       // [nle]     first row of every local expert (multiple of 128)
  int* group_flag_base;  // [nle]     group_offs / 128: first arrival counter of the expert
  int* dst_base;         // [E]       row in the owner's buffer where this rank's run for expert e starts
  int* slot_start;       // [E + 1]   first slot of expert e in this rank's permuted order
  int* before;           // [P * nle] rows of local expert j that come from ranks < r
  int* src_prefix;       // [P * E]   slot_start of every rank
  int* recv_expected;    // [P]       rows coming back from rank p, times `expected_mult`
  int* totals;           // [2]       rows of the local expert-major buffer in use; 1 if the plan was refused
} FmDroplessPlan;
// Exchange the per-expert counts with every peer (peer stores + flag, bounded wait) and derive the
// plan; then fill, for every local expert-major row, the rank and permuted-order row it returns to
// (-1 for padding rows).  `table_ptrs[p]`: rank p's int[2][P][E]; `flag_ptrs[p]`: rank p's int[P];
// `epoch` must grow by one per call.  A plan needing more than `max_rows` rows on any rank is
// refused by all ranks alike: nothing is sent and a status record is written.
int fm_dropless_plan(const int* counts, int* const* table_ptrs, int* const* flag_ptrs, int epoch, int P,
                     int me, int E, int nle, int expected_mult, int max_rows, const FmDroplessPlan* out,
                     int* row_dst_rank, int* row_dst_row, unsigned long long timeout_ns, int* status,
                     cudaStream_t stream);
// Gather the routed rows and store them into their owners' buffers, one arrival per row on the
// counter of the row's 128-row block; probs may be null.
int fm_dropless_dispatch(const void* x, const long long* sorted_idx, const float* probs,
                         const FmDroplessPlan* pl, void* const* dst_tokens, float* const* dst_probs,
                         int* const* dst_flags, long long total_slots, int H, int E, int nle, int P, int me,
                         int num_ctas, cudaStream_t stream);
// Zero the rows that pad every group to a whole 128-row block.
int fm_zero_group_padding(void* buf, long long row_bytes, const int* group_rows, const int* group_offs,
                          int num_groups, cudaStream_t stream);

// Two-shot all-reduce (sum) over peer memory: every rank's `buf_ptrs[p]` points at its copy of
// the same symmetric buffer of `count` elements (fp32 or bf16, in place).  Rank r reduces
// chunk r by reading all peers, scales by `scale`, and writes the result to every peer.
int fm_allreduce_p2p(void* const* buf_ptrs_dev, long long count, int dtype_fp32, float scale,
                     int* const* flag_ptrs_dev, int my_rank, int nranks, int epoch, int num_ctas,
                     unsigned long long timeout_ns, int* status, cudaStream_t stream);

// Same on the slice [elem_offset, elem_offset + count) of the buffers (the slice must start on a
// 16-byte boundary): what a scheduler that reduces a flat gradient buffer piece by piece calls.
int fm_allreduce_p2p_slice(void* const* buf_ptrs_dev, long long elem_offset, long long count, int dtype_fp32,
                           float scale, int* const* flag_ptrs_dev, int my_rank, int nranks, int epoch,
                           int num_ctas, unsigned long long timeout_ns, int* status, cudaStream_t stream);

// In-switch (NVLS) sum all-reduce of `count` fp32 elements in place.  `multicast_ptr` is the
// multicast address of a buffer that every rank bound to the same NVLink multicast object (the
// caller obtains it from a VMM-based symmetric allocator); the flags live in this library's own
// symmetric heap.  Rank r reduces slice r with multimem.ld_reduce and broadcasts it with multimem.st.
int fm_allreduce_nvls(float* multicast_ptr, long long count, float scale, int* const* flag_ptrs_dev,
                      int my_rank, int nranks, int epoch, int num_ctas, unsigned long long timeout_ns,
                      int* status, cudaStream_t stream);

// One-sided put + signal: copy `bytes` (16-byte multiple) from `src` to `dst` (a peer address),
// then store `value` to `flag` (a peer address) with a system-scope release.
int fm_put_signal(const void* src, long long bytes, void* dst, int* flag, int value, int num_ctas,
                  int* local_counter, cudaStream_t stream);

// Test hook for bounded waits: waits for *flag >= expected and reports a status on timeout.
int fm_wait_flag(const int* flag, int expected, unsigned long long timeout_ns, int* status,
                 cudaStream_t stream);

#ifdef __cplusplus
}
#endif
