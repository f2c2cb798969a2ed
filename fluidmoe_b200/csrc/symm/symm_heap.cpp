// Host side of the symmetric-memory runtime: slab allocation and CUDA IPC mapping.
#include <stdio.h>
#include <string.h>

#include "../include/fm_symm.h"

extern "C" void fm_set_error(const char* msg);

static int fail(cudaError_t e, const char* what) {
  char buf[256];
  snprintf(buf, sizeof(buf), "%s: %s", what, cudaGetErrorString(e));
  fm_set_error(buf);
  (void)cudaGetLastError();
  return (int)e;
}

extern "C" int fm_symm_alloc(size_t bytes, void** ptr, unsigned char handle[FM_IPC_HANDLE_BYTES]) {
  static_assert(sizeof(cudaIpcMemHandle_t) == FM_IPC_HANDLE_BYTES, "IPC handle size");
  cudaError_t e = cudaMalloc(ptr, bytes);
  if (e != cudaSuccess) return fail(e, "cudaMalloc(slab)");
  e = cudaMemset(*ptr, 0, bytes);
  if (e != cudaSuccess) return fail(e, "cudaMemset(slab)");
  cudaIpcMemHandle_t h;
  e = cudaIpcGetMemHandle(&h, *ptr);
  if (e != cudaSuccess) {
    // Memory stays usable locally (single-rank runs need no handle).
    memset(handle, 0, FM_IPC_HANDLE_BYTES);
    (void)cudaGetLastError();
    return 0;
  }
  memcpy(handle, &h, FM_IPC_HANDLE_BYTES);
  return 0;
}

extern "C" int fm_symm_open(const unsigned char handle[FM_IPC_HANDLE_BYTES], void** peer_ptr) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, FM_IPC_HANDLE_BYTES);
  cudaError_t e = cudaIpcOpenMemHandle(peer_ptr, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return fail(e, "cudaIpcOpenMemHandle");
  return 0;
}

extern "C" int fm_symm_close(void* peer_ptr) {
  cudaError_t e = cudaIpcCloseMemHandle(peer_ptr);
  if (e != cudaSuccess) return fail(e, "cudaIpcCloseMemHandle");
  return 0;
}

extern "C" int fm_symm_free(void* ptr) {
  cudaError_t e = cudaFree(ptr);
  if (e != cudaSuccess) return fail(e, "cudaFree(slab)");
  return 0;
}

extern "C" int fm_symm_can_access_peer(int dev, int peer_dev) {
  int ok = 0;
  if (cudaDeviceCanAccessPeer(&ok, dev, peer_dev) != cudaSuccess) {
    (void)cudaGetLastError();
    return 0;
  }
  return ok;
}
