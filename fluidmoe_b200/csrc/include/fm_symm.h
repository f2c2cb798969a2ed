// C ABI of the symmetric-memory runtime (see csrc/symm/symm_heap.cpp).
#pragma once
#include <stdint.h>
#include <cuda_runtime.h>
#ifdef __cplusplus
extern "C" {
#endif
#ifdef __cplusplus
}
#endif
