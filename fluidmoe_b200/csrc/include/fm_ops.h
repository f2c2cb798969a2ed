// C ABI of the element-wise / reduction kernels (see csrc/ops/*.cu).
#pragma once
#include <stdint.h>
#include <cuda_runtime.h>
#ifdef __cplusplus
extern "C" {
#endif
#ifdef __cplusplus
}
#endif
