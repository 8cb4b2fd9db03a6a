// C launchers of the non-GEMM kernels (implemented in the .cu files under csrc/).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#ifdef __cplusplus
}
#endif
