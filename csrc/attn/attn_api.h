// C entry points of the tcgen05 flash-attention kernels (causal, grouped-query, head_dim 128).
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// q [B,S,nh,128], k/v [B,S,nkv,128], o [B,S,nh,128]: bf16, contiguous.  lse [B,nh,S] fp32 holds the
// base-2 log-sum-exp of the scaled scores (what backward needs to rebuild the probabilities).
// S must be a multiple of 128 and nh a multiple of nkv.  Returns 0 or a negative argument / launch code;
// a wait that ran out inside the kernel is reported through `status` (see common/ptx.cuh).
int b200_flash_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int B, int S, int nh, int nkv,
                   float softmax_scale, int* status, cudaStream_t stream);

// Gradients of the same attention.  delta [B,nh,S] fp32 is scratch (row sums of dO*O); dq_acc [B,S,nh,128]
// fp32 is scratch that must be zero on entry and holds dQ on exit (dq, bf16, is written from it);
// dk/dv [B,S,nkv,128] bf16.
int b200_flash_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o, const float* lse,
                   float* delta, float* dq_acc, void* dq, void* dk, void* dv, int B, int S, int nh, int nkv,
                   float softmax_scale, int* status, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
