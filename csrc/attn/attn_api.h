// C entry points of the tcgen05 flash-attention kernels (causal, grouped-query, head_dim 128 or 64).
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// q [B,S,nh,hd], k/v [B,S,nkv,hd], o [B,S,nh,hd]: bf16; hd = head_dim is 128 or 64.  o is contiguous; q, k, v may be
// slices of a wider row (the fused QKV activation): ldq / ldk / ldv give the distance between consecutive tokens
// in elements (0 = contiguous), a token's heads are contiguous and batches follow each other after S tokens.  lse [B,nh,S] fp32 holds the
// base-2 log-sum-exp of the scaled scores (what backward needs to rebuild the probabilities).
// S must be a multiple of 128 and nh a multiple of nkv.  Returns 0 or a negative argument / launch code;
// a wait that ran out inside the kernel is reported through `status` (see common/ptx.cuh).
int b200_flash_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int B, int S, int nh, int nkv,
                   int head_dim, long long ldq, long long ldk, long long ldv, float softmax_scale, int* status,
                   cudaStream_t stream);

// Gradients of the same attention (same shape rules).  delta [B,nh,S] fp32 is scratch: it receives
// softmax_scale * rowsum(dO * O).  dq [B,S,nh,hd], dk/dv [B,S,nkv,hd] bf16 are overwritten.  Three
// launches: delta, dQ (one query tile per work item, loops over key tiles) and dK/dV (one key tile per
// work item, loops over the query heads of its group and their query tiles).
int b200_flash_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o, const float* lse,
                   float* delta, void* dq, void* dk, void* dv, int B, int S, int nh, int nkv, int head_dim,
                   long long ldq, long long ldk, long long ldv, float softmax_scale, int* status, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
