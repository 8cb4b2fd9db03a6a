// C interface of the tcgen05 GEMM family (implemented in gemm_sm100.cu).
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Problem modes / epilogues: numeric values match b200::GemmMode / b200::GemmEpi.
typedef struct B200GemmDesc {
  int mode;  // 0 dense, 1 grouped by rows (padded expert segments), 2 grouped by contraction (per-expert dW)
  int epi;   // 0 bf16, 1 fp32 (beta), 2 swiglu, 3 swiglu backward, 4 bf16 + softmax partials, 5 bf16 scatter to peers,
             // 6 fused QKV projection: raw bf16 output + per-head RMSNorm and RoPE of the q / k heads (pair-tile kernel)
  int bn;    // tile width: 256, 128 or 64
  int cta2;  // 1: pair-tile kernel (two CTAs per 256-row tile, TMA-store epilogue); bn 256 or 128
  int a_mn;  // A stored with the M index contiguous (rows = contraction index)
  int b_mn;  // B stored with the N index contiguous (rows = contraction index)
  int M, N, K;
  int num_experts;
  int m_fast;
  int beta;
  int n_half;
  // A tensor (bf16): `a_inner` contiguous elements per row, `a_rows` rows, row pitch lda (elements)
  const void* A;
  long long lda;
  long long a_inner, a_rows;
  // B tensor (bf16): [b_experts][b_rows][b_inner], row pitch ldb, expert pitch b_expert_stride (elements)
  const void* B;
  long long ldb, b_expert_stride;
  long long b_inner, b_rows;
  int b_experts;
  const int* tile_expert;
  const int* num_m_tiles;
  const int* seg_off;
  // pair-tile kernel, grouped by rows: int2 per tile (first row, expert | live 128-row halves << 16);
  // num_m_tiles then holds the number of pair tiles
  const int* pair_tiles;
  int max_pair_tiles;
  // pair-tile kernel: fetch operand rows by index with TMA gather.  a_gather: A (K-major) is then the SOURCE
  // tensor [a_rows, a_inner] and a_gather[r] names the source row of output row r; b_gather: B (MN-major,
  // grouped by contraction) is the source tensor [b_rows, b_inner] and b_gather[k] the source row of contraction
  // row k.  Indices outside the source give zero rows.
  const int* a_gather;
  const int* b_gather;
  // pair-tile SwiGLU epilogues: fold the routing weight row_w[row_slot[r]] of sorted row r into the stored
  // activation (forward) / the incoming gradient (backward, which also writes row_dot[r * n_tiles + n])
  const int* row_slot;
  const float* row_w;
  float* row_dot;
  // epi 6 (head_dim 128; C = raw projection [M, N], aux0 = same layout with q / k heads normalised and rotated, v
  // heads copied): rope_cs [S, 64, 2] fp32 (cos, sin), rope_w / rope_kw [128] fp32 (q-norm / k-norm weight), rope_rstd
  // [M, nh + nkv] fp32 receives the reciprocal RMS of every q / k head; the position of row r is r % rope_S
  const float* rope_cs;
  const float* rope_w;
  const float* rope_kw;
  float* rope_rstd;
  int rope_S, rope_nh, rope_nkv;
  float rope_eps;
  void* C;
  long long ldc, c_expert_stride;
  void* aux0;
  long long ld_aux0;
  void* aux1;
  long long ld_aux1;
  int* status;  // device int, 0 = ok; a bounded wait that ran out writes its code here
  // ---- expert-parallel hooks (see b200::GemmEp); leave zeroed when unused
  const int* ep_wait_flags;
  int ep_wait_n;
  const int* ep_epoch_base;
  int ep_wait_epoch_off;
  void* ep_scatter_dst[8];
  const int* ep_scatter_meta;
  int* ep_post_flags[8];
  int ep_post_index;
  int ep_post_epoch_off;
  int ep_world;
  int* ep_counter;
  unsigned long long ep_limit_ns;
} B200GemmDesc;

// Enqueue one GEMM on `stream`. Returns 0 on success, a negative code on a host-side error.
int b200_gemm(const B200GemmDesc* desc, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
