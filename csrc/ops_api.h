// C launchers of the non-GEMM kernels (implemented in the .cu files under csrc/).
// All pointers are device pointers; bf16 tensors are passed as void*. Every function only
// enqueues work on `stream` and returns 0, or a negative code for a rejected argument.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// ---- norm/rmsnorm.cu
int b200_rmsnorm_fwd(const void* x, const void* res, const float* w, void* h_out, void* y, float* rstd, int T, int H,
                     float eps, cudaStream_t stream);
int b200_rmsnorm_bwd_blocks(int T);  // rows of the dw scratch: float[blocks * H]
int b200_rmsnorm_bwd(const void* dy, const void* x, const float* rstd, const float* w, const void* dres, void* dx,
                     float* dw_part, float* dw_out, int dw_accumulate, int T, int H, cudaStream_t stream);

// ---- rope/qknorm_rope.cu
int b200_qknorm_rope_blocks(long long items);  // dw scratch: float[blocks * 2 * hd]
int b200_qknorm_rope_fwd(const void* qkv, int ld, const float* qw, const float* kw, const float* cs, void* q_out,
                         void* k_out, void* v_out, float* rstd, int T, int S, int nh, int nkv, int hd, float eps,
                         cudaStream_t stream);
int b200_qknorm_rope_bwd(const void* dq, const void* dk, const void* dv, const void* qkv, int ld, const float* rstd,
                         const float* qw, const float* kw, const float* cs, void* dqkv, float* dw_part, float* dqw,
                         float* dkw, int dw_accumulate, int T, int S, int nh, int nkv, int hd, cudaStream_t stream);

// ---- moe/router.cu
// Optional statistics (null = off): cnt_sel / cnt_unb int [B, E] (zeroed by the caller; pass the same pointer
// for both when there is neither bias nor group-limited routing), tokens_acc float [E], rsum / margin float [T].
int b200_router_fwd(const float* logits, const float* bias, float* scores, float* topk_w, int* topk_idx, int T, int E,
                    int K, int mode, int norm, float scale, int num_groups, int group_topk, int* cnt_sel,
                    int* cnt_unb, float* tokens_acc, float* rsum, float* margin, float* part, int S,
                    cudaStream_t stream);
// consecutive tokens one block of b200_router_fwd covers (its `part` output has one [2, E] row per block)
int b200_router_tokens_per_block(int E);
// per-sequence sums of the per-block partials: psum / pn [B, E]
int b200_router_part_reduce(const float* part, int B, int blocks_per_seq, int E, float* psum, float* pn,
                            cudaStream_t stream);
// per-sequence column sums of the scores (psum) and of the row-normalised scores (pn, optional), [B, E]
int b200_router_colsum(const float* scores, const float* rsum, int B, int S, int E, float* psum, float* pn,
                       cudaStream_t stream);
// Switch loss and sequence-level loss from stacked [L, B, E] statistics; g[E] = d(aux)/d(score of expert e)
int b200_moe_aux(const int* cnt_unb, const int* cnt_sel, const float* psum, const float* pn, int L, int B, int E,
                 int K, int S, float* g, float* out, cudaStream_t stream);
// aux_g / seq_cnt (optional) add the balance-loss gradients; d_aux = device pair of upstream gradients
int b200_router_bwd(const float* dscores, const float* dtopk_w, const float* scores, const int* topk_idx,
                    void* dlogits, int T, int E, int K, int mode, int norm, float scale, const float* aux_g,
                    const float* d_aux, const int* seq_cnt, const float* rsum, float seq_scale, int S,
                    cudaStream_t stream);

// ---- moe/dispatch.cu
int b200_moe_plan_blocks(int n);  // plan scratch: int[blocks * E]
// pair_tiles (optional): int2 per pair tile for the pair-tile GEMM kernel, capacity max_pairs;
// row_tok (optional): int[capacity], source token (assignment / K) of every sorted row, 0x7f7f7f7f for padding
int b200_moe_plan(const int* idx, int n, int E, int* scratch, int* counts, int* seg_off, int* tile_expert,
                  int* num_m_tiles, int* pos, int* row_slot, int capacity, int* pair_tiles, int max_pairs,
                  int* num_pair_tiles, int* row_tok, int K, cudaStream_t stream);
// dw[row_slot[r]] = sum_n row_dot[r * n_tiles + n] for the live sorted rows (routing-weight gradient)
int b200_moe_row_dot_reduce(const float* row_dot, const int* row_slot, const int* seg_off, int E, int n_tiles,
                            int capacity, float* dw, cudaStream_t stream);
// dw[t * K + k] = <dout[t], y[t * K + k]> (bf16 rows of H elements)
int b200_moe_slot_dot(const void* dout, const void* y, int T, int K, int H, float* dw, cudaStream_t stream);
int b200_moe_gather(const void* x, const int* row_slot, const int* seg_off, int E, int K, int H, void* xs,
                    int capacity, cudaStream_t stream);
int b200_moe_combine(const void* ys, const int* pos, const float* w, const void* res, int T, int K, int H, void* out,
                     const int* wait_flags, int wait_n, const int* epoch_base, int epoch_off, int* status,
                     cudaStream_t stream);
int b200_moe_combine_bwd(const void* dout, const void* ys, const int* row_slot, const int* seg_off, const float* w,
                         int E, int K, int H, void* dys, float* dw, int capacity, cudaStream_t stream);

// ---- lce/lce.cu
// per row: log-sum-exp and loss (0 where the label is ignored); no atomics
int b200_lse_loss(const float* part, int n_tiles, const void* logits, long long ld, const long long* labels,
                  int ignore_index, int T, int V, float* lse, float* row_loss, cudaStream_t stream);
// fixed-order reductions into acc[3]: row_loss == null -> acc[1] = valid labels; else acc[0] = sum, acc[2] = mean
int b200_lce_reduce(const float* row_loss, const long long* labels, int ignore_index, int T, int V, float* acc,
                    cudaStream_t stream);
int b200_dlogits(void* logits, long long ld, const float* lse, const long long* labels, int ignore_index, int T, int V,
                 const float* loss_acc, float upstream, cudaStream_t stream);
int b200_embed_fwd(const long long* ids, const void* table, int T, int H, int V, void* out, cudaStream_t stream);
int b200_embed_sort_capacity();  // tokens the built-in key sort handles
int b200_embed_sort(const long long* ids, int T, int V, unsigned long long* keys, cudaStream_t stream);
// deterministic: (id, position) keys are sorted (here, or by the caller: presorted) and every id's rows are
// added in position order by one warp; keys = uint64[T] scratch
int b200_embed_bwd(const long long* ids, const void* dout, int T, int H, int V, float* grad,
                   unsigned long long* keys, int presorted, int accumulate, cudaStream_t stream);

// ---- optim/optim.cu
int b200_sumsq_blocks(long long n);  // scratch: float[blocks]
int b200_sumsq(const float* g, long long n, float* scratch, float* out, int accumulate, cudaStream_t stream);
int b200_clip_coef(const float* sumsq, float max_norm, float* coef, cudaStream_t stream);
// hyper: device float[3] = {lr, 1 - beta1^t, 1 - beta2^t}
// p16_peers (optional, `world` entries): the same slice of every rank's bf16 compute copy; when given the
// new weights are also stored there (sharded optimizer: update + parameter all-gather in one pass).
// p16_mc (optional): NVSwitch multicast address of that slice; one `multimem.st` then replaces the peer stores.
int b200_adamw(float* p, const float* g, float* m, float* v, void* p16, long long n, const float* hyper, float beta1,
               float beta2, float eps, float wd, const float* grad_coef, void* const* p16_peers, int world,
               void* p16_mc, cudaStream_t stream);
int b200_cast_bf16(const float* src, void* dst, long long n, cudaStream_t stream);
// out[i] (+)= sum_p part[p * n + i], p in fixed order (split-K partial sums; bitwise reproducible)
int b200_sum_partials(const float* part, float* out, int nparts, int n, int accumulate, cudaStream_t stream);

// ---- comm/allreduce.cu
#define B200_MAX_RANKS 8
typedef struct B200Peers {
  void* buf[B200_MAX_RANKS];    // every rank's flat fp32 gradient buffer (symmetric memory)
  void* flags[B200_MAX_RANKS];  // every rank's int[2 * B200_MAX_RANKS] flag words, zero-initialised
  void* norm[B200_MAX_RANKS];   // every rank's float[B200_MAX_RANKS] squared-norm slots
  void* mc_buf;                 // NVSwitch multicast address of the gradient buffers, or null
} B200Peers;
// One bucket [off, off+n) of the gradient buffer: average over ranks in place on every rank.
// epoch = *epoch_base + epoch_off must grow with every launch and agree across ranks.
// state_i: int[2], state_f: float[2 + 148] (running sum + one partial per block), both zero-initialised
// local scratch.
int b200_allreduce(const B200Peers* p, int rank, int world, long long off, long long n, float scale,
                   const int* epoch_base, int epoch_off, int final_bucket, int publish, int use_multimem, int blocks,
                   int* state_i, float* state_f, int* status, unsigned long long limit_ns, cudaStream_t stream);
// flags must then hold 4 * B200_MAX_RANKS words; channels 0/1 belong to b200_allreduce
int b200_peer_barrier(const B200Peers* p, int rank, int world, int chan, const int* epoch_base, int epoch_off,
                      int* status, unsigned long long limit_ns, cudaStream_t stream);
int b200_clip_coef_multi(const float* parts, int world, float max_norm, float* coef, cudaStream_t stream);
// all-gather of one sharded parameter unit into a local buffer: dst[r * per + i] = shards[r][i], i < per,
// clipped to n elements overall (bf16; per and n multiples of 8)
int b200_allgather_bf16(const void* const* shards, int world, long long per, long long n, void* dst, int blocks,
                        cudaStream_t stream);

// ---- moe/ep.cu (expert parallelism over peer memory; pointer arrays have B200_MAX_RANKS entries)
#define B200_EP_CH_COUNTS 0
#define B200_EP_CH_DISPATCH 1
#define B200_EP_CH_RETURN 2
int b200_ep_exchange(const int* counts, void* const* cmat, void* const* flags, int chan, const int* epoch_base,
                     int epoch_off, int rank, int world, int E, int H, int capacity, int* send_base, int* recv_seg_off,
                     int* recv_tile_expert, int* recv_num_m_tiles, void* recv_buf, int* recv_meta, int* status,
                     unsigned long long limit_ns, int* recv_pair_tiles, int max_pairs,
                     int* recv_num_pair_tiles, cudaStream_t stream);
int b200_ep_dispatch(const void* rows, const float* scale, const int* idx, const int* pos, const int* local_seg_off,
                     const int* send_base, void* const* recv_buf, void* const* recv_meta, void* const* flags, int chan,
                     const int* epoch_base, int epoch_off, int rank, int world, int E, int n, int K, int H,
                     int capacity, int* counter, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
