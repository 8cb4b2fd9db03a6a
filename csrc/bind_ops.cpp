// Bindings of the non-GEMM kernels. Shapes and dtypes are validated here; the launchers only
// see raw pointers.
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include "ops_api.h"
#include "common/tma_host.h"
#include "attn/attn_api.h"

#include <cstring>
#include <vector>

namespace {

using torch::Tensor;
using OptT = c10::optional<Tensor>;

cudaStream_t stream() { return at::cuda::getCurrentCUDAStream().stream(); }

template <typename T>
T* optp(const OptT& t) {
  return t.has_value() && t->defined() ? reinterpret_cast<T*>(t->data_ptr()) : nullptr;
}
void need(bool ok, const char* what) { TORCH_CHECK(ok, "moe_b200: ", what); }
void bf16c(const Tensor& t, const char* n) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kBFloat16 && t.is_contiguous(), n, ": contiguous CUDA bf16 expected");
}
// [B,S,h,hd] bf16 whose heads are contiguous per token while tokens may be further apart (a slice of a wider row);
// returns the token pitch in elements
int64_t bf16_rows4(const Tensor& t, const char* n) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kBFloat16 && t.dim() == 4, n, ": 4-D CUDA bf16 expected");
  TORCH_CHECK(t.stride(3) == 1 && t.stride(2) == t.size(3) && t.stride(1) >= t.size(2) * t.size(3) &&
                  (t.size(0) == 1 || t.stride(0) == t.stride(1) * t.size(1)) && t.stride(1) % 8 == 0 &&
                  reinterpret_cast<uintptr_t>(t.data_ptr()) % 16 == 0,
              n, ": heads must be contiguous per token, tokens evenly spaced, 16-byte aligned");
  return t.stride(1);
}
void f32c(const Tensor& t, const char* n) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kFloat && t.is_contiguous(), n, ": contiguous CUDA fp32 expected");
}
void i32c(const Tensor& t, const char* n) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kInt && t.is_contiguous(), n, ": contiguous CUDA int32 expected");
}
void rc_ok(int rc, const char* fn) {
  TORCH_CHECK(rc == 0, fn, " rejected its arguments (code ", rc, ", last tensor-map encode result ",
              b200::tma_last_encode_result(), ")");
}

// ------------------------------------------------------------------ rmsnorm
void rmsnorm_fwd(const Tensor& x, const OptT& res, const Tensor& w, const OptT& h_out, Tensor& y, const OptT& rstd,
                 double eps) {
  bf16c(x, "x"); f32c(w, "w"); bf16c(y, "y");
  c10::cuda::CUDAGuard g(x.device());
  const int H = (int)x.size(-1);
  const int T = (int)(x.numel() / H);
  need(w.numel() == H, "rmsnorm weight size");
  rc_ok(b200_rmsnorm_fwd(x.data_ptr(), optp<const void>(res), w.data_ptr<float>(), optp<void>(h_out), y.data_ptr(),
                         optp<float>(rstd), T, H, (float)eps, stream()), "rmsnorm_fwd");
}
int64_t rmsnorm_bwd_blocks(int64_t T) { return b200_rmsnorm_bwd_blocks((int)T); }
void rmsnorm_bwd(const Tensor& dy, const Tensor& x, const Tensor& rstd, const Tensor& w, const OptT& dres, Tensor& dx,
                 Tensor& dw_part, Tensor& dw_out, bool accumulate) {
  bf16c(dy, "dy"); bf16c(x, "x"); f32c(rstd, "rstd"); f32c(w, "w"); bf16c(dx, "dx"); f32c(dw_part, "dw_part");
  f32c(dw_out, "dw_out");
  c10::cuda::CUDAGuard g(x.device());
  const int H = (int)x.size(-1);
  const int T = (int)(x.numel() / H);
  need(dw_part.numel() >= (int64_t)b200_rmsnorm_bwd_blocks(T) * H, "rmsnorm dw scratch too small");
  rc_ok(b200_rmsnorm_bwd(dy.data_ptr(), x.data_ptr(), rstd.data_ptr<float>(), w.data_ptr<float>(),
                         optp<const void>(dres), dx.data_ptr(), dw_part.data_ptr<float>(), dw_out.data_ptr<float>(),
                         accumulate ? 1 : 0, T, H, stream()), "rmsnorm_bwd");
}

// ------------------------------------------------------------- qknorm + rope
int64_t qknorm_rope_blocks(int64_t items) { return b200_qknorm_rope_blocks(items); }
void qknorm_rope_fwd(const Tensor& qkv, const Tensor& qw, const Tensor& kw, const Tensor& cs, Tensor& q, Tensor& k,
                     Tensor& v, Tensor& rstd, int64_t S, int64_t nh, int64_t nkv, int64_t hd, double eps) {
  bf16c(qkv, "qkv"); f32c(qw, "qw"); f32c(kw, "kw"); f32c(cs, "cs"); bf16c(q, "q"); bf16c(k, "k"); bf16c(v, "v"); f32c(rstd, "rstd");
  c10::cuda::CUDAGuard g(qkv.device());
  const int ld = (int)qkv.size(-1);
  const int T = (int)(qkv.numel() / ld);
  need(ld == (nh + 2 * nkv) * hd, "qkv width");
  need(cs.numel() >= S * hd, "rope table too small");
  rc_ok(b200_qknorm_rope_fwd(qkv.data_ptr(), ld, qw.data_ptr<float>(), kw.data_ptr<float>(), cs.data_ptr<float>(),
                             q.data_ptr(), k.data_ptr(), v.data_ptr(), rstd.data_ptr<float>(), T, (int)S, (int)nh, (int)nkv,
                             (int)hd, (float)eps, stream()), "qknorm_rope_fwd");
}
void qknorm_rope_bwd(const Tensor& dq, const Tensor& dk, const Tensor& dv, const Tensor& qkv, const Tensor& rstd,
                     const Tensor& qw, const Tensor& kw, const Tensor& cs, Tensor& dqkv, Tensor& dw_part, Tensor& dqw,
                     Tensor& dkw, bool accumulate, int64_t S, int64_t nh, int64_t nkv, int64_t hd) {
  bf16c(dq, "dq"); bf16c(dk, "dk"); bf16c(dv, "dv"); bf16c(qkv, "qkv"); bf16c(dqkv, "dqkv");
  f32c(dw_part, "dw_part"); f32c(dqw, "dqw"); f32c(dkw, "dkw");
  c10::cuda::CUDAGuard g(qkv.device());
  const int ld = (int)qkv.size(-1);
  const int T = (int)(qkv.numel() / ld);
  need(dw_part.numel() >= b200_qknorm_rope_blocks((int64_t)T) * 2 * hd, "qk dw scratch too small");
  rc_ok(b200_qknorm_rope_bwd(dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), qkv.data_ptr(), ld, rstd.data_ptr<float>(),
                             qw.data_ptr<float>(), kw.data_ptr<float>(), cs.data_ptr<float>(), dqkv.data_ptr(),
                             dw_part.data_ptr<float>(), dqw.data_ptr<float>(), dkw.data_ptr<float>(),
                             accumulate ? 1 : 0, T, (int)S, (int)nh, (int)nkv, (int)hd, stream()), "qknorm_rope_bwd");
}

// ---------------------------------------------------------------- attention
void flash_fwd(const Tensor& q, const Tensor& k, const Tensor& v, Tensor& o, Tensor& lse, double scale, Tensor& status) {
  const int64_t ldq = bf16_rows4(q, "q"), ldk = bf16_rows4(k, "k"), ldv = bf16_rows4(v, "v");
  bf16c(o, "o"); f32c(lse, "lse"); i32c(status, "status");
  need(q.dim() == 4 && k.dim() == 4 && (q.size(3) == 128 || q.size(3) == 64) && k.size(3) == q.size(3),
       "flash attention: [B,S,h,128] or [B,S,h,64] expected");
  need(k.sizes() == v.sizes() && o.sizes() == q.sizes(), "flash attention: shape mismatch");
  const int B = (int)q.size(0), S = (int)q.size(1), nh = (int)q.size(2), nkv = (int)k.size(2);
  need(k.size(0) == B && k.size(1) == S, "flash attention: k/v batch or length");
  need(lse.numel() == (int64_t)B * nh * S, "flash attention: lse size");
  c10::cuda::CUDAGuard g(q.device());
  rc_ok(b200_flash_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr<float>(), B, S, nh, nkv,
                       (int)q.size(3), ldq, ldk, ldv, (float)scale, status.data_ptr<int>(), stream()), "flash_fwd");
}

void flash_bwd(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& o, const Tensor& d_o, const Tensor& lse,
               Tensor& delta, Tensor& dq, Tensor& dk, Tensor& dv, double scale, Tensor& status) {
  const int64_t ldq = bf16_rows4(q, "q"), ldk = bf16_rows4(k, "k"), ldv = bf16_rows4(v, "v");
  bf16c(o, "o"); bf16c(d_o, "d_o"); f32c(lse, "lse"); f32c(delta, "delta");
  bf16c(dq, "dq"); bf16c(dk, "dk"); bf16c(dv, "dv"); i32c(status, "status");
  need(q.dim() == 4 && k.dim() == 4 && (q.size(3) == 128 || q.size(3) == 64) && k.size(3) == q.size(3),
       "flash attention: [B,S,h,128] or [B,S,h,64] expected");
  need(k.sizes() == v.sizes() && o.sizes() == q.sizes() && d_o.sizes() == q.sizes() && dq.sizes() == q.sizes() &&
           dk.sizes() == k.sizes() && dv.sizes() == k.sizes(), "flash attention backward: shape mismatch");
  const int B = (int)q.size(0), S = (int)q.size(1), nh = (int)q.size(2), nkv = (int)k.size(2);
  need(lse.numel() == (int64_t)B * nh * S && delta.numel() == lse.numel(), "flash attention backward: statistics size");
  c10::cuda::CUDAGuard g(q.device());
  rc_ok(b200_flash_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), d_o.data_ptr(), lse.data_ptr<float>(),
                       delta.data_ptr<float>(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), B, S, nh, nkv, (int)q.size(3),
                       ldq, ldk, ldv, (float)scale, status.data_ptr<int>(), stream()), "flash_bwd");
}

// ------------------------------------------------------------------- router
void router_fwd(const Tensor& logits, const OptT& bias, Tensor& scores, Tensor& topk_w, Tensor& topk_idx, int64_t K,
                int64_t mode, bool norm, double scale, int64_t num_groups, int64_t group_topk, const OptT& cnt_sel,
                const OptT& cnt_unb, const OptT& tokens_acc, const OptT& rsum, const OptT& margin, const OptT& part,
                int64_t S) {
  f32c(logits, "logits"); f32c(scores, "scores"); f32c(topk_w, "topk_w"); i32c(topk_idx, "topk_idx");
  c10::cuda::CUDAGuard g(logits.device());
  const int T = (int)logits.size(0), E = (int)logits.size(1);
  const bool stats = cnt_sel.has_value() && cnt_sel->defined();
  if (stats) {
    i32c(*cnt_sel, "cnt_sel");
    need(S > 0 && T % S == 0 && cnt_sel->numel() == (int64_t)(T / S) * E, "cnt_sel must be int32 [T / S, E]");
    if (cnt_unb.has_value() && cnt_unb->defined()) {
      i32c(*cnt_unb, "cnt_unb");
      need(cnt_unb->numel() == cnt_sel->numel(), "cnt_unb size");
    }
  }
  if (tokens_acc.has_value() && tokens_acc->defined()) { f32c(*tokens_acc, "tokens_acc"); need(tokens_acc->numel() == E, "tokens_acc size"); }
  if (rsum.has_value() && rsum->defined()) { f32c(*rsum, "rsum"); need(rsum->numel() >= T, "rsum size"); }
  if (margin.has_value() && margin->defined()) { f32c(*margin, "margin"); need(margin->numel() >= T, "margin size"); }
  if (part.has_value() && part->defined()) {
    f32c(*part, "part");
    const int bt = b200_router_tokens_per_block(E);
    need(part->numel() >= (int64_t)((T + bt - 1) / bt) * 2 * E, "part must hold [blocks, 2, E] floats");
  }
  rc_ok(b200_router_fwd(logits.data_ptr<float>(), optp<const float>(bias), scores.data_ptr<float>(),
                        topk_w.data_ptr<float>(), topk_idx.data_ptr<int>(), T, E, (int)K, (int)mode, norm ? 1 : 0,
                        (float)scale, (int)num_groups, (int)group_topk, optp<int>(cnt_sel), optp<int>(cnt_unb),
                        optp<float>(tokens_acc), optp<float>(rsum), optp<float>(margin), optp<float>(part), (int)S,
                        stream()),
        "router_fwd");
}
void router_colsum(const Tensor& scores, const OptT& rsum, int64_t S, Tensor& psum, const OptT& pn) {
  f32c(scores, "scores"); f32c(psum, "psum");
  c10::cuda::CUDAGuard g(scores.device());
  const int T = (int)scores.size(0), E = (int)scores.size(1);
  need(S > 0 && T % S == 0, "router_colsum: T must be a multiple of S");
  const int B = T / (int)S;
  need(psum.numel() == (int64_t)B * E, "psum must be [T / S, E]");
  if (pn.has_value() && pn->defined()) { f32c(*pn, "pn"); need(pn->numel() == psum.numel(), "pn size"); }
  rc_ok(b200_router_colsum(scores.data_ptr<float>(), optp<const float>(rsum), B, (int)S, E, psum.data_ptr<float>(),
                           optp<float>(pn), stream()), "router_colsum");
}
int64_t router_tokens_per_block(int64_t E) { return b200_router_tokens_per_block((int)E); }
void router_part_reduce(const Tensor& part, int64_t blocks_per_seq, Tensor& psum, Tensor& pn) {
  f32c(part, "part"); f32c(psum, "psum"); f32c(pn, "pn");
  need(psum.dim() == 2 && pn.sizes() == psum.sizes(), "psum / pn must be [B, E]");
  const int B = (int)psum.size(0), E = (int)psum.size(1);
  need(part.numel() >= (int64_t)B * blocks_per_seq * 2 * E, "part too small");
  c10::cuda::CUDAGuard g(part.device());
  rc_ok(b200_router_part_reduce(part.data_ptr<float>(), B, (int)blocks_per_seq, E, psum.data_ptr<float>(),
                                pn.data_ptr<float>(), stream()), "router_part_reduce");
}
void moe_aux(const Tensor& cnt_unb, const OptT& cnt_sel, const Tensor& psum, const OptT& pn, int64_t K, int64_t S,
             const OptT& gvec, Tensor& out) {
  i32c(cnt_unb, "cnt_unb"); f32c(psum, "psum"); f32c(out, "out");
  need(cnt_unb.dim() == 3 && psum.sizes() == cnt_unb.sizes() && out.numel() >= 2, "moe_aux: [L, B, E] statistics");
  c10::cuda::CUDAGuard g(psum.device());
  const int L = (int)cnt_unb.size(0), B = (int)cnt_unb.size(1), E = (int)cnt_unb.size(2);
  if (cnt_sel.has_value() && cnt_sel->defined()) { i32c(*cnt_sel, "cnt_sel"); need(cnt_sel->sizes() == cnt_unb.sizes(), "cnt_sel shape"); }
  if (pn.has_value() && pn->defined()) { f32c(*pn, "pn"); need(pn->sizes() == cnt_unb.sizes(), "pn shape"); }
  if (gvec.has_value() && gvec->defined()) { f32c(*gvec, "g"); need(gvec->numel() == E, "g size"); }
  rc_ok(b200_moe_aux(cnt_unb.data_ptr<int>(), optp<const int>(cnt_sel), psum.data_ptr<float>(), optp<const float>(pn),
                     L, B, E, (int)K, (int)S, optp<float>(gvec), out.data_ptr<float>(), stream()), "moe_aux");
}
void router_bwd(const OptT& dscores, const Tensor& dtopk_w, const Tensor& scores, const Tensor& topk_idx,
                Tensor& dlogits, int64_t K, int64_t mode, bool norm, double scale, const OptT& aux_g,
                const OptT& d_aux, const OptT& seq_cnt, const OptT& rsum, double seq_scale, int64_t S) {
  f32c(dtopk_w, "dtopk_w"); f32c(scores, "scores"); i32c(topk_idx, "topk_idx"); bf16c(dlogits, "dlogits");
  c10::cuda::CUDAGuard g(scores.device());
  const int T = (int)scores.size(0), E = (int)scores.size(1);
  if (dscores.has_value() && dscores->defined()) { f32c(*dscores, "dscores"); need(dscores->numel() == scores.numel(), "dscores size"); }
  if (aux_g.has_value() && aux_g->defined()) { f32c(*aux_g, "aux_g"); need(aux_g->numel() == E, "aux_g size"); }
  if (d_aux.has_value() && d_aux->defined()) { f32c(*d_aux, "d_aux"); need(d_aux->numel() >= 2, "d_aux holds two floats"); }
  if (seq_cnt.has_value() && seq_cnt->defined()) {
    i32c(*seq_cnt, "seq_cnt");
    need(S > 0 && T % S == 0 && seq_cnt->numel() == (int64_t)(T / S) * E, "seq_cnt must be int32 [T / S, E]");
  }
  if (rsum.has_value() && rsum->defined()) { f32c(*rsum, "rsum"); need(rsum->numel() >= T, "rsum size"); }
  rc_ok(b200_router_bwd(optp<const float>(dscores), dtopk_w.data_ptr<float>(), scores.data_ptr<float>(),
                        topk_idx.data_ptr<int>(), dlogits.data_ptr(), T, E, (int)K, (int)mode, norm ? 1 : 0,
                        (float)scale, optp<const float>(aux_g), optp<const float>(d_aux), optp<const int>(seq_cnt),
                        optp<const float>(rsum), (float)seq_scale, (int)S, stream()), "router_bwd");
}

// ----------------------------------------------------------------- dispatch
int64_t moe_plan_blocks(int64_t n) { return b200_moe_plan_blocks((int)n); }
void moe_plan(const Tensor& idx, int64_t E, Tensor& scratch, Tensor& counts, Tensor& seg_off, Tensor& tile_expert,
              Tensor& num_m_tiles, Tensor& pos, Tensor& row_slot, const OptT& pair_tiles,
              const OptT& num_pair_tiles, const OptT& row_tok, int64_t K) {
  i32c(idx, "idx"); i32c(scratch, "scratch"); i32c(counts, "counts"); i32c(seg_off, "seg_off");
  i32c(tile_expert, "tile_expert"); i32c(num_m_tiles, "num_m_tiles"); i32c(pos, "pos"); i32c(row_slot, "row_slot");
  c10::cuda::CUDAGuard g(idx.device());
  const int n = (int)idx.numel();
  const int cap = (int)row_slot.numel();
  need(scratch.numel() >= (int64_t)b200_moe_plan_blocks(n) * E, "plan scratch too small");
  need(seg_off.numel() >= E + 1 && counts.numel() >= E && tile_expert.numel() >= cap / 128 && pos.numel() >= n,
       "plan output sizes");
  rc_ok(b200_moe_plan(idx.data_ptr<int>(), n, (int)E, scratch.data_ptr<int>(), counts.data_ptr<int>(),
                      seg_off.data_ptr<int>(), tile_expert.data_ptr<int>(), num_m_tiles.data_ptr<int>(),
                      pos.data_ptr<int>(), row_slot.data_ptr<int>(), cap, optp<int>(pair_tiles),
                      pair_tiles.has_value() && pair_tiles->defined() ? (int)(pair_tiles->numel() / 2) : 0,
                      optp<int>(num_pair_tiles), optp<int>(row_tok), (int)K, stream()), "moe_plan");
}
void moe_row_dot_reduce(const Tensor& row_dot, const Tensor& row_slot, const Tensor& seg_off, int64_t E, Tensor& dw) {
  f32c(row_dot, "row_dot"); i32c(row_slot, "row_slot"); i32c(seg_off, "seg_off"); f32c(dw, "dw");
  const int cap = (int)row_slot.numel();
  need(row_dot.numel() % cap == 0 && row_dot.numel() >= cap, "row_dot must be [capacity, n_tiles]");
  c10::cuda::CUDAGuard g(row_dot.device());
  rc_ok(b200_moe_row_dot_reduce(row_dot.data_ptr<float>(), row_slot.data_ptr<int>(), seg_off.data_ptr<int>(), (int)E,
                                (int)(row_dot.numel() / cap), cap, dw.data_ptr<float>(), stream()),
        "moe_row_dot_reduce");
}
void moe_slot_dot(const Tensor& dout, const Tensor& y, int64_t K, Tensor& dw) {
  bf16c(dout, "dout"); bf16c(y, "y"); f32c(dw, "dw");
  const int T = (int)dout.size(0), H = (int)dout.size(1);
  need(y.numel() == (int64_t)T * K * H && dw.numel() == (int64_t)T * K, "moe_slot_dot: shapes");
  c10::cuda::CUDAGuard g(dout.device());
  rc_ok(b200_moe_slot_dot(dout.data_ptr(), y.data_ptr(), T, (int)K, H, dw.data_ptr<float>(), stream()), "moe_slot_dot");
}
void moe_gather(const Tensor& x, const Tensor& row_slot, const Tensor& seg_off, int64_t E, int64_t K, Tensor& xs) {
  bf16c(x, "x"); bf16c(xs, "xs"); i32c(row_slot, "row_slot"); i32c(seg_off, "seg_off");
  c10::cuda::CUDAGuard g(x.device());
  rc_ok(b200_moe_gather(x.data_ptr(), row_slot.data_ptr<int>(), seg_off.data_ptr<int>(), (int)E, (int)K,
                        (int)x.size(1), xs.data_ptr(), (int)xs.size(0), stream()), "moe_gather");
}
void moe_combine(const Tensor& ys, const OptT& pos, const OptT& w, const OptT& res, Tensor& out, int64_t K,
                 const OptT& wait_flags, int64_t wait_n, const OptT& epoch_base, int64_t epoch_off,
                 const OptT& status) {
  bf16c(ys, "ys"); bf16c(out, "out");
  c10::cuda::CUDAGuard g(ys.device());
  rc_ok(b200_moe_combine(ys.data_ptr(), optp<const int>(pos), optp<const float>(w), optp<const void>(res),
                         (int)out.size(0), (int)K, (int)out.size(1), out.data_ptr(), optp<const int>(wait_flags),
                         (int)wait_n, optp<const int>(epoch_base), (int)epoch_off, optp<int>(status), stream()),
        "moe_combine");
}

std::vector<void*> ptrs8(const std::vector<int64_t>& v) {
  std::vector<void*> p(B200_MAX_RANKS, nullptr);
  for (size_t i = 0; i < v.size() && i < B200_MAX_RANKS; ++i) p[i] = reinterpret_cast<void*>(v[i]);
  return p;
}

void ep_exchange(const Tensor& counts, const std::vector<int64_t>& cmat, const std::vector<int64_t>& flags,
                 const Tensor& epoch_base, int64_t epoch_off, int64_t rank, int64_t world, int64_t E, int64_t H,
                 Tensor& send_base, Tensor& recv_seg_off, Tensor& recv_tile_expert, Tensor& recv_num_m_tiles,
                 Tensor& recv_buf, Tensor& recv_meta, Tensor& status, const OptT& recv_pair_tiles,
                 const OptT& recv_num_pair_tiles) {
  i32c(counts, "counts"); i32c(send_base, "send_base"); i32c(recv_seg_off, "recv_seg_off");
  i32c(recv_tile_expert, "recv_tile_expert"); i32c(recv_num_m_tiles, "recv_num_m_tiles"); bf16c(recv_buf, "recv_buf");
  i32c(recv_meta, "recv_meta"); i32c(epoch_base, "epoch_base");
  c10::cuda::CUDAGuard g(counts.device());
  auto cm = ptrs8(cmat), fl = ptrs8(flags);
  rc_ok(b200_ep_exchange(counts.data_ptr<int>(), cm.data(), fl.data(), B200_EP_CH_COUNTS, epoch_base.data_ptr<int>(),
                         (int)epoch_off, (int)rank, (int)world, (int)E, (int)H, (int)recv_buf.size(0),
                         send_base.data_ptr<int>(), recv_seg_off.data_ptr<int>(), recv_tile_expert.data_ptr<int>(),
                         recv_num_m_tiles.data_ptr<int>(), recv_buf.data_ptr(), recv_meta.data_ptr<int>(),
                         status.data_ptr<int>(), 0, optp<int>(recv_pair_tiles),
                         recv_pair_tiles.has_value() && recv_pair_tiles->defined() ? (int)(recv_pair_tiles->numel() / 2) : 0,
                         optp<int>(recv_num_pair_tiles), stream()), "ep_exchange");
}

void ep_dispatch(const Tensor& rows, const OptT& scale, const Tensor& idx, const Tensor& pos,
                 const Tensor& local_seg_off, const Tensor& send_base, const std::vector<int64_t>& recv_buf,
                 const std::vector<int64_t>& recv_meta, const std::vector<int64_t>& flags, const Tensor& epoch_base,
                 int64_t epoch_off, int64_t rank, int64_t world, int64_t E, int64_t K, int64_t capacity,
                 Tensor& counter) {
  bf16c(rows, "rows"); i32c(idx, "idx"); i32c(pos, "pos"); i32c(local_seg_off, "local_seg_off");
  i32c(send_base, "send_base"); i32c(epoch_base, "epoch_base"); i32c(counter, "counter");
  c10::cuda::CUDAGuard g(rows.device());
  auto rb = ptrs8(recv_buf), rm = ptrs8(recv_meta), fl = ptrs8(flags);
  rc_ok(b200_ep_dispatch(rows.data_ptr(), optp<const float>(scale), idx.data_ptr<int>(), pos.data_ptr<int>(),
                         local_seg_off.data_ptr<int>(), send_base.data_ptr<int>(), rb.data(), rm.data(), fl.data(),
                         B200_EP_CH_DISPATCH, epoch_base.data_ptr<int>(), (int)epoch_off, (int)rank, (int)world, (int)E,
                         (int)idx.numel(), (int)K, (int)rows.size(1), (int)capacity, counter.data_ptr<int>(), stream()),
        "ep_dispatch");
}
void moe_combine_bwd(const Tensor& dout, const Tensor& ys, const Tensor& row_slot, const Tensor& seg_off,
                     const Tensor& w, int64_t E, int64_t K, Tensor& dys, Tensor& dw) {
  bf16c(dout, "dout"); bf16c(ys, "ys"); bf16c(dys, "dys"); f32c(w, "w"); f32c(dw, "dw");
  c10::cuda::CUDAGuard g(ys.device());
  rc_ok(b200_moe_combine_bwd(dout.data_ptr(), ys.data_ptr(), row_slot.data_ptr<int>(), seg_off.data_ptr<int>(),
                             w.data_ptr<float>(), (int)E, (int)K, (int)dout.size(1), dys.data_ptr(),
                             dw.data_ptr<float>(), (int)dys.size(0), stream()), "moe_combine_bwd");
}

// ---------------------------------------------------------------------- lce
void lce_reduce(const OptT& row_loss, const Tensor& labels, int64_t ignore_index, int64_t V, Tensor& acc) {
  f32c(acc, "acc");
  need(acc.numel() >= 3, "acc must hold 3 floats");
  need(labels.is_cuda() && labels.scalar_type() == at::kLong && labels.is_contiguous(), "labels must be int64");
  c10::cuda::CUDAGuard g(labels.device());
  const int T = (int)labels.numel();
  if (row_loss.has_value() && row_loss->defined()) {
    f32c(*row_loss, "row_loss");
    need(row_loss->numel() >= T, "row_loss size");
  }
  rc_ok(b200_lce_reduce(optp<const float>(row_loss), reinterpret_cast<const long long*>(labels.data_ptr<int64_t>()),
                        (int)ignore_index, T, (int)V, acc.data_ptr<float>(), stream()), "lce_reduce");
}
void lse_loss(const Tensor& part, const Tensor& logits, const Tensor& labels, int64_t ignore_index, Tensor& lse,
              Tensor& loss_acc) {
  f32c(part, "part"); f32c(lse, "lse"); f32c(loss_acc, "row_loss");
  need(lse.numel() >= logits.size(0) && loss_acc.numel() >= logits.size(0), "lse / row_loss size");
  need(labels.is_cuda() && labels.scalar_type() == at::kLong && labels.is_contiguous(), "labels must be int64");
  c10::cuda::CUDAGuard g(logits.device());
  const int T = (int)logits.size(0), V = (int)logits.size(1);
  rc_ok(b200_lse_loss(part.data_ptr<float>(), (int)part.size(1), logits.data_ptr(), logits.stride(0),
                      reinterpret_cast<const long long*>(labels.data_ptr<int64_t>()), (int)ignore_index, T, V,
                      lse.data_ptr<float>(), loss_acc.data_ptr<float>(), stream()), "lse_loss");
}
void dlogits_(Tensor& logits, const Tensor& lse, const Tensor& labels, int64_t ignore_index, const Tensor& loss_acc,
              double upstream) {
  c10::cuda::CUDAGuard g(logits.device());
  const int T = (int)logits.size(0), V = (int)logits.size(1);
  rc_ok(b200_dlogits(logits.data_ptr(), logits.stride(0), lse.data_ptr<float>(),
                     reinterpret_cast<const long long*>(labels.data_ptr<int64_t>()), (int)ignore_index, T, V,
                     loss_acc.data_ptr<float>(), (float)upstream, stream()), "dlogits");
}
void embed_fwd(const Tensor& ids, const Tensor& table, Tensor& out) {
  bf16c(table, "table"); bf16c(out, "out");
  need(ids.is_cuda() && ids.scalar_type() == at::kLong && ids.is_contiguous(), "ids must be int64");
  c10::cuda::CUDAGuard g(table.device());
  rc_ok(b200_embed_fwd(reinterpret_cast<const long long*>(ids.data_ptr<int64_t>()), table.data_ptr(),
                       (int)ids.numel(), (int)table.size(1), (int)table.size(0), out.data_ptr(), stream()),
        "embed_fwd");
}
int64_t embed_sort_capacity() { return b200_embed_sort_capacity(); }
void embed_sort(const Tensor& ids, int64_t V, Tensor& keys) {
  need(ids.is_cuda() && ids.scalar_type() == at::kLong && ids.is_contiguous(), "ids must be int64");
  need(keys.is_cuda() && keys.scalar_type() == at::kLong && keys.is_contiguous() && keys.numel() >= ids.numel(),
       "keys must be an int64 scratch of at least ids.numel() elements");
  c10::cuda::CUDAGuard g(ids.device());
  rc_ok(b200_embed_sort(reinterpret_cast<const long long*>(ids.data_ptr<int64_t>()), (int)ids.numel(), (int)V,
                        reinterpret_cast<unsigned long long*>(keys.data_ptr<int64_t>()), stream()), "embed_sort");
}
void embed_bwd(const Tensor& ids, const Tensor& dout, Tensor& grad, Tensor& keys, bool presorted, bool accumulate) {
  bf16c(dout, "dout"); f32c(grad, "grad");
  need(ids.is_cuda() && ids.scalar_type() == at::kLong && ids.is_contiguous(), "ids must be int64");
  need(keys.is_cuda() && keys.scalar_type() == at::kLong && keys.is_contiguous() && keys.numel() >= ids.numel(),
       "keys must be an int64 scratch of at least ids.numel() elements");
  c10::cuda::CUDAGuard g(dout.device());
  rc_ok(b200_embed_bwd(reinterpret_cast<const long long*>(ids.data_ptr<int64_t>()), dout.data_ptr(),
                       (int)ids.numel(), (int)dout.size(-1), (int)grad.size(0), grad.data_ptr<float>(),
                       reinterpret_cast<unsigned long long*>(keys.data_ptr<int64_t>()), presorted ? 1 : 0,
                       accumulate ? 1 : 0, stream()), "embed_bwd");
}

// -------------------------------------------------------------------- optim
int64_t sumsq_blocks(int64_t n) { return b200_sumsq_blocks(n); }
void sumsq(const Tensor& g, Tensor& scratch, Tensor& out, bool accumulate) {
  f32c(g, "g"); f32c(scratch, "scratch"); f32c(out, "out");
  c10::cuda::CUDAGuard gd(g.device());
  need(scratch.numel() >= b200_sumsq_blocks(g.numel()), "sumsq scratch too small");
  rc_ok(b200_sumsq(g.data_ptr<float>(), g.numel(), scratch.data_ptr<float>(), out.data_ptr<float>(),
                   accumulate ? 1 : 0, stream()), "sumsq");
}
void clip_coef(const Tensor& ss, double max_norm, Tensor& coef) {
  f32c(ss, "sumsq"); f32c(coef, "coef");
  c10::cuda::CUDAGuard gd(ss.device());
  rc_ok(b200_clip_coef(ss.data_ptr<float>(), (float)max_norm, coef.data_ptr<float>(), stream()), "clip_coef");
}
void adamw(Tensor& p, const Tensor& g, Tensor& m, Tensor& v, const OptT& p16, const Tensor& hyper, double beta1,
           double beta2, double eps, double wd, const OptT& grad_coef, const std::vector<int64_t>& p16_peers,
           int64_t p16_mc) {
  f32c(p, "p"); f32c(g, "g"); f32c(m, "m"); f32c(v, "v"); f32c(hyper, "hyper");
  need(hyper.numel() >= 3, "hyper must hold {lr, bc1, bc2}");
  std::vector<void*> peers;
  for (auto a : p16_peers) peers.push_back(reinterpret_cast<void*>(a));
  c10::cuda::CUDAGuard gd(p.device());
  need(g.numel() == p.numel() && m.numel() == p.numel() && v.numel() == p.numel(), "adamw sizes");
  rc_ok(b200_adamw(p.data_ptr<float>(), g.data_ptr<float>(), m.data_ptr<float>(), v.data_ptr<float>(),
                   optp<void>(p16), p.numel(), hyper.data_ptr<float>(), (float)beta1, (float)beta2, (float)eps,
                   (float)wd, optp<const float>(grad_coef), p16_peers.empty() ? nullptr : peers.data(),
                   (int)p16_peers.size(), reinterpret_cast<void*>(p16_mc), stream()), "adamw");
}
void sum_partials(const Tensor& part, Tensor& out, bool accumulate) {
  f32c(part, "part"); f32c(out, "out");
  need(out.numel() > 0 && part.numel() % out.numel() == 0 && out.numel() < (1ll << 31), "sum_partials sizes");
  c10::cuda::CUDAGuard gd(part.device());
  rc_ok(b200_sum_partials(part.data_ptr<float>(), out.data_ptr<float>(), (int)(part.numel() / out.numel()),
                          (int)out.numel(), accumulate ? 1 : 0, stream()), "sum_partials");
}
void cast_bf16(const Tensor& src, Tensor& dst) {
  f32c(src, "src"); bf16c(dst, "dst");
  c10::cuda::CUDAGuard gd(src.device());
  rc_ok(b200_cast_bf16(src.data_ptr<float>(), dst.data_ptr(), src.numel(), stream()), "cast_bf16");
}

// --------------------------------------------------------------------- comm
void allreduce(const std::vector<int64_t>& bufs, const std::vector<int64_t>& flags, const std::vector<int64_t>& norms,
               int64_t mc_buf, int64_t rank, int64_t world, int64_t off, int64_t n, double scale,
               const Tensor& epoch_base, int64_t epoch_off, bool final_bucket, bool publish, bool use_multimem,
               int64_t blocks, Tensor& state_i, Tensor& state_f, Tensor& status, int64_t limit_ns) {
  i32c(epoch_base, "epoch_base"); i32c(state_i, "state_i"); f32c(state_f, "state_f"); i32c(status, "status");
  need(state_f.numel() >= 2 + 148, "allreduce: state_f holds 2 + 148 floats");
  need((int64_t)bufs.size() >= world && (int64_t)flags.size() >= world && (int64_t)norms.size() >= world,
       "peer pointer lists shorter than world");
  c10::cuda::CUDAGuard g(status.device());
  B200Peers p;
  for (int r = 0; r < B200_MAX_RANKS; ++r) {
    p.buf[r] = r < world ? reinterpret_cast<void*>(bufs[r]) : nullptr;
    p.flags[r] = r < world ? reinterpret_cast<void*>(flags[r]) : nullptr;
    p.norm[r] = r < world ? reinterpret_cast<void*>(norms[r]) : nullptr;
  }
  p.mc_buf = reinterpret_cast<void*>(mc_buf);
  rc_ok(b200_allreduce(&p, (int)rank, (int)world, off, n, (float)scale, epoch_base.data_ptr<int>(), (int)epoch_off,
                       final_bucket ? 1 : 0, publish ? 1 : 0, use_multimem ? 1 : 0, (int)blocks, state_i.data_ptr<int>(),
                       state_f.data_ptr<float>(), status.data_ptr<int>(), (unsigned long long)limit_ns, stream()),
        "allreduce");
}
void peer_barrier(const std::vector<int64_t>& flags, int64_t rank, int64_t world, int64_t chan,
                  const Tensor& epoch_base, int64_t epoch_off, Tensor& status) {
  i32c(epoch_base, "epoch_base"); i32c(status, "status");
  c10::cuda::CUDAGuard g(status.device());
  B200Peers p;
  std::memset(&p, 0, sizeof(p));
  for (int r = 0; r < B200_MAX_RANKS && r < (int)flags.size(); ++r) p.flags[r] = reinterpret_cast<void*>(flags[r]);
  rc_ok(b200_peer_barrier(&p, (int)rank, (int)world, (int)chan, epoch_base.data_ptr<int>(), (int)epoch_off,
                          status.data_ptr<int>(), 0, stream()), "peer_barrier");
}
void allgather_bf16(const std::vector<int64_t>& shards, int64_t per, int64_t n, Tensor& dst, int64_t blocks) {
  bf16c(dst, "dst");
  need(dst.numel() >= n, "allgather_bf16: destination too small");
  need(!shards.empty() && (int)shards.size() <= B200_MAX_RANKS, "allgather_bf16: 1..8 ranks");
  c10::cuda::CUDAGuard g(dst.device());
  const void* ptrs[B200_MAX_RANKS] = {nullptr};
  for (size_t r = 0; r < shards.size(); ++r) ptrs[r] = reinterpret_cast<const void*>(shards[r]);
  rc_ok(b200_allgather_bf16(ptrs, (int)shards.size(), per, n, dst.data_ptr(), (int)blocks, stream()), "allgather_bf16");
}
void clip_coef_multi(const Tensor& parts, int64_t world, double max_norm, Tensor& coef) {
  f32c(parts, "parts"); f32c(coef, "coef");
  c10::cuda::CUDAGuard g(parts.device());
  rc_ok(b200_clip_coef_multi(parts.data_ptr<float>(), (int)world, (float)max_norm, coef.data_ptr<float>(), stream()),
        "clip_coef_multi");
}

}  // namespace

void bind_ops(pybind11::module_& m) {
  m.def("allreduce", &allreduce);
  m.def("peer_barrier", &peer_barrier);
  m.def("allgather_bf16", &allgather_bf16);
  m.def("ep_exchange", &ep_exchange, pybind11::arg("counts"), pybind11::arg("cmat"), pybind11::arg("flags"),
        pybind11::arg("epoch_base"), pybind11::arg("epoch_off"), pybind11::arg("rank"), pybind11::arg("world"),
        pybind11::arg("E"), pybind11::arg("H"), pybind11::arg("send_base"), pybind11::arg("recv_seg_off"),
        pybind11::arg("recv_tile_expert"), pybind11::arg("recv_num_m_tiles"), pybind11::arg("recv_buf"),
        pybind11::arg("recv_meta"), pybind11::arg("status"), pybind11::arg("recv_pair_tiles") = pybind11::none(),
        pybind11::arg("recv_num_pair_tiles") = pybind11::none());
  m.def("ep_dispatch", &ep_dispatch);
  m.def("clip_coef_multi", &clip_coef_multi);
  m.def("rmsnorm_fwd", &rmsnorm_fwd);
  m.def("rmsnorm_bwd_blocks", &rmsnorm_bwd_blocks);
  m.def("rmsnorm_bwd", &rmsnorm_bwd);
  m.def("qknorm_rope_blocks", &qknorm_rope_blocks);
  m.def("qknorm_rope_fwd", &qknorm_rope_fwd);
  m.def("qknorm_rope_bwd", &qknorm_rope_bwd);
  m.def("flash_fwd", &flash_fwd);
  m.def("flash_bwd", &flash_bwd);
  {
    namespace py = pybind11;
    m.def("router_fwd", &router_fwd, py::arg("logits"), py::arg("bias"), py::arg("scores"), py::arg("topk_w"),
          py::arg("topk_idx"), py::arg("K"), py::arg("mode"), py::arg("norm"), py::arg("scale"),
          py::arg("num_groups"), py::arg("group_topk"), py::arg("cnt_sel") = py::none(),
          py::arg("cnt_unb") = py::none(), py::arg("tokens_acc") = py::none(), py::arg("rsum") = py::none(),
          py::arg("margin") = py::none(), py::arg("part") = py::none(), py::arg("S") = 0);
    m.def("router_tokens_per_block", &router_tokens_per_block);
    m.def("router_part_reduce", &router_part_reduce);
    m.def("router_colsum", &router_colsum);
    m.def("moe_aux", &moe_aux);
  }
  {
    namespace py = pybind11;
    m.def("router_bwd", &router_bwd, py::arg("dscores"), py::arg("dtopk_w"), py::arg("scores"), py::arg("topk_idx"),
          py::arg("dlogits"), py::arg("K"), py::arg("mode"), py::arg("norm"), py::arg("scale"),
          py::arg("aux_g") = py::none(), py::arg("d_aux") = py::none(), py::arg("seq_cnt") = py::none(),
          py::arg("rsum") = py::none(), py::arg("seq_scale") = 0.0, py::arg("S") = 0);
  }
  m.def("moe_plan_blocks", &moe_plan_blocks);
  m.def("moe_plan", &moe_plan, pybind11::arg("idx"), pybind11::arg("E"), pybind11::arg("scratch"),
        pybind11::arg("counts"), pybind11::arg("seg_off"), pybind11::arg("tile_expert"), pybind11::arg("num_m_tiles"),
        pybind11::arg("pos"), pybind11::arg("row_slot"), pybind11::arg("pair_tiles") = pybind11::none(),
        pybind11::arg("num_pair_tiles") = pybind11::none(), pybind11::arg("row_tok") = pybind11::none(),
        pybind11::arg("K") = 1);
  m.def("moe_gather", &moe_gather);
  m.def("moe_slot_dot", &moe_slot_dot);
  m.def("moe_row_dot_reduce", &moe_row_dot_reduce);
  m.def("moe_combine", &moe_combine);
  m.def("moe_combine_bwd", &moe_combine_bwd);
  m.def("lse_loss", &lse_loss);
  m.def("lce_reduce", &lce_reduce);
  m.def("dlogits_", &dlogits_);
  m.def("embed_fwd", &embed_fwd);
  m.def("embed_bwd", &embed_bwd);
  m.def("embed_sort_capacity", &embed_sort_capacity);
  m.def("embed_sort", &embed_sort);
  m.def("sumsq_blocks", &sumsq_blocks);
  m.def("sumsq", &sumsq);
  m.def("clip_coef", &clip_coef);
  m.def("adamw", &adamw, pybind11::arg("p"), pybind11::arg("g"), pybind11::arg("m"), pybind11::arg("v"),
        pybind11::arg("p16"), pybind11::arg("hyper"), pybind11::arg("beta1"), pybind11::arg("beta2"), pybind11::arg("eps"),
        pybind11::arg("wd"), pybind11::arg("grad_coef"), pybind11::arg("p16_peers") = std::vector<int64_t>(),
        pybind11::arg("p16_mc") = 0);
  m.def("cast_bf16", &cast_bf16);
  m.def("sum_partials", &sum_partials);
}
