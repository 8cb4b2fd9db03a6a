// Router scoring and selection on fp32 logits: softmax or sigmoid(+selection bias), optional
// group-limited routing, top-k with ties to the lowest index, weight normalisation and scaling.
// One warp per token; the token's score row lives in shared memory during selection.
#include "../common/ptx.cuh"
#include "../ops_api.h"

namespace b200 {

constexpr int ROUTER_WARPS = 4;

struct ArgMax {
  float v;
  int i;
};
__device__ __forceinline__ ArgMax better(ArgMax a, ArgMax b) {
  return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a;
}
__device__ __forceinline__ ArgMax warp_argmax(ArgMax a) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgMax b;
    b.v = __shfl_xor_sync(0xffffffffu, a.v, o);
    b.i = __shfl_xor_sync(0xffffffffu, a.i, o);
    a = better(a, b);
  }
  return a;
}
// arg max over buf[lo, hi), lowest index on ties; every lane returns the same result
__device__ __forceinline__ ArgMax row_argmax(const float* buf, int lo, int hi, int lane) {
  ArgMax a{-INFINITY, 0x7fffffff};
  for (int e = lo + lane; e < hi; e += 32) {
    const float v = buf[e];
    if (v > a.v) {
      a.v = v;
      a.i = e;
    }
  }
  a = warp_argmax(a);
  if (a.i == 0x7fffffff) a.i = lo;  // whole range is -inf
  return a;
}

// Statistics the losses and the routing report need, produced while the token's scores are on chip
// (all optional, null = off).  Counts are integers added with atomics, so their value does not depend
// on the order; floating-point sums are left to fixed-order reductions elsewhere.
struct RouterStats {
  int* cnt_sel;       // [B, E] tokens routed to each expert per sequence (the actual, bias-steered choice)
  int* cnt_unb;       // [B, E] the same from the top-k of the unbiased scores (Switch loss, routing report)
  float* tokens_acc;  // [E] running token counter of the router (selection counts are added)
  float* rsum;        // [T] sum of the token's scores over the experts
  float* margin;      // [T] k-th minus (k+1)-th unbiased score
  float* part;        // [blocks, 2, E] per-block sums of the scores and of the row-normalised scores (needs rsum,
                      // and S a multiple of the block's token count)
  int S;              // tokens per sequence
  int separate_unb;   // the unbiased top-k can differ from the selection (bias or group-limited routing)
  int tpw;            // consecutive tokens per warp (a block covers ROUTER_WARPS * tpw consecutive tokens)
};

// mode 0: softmax, mode 1: sigmoid.  bias (may be null) only steers selection.
__global__ void router_fwd_kernel(const float* __restrict__ logits, const float* __restrict__ bias,
                                  float* __restrict__ scores, float* __restrict__ topk_w, int* __restrict__ topk_idx,
                                  int T, int E, int K, int mode, int norm, float scale, int num_groups,
                                  int group_topk, const RouterStats st) {
  extern __shared__ float sm[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* buf = sm + static_cast<size_t>(warp) * (E + 32);
  float* gsc = buf + E;  // group scores
  // block-level histograms (one sequence per block when S is a multiple of the block's token count)
  int* hsel = reinterpret_cast<int*>(sm + static_cast<size_t>(ROUTER_WARPS) * (E + 32));
  int* hunb = hsel + E;
  // per-warp running sums over this warp's tokens (fixed order): [warp][raw | normalised][E]
  float* psw = reinterpret_cast<float*>(hunb + E) + static_cast<size_t>(warp) * 2 * E;
  const int block_tokens = ROUTER_WARPS * st.tpw;
  const bool want_cnt = st.cnt_sel != nullptr;
  const bool block_hist = want_cnt && (st.S % block_tokens == 0);
  const bool want_part = st.part != nullptr;
  if (block_hist) {
    for (int e = threadIdx.x; e < 2 * E; e += blockDim.x) hsel[e] = 0;
  }
  if (want_part) {
    for (int e = lane; e < 2 * E; e += 32) psw[e] = 0.f;
  }
  __syncthreads();
  const int t_begin = blockIdx.x * block_tokens + warp * st.tpw;
  for (int t = t_begin; t < t_begin + st.tpw && t < T; ++t) {
    const float* lr = logits + static_cast<size_t>(t) * E;
    float* sr = scores + static_cast<size_t>(t) * E;
    if (mode == 0) {
      float mx = -INFINITY;
      for (int e = lane; e < E; e += 32) {
        const float v = lr[e];
        buf[e] = v;
        mx = fmaxf(mx, v);
      }
      mx = warp_max(mx);
      float sum = 0.f;
      for (int e = lane; e < E; e += 32) {
        const float p = expf(buf[e] - mx);
        buf[e] = p;
        sum += p;
      }
      sum = warp_sum(sum);
      const float inv = 1.f / sum;
      for (int e = lane; e < E; e += 32) {
        const float p = buf[e] * inv;
        sr[e] = p;
        buf[e] = bias ? p + bias[e] : p;
      }
    } else {
      for (int e = lane; e < E; e += 32) {
        const float s = 1.f / (1.f + expf(-lr[e]));
        sr[e] = s;
        buf[e] = bias ? s + bias[e] : s;
      }
    }
    __syncwarp();
    if (num_groups > 1) {
      const int per = E / num_groups;
      const int m = K / group_topk;
      for (int g = 0; g < num_groups; ++g) {
        // sum of the top-m biased scores of the group; picked entries are parked as -inf and restored
        float acc = 0.f;
        int picked[8];
        float pv[8];
        for (int j = 0; j < m; ++j) {
          const ArgMax a = row_argmax(buf, g * per, (g + 1) * per, lane);
          acc += a.v;
          picked[j] = a.i;
          pv[j] = a.v;
          __syncwarp();
          if (lane == 0) buf[a.i] = -INFINITY;
          __syncwarp();
        }
        if (lane == 0) {
          for (int j = 0; j < m; ++j) buf[picked[j]] = pv[j];
          gsc[g] = acc;
        }
        __syncwarp();
      }
      unsigned keep = 0u;
      for (int j = 0; j < group_topk; ++j) {
        const ArgMax a = row_argmax(gsc, 0, num_groups, lane);
        keep |= 1u << a.i;
        __syncwarp();
        if (lane == 0) gsc[a.i] = -INFINITY;
        __syncwarp();
      }
      for (int e = lane; e < E; e += 32)
        if (!((keep >> (e / per)) & 1u)) buf[e] = -INFINITY;
      __syncwarp();
    }
    float myw = 0.f;
    int myi = 0;
    float wsum = 0.f;
    float last_un = 0.f;
    for (int k = 0; k < K; ++k) {
      const ArgMax a = row_argmax(buf, 0, E, lane);
      const float un = sr[a.i];  // unbiased score (written above by this warp)
      wsum += un;
      last_un = un;
      if (lane == k) {
        myw = un;
        myi = a.i;
      }
      __syncwarp();
      if (lane == 0) buf[a.i] = -INFINITY;
      __syncwarp();
    }
    if (norm) myw = mode == 0 ? myw / wsum : myw / (wsum + 1e-20f);
    myw *= scale;
    if (lane < K) {
      topk_w[static_cast<size_t>(t) * K + lane] = myw;
      topk_idx[static_cast<size_t>(t) * K + lane] = myi;
    }
    // ---- statistics
    const int seq = st.S > 0 ? t / st.S : 0;
    if (want_cnt && lane < K) {
      if (block_hist) {
        atomicAdd(&hsel[myi], 1);
      } else {
        atomicAdd(&st.cnt_sel[static_cast<size_t>(seq) * E + myi], 1);
        if (st.tokens_acc != nullptr) atomicAdd(&st.tokens_acc[myi], 1.f);
      }
    }
    if (st.rsum != nullptr) {
      float rs = 0.f;
      for (int e = lane; e < E; e += 32) rs += sr[e];
      rs = warp_sum(rs);
      if (lane == 0) st.rsum[t] = rs;
      if (want_part) {
        const float inv = 1.f / (rs + 1e-20f);
        for (int e = lane; e < E; e += 32) {
          const float v = sr[e];
          psw[e] += v;
          psw[E + e] += v * inv;
        }
      }
    }
    if (st.separate_unb && (st.cnt_unb != nullptr || st.margin != nullptr)) {
      // top-(k+1) of the unbiased scores: counts for the Switch loss / report, margin between k and k+1
      __syncwarp();
      for (int e = lane; e < E; e += 32) buf[e] = sr[e];
      __syncwarp();
      float vk = 0.f, vk1 = 0.f;
      const int rounds = K < E ? K + 1 : K;
      for (int k = 0; k < rounds; ++k) {
        const ArgMax a = row_argmax(buf, 0, E, lane);
        if (k == K - 1) vk = a.v;
        if (k == K) vk1 = a.v;
        if (k < K && lane == 0 && st.cnt_unb != nullptr) {
          if (block_hist) atomicAdd(&hunb[a.i], 1);
          else atomicAdd(&st.cnt_unb[static_cast<size_t>(seq) * E + a.i], 1);
        }
        __syncwarp();
        if (lane == 0) buf[a.i] = -INFINITY;
        __syncwarp();
      }
      if (st.margin != nullptr && lane == 0) st.margin[t] = K < E ? vk - vk1 : 0.f;
    } else if (st.margin != nullptr) {
      // selection == unbiased top-k: one more round gives the (k+1)-th score
      float m = 0.f;
      if (K < E) {
        const ArgMax a = row_argmax(buf, 0, E, lane);
        m = last_un - sr[a.i];
      }
      if (lane == 0) st.margin[t] = m;
    }
    __syncwarp();
  }
  if (want_part) {
    __syncthreads();
    const float* all = reinterpret_cast<const float*>(hunb + E);
    for (int e = threadIdx.x; e < 2 * E; e += blockDim.x) {
      float a = 0.f;
#pragma unroll
      for (int w = 0; w < ROUTER_WARPS; ++w) a += all[static_cast<size_t>(w) * 2 * E + e];  // warp order: fixed
      st.part[static_cast<size_t>(blockIdx.x) * 2 * E + e] = a;
    }
  }
  if (block_hist) {
    __syncthreads();
    const int t0 = blockIdx.x * block_tokens;
    if (t0 < T) {
      const int seq = t0 / st.S;
      for (int e = threadIdx.x; e < E; e += blockDim.x) {
        const int c = hsel[e];
        if (c) {
          atomicAdd(&st.cnt_sel[static_cast<size_t>(seq) * E + e], c);
          if (st.tokens_acc != nullptr) atomicAdd(&st.tokens_acc[e], static_cast<float>(c));
        }
        if (st.separate_unb && st.cnt_unb != nullptr && hunb[e])
          atomicAdd(&st.cnt_unb[static_cast<size_t>(seq) * E + e], hunb[e]);
      }
    }
  }
}

// Column sums of the scores per sequence, in a fixed order: psum[b, e] = sum over the tokens t of sequence
// b of s[t, e], and pn[b, e] = the same of s[t, e] / (rsum[t] + 1e-20) (normalised scores).  One block per
// (32-column tile, sequence); warps walk the rows w, w + 8, ..., and are added up in warp order.
__global__ void router_colsum_kernel(const float* __restrict__ scores, const float* __restrict__ rsum, int S, int E,
                                     float* __restrict__ psum, float* __restrict__ pn) {
  __shared__ float sh[2][8][32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int e = blockIdx.x * 32 + lane;
  const int b = blockIdx.y;
  float a = 0.f, n = 0.f;
  if (e < E) {
    for (int r = warp; r < S; r += 8) {
      const size_t t = static_cast<size_t>(b) * S + r;
      const float v = scores[t * E + e];
      a += v;
      if (rsum != nullptr) n += v / (rsum[t] + 1e-20f);
    }
  }
  sh[0][warp][lane] = a;
  sh[1][warp][lane] = n;
  __syncthreads();
  if (warp == 0 && e < E) {
    float x = 0.f, y = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) {
      x += sh[0][w][lane];
      y += sh[1][w][lane];
    }
    psum[static_cast<size_t>(b) * E + e] = x;
    if (pn != nullptr) pn[static_cast<size_t>(b) * E + e] = y;
  }
}

// Per-sequence sums from the per-block partials router_fwd_kernel wrote: psum[b, e] (and pn[b, e]) = sum over the
// `bps` blocks of sequence b, in a fixed order (32 warps stride over the blocks, then warp order).
__global__ void __launch_bounds__(1024)
router_part_reduce_kernel(const float* __restrict__ part, int bps, int E, float* __restrict__ psum,
                          float* __restrict__ pn) {
  __shared__ float sh[2][32][33];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int e = blockIdx.x * 32 + lane;
  const int b = blockIdx.y;
  float a = 0.f, n = 0.f;
  if (e < E) {
    for (int k = warp; k < bps; k += 32) {
      const float* p = part + (static_cast<size_t>(b) * bps + k) * 2 * E;
      a += p[e];
      n += p[E + e];
    }
  }
  sh[0][warp][lane] = a;
  sh[1][warp][lane] = n;
  __syncthreads();
  if (warp == 0 && e < E) {
    float x = 0.f, y = 0.f;
#pragma unroll
    for (int w = 0; w < 32; ++w) {
      x += sh[0][w][lane];
      y += sh[1][w][lane];
    }
    psum[static_cast<size_t>(b) * E + e] = x;
    pn[static_cast<size_t>(b) * E + e] = y;
  }
}

// Both balance losses from the per-layer statistics, single block, fixed order.
//   Switch loss (all layers pooled):  aux = E * sum_e (cnt_e / N) * (psum_e / N),  N = L * B * S,
//     cnt from the unbiased top-k; g[e] = E * cnt_e / N^2 is its gradient w.r.t. every score of expert e.
//   Sequence-level loss: mean over layers and sequences of sum_e f[b,e] * P[b,e],
//     f = cnt_sel * E / (K * S),  P = pn / S.
// out[0] = aux, out[1] = seq aux.
__global__ void moe_aux_kernel(const int* __restrict__ cnt_unb, const int* __restrict__ cnt_sel,
                               const float* __restrict__ psum, const float* __restrict__ pn, int L, int B, int E,
                               int K, int S, float* __restrict__ g, float* __restrict__ out) {
  __shared__ float red[2][32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const float N = static_cast<float>(L) * B * S;
  float aux = 0.f, seq = 0.f;
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    float c = 0.f, p = 0.f;
    for (int lb = 0; lb < L * B; ++lb) {
      c += static_cast<float>(cnt_unb[static_cast<size_t>(lb) * E + e]);
      p += psum[static_cast<size_t>(lb) * E + e];
      if (pn != nullptr)
        seq += static_cast<float>(cnt_sel[static_cast<size_t>(lb) * E + e]) * pn[static_cast<size_t>(lb) * E + e];
    }
    aux += (c / N) * (p / N);
    if (g != nullptr) g[e] = static_cast<float>(E) * c / (N * N);
  }
  aux = warp_sum(aux);
  seq = warp_sum(seq);
  if (lane == 0) {
    red[0][warp] = aux;
    red[1][warp] = seq;
  }
  __syncthreads();
  if (warp == 0) {
    float a = lane < nw ? red[0][lane] : 0.f, s2 = lane < nw ? red[1][lane] : 0.f;
    a = warp_sum(a);
    s2 = warp_sum(s2);
    if (lane == 0) {
      out[0] = a * static_cast<float>(E);
      out[1] = s2 * static_cast<float>(E) / (static_cast<float>(K) * S * S * L * B);
    }
  }
}

// Gradient of the two balance losses w.r.t. the scores, applied on the fly (nothing of size [T, E] is built):
//   Switch:   d_aux[0] * g[e]
//   sequence: d_aux[1] * seq_scale / rsum_t * (c[b,e] - sum_e' c[b,e'] * s[t,e'] / rsum_t),  c = cnt_sel
struct RouterAuxGrad {
  const float* g;        // [E] or null
  const float* d_aux;    // device pair: upstream gradients of (aux, seq aux)
  const int* cnt_sel;    // [B, E] or null (sequence-level loss off)
  const float* rsum;     // [T]
  float seq_scale;       // E / (K * S) / (L * B * S)
  int S;
};

// d(logits) in bf16 from d(scores) (may be null), d(topk weights) and the balance-loss terms.
__global__ void router_bwd_kernel(const float* __restrict__ dscores, const float* __restrict__ dtopk_w,
                                  const float* __restrict__ scores, const int* __restrict__ topk_idx,
                                  __nv_bfloat16* __restrict__ dlogits, int T, int E, int K, int mode, int norm,
                                  float scale, const RouterAuxGrad ag) {
  extern __shared__ float sm[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* buf = sm + static_cast<size_t>(warp) * E;
  const float da = ag.g != nullptr ? ag.d_aux[0] : 0.f;
  const float ds = ag.cnt_sel != nullptr ? ag.d_aux[1] * ag.seq_scale : 0.f;
  for (int t = blockIdx.x * ROUTER_WARPS + warp; t < T; t += gridDim.x * ROUTER_WARPS) {
    const float* sr = scores + static_cast<size_t>(t) * E;
    for (int e = lane; e < E; e += 32) {
      float v = dscores ? dscores[static_cast<size_t>(t) * E + e] : 0.f;
      if (ag.g != nullptr) v += da * ag.g[e];
      buf[e] = v;
    }
    if (ag.cnt_sel != nullptr) {
      const int* c = ag.cnt_sel + static_cast<size_t>(t / ag.S) * E;
      const float inv = 1.f / (ag.rsum[t] + 1e-20f);
      float dot = 0.f;
      for (int e = lane; e < E; e += 32) dot += static_cast<float>(c[e]) * sr[e];
      dot = warp_sum(dot) * inv;
      for (int e = lane; e < E; e += 32) buf[e] += ds * inv * (static_cast<float>(c[e]) - dot);
    }
    __syncwarp();
    // selected entries
    int idx = 0;
    float sk = 0.f, dwk = 0.f;
    if (lane < K) {
      idx = topk_idx[static_cast<size_t>(t) * K + lane];
      sk = sr[idx];
      dwk = dtopk_w[static_cast<size_t>(t) * K + lane] * scale;
    }
    float add;
    if (norm) {
      const float S = warp_sum(sk) + (mode == 0 ? 0.f : 1e-20f);
      const float dot = warp_sum(dwk * sk) / S;
      add = (dwk - dot) / S;
    } else {
      add = dwk;
    }
    if (lane < K) buf[idx] += add;
    __syncwarp();
    __nv_bfloat16* out = dlogits + static_cast<size_t>(t) * E;
    if (mode == 0) {
      float dot = 0.f;
      for (int e = lane; e < E; e += 32) dot += buf[e] * sr[e];
      dot = warp_sum(dot);
      for (int e = lane; e < E; e += 32) out[e] = __float2bfloat16(sr[e] * (buf[e] - dot));
    } else {
      for (int e = lane; e < E; e += 32) {
        const float s = sr[e];
        out[e] = __float2bfloat16(buf[e] * s * (1.f - s));
      }
    }
    __syncwarp();
  }
}

}  // namespace b200

using namespace b200;

// tokens per warp: few for small expert counts (many blocks in flight), more when a token's row is long
extern "C" int b200_router_tokens_per_block(int E) { return ROUTER_WARPS * (E <= 256 ? 2 : 8); }

static int router_grid(int T) {
  int g = (T + ROUTER_WARPS - 1) / ROUTER_WARPS;
  return g < 1 ? 1 : (g > 1184 ? 1184 : g);
}

extern "C" int b200_router_fwd(const float* logits, const float* bias, float* scores, float* topk_w, int* topk_idx,
                               int T, int E, int K, int mode, int norm, float scale, int num_groups, int group_topk,
                               int* cnt_sel, int* cnt_unb, float* tokens_acc, float* rsum, float* margin, float* part,
                               int S, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (K > 32 || K > E || num_groups > 32) return -1;
  if (num_groups > 1 && (E % num_groups != 0 || group_topk <= 0 || K % group_topk != 0 || K / group_topk > 8))
    return -1;
  if (cnt_sel != nullptr && (S <= 0 || T % S != 0)) return -1;
  RouterStats st;
  st.cnt_sel = cnt_sel;
  st.cnt_unb = cnt_unb;
  st.tokens_acc = tokens_acc;
  st.rsum = rsum;
  st.margin = margin;
  st.part = part;
  st.S = S > 0 ? S : T;
  st.separate_unb = (bias != nullptr || num_groups > 1) ? 1 : 0;
  st.tpw = b200_router_tokens_per_block(E) / ROUTER_WARPS;
  if (!st.separate_unb && cnt_unb != nullptr && cnt_unb != cnt_sel) return -1;  // identical by construction
  const int block_tokens = ROUTER_WARPS * st.tpw;
  if (part != nullptr && (rsum == nullptr || st.S % block_tokens != 0)) return -1;
  const size_t smem = (static_cast<size_t>(ROUTER_WARPS) * (E + 32) + 2 * static_cast<size_t>(E) +
                       (part != nullptr ? static_cast<size_t>(ROUTER_WARPS) * 2 * E : 0)) * sizeof(float);
  if (smem > 48 * 1024) {
    if (smem > 200 * 1024) return -1;
    cudaFuncSetAttribute(router_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  }
  router_fwd_kernel<<<(T + block_tokens - 1) / block_tokens, ROUTER_WARPS * 32, smem, stream>>>(
      logits, bias, scores, topk_w, topk_idx, T, E, K, mode, norm, scale, num_groups, group_topk, st);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int b200_router_colsum(const float* scores, const float* rsum, int B, int S, int E, float* psum, float* pn,
                                  cudaStream_t stream) {
  if (B <= 0 || S <= 0 || E <= 0) return 0;
  if (pn != nullptr && rsum == nullptr) return -1;
  router_colsum_kernel<<<dim3((E + 31) / 32, B), 256, 0, stream>>>(scores, rsum, S, E, psum, pn);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int b200_router_part_reduce(const float* part, int B, int blocks_per_seq, int E, float* psum, float* pn,
                                       cudaStream_t stream) {
  if (B <= 0 || blocks_per_seq <= 0 || E <= 0) return -1;
  router_part_reduce_kernel<<<dim3((E + 31) / 32, B), 1024, 0, stream>>>(part, blocks_per_seq, E, psum, pn);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int b200_moe_aux(const int* cnt_unb, const int* cnt_sel, const float* psum, const float* pn, int L, int B,
                            int E, int K, int S, float* g, float* out, cudaStream_t stream) {
  if (L <= 0 || B <= 0 || E <= 0) return -1;
  if (pn != nullptr && cnt_sel == nullptr) return -1;
  moe_aux_kernel<<<1, 1024, 0, stream>>>(cnt_unb, cnt_sel, psum, pn, L, B, E, K, S, g, out);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int b200_router_bwd(const float* dscores, const float* dtopk_w, const float* scores, const int* topk_idx,
                               void* dlogits, int T, int E, int K, int mode, int norm, float scale,
                               const float* aux_g, const float* d_aux, const int* seq_cnt, const float* rsum,
                               float seq_scale, int S, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (K > 32) return -1;
  if ((aux_g != nullptr || seq_cnt != nullptr) && d_aux == nullptr) return -1;
  if (seq_cnt != nullptr && (rsum == nullptr || S <= 0)) return -1;
  RouterAuxGrad ag;
  ag.g = aux_g;
  ag.d_aux = d_aux;
  ag.cnt_sel = seq_cnt;
  ag.rsum = rsum;
  ag.seq_scale = seq_scale;
  ag.S = S > 0 ? S : T;
  const size_t smem = static_cast<size_t>(ROUTER_WARPS) * E * sizeof(float);
  if (smem > 48 * 1024) {
    if (smem > 200 * 1024) return -1;
    cudaFuncSetAttribute(router_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  }
  router_bwd_kernel<<<router_grid(T), ROUTER_WARPS * 32, smem, stream>>>(
      dscores, dtopk_w, scores, topk_idx, reinterpret_cast<__nv_bfloat16*>(dlogits), T, E, K, mode, norm, scale, ag);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
