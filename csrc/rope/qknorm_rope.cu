// Per-head QK RMSNorm (weight shared across heads) fused with rotate-half RoPE, forward and backward.
// Input is the fused QKV projection output [T, (nh + 2 nkv) * hd]; one warp per token, several heads per pass.
#include "../common/ptx.cuh"
#include "../ops_api.h"

namespace b200 {

// Lane layout: 16 bytes (8 elements) per lane, HD / 8 lanes per head, so a warp works on 32 / (HD / 8) heads of
// one token at a time and every global access is a full 16-byte vector.  The rotate-half partner of a lane
// sits LPH / 2 lanes away, the per-head sum of squares is a shuffle reduction over the head's lanes.
template <int HD>
struct QkLayout {
  static constexpr int LPH = HD / 8;    // lanes per head
  static constexpr int HPW = 32 / LPH;  // heads per warp pass
  static constexpr int HALF = HD / 2;
};

__device__ __forceinline__ void unpack8(const uint4 q, float (&f)[8]) {
  const float2 a = unpack_bf16x2(q.x), b = unpack_bf16x2(q.y), c = unpack_bf16x2(q.z), d = unpack_bf16x2(q.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  return make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]), pack_bf16x2(f[6], f[7]));
}
template <int LPH>
__device__ __forceinline__ float head_sum(float v) {
#pragma unroll
  for (int o = LPH / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// One warp per token, HPW heads per pass, QK_UNROLL passes in flight.
constexpr int QK_UNROLL = 8;

template <int HD>
__global__ void __launch_bounds__(256)
qknorm_rope_fwd_kernel(const __nv_bfloat16* __restrict__ qkv, int ld, const float* __restrict__ qw,
                       const float* __restrict__ kw, const float* __restrict__ cs,  // [S, hd/2, 2]
                       __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ k_out,
                       __nv_bfloat16* __restrict__ v_out, float* __restrict__ rstd_out, int T, int S, int nh, int nkv,
                       float eps) {
  using L = QkLayout<HD>;
  const int lane = threadIdx.x & 31;
  const int sub = lane / L::LPH, li = lane % L::LPH;
  const int nqk = nh + nkv, nall = nh + 2 * nkv;
  const int wid = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int nw = (gridDim.x * blockDim.x) >> 5;
  float wq[8], wk[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    wq[i] = qw[li * 8 + i];
    wk[i] = kw[li * 8 + i];
  }
  const bool lower = li < L::LPH / 2;  // this lane's elements lie in the first half of the head
  const int passes = (nall + L::HPW - 1) / L::HPW;
  for (int t = wid; t < T; t += nw) {
    const float* csr = cs + (static_cast<size_t>(t % S) * L::HALF + (li * 8) % L::HALF) * 2;
    float c[8], sn[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float4 v = *reinterpret_cast<const float4*>(csr + 4 * i);
      c[2 * i] = v.x;
      sn[2 * i] = lower ? -v.y : v.y;
      c[2 * i + 1] = v.z;
      sn[2 * i + 1] = lower ? -v.w : v.w;
    }
    const __nv_bfloat16* row = qkv + static_cast<size_t>(t) * ld + li * 8;
    for (int p0 = 0; p0 < passes; p0 += QK_UNROLL) {
      uint4 raw[QK_UNROLL];
#pragma unroll
      for (int u = 0; u < QK_UNROLL; ++u) {
        const int h = (p0 + u) * L::HPW + sub;
        if (p0 + u < passes && h < nall) raw[u] = *reinterpret_cast<const uint4*>(row + h * HD);
      }
#pragma unroll
      for (int u = 0; u < QK_UNROLL; ++u) {
        if (p0 + u >= passes) break;  // warp-uniform
        const int h = (p0 + u) * L::HPW + sub;
        const bool active = h < nall;
        if (active && h >= nqk) {  // v head: plain copy into the attention layout
          *reinterpret_cast<uint4*>(v_out + (static_cast<size_t>(t) * nkv + (h - nqk)) * HD + li * 8) = raw[u];
        }
        const bool qk = active && h < nqk;
        float x[8];
        if (qk) {
          unpack8(raw[u], x);
        } else {
#pragma unroll
          for (int i = 0; i < 8; ++i) x[i] = 0.f;
        }
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) ss += x[i] * x[i];
        ss = head_sum<L::LPH>(ss);  // all lanes take part in the shuffles
        const float rstd = rsqrtf(ss * (1.0f / HD) + eps);
        const bool is_q = h < nh;
        float xn[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) xn[i] = x[i] * rstd;
        // round-trip through bf16 (what the unfused module sequence would have stored)
        unpack8(pack8(xn), xn);
        float y[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          xn[i] *= is_q ? wq[i] : wk[i];
          const float other = __shfl_xor_sync(0xffffffffu, xn[i], L::LPH / 2);
          y[i] = xn[i] * c[i] + other * sn[i];
        }
        if (qk) {
          if (li == 0) rstd_out[t * nqk + h] = rstd;
          __nv_bfloat16* dst = is_q ? q_out + (static_cast<size_t>(t) * nh + h) * HD
                                    : k_out + (static_cast<size_t>(t) * nkv + (h - nh)) * HD;
          *reinterpret_cast<uint4*>(dst + li * 8) = pack8(y);
        }
      }
    }
  }
}

// dq/dk -> d(qkv) for the q and k heads, dv copied into the v slice; dw partials [grid, 2, hd].
template <int HD>
__global__ void __launch_bounds__(256)
qknorm_rope_bwd_kernel(const __nv_bfloat16* __restrict__ dq, const __nv_bfloat16* __restrict__ dk,
                       const __nv_bfloat16* __restrict__ dv, const __nv_bfloat16* __restrict__ qkv, int ld,
                       const float* __restrict__ rstd_in, const float* __restrict__ qw, const float* __restrict__ kw,
                       const float* __restrict__ cs, __nv_bfloat16* __restrict__ dqkv, float* __restrict__ dw_part,
                       int T, int S, int nh, int nkv) {
  using L = QkLayout<HD>;
  __shared__ float sm[8][2][HD];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int sub = lane / L::LPH, li = lane % L::LPH;
  const int nqk = nh + nkv, nall = nh + 2 * nkv;
  const int wid = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int nw = (gridDim.x * blockDim.x) >> 5;
  float dwq[8], dwk[8], wq[8], wk[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    dwq[i] = dwk[i] = 0.f;
    wq[i] = qw[li * 8 + i];
    wk[i] = kw[li * 8 + i];
  }
  const bool lower = li < L::LPH / 2;
  const int passes = (nall + L::HPW - 1) / L::HPW;
  constexpr int U = 2;
  for (int t = wid; t < T; t += nw) {
    const float* csr = cs + (static_cast<size_t>(t % S) * L::HALF + (li * 8) % L::HALF) * 2;
    float c[8], sn[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float4 v = *reinterpret_cast<const float4*>(csr + 4 * i);
      c[2 * i] = v.x;
      sn[2 * i] = v.y;
      c[2 * i + 1] = v.z;
      sn[2 * i + 1] = v.w;
    }
    const __nv_bfloat16* row = qkv + static_cast<size_t>(t) * ld + li * 8;
    __nv_bfloat16* drow = dqkv + static_cast<size_t>(t) * ld + li * 8;
    for (int p0 = 0; p0 < passes; p0 += U) {
      uint4 graw[U], xraw[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int h = (p0 + u) * L::HPW + sub;
        if (p0 + u < passes && h < nall) {
          const __nv_bfloat16* gsrc = h < nh    ? dq + (static_cast<size_t>(t) * nh + h) * HD
                                      : h < nqk ? dk + (static_cast<size_t>(t) * nkv + (h - nh)) * HD
                                                : dv + (static_cast<size_t>(t) * nkv + (h - nqk)) * HD;
          graw[u] = *reinterpret_cast<const uint4*>(gsrc + li * 8);
          if (h < nqk) xraw[u] = *reinterpret_cast<const uint4*>(row + h * HD);
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (p0 + u >= passes) break;
        const int h = (p0 + u) * L::HPW + sub;
        const bool active = h < nall;
        if (active && h >= nqk) *reinterpret_cast<uint4*>(drow + h * HD) = graw[u];  // v head: plain copy
        const bool qk = active && h < nqk;
        const bool is_q = h < nh;
        float g[8], x[8];
        if (qk) {
          unpack8(graw[u], g);
          unpack8(xraw[u], x);
        } else {
#pragma unroll
          for (int i = 0; i < 8; ++i) g[i] = x[i] = 0.f;
        }
        const float rstd = qk ? rstd_in[t * nqk + h] : 0.f;
        float xh[8], wd[8];
        float dot = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float gs = g[i] * sn[i];
          const float other = __shfl_xor_sync(0xffffffffu, gs, L::LPH / 2);
          // transpose of the rotation: lower half receives +z[i+HALF], upper half -z[i-HALF]
          const float dxn = g[i] * c[i] + (lower ? other : -other);
          xh[i] = x[i] * rstd;
          wd[i] = dxn * (is_q ? wq[i] : wk[i]);
          dot += wd[i] * xh[i];
          if (is_q) dwq[i] += dxn * xh[i]; else dwk[i] += dxn * xh[i];
        }
        dot = head_sum<L::LPH>(dot) * (1.0f / HD);
        if (qk) {
          float o[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] = rstd * (wd[i] - xh[i] * dot);
          *reinterpret_cast<uint4*>(drow + h * HD) = pack8(o);
        }
      }
    }
  }
  // lanes with the same position inside a head (same li) hold partial sums for the same weight elements
#pragma unroll
  for (int i = 0; i < 8; ++i) {
#pragma unroll
    for (int o = L::LPH; o < 32; o <<= 1) {
      dwq[i] += __shfl_xor_sync(0xffffffffu, dwq[i], o);
      dwk[i] += __shfl_xor_sync(0xffffffffu, dwk[i], o);
    }
  }
  if (sub == 0) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      sm[warp][0][li * 8 + i] = dwq[i];
      sm[warp][1][li * 8 + i] = dwk[i];
    }
  }
  __syncthreads();
  const int nwarps = blockDim.x >> 5;
  for (int cc = threadIdx.x; cc < 2 * HD; cc += blockDim.x) {
    float s2 = 0.f;
    for (int wv = 0; wv < nwarps; ++wv) s2 += sm[wv][cc / HD][cc % HD];
    dw_part[static_cast<size_t>(blockIdx.x) * 2 * HD + cc] = s2;
  }
}

__global__ void qk_dw_reduce_kernel(const float* __restrict__ part, int nblocks, int hd, float* __restrict__ dqw,
                                    float* __restrict__ dkw, int accumulate) {
  // block = 32 columns of the [nblocks, 2*hd] partials, 32 warps stride over the rows; fixed summation order
  __shared__ float sm[32][33];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + lane;
  float s = 0.f;
  if (c < 2 * hd)
    for (int b = warp; b < nblocks; b += 32) s += part[static_cast<size_t>(b) * 2 * hd + c];
  sm[warp][lane] = s;
  __syncthreads();
  if (warp == 0 && c < 2 * hd) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < 32; ++w) t += sm[w][lane];
    float* out = c < hd ? dqw + c : dkw + (c - hd);
    *out = accumulate ? *out + t : t;
  }
}

}  // namespace b200

using namespace b200;

// `items` = number of tokens; one warp per token, eight warps per block
extern "C" int b200_qknorm_rope_blocks(long long items) {
  long long g = (items + 7) / 8;
  return static_cast<int>(g < 1 ? 1 : (g > 592 ? 592 : g));
}

extern "C" int b200_qknorm_rope_fwd(const void* qkv, int ld, const float* qw, const float* kw, const float* cs,
                                    void* q_out, void* k_out, void* v_out, float* rstd, int T, int S, int nh, int nkv,
                                    int hd, float eps, cudaStream_t stream) {
  if (T <= 0) return 0;
  const int grid = b200_qknorm_rope_blocks(T);
#define ARGS reinterpret_cast<const __nv_bfloat16*>(qkv), ld, qw, kw, cs, reinterpret_cast<__nv_bfloat16*>(q_out), \
             reinterpret_cast<__nv_bfloat16*>(k_out), reinterpret_cast<__nv_bfloat16*>(v_out), rstd, T, S, nh, nkv, eps
  if (hd == 128) qknorm_rope_fwd_kernel<128><<<grid, 256, 0, stream>>>(ARGS);
  else if (hd == 64) qknorm_rope_fwd_kernel<64><<<grid, 256, 0, stream>>>(ARGS);
  else if (hd == 32) qknorm_rope_fwd_kernel<32><<<grid, 256, 0, stream>>>(ARGS);
  else return -1;
#undef ARGS
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int b200_qknorm_rope_bwd(const void* dq, const void* dk, const void* dv, const void* qkv, int ld,
                                    const float* rstd, const float* qw, const float* kw, const float* cs, void* dqkv,
                                    float* dw_part, float* dqw, float* dkw, int dw_accumulate, int T, int S, int nh,
                                    int nkv, int hd, cudaStream_t stream) {
  if (T <= 0) return 0;
  const int grid = b200_qknorm_rope_blocks(T);
#define ARGS reinterpret_cast<const __nv_bfloat16*>(dq), reinterpret_cast<const __nv_bfloat16*>(dk),             \
             reinterpret_cast<const __nv_bfloat16*>(dv), reinterpret_cast<const __nv_bfloat16*>(qkv), ld, rstd, \
             qw, kw, cs, reinterpret_cast<__nv_bfloat16*>(dqkv), dw_part, T, S, nh, nkv
  if (hd == 128) qknorm_rope_bwd_kernel<128><<<grid, 256, 0, stream>>>(ARGS);
  else if (hd == 64) qknorm_rope_bwd_kernel<64><<<grid, 256, 0, stream>>>(ARGS);
  else if (hd == 32) qknorm_rope_bwd_kernel<32><<<grid, 256, 0, stream>>>(ARGS);
  else return -1;
#undef ARGS
  qk_dw_reduce_kernel<<<(2 * hd + 31) / 32, 1024, 0, stream>>>(dw_part, grid, hd, dqw, dkw, dw_accumulate);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
