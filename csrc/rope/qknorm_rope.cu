// Per-head QK RMSNorm (weight shared across heads) fused with rotate-half RoPE, forward and backward.
// Input is the fused QKV projection output [T, (nh + 2 nkv) * hd]; one warp handles one (token, head).
#include "../common/ptx.cuh"
#include "../ops_api.h"

namespace b200 {

template <int EPL>  // elements per lane = hd / 32
__device__ __forceinline__ void load_lane(const __nv_bfloat16* p, int lane, float (&f)[EPL]) {
  if constexpr (EPL == 4) {
    const uint2 q = *reinterpret_cast<const uint2*>(p + lane * 4);
    const float2 a = unpack_bf16x2(q.x), b = unpack_bf16x2(q.y);
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
  } else if constexpr (EPL == 2) {
    const float2 a = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(p + lane * 2));
    f[0] = a.x; f[1] = a.y;
  } else {
    f[0] = __bfloat162float(p[lane]);
  }
}
template <int EPL>
__device__ __forceinline__ void store_lane(__nv_bfloat16* p, int lane, const float (&f)[EPL]) {
  if constexpr (EPL == 4) {
    *reinterpret_cast<uint2*>(p + lane * 4) = make_uint2(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]));
  } else if constexpr (EPL == 2) {
    *reinterpret_cast<uint32_t*>(p + lane * 2) = pack_bf16x2(f[0], f[1]);
  } else {
    p[lane] = __float2bfloat16(f[0]);
  }
}

// round-trip through bf16 (what the unfused module sequence would have stored), two lanes of work at a time
template <int EPL>
__device__ __forceinline__ void round_bf16(float (&v)[EPL]) {
  if constexpr (EPL >= 2) {
#pragma unroll
    for (int i = 0; i < EPL; i += 2) {
      const float2 f = unpack_bf16x2(pack_bf16x2(v[i], v[i + 1]));
      v[i] = f.x;
      v[i + 1] = f.y;
    }
  } else {
    v[0] = __bfloat162float(__float2bfloat16(v[0]));
  }
}

// One warp per token, looping over that token's heads: the position, the cos/sin values and the norm
// weights of a lane's elements are loaded once per token instead of once per (token, head), and no
// index division is left in the inner loop.
template <int EPL>
__global__ void qknorm_rope_fwd_kernel(const __nv_bfloat16* __restrict__ qkv, int ld, const float* __restrict__ qw,
                                       const float* __restrict__ kw, const float* __restrict__ cs,  // [S, hd/2, 2]
                                       __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ k_out,
                                       __nv_bfloat16* __restrict__ v_out, float* __restrict__ rstd_out, int T, int S,
                                       int nh, int nkv, float eps) {
  constexpr int HD = EPL * 32, HALF = HD / 2;
  const int lane = threadIdx.x & 31;
  const int nqk = nh + nkv, nall = nh + 2 * nkv;
  const int wid = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int nw = (gridDim.x * blockDim.x) >> 5;
  float wq[EPL], wk[EPL];
#pragma unroll
  for (int i = 0; i < EPL; ++i) {
    wq[i] = qw[lane * EPL + i];
    wk[i] = kw[lane * EPL + i];
  }
  const bool lower = lane < 16;  // elements of this lane lie in the first half of the head
  for (int t = wid; t < T; t += nw) {
    const float* csr = cs + static_cast<size_t>(t % S) * HALF * 2;
    float c[EPL], sn[EPL];
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
      const int j = (lane * EPL + i) % HALF;
      const float2 v = *reinterpret_cast<const float2*>(csr + 2 * j);
      c[i] = v.x;
      sn[i] = lower ? -v.y : v.y;
    }
    const __nv_bfloat16* row = qkv + static_cast<size_t>(t) * ld;
#pragma unroll 2
    for (int h = 0; h < nall; ++h) {
      float x[EPL];
      load_lane<EPL>(row + h * HD, lane, x);
      if (h >= nqk) {  // v head: plain copy into the attention layout
        store_lane<EPL>(v_out + (static_cast<size_t>(t) * nkv + (h - nqk)) * HD, lane, x);
        continue;
      }
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < EPL; ++i) ss += x[i] * x[i];
      ss = warp_sum(ss);
      const float rstd = rsqrtf(ss * (1.0f / HD) + eps);
      if (lane == 0) rstd_out[t * nqk + h] = rstd;
      const bool is_q = h < nh;
      float xn[EPL];
#pragma unroll
      for (int i = 0; i < EPL; ++i) xn[i] = x[i] * rstd;
      round_bf16<EPL>(xn);
      float y[EPL];
#pragma unroll
      for (int i = 0; i < EPL; ++i) {
        xn[i] *= is_q ? wq[i] : wk[i];
        const float other = __shfl_xor_sync(0xffffffffu, xn[i], 16);
        y[i] = xn[i] * c[i] + other * sn[i];
      }
      __nv_bfloat16* dst = is_q ? q_out + (static_cast<size_t>(t) * nh + h) * HD
                                : k_out + (static_cast<size_t>(t) * nkv + (h - nh)) * HD;
      store_lane<EPL>(dst, lane, y);
    }
  }
}

// dq/dk -> d(qkv) for the q and k heads, dv copied into the v slice; dw partials [grid, 2, hd].
template <int EPL>
__global__ void qknorm_rope_bwd_kernel(const __nv_bfloat16* __restrict__ dq, const __nv_bfloat16* __restrict__ dk,
                                       const __nv_bfloat16* __restrict__ dv, const __nv_bfloat16* __restrict__ qkv,
                                       int ld, const float* __restrict__ rstd_in, const float* __restrict__ qw,
                                       const float* __restrict__ kw, const float* __restrict__ cs,
                                       __nv_bfloat16* __restrict__ dqkv, float* __restrict__ dw_part, int T, int S,
                                       int nh, int nkv) {
  constexpr int HD = EPL * 32, HALF = HD / 2;
  __shared__ float sm[8][2][HD];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nqk = nh + nkv, nall = nh + 2 * nkv;
  const int wid = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int nw = (gridDim.x * blockDim.x) >> 5;
  float dwq[EPL], dwk[EPL], wq[EPL], wk[EPL];
#pragma unroll
  for (int i = 0; i < EPL; ++i) {
    dwq[i] = dwk[i] = 0.f;
    wq[i] = qw[lane * EPL + i];
    wk[i] = kw[lane * EPL + i];
  }
  const bool lower = lane < 16;
  for (int t = wid; t < T; t += nw) {
    const float* csr = cs + static_cast<size_t>(t % S) * HALF * 2;
    float c[EPL], sn[EPL];
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
      const int j = (lane * EPL + i) % HALF;
      const float2 v = *reinterpret_cast<const float2*>(csr + 2 * j);
      c[i] = v.x;
      sn[i] = v.y;
    }
    const __nv_bfloat16* row = qkv + static_cast<size_t>(t) * ld;
    __nv_bfloat16* drow = dqkv + static_cast<size_t>(t) * ld;
#pragma unroll 2
    for (int h = 0; h < nall; ++h) {
      __nv_bfloat16* dst = drow + h * HD;
      if (h >= nqk) {  // v head: plain copy
        float g[EPL];
        load_lane<EPL>(dv + (static_cast<size_t>(t) * nkv + (h - nqk)) * HD, lane, g);
        store_lane<EPL>(dst, lane, g);
        continue;
      }
      const bool is_q = h < nh;
      const __nv_bfloat16* gsrc = is_q ? dq + (static_cast<size_t>(t) * nh + h) * HD
                                       : dk + (static_cast<size_t>(t) * nkv + (h - nh)) * HD;
      float g[EPL], x[EPL];
      load_lane<EPL>(gsrc, lane, g);
      load_lane<EPL>(row + h * HD, lane, x);
      const float rstd = rstd_in[t * nqk + h];
      float xh[EPL], wd[EPL];
      float dot = 0.f;
#pragma unroll
      for (int i = 0; i < EPL; ++i) {
        const float gs = g[i] * sn[i];
        const float other = __shfl_xor_sync(0xffffffffu, gs, 16);
        // transpose of the rotation: lower half receives +z[i+HALF], upper half -z[i-HALF]
        const float dxn = g[i] * c[i] + (lower ? other : -other);
        xh[i] = x[i] * rstd;
        wd[i] = dxn * (is_q ? wq[i] : wk[i]);
        dot += wd[i] * xh[i];
        if (is_q) dwq[i] += dxn * xh[i]; else dwk[i] += dxn * xh[i];
      }
      dot = warp_sum(dot) * (1.0f / HD);
      float o[EPL];
#pragma unroll
      for (int i = 0; i < EPL; ++i) o[i] = rstd * (wd[i] - xh[i] * dot);
      store_lane<EPL>(dst, lane, o);
    }
  }
#pragma unroll
  for (int i = 0; i < EPL; ++i) {
    sm[warp][0][lane * EPL + i] = dwq[i];
    sm[warp][1][lane * EPL + i] = dwk[i];
  }
  __syncthreads();
  const int nwarps = blockDim.x >> 5;
  for (int cc = threadIdx.x; cc < 2 * HD; cc += blockDim.x) {
    float s = 0.f;
    for (int wv = 0; wv < nwarps; ++wv) s += sm[wv][cc / HD][cc % HD];
    dw_part[static_cast<size_t>(blockIdx.x) * 2 * HD + cc] = s;
  }
}

__global__ void qk_dw_reduce_kernel(const float* __restrict__ part, int nblocks, int hd, float* __restrict__ dqw,
                                    float* __restrict__ dkw, int accumulate) {
  // block = 32 columns of the [nblocks, 2*hd] partials, 8 warps stride over the rows; fixed summation order
  __shared__ float sm[8][33];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + lane;
  float s = 0.f;
  if (c < 2 * hd)
    for (int b = warp; b < nblocks; b += 8) s += part[static_cast<size_t>(b) * 2 * hd + c];
  sm[warp][lane] = s;
  __syncthreads();
  if (warp == 0 && c < 2 * hd) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) t += sm[w][lane];
    float* out = c < hd ? dqw + c : dkw + (c - hd);
    *out = accumulate ? *out + t : t;
  }
}

}  // namespace b200

using namespace b200;

// `items` = number of tokens; one warp per token, eight warps per block
extern "C" int b200_qknorm_rope_blocks(long long items) {
  long long g = (items + 7) / 8;
  return static_cast<int>(g < 1 ? 1 : (g > 1184 ? 1184 : g));
}

extern "C" int b200_qknorm_rope_fwd(const void* qkv, int ld, const float* qw, const float* kw, const float* cs,
                                    void* q_out, void* k_out, void* v_out, float* rstd, int T, int S, int nh, int nkv,
                                    int hd, float eps, cudaStream_t stream) {
  if (T <= 0) return 0;
  const int grid = b200_qknorm_rope_blocks(T);
#define ARGS reinterpret_cast<const __nv_bfloat16*>(qkv), ld, qw, kw, cs, reinterpret_cast<__nv_bfloat16*>(q_out), \
             reinterpret_cast<__nv_bfloat16*>(k_out), reinterpret_cast<__nv_bfloat16*>(v_out), rstd, T, S, nh, nkv, eps
  if (hd == 128) qknorm_rope_fwd_kernel<4><<<grid, 256, 0, stream>>>(ARGS);
  else if (hd == 64) qknorm_rope_fwd_kernel<2><<<grid, 256, 0, stream>>>(ARGS);
  else if (hd == 32) qknorm_rope_fwd_kernel<1><<<grid, 256, 0, stream>>>(ARGS);
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
  if (hd == 128) qknorm_rope_bwd_kernel<4><<<grid, 256, 0, stream>>>(ARGS);
  else if (hd == 64) qknorm_rope_bwd_kernel<2><<<grid, 256, 0, stream>>>(ARGS);
  else if (hd == 32) qknorm_rope_bwd_kernel<1><<<grid, 256, 0, stream>>>(ARGS);
  else return -1;
#undef ARGS
  qk_dw_reduce_kernel<<<(2 * hd + 31) / 32, 256, 0, stream>>>(dw_part, grid, hd, dqw, dkw, dw_accumulate);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
