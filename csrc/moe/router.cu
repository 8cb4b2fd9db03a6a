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

// mode 0: softmax, mode 1: sigmoid.  bias (may be null) only steers selection.
__global__ void router_fwd_kernel(const float* __restrict__ logits, const float* __restrict__ bias,
                                  float* __restrict__ scores, float* __restrict__ topk_w, int* __restrict__ topk_idx,
                                  int T, int E, int K, int mode, int norm, float scale, int num_groups,
                                  int group_topk) {
  extern __shared__ float sm[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* buf = sm + static_cast<size_t>(warp) * (E + 32);
  float* gsc = buf + E;  // group scores
  for (int t = blockIdx.x * ROUTER_WARPS + warp; t < T; t += gridDim.x * ROUTER_WARPS) {
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
    for (int k = 0; k < K; ++k) {
      const ArgMax a = row_argmax(buf, 0, E, lane);
      const float un = sr[a.i];  // unbiased score (written above by this warp)
      wsum += un;
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
    __syncwarp();
  }
}

// d(logits) in bf16 from d(scores) (may be null) and d(topk weights).
__global__ void router_bwd_kernel(const float* __restrict__ dscores, const float* __restrict__ dtopk_w,
                                  const float* __restrict__ scores, const int* __restrict__ topk_idx,
                                  __nv_bfloat16* __restrict__ dlogits, int T, int E, int K, int mode, int norm,
                                  float scale) {
  extern __shared__ float sm[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* buf = sm + static_cast<size_t>(warp) * E;
  for (int t = blockIdx.x * ROUTER_WARPS + warp; t < T; t += gridDim.x * ROUTER_WARPS) {
    const float* sr = scores + static_cast<size_t>(t) * E;
    for (int e = lane; e < E; e += 32) buf[e] = dscores ? dscores[static_cast<size_t>(t) * E + e] : 0.f;
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

static int router_grid(int T) {
  int g = (T + ROUTER_WARPS - 1) / ROUTER_WARPS;
  return g < 1 ? 1 : (g > 1184 ? 1184 : g);
}

extern "C" int b200_router_fwd(const float* logits, const float* bias, float* scores, float* topk_w, int* topk_idx,
                               int T, int E, int K, int mode, int norm, float scale, int num_groups, int group_topk,
                               cudaStream_t stream) {
  if (T <= 0) return 0;
  if (K > 32 || K > E || num_groups > 32) return -1;
  if (num_groups > 1 && (E % num_groups != 0 || group_topk <= 0 || K % group_topk != 0 || K / group_topk > 8))
    return -1;
  const size_t smem = static_cast<size_t>(ROUTER_WARPS) * (E + 32) * sizeof(float);
  if (smem > 48 * 1024) {
    if (smem > 200 * 1024) return -1;
    cudaFuncSetAttribute(router_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  }
  router_fwd_kernel<<<router_grid(T), ROUTER_WARPS * 32, smem, stream>>>(logits, bias, scores, topk_w, topk_idx, T,
                                                                         E, K, mode, norm, scale, num_groups,
                                                                         group_topk);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int b200_router_bwd(const float* dscores, const float* dtopk_w, const float* scores, const int* topk_idx,
                               void* dlogits, int T, int E, int K, int mode, int norm, float scale,
                               cudaStream_t stream) {
  if (T <= 0) return 0;
  if (K > 32) return -1;
  const size_t smem = static_cast<size_t>(ROUTER_WARPS) * E * sizeof(float);
  if (smem > 48 * 1024) {
    if (smem > 200 * 1024) return -1;
    cudaFuncSetAttribute(router_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  }
  router_bwd_kernel<<<router_grid(T), ROUTER_WARPS * 32, smem, stream>>>(
      dscores, dtopk_w, scores, topk_idx, reinterpret_cast<__nv_bfloat16*>(dlogits), T, E, K, mode, norm, scale);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
