// Flat-buffer optimiser kernels: squared-norm reduction, clip coefficient, fused AdamW that also
// refreshes the bf16 compute copy of the parameters, and an fp32 -> bf16 cast.
#include "../common/ptx.cuh"
#include "../ops_api.h"
#include <cmath>

namespace b200 {

constexpr int RED_THREADS = 256;

struct AdamPeers {
  __nv_bfloat16* p16[8];  // same slice of the bf16 compute copy on every rank (null entries unused)
};

// partial[b] = sum over this block's grid-stride slice of g^2
__global__ void sumsq_partial_kernel(const float* __restrict__ g, long long n, float* __restrict__ partial) {
  __shared__ float sh[RED_THREADS / 32];
  float acc = 0.f;
  const long long n4 = n >> 2;
  const float4* g4 = reinterpret_cast<const float4*>(g);
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float4 v = g4[i];
    acc += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  if (blockIdx.x == 0 && threadIdx.x < (n & 3)) {
    const float v = g[(n4 << 2) + threadIdx.x];
    acc += v * v;
  }
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < RED_THREADS / 32; ++i) s += sh[i];
    partial[blockIdx.x] = s;
  }
}

// out[0] (+)= sum(partial) in a fixed order
__global__ void sumsq_final_kernel(const float* __restrict__ partial, int nb, float* __restrict__ out, int accumulate) {
  __shared__ float sh[RED_THREADS];
  float acc = 0.f;
  for (int i = threadIdx.x; i < nb; i += RED_THREADS) acc += partial[i];
  sh[threadIdx.x] = acc;
  __syncthreads();
  for (int s = RED_THREADS / 2; s > 0; s >>= 1) {
    if (threadIdx.x < s) sh[threadIdx.x] += sh[threadIdx.x + s];
    __syncthreads();
  }
  if (threadIdx.x == 0) out[0] = accumulate ? out[0] + sh[0] : sh[0];
}

// coef[0] = min(1, max_norm / (sqrt(sumsq) + 1e-6)), coef[1] = sqrt(sumsq)
__global__ void clip_coef_kernel(const float* __restrict__ sumsq, float max_norm, float* __restrict__ coef) {
  const float norm = sqrtf(sumsq[0]);
  float c = 1.f;
  if (max_norm > 0.f) c = fminf(1.f, max_norm / (norm + 1e-6f));
  coef[0] = c;
  coef[1] = norm;
}

// AdamW with decoupled weight decay over a flat slice; gradients are scaled by *grad_coef (clip).
__global__ void adamw_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m,
                             float* __restrict__ v, __nv_bfloat16* __restrict__ p16, long long n,
                             const float* __restrict__ hyper, float beta1, float beta2, float eps, float wd,
                             const float* __restrict__ grad_coef, AdamPeers peers, int world,
                             __nv_bfloat16* p16_mc) {
  // hyper = {learning rate, 1 - beta1^t, 1 - beta2^t}: device-resident so that a captured CUDA graph
  // can be replayed with new values
  const float lr = hyper[0], bc1 = hyper[1], bc2 = hyper[2];
  const float gc = grad_coef ? grad_coef[0] : 1.f;
  const float rs_bc2 = rsqrtf(bc2);
  const float step = lr / bc1;
  const long long n4 = n >> 2;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float4 pv = reinterpret_cast<float4*>(p)[i];
    const float4 gv = reinterpret_cast<const float4*>(g)[i];
    float4 mv = reinterpret_cast<float4*>(m)[i];
    float4 vv = reinterpret_cast<float4*>(v)[i];
    float* pp = &pv.x;
    const float* gg = &gv.x;
    float* mm = &mv.x;
    float* vw = &vv.x;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float gr = gg[j] * gc;
      pp[j] *= 1.f - lr * wd;
      mm[j] = beta1 * mm[j] + (1.f - beta1) * gr;
      vw[j] = beta2 * vw[j] + (1.f - beta2) * gr * gr;
      pp[j] -= step * mm[j] / (sqrtf(vw[j]) * rs_bc2 + eps);
    }
    reinterpret_cast<float4*>(p)[i] = pv;
    reinterpret_cast<float4*>(m)[i] = mv;
    reinterpret_cast<float4*>(v)[i] = vv;
    const uint2 packed = make_uint2(pack_bf16x2(pv.x, pv.y), pack_bf16x2(pv.z, pv.w));
    if (p16) reinterpret_cast<uint2*>(p16)[i] = packed;
    // sharded optimizer: the owner of this slice publishes the new bf16 weights to every rank: one multicast
    // store that the NVSwitch fans out to all ranks (own copy included), or `world` peer stores
    if (p16_mc != nullptr) {
      asm volatile("multimem.st.relaxed.sys.global.v2.f32 [%0], {%1, %2};" ::"l"(reinterpret_cast<uint2*>(p16_mc) + i),
                   "f"(__uint_as_float(packed.x)), "f"(__uint_as_float(packed.y))
                   : "memory");
    } else {
      for (int r = 0; r < world; ++r) reinterpret_cast<uint2*>(peers.p16[r])[i] = packed;
    }
  }
  if (world > 0) __threadfence_system();
  // tail (n not a multiple of 4)
  if (blockIdx.x == 0 && threadIdx.x < (n & 3)) {
    const long long i = (n4 << 2) + threadIdx.x;
    const float gr = g[i] * gc;
    float pv = p[i] * (1.f - lr * wd);
    const float mv = beta1 * m[i] + (1.f - beta1) * gr;
    const float vv = beta2 * v[i] + (1.f - beta2) * gr * gr;
    pv -= step * mv / (sqrtf(vv) * rs_bc2 + eps);
    p[i] = pv;
    m[i] = mv;
    v[i] = vv;
    if (p16) p16[i] = __float2bfloat16(pv);
  }
}

__global__ void cast_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, long long n) {
  const long long n4 = n >> 2;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float4 v = reinterpret_cast<const float4*>(src)[i];
    reinterpret_cast<uint2*>(dst)[i] = make_uint2(pack_bf16x2(v.x, v.y), pack_bf16x2(v.z, v.w));
  }
  if (blockIdx.x == 0 && threadIdx.x < (n & 3)) {
    const long long i = (n4 << 2) + threadIdx.x;
    dst[i] = __float2bfloat16(src[i]);
  }
}

}  // namespace b200

using namespace b200;

extern "C" int b200_sumsq_blocks(long long n) {
  long long b = (n / 4 + RED_THREADS - 1) / RED_THREADS;
  return static_cast<int>(b < 1 ? 1 : (b > 1184 ? 1184 : b));
}

// scratch: float[b200_sumsq_blocks(n)]
extern "C" int b200_sumsq(const float* g, long long n, float* scratch, float* out, int accumulate,
                          cudaStream_t stream) {
  if (n <= 0) return 0;
  if ((reinterpret_cast<uintptr_t>(g) & 15u) != 0) return -1;
  const int nb = b200_sumsq_blocks(n);
  sumsq_partial_kernel<<<nb, RED_THREADS, 0, stream>>>(g, n, scratch);
  sumsq_final_kernel<<<1, RED_THREADS, 0, stream>>>(scratch, nb, out, accumulate);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int b200_clip_coef(const float* sumsq, float max_norm, float* coef, cudaStream_t stream) {
  clip_coef_kernel<<<1, 1, 0, stream>>>(sumsq, max_norm, coef);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int b200_adamw(float* p, const float* g, float* m, float* v, void* p16, long long n, const float* hyper,
                          float beta1, float beta2, float eps, float wd, const float* grad_coef, void* const* p16_peers,
                          int world, void* p16_mc, cudaStream_t stream) {
  if (n <= 0) return 0;
  AdamPeers peers;
  for (int r = 0; r < 8; ++r) peers.p16[r] = (p16_peers && r < world) ? reinterpret_cast<__nv_bfloat16*>(p16_peers[r]) : nullptr;
  if (p16_peers == nullptr) world = 0;
  if (world == 0) p16_mc = nullptr;
  if (world > 0 && (n & 3) != 0) return -1;  // published slices are whole float4 groups
  if (p16_mc != nullptr && (reinterpret_cast<uintptr_t>(p16_mc) & 7) != 0) return -3;
  long long b = (n / 4 + 255) / 256;
  const int grid = static_cast<int>(b < 1 ? 1 : (b > 148 * 16 ? 148 * 16 : b));
  adamw_kernel<<<grid, 256, 0, stream>>>(p, g, m, v, reinterpret_cast<__nv_bfloat16*>(p16), n, hyper, beta1, beta2,
                                         eps, wd, grad_coef, peers, world, reinterpret_cast<__nv_bfloat16*>(p16_mc));
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int b200_cast_bf16(const float* src, void* dst, long long n, cudaStream_t stream) {
  if (n <= 0) return 0;
  long long b = (n / 4 + 255) / 256;
  const int grid = static_cast<int>(b < 1 ? 1 : (b > 148 * 16 ? 148 * 16 : b));
  cast_bf16_kernel<<<grid, 256, 0, stream>>>(src, reinterpret_cast<__nv_bfloat16*>(dst), n);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
