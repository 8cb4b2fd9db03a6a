// RMSNorm forward (optionally fused with the residual add that precedes it) and backward.
// One warp per row; each lane owns 8-element (16-byte) column chunks lane, lane+32, ...
// Memory-bound: x is read once from DRAM (the second pass hits L1/L2), y written once.
#include "../common/ptx.cuh"
#include "../ops_api.h"

namespace b200 {

constexpr int NORM_WARPS = 4;

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&f)[8]) {
  const uint4 q = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = unpack_bf16x2(w[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&f)[8]) {
  *reinterpret_cast<uint4*>(p) = make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]),
                                            pack_bf16x2(f[4], f[5]), pack_bf16x2(f[6], f[7]));
}

// y = w * bf16(h * rstd),  h = x (+ res).  When res != null the sum is also written to h_out.
__global__ void rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                                   const float* __restrict__ w, __nv_bfloat16* __restrict__ h_out,
                                   __nv_bfloat16* __restrict__ y, float* __restrict__ rstd_out, int T, int H,
                                   float eps) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * NORM_WARPS + warp;
  if (row >= T) return;
  const __nv_bfloat16* xr = x + static_cast<size_t>(row) * H;
  const __nv_bfloat16* rr = res ? res + static_cast<size_t>(row) * H : nullptr;
  __nv_bfloat16* hr = h_out ? h_out + static_cast<size_t>(row) * H : nullptr;
  const int nch = H >> 3;
  float ss = 0.f;
  for (int c = lane; c < nch; c += 32) {
    float f[8];
    load8(xr + c * 8, f);
    if (rr) {
      float g[8];
      load8(rr + c * 8, g);
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] += g[i];
      // the residual stream is stored in bf16: normalise exactly what later layers will read
      uint4 packed = make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]),
                                pack_bf16x2(f[6], f[7]));
      *reinterpret_cast<uint4*>(hr + c * 8) = packed;
      const uint32_t pw[4] = {packed.x, packed.y, packed.z, packed.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 t = unpack_bf16x2(pw[i]);
        f[2 * i] = t.x;
        f[2 * i + 1] = t.y;
      }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) ss += f[i] * f[i];
  }
  ss = warp_sum(ss);
  const float rstd = rsqrtf(ss / static_cast<float>(H) + eps);
  if (lane == 0 && rstd_out) rstd_out[row] = rstd;
  const __nv_bfloat16* src = rr ? hr : xr;
  __nv_bfloat16* yr = y + static_cast<size_t>(row) * H;
  for (int c = lane; c < nch; c += 32) {
    float f[8];
    load8(src + c * 8, f);
    const float4 w0 = *reinterpret_cast<const float4*>(w + c * 8);
    const float4 w1 = *reinterpret_cast<const float4*>(w + c * 8 + 4);
    const float wv[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = wv[i] * __bfloat162float(__float2bfloat16(f[i] * rstd));
    store8(yr + c * 8, f);
  }
}

// dx = rstd * (w*dy - xhat * mean(w*dy*xhat)) (+ dres);  dw partials per block in `dw_part[grid, H]`.
template <int MAXCH>
__global__ void rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                                   const float* __restrict__ rstd, const float* __restrict__ w,
                                   const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx,
                                   float* __restrict__ dw_part, int T, int H) {
  extern __shared__ float sm_dw[];  // [NORM_WARPS][H]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nch = H >> 3;
  float dwacc[MAXCH][8];
#pragma unroll
  for (int i = 0; i < MAXCH; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) dwacc[i][j] = 0.f;

  for (int row = blockIdx.x * NORM_WARPS + warp; row < T; row += gridDim.x * NORM_WARPS) {
    const size_t off = static_cast<size_t>(row) * H;
    const float rs = rstd[row];
    float wdy[MAXCH][8], xh[MAXCH][8];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < MAXCH; ++i) {
      const int c = lane + 32 * i;
      if (c < nch) {
        float a[8], b[8];
        load8(dy + off + c * 8, a);
        load8(x + off + c * 8, b);
        const float4 w0 = *reinterpret_cast<const float4*>(w + c * 8);
        const float4 w1 = *reinterpret_cast<const float4*>(w + c * 8 + 4);
        const float wv[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xh[i][j] = b[j] * rs;
          dwacc[i][j] += a[j] * xh[i][j];
          wdy[i][j] = a[j] * wv[j];
          dot += wdy[i][j] * xh[i][j];
        }
      }
    }
    dot = warp_sum(dot) / static_cast<float>(H);
#pragma unroll
    for (int i = 0; i < MAXCH; ++i) {
      const int c = lane + 32 * i;
      if (c < nch) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = rs * (wdy[i][j] - xh[i][j] * dot);
        if (dres) {
          float r[8];
          load8(dres + off + c * 8, r);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += r[j];
        }
        store8(dx + off + c * 8, o);
      }
    }
  }
  // block partial of dw: warps -> shared -> one row of dw_part
#pragma unroll
  for (int i = 0; i < MAXCH; ++i) {
    const int c = lane + 32 * i;
    if (c < nch)
#pragma unroll
      for (int j = 0; j < 8; ++j) sm_dw[warp * H + c * 8 + j] = dwacc[i][j];
  }
  __syncthreads();
  for (int col = threadIdx.x; col < H; col += blockDim.x) {
    float s = 0.f;
#pragma unroll
    for (int wv = 0; wv < NORM_WARPS; ++wv) s += sm_dw[wv * H + col];
    dw_part[static_cast<size_t>(blockIdx.x) * H + col] = s;
  }
}

// out[col] (+)= sum_b part[b, col]   (fixed order: deterministic).  Block = 32 columns x 8 row-strided warps.
__global__ void colsum_kernel(const float* __restrict__ part, float* __restrict__ out, int nblocks, int H,
                              int accumulate) {
  __shared__ float sm[8][33];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int col = blockIdx.x * 32 + lane;
  float s = 0.f;
  if (col < H)
    for (int b = warp; b < nblocks; b += 8) s += part[static_cast<size_t>(b) * H + col];
  sm[warp][lane] = s;
  __syncthreads();
  if (warp == 0 && col < H) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) t += sm[w][lane];
    out[col] = accumulate ? out[col] + t : t;
  }
}

}  // namespace b200

using namespace b200;

extern "C" int b200_sum_partials(const float* part, float* out, int nparts, int n, int accumulate, cudaStream_t stream) {
  if (nparts <= 0 || n <= 0) return -1;
  colsum_kernel<<<(n + 31) / 32, 256, 0, stream>>>(part, out, nparts, n, accumulate);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int b200_rmsnorm_fwd(const void* x, const void* res, const float* w, void* h_out, void* y, float* rstd,
                                int T, int H, float eps, cudaStream_t stream) {
  if (H % 8 != 0 || T <= 0) return T == 0 ? 0 : -1;
  const int grid = (T + NORM_WARPS - 1) / NORM_WARPS;
  rmsnorm_fwd_kernel<<<grid, NORM_WARPS * 32, 0, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<const __nv_bfloat16*>(res), w,
      reinterpret_cast<__nv_bfloat16*>(h_out), reinterpret_cast<__nv_bfloat16*>(y), rstd, T, H, eps);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int b200_rmsnorm_bwd_blocks(int T) {
  int g = (T + NORM_WARPS - 1) / NORM_WARPS;
  return g < 592 ? (g < 1 ? 1 : g) : 592;  // 148 SMs x 4 resident blocks
}

extern "C" int b200_rmsnorm_bwd(const void* dy, const void* x, const float* rstd, const float* w, const void* dres,
                                void* dx, float* dw_part, float* dw_out, int dw_accumulate, int T, int H,
                                cudaStream_t stream) {
  if (H % 8 != 0 || H > 4096) return -1;
  if (T <= 0) return 0;
  const int grid = b200_rmsnorm_bwd_blocks(T);
  const size_t smem = static_cast<size_t>(NORM_WARPS) * H * sizeof(float);
  const int nch32 = (H / 8 + 31) / 32;
#define LAUNCH(MC)                                                                                               \
  rmsnorm_bwd_kernel<MC><<<grid, NORM_WARPS * 32, smem, stream>>>(                                               \
      reinterpret_cast<const __nv_bfloat16*>(dy), reinterpret_cast<const __nv_bfloat16*>(x), rstd, w,            \
      reinterpret_cast<const __nv_bfloat16*>(dres), reinterpret_cast<__nv_bfloat16*>(dx), dw_part, T, H)
  if (smem > 48 * 1024) {
    cudaFuncSetAttribute(rmsnorm_bwd_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
  }
  if (nch32 <= 1) LAUNCH(1);
  else if (nch32 <= 2) LAUNCH(2);
  else if (nch32 <= 4) LAUNCH(4);
  else if (nch32 <= 8) LAUNCH(8);
  else LAUNCH(16);
#undef LAUNCH
  colsum_kernel<<<(H + 31) / 32, 256, 0, stream>>>(dw_part, dw_out, grid, H, dw_accumulate);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// --------------------------------------------------------------------------------------------
// Allocation-free variant of the backward pass (declared and documented in rmsnorm_noalloc.h).
// The per-block partial sums live in a file-scope device array instead of caller memory.
#include "rmsnorm_noalloc.h"

#include <atomic>

namespace b200 {
static __device__ __align__(256) float g_noalloc_dw_scratch[B200_NOALLOC_MAX_BLOCKS * B200_NOALLOC_MAX_H];
}

// In host code the array's name is only a handle: the device address has to be asked for, once per
// device and with that device current.
// Host threads may make the first call on a device at the same time: the per-device slots are atomics
// (every thread that looks the address up stores the same value).
static float* noalloc_scratch_for_current_device() {
  constexpr int kMaxDevices = 64;
  static std::atomic<float*> cache[kMaxDevices];
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  float* p = cache[dev].load(std::memory_order_acquire);
  if (p == nullptr) {
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), b200::g_noalloc_dw_scratch) != cudaSuccess) {
      (void)cudaGetLastError();
      return nullptr;
    }
    cache[dev].store(p, std::memory_order_release);
  }
  return p;
}

extern "C" int b200_rmsnorm_bwd_noalloc(const void* dy, const void* x, const float* rstd, const float* w,
                                        const void* dres, void* dx, float* dw_out, int dw_accumulate, int T, int H,
                                        cudaStream_t stream) {
  if (T < 0 || H <= 0 || H % 8 != 0 || H > B200_NOALLOC_MAX_H) return B200_NOALLOC_ERR_SIZE;
  if (T == 0) return B200_NOALLOC_OK;
  if (!dy || !x || !rstd || !w || !dx || !dw_out) return B200_NOALLOC_ERR_ARG;
  // an error left behind by an earlier, unrelated call must not be reported as a failed launch of ours
  if (cudaPeekAtLastError() != cudaSuccess) return B200_NOALLOC_ERR_PRIOR;
  float* scratch = noalloc_scratch_for_current_device();
  if (scratch == nullptr) return B200_NOALLOC_ERR_SETUP;
  const int grid = b200_rmsnorm_bwd_blocks(T);  // <= B200_NOALLOC_MAX_BLOCKS; rows [0, grid) are rewritten below
  const size_t smem = static_cast<size_t>(NORM_WARPS) * H * sizeof(float);  // <= 32 KiB for H <= 2048
  const int nch32 = (H / 8 + 31) / 32;
#define LAUNCH(MC)                                                                                               \
  rmsnorm_bwd_kernel<MC><<<grid, NORM_WARPS * 32, smem, stream>>>(                                               \
      reinterpret_cast<const __nv_bfloat16*>(dy), reinterpret_cast<const __nv_bfloat16*>(x), rstd, w,            \
      reinterpret_cast<const __nv_bfloat16*>(dres), reinterpret_cast<__nv_bfloat16*>(dx), scratch, T, H)
  if (nch32 <= 1) LAUNCH(1);
  else if (nch32 <= 2) LAUNCH(2);
  else if (nch32 <= 4) LAUNCH(4);
  else LAUNCH(8);
#undef LAUNCH
  colsum_kernel<<<(H + 31) / 32, 256, 0, stream>>>(scratch, dw_out, grid, H, dw_accumulate);
  return cudaGetLastError() == cudaSuccess ? B200_NOALLOC_OK : B200_NOALLOC_ERR_LAUNCH;
}

extern "C" const char* b200_rmsnorm_bwd_noalloc_strerror(int code) {
  switch (code) {
    case B200_NOALLOC_OK: return "ok";
    case B200_NOALLOC_ERR_SIZE:
      return "size not supported: H must be a positive multiple of 8 and at most 2048 (B200_NOALLOC_MAX_H), T >= 0";
    case B200_NOALLOC_ERR_SETUP: return "could not obtain the device address of the built-in scratch array";
    case B200_NOALLOC_ERR_LAUNCH: return "a kernel launch was refused by the CUDA runtime";
    case B200_NOALLOC_ERR_ARG: return "a required pointer argument is null";
    case B200_NOALLOC_ERR_PRIOR:
      return "a CUDA error from an earlier call is pending on this thread; nothing was enqueued";
    default: return "unknown code";
  }
}
