// Cross-entropy pieces around the vocabulary GEMM.
//   1. lse_loss: combine the per-(row, n-tile) (max, sum exp) partials written by the GEMM epilogue into
//      the row log-sum-exp, pick the label logit, and reduce the summed loss / valid-token count.
//   2. dlogits: turn the stored bf16 logits into d(loss)/d(logits) in place:
//      (softmax - onehot) * upstream / n_valid, rows with an ignored label become zero.
#include "../common/ptx.cuh"
#include "../ops_api.h"

namespace b200 {

// One warp per row: row log-sum-exp and row loss (0 for an ignored label).  No atomics: the sum over rows
// is taken afterwards in a fixed order by lce_reduce_kernel, so the loss has the same bits on every run.
__global__ void lse_loss_kernel(const float2* __restrict__ part, int n_tiles, const __nv_bfloat16* __restrict__ logits,
                                long long ld, const long long* __restrict__ labels, int ignore_index, int T, int V,
                                float* __restrict__ lse_out, float* __restrict__ row_loss) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * 8 + warp;
  if (row < T) {
    const float2* pr = part + static_cast<size_t>(row) * n_tiles;
    float mx = -INFINITY;
    for (int i = lane; i < n_tiles; i += 32) mx = fmaxf(mx, pr[i].x);
    mx = warp_max(mx);
    float sum = 0.f;
    for (int i = lane; i < n_tiles; i += 32) {
      const float2 p = pr[i];
      sum += p.y * __expf(p.x - mx);
    }
    sum = warp_sum(sum);
    const float lse = mx + __logf(sum);
    if (lane == 0) {
      lse_out[row] = lse;
      const long long lab = labels[row];
      float loss = 0.f;
      if (lab != ignore_index && lab >= 0 && lab < V)
        loss = lse - __bfloat162float(logits[static_cast<size_t>(row) * ld + lab]);
      row_loss[row] = loss;
    }
  }
}

// Single block, fixed order.  row_loss == null: acc[1] = number of rows with a valid label (needed before
// the first gradient tile can be scaled).  Otherwise acc[0] = sum of row losses, acc[2] = mean loss.
__global__ void lce_reduce_kernel(const float* __restrict__ row_loss, const long long* __restrict__ labels,
                                  int ignore_index, int T, int V, float* __restrict__ acc) {
  __shared__ float sh[32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float v = 0.f;
  for (int i = threadIdx.x; i < T; i += blockDim.x) {
    if (row_loss != nullptr) {
      v += row_loss[i];
    } else {
      const long long lab = labels[i];
      v += (lab != ignore_index && lab >= 0 && lab < V) ? 1.f : 0.f;
    }
  }
  v = warp_sum(v);
  if (lane == 0) sh[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < (blockDim.x >> 5) ? sh[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) {
      if (row_loss != nullptr) {
        acc[0] = t;
        acc[2] = t / fmaxf(acc[1], 1.f);
      } else {
        acc[1] = t;
      }
    }
  }
}

// In place over [T, V] bf16; 8 elements per thread step.  V must be a multiple of 8.
__global__ void dlogits_kernel(__nv_bfloat16* __restrict__ logits, long long ld, const float* __restrict__ lse,
                               const long long* __restrict__ labels, int ignore_index, int T, int V,
                               const float* __restrict__ loss_acc, float upstream) {
  const int vch = V >> 3;
  const long long total = static_cast<long long>(T) * vch;
  const float nvalid = loss_acc[1];
  const float sc = nvalid > 0.f ? upstream / nvalid : 0.f;
  constexpr float kLog2e = 1.4426950408889634f;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int row = static_cast<int>(i / vch);
    const int c = static_cast<int>(i - static_cast<long long>(row) * vch);
    uint4* p = reinterpret_cast<uint4*>(logits + static_cast<size_t>(row) * ld + c * 8);
    const long long lab = labels[row];
    if (lab == ignore_index || lab < 0 || lab >= V) {
      *p = make_uint4(0, 0, 0, 0);
      continue;
    }
    const float nl = -lse[row] * kLog2e;
    const uint4 q = *p;
    const uint32_t u[4] = {q.x, q.y, q.z, q.w};
    uint32_t o[4];
    const int col0 = c * 8;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = unpack_bf16x2(u[j]);
      float g0 = ex2_approx(fmaf(f.x, kLog2e, nl)), g1 = ex2_approx(fmaf(f.y, kLog2e, nl));
      if (col0 + 2 * j == lab) g0 -= 1.f;
      if (col0 + 2 * j + 1 == lab) g1 -= 1.f;
      o[j] = pack_bf16x2(g0 * sc, g1 * sc);
    }
    *p = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// ------------------------------------------------------------------ embedding
__global__ void embed_fwd_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ table, int T,
                                 int H, int V, __nv_bfloat16* __restrict__ out) {
  const int nch = H >> 3;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
  for (int t = blockIdx.x * wpb + warp; t < T; t += gridDim.x * wpb) {
    long long id = ids[t];
    if (id < 0 || id >= V) id = 0;
    const uint4* src = reinterpret_cast<const uint4*>(table + static_cast<size_t>(id) * H);
    uint4* dst = reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * H);
    for (int c = lane; c < nch; c += 32) dst[c] = src[c];
  }
}

// ---- embedding backward, deterministic: sort (id, position) keys, then one warp per run of equal ids
// adds that id's rows in position order.  No atomics, so the gradient has the same bits on every run.

// Single block bitonic sort of n <= capacity 64-bit keys in shared memory (capacity = power of two).
__global__ void embed_sort_kernel(const long long* __restrict__ ids, int T, int V, int capacity,
                                  unsigned long long* __restrict__ keys_out) {
  extern __shared__ unsigned long long keys[];
  for (int i = threadIdx.x; i < capacity; i += blockDim.x) {
    unsigned long long k = ~0ull;  // padding sorts last
    if (i < T) {
      const long long id = ids[i];
      if (id >= 0 && id < V) k = (static_cast<unsigned long long>(id) << 32) | static_cast<unsigned>(i);
    }
    keys[i] = k;
  }
  __syncthreads();
  for (int size = 2; size <= capacity; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      for (int i = threadIdx.x; i < capacity / 2; i += blockDim.x) {
        const int lo = 2 * i - (i & (stride - 1));
        const int hi = lo + stride;
        const bool up = (lo & size) == 0;
        const unsigned long long a = keys[lo], b = keys[hi];
        if ((a > b) == up) {
          keys[lo] = b;
          keys[hi] = a;
        }
      }
      __syncthreads();
    }
  }
  for (int i = threadIdx.x; i < T; i += blockDim.x) keys_out[i] = keys[i];
}

// keys sorted ascending, (id << 32 | position), invalid ids as ~0.  Warp w looks at sorted slot w; if a run
// of one id starts there it sums the run's rows in order and writes (or adds to) grad[id].
__global__ void embed_bwd_sorted_kernel(const unsigned long long* __restrict__ keys, const __nv_bfloat16* __restrict__ dout,
                                        int T, int H, float* __restrict__ grad, int accumulate) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
  const int nch = H >> 3;
  for (int i = blockIdx.x * wpb + warp; i < T; i += gridDim.x * wpb) {
    const unsigned long long k = keys[i];
    if (k == ~0ull) continue;
    const unsigned id = static_cast<unsigned>(k >> 32);
    if (i > 0 && static_cast<unsigned>(keys[i - 1] >> 32) == id) continue;  // not the start of a run
    float* dst = grad + static_cast<size_t>(id) * H;
    for (int c = lane; c < nch; c += 32) {
      float acc[8];
      if (accumulate) {
        const float4 a = *reinterpret_cast<const float4*>(dst + c * 8);
        const float4 b = *reinterpret_cast<const float4*>(dst + c * 8 + 4);
        acc[0] = a.x; acc[1] = a.y; acc[2] = a.z; acc[3] = a.w;
        acc[4] = b.x; acc[5] = b.y; acc[6] = b.z; acc[7] = b.w;
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.f;
      }
      for (int r = i; r < T; ++r) {
        const unsigned long long kr = keys[r];
        if (static_cast<unsigned>(kr >> 32) != id || kr == ~0ull) break;
        const unsigned t = static_cast<unsigned>(kr & 0xffffffffu);
        const uint4 q = *reinterpret_cast<const uint4*>(dout + static_cast<size_t>(t) * H + c * 8);
        const uint32_t u[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = unpack_bf16x2(u[j]);
          acc[2 * j] += f.x;
          acc[2 * j + 1] += f.y;
        }
      }
      *reinterpret_cast<float4*>(dst + c * 8) = make_float4(acc[0], acc[1], acc[2], acc[3]);
      *reinterpret_cast<float4*>(dst + c * 8 + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
    }
  }
}

}  // namespace b200

using namespace b200;

extern "C" int b200_lse_loss(const float* part, int n_tiles, const void* logits, long long ld, const long long* labels,
                             int ignore_index, int T, int V, float* lse, float* row_loss, cudaStream_t stream) {
  if (T <= 0) return 0;
  lse_loss_kernel<<<(T + 7) / 8, 256, 0, stream>>>(reinterpret_cast<const float2*>(part), n_tiles,
                                                   reinterpret_cast<const __nv_bfloat16*>(logits), ld, labels,
                                                   ignore_index, T, V, lse, row_loss);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int b200_lce_reduce(const float* row_loss, const long long* labels, int ignore_index, int T, int V,
                               float* acc, cudaStream_t stream) {
  if (T <= 0) return 0;
  lce_reduce_kernel<<<1, 1024, 0, stream>>>(row_loss, labels, ignore_index, T, V, acc);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int b200_dlogits(void* logits, long long ld, const float* lse, const long long* labels, int ignore_index,
                            int T, int V, const float* loss_acc, float upstream, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (V % 8 != 0) return -1;
  dlogits_kernel<<<148 * 16, 256, 0, stream>>>(reinterpret_cast<__nv_bfloat16*>(logits), ld, lse, labels,
                                               ignore_index, T, V, loss_acc, upstream);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int b200_embed_fwd(const long long* ids, const void* table, int T, int H, int V, void* out,
                              cudaStream_t stream) {
  if (T <= 0) return 0;
  if (H % 8 != 0) return -1;
  int grid = (T + 7) / 8;
  if (grid > 1184) grid = 1184;
  embed_fwd_kernel<<<grid, 256, 0, stream>>>(ids, reinterpret_cast<const __nv_bfloat16*>(table), T, H, V,
                                             reinterpret_cast<__nv_bfloat16*>(out));
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// Largest token count the single-block sort handles (64-bit keys in shared memory).
extern "C" int b200_embed_sort_capacity() { return 16384; }

// Sort the (id, position) keys of `ids` into keys[T] (at most b200_embed_sort_capacity() tokens).  The ids are
// known when the forward pass starts, so a caller can run this early, beside other work.
extern "C" int b200_embed_sort(const long long* ids, int T, int V, unsigned long long* keys, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (T > b200_embed_sort_capacity() || keys == nullptr) return -3;
  int cap = 1;
  while (cap < T) cap <<= 1;
  const size_t smem = static_cast<size_t>(cap) * sizeof(unsigned long long);
  if (smem > 48 * 1024) {
    static bool raised = false;
    if (!raised) {
      if (cudaFuncSetAttribute(embed_sort_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 128 * 1024) !=
          cudaSuccess)
        return -4;
      raised = true;
    }
  }
  embed_sort_kernel<<<1, 1024, smem, stream>>>(ids, T, V, cap, keys);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// keys: uint64[T] scratch.  The caller zeroes `grad` first unless `accumulate`; rows of ids that do not
// occur are left as they are.
extern "C" int b200_embed_bwd(const long long* ids, const void* dout, int T, int H, int V, float* grad,
                              unsigned long long* keys, int presorted, int accumulate, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (H % 8 != 0 || keys == nullptr) return -1;
  if (!presorted) {
    const int rc = b200_embed_sort(ids, T, V, keys, stream);
    if (rc) return rc;
  }
  int grid = (T + 7) / 8;
  if (grid > 2368) grid = 2368;
  embed_bwd_sorted_kernel<<<grid, 256, 0, stream>>>(keys, reinterpret_cast<const __nv_bfloat16*>(dout), T, H, grad,
                                                    accumulate);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
