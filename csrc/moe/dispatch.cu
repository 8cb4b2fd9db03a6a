// Token dispatch plan for the grouped expert GEMMs, and the row movers around them.
//
// The (token, slot) -> expert assignment is turned into an expert-sorted row layout in which every
// expert's segment is padded to a multiple of 128 rows, so that a 128-row GEMM tile never straddles
// two experts.  The sort is a deterministic counting sort (stable in token order): block histograms,
// a scan, and a ranked scatter - no atomics on the ordering path, no host synchronisation.
#include "../common/ptx.cuh"
#include "../ops_api.h"

namespace b200 {

constexpr int PLAN_CHUNK = 512;  // assignments per block

// block_hist[b][e] = number of assignments to expert e among entries [b*CHUNK, (b+1)*CHUNK)
__global__ void plan_hist_kernel(const int* __restrict__ idx, int n, int E, int* __restrict__ block_hist) {
  extern __shared__ int sh[];
  for (int e = threadIdx.x; e < E; e += blockDim.x) sh[e] = 0;
  __syncthreads();
  const int base = blockIdx.x * PLAN_CHUNK;
  for (int i = threadIdx.x; i < PLAN_CHUNK; i += blockDim.x) {
    const int g = base + i;
    if (g < n) {
      const int e = idx[g];
      if (e >= 0 && e < E) atomicAdd(&sh[e], 1);
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) block_hist[static_cast<size_t>(blockIdx.x) * E + e] = sh[e];
}

// Single block: per-expert exclusive scan over blocks (in place), counts, padded segment offsets,
// tile -> expert map and live tile count; and the same rows as a list of pair tiles (two consecutive
// 128-row tiles of ONE expert, or a single last tile) for the pair-tile GEMM kernel.
// The scan over experts is a block-wide scan (contiguous experts per thread, shuffles across threads).
__global__ void plan_scan_kernel(int* __restrict__ block_hist, int nblocks, int E, int* __restrict__ counts,
                                 int* __restrict__ seg_off, int* __restrict__ tile_expert, int max_tiles,
                                 int* __restrict__ num_m_tiles, int* __restrict__ pair_tiles, int max_pairs,
                                 int* __restrict__ num_pair_tiles) {
  extern __shared__ int sh[];  // [E] padded sizes, then [E + 1] row offsets, then [E + 1] pair offsets
  int* rows_off = sh + E;
  int* pair_off = rows_off + E + 1;
  __shared__ int wr[32], wp[32];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
  // exclusive scan over the chunk histograms, one warp per expert, 32 chunks per shuffle scan
  for (int e = warp; e < E; e += nwarps) {
    int run = 0;
    for (int b0 = 0; b0 < nblocks; b0 += 32) {
      const int b = b0 + lane;
      const size_t o = static_cast<size_t>(b) * E + e;
      const int c = b < nblocks ? block_hist[o] : 0;
      int inc = c;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int x = __shfl_up_sync(0xffffffffu, inc, d);
        if (lane >= d) inc += x;
      }
      if (b < nblocks) block_hist[o] = run + inc - c;
      run += __shfl_sync(0xffffffffu, inc, 31);
    }
    if (lane == 0) {
      counts[e] = run;
      sh[e] = (run + 127) / 128 * 128;
    }
  }
  __syncthreads();
  const int per = (E + blockDim.x - 1) / blockDim.x;
  const int lo = tid * per < E ? tid * per : E;
  const int hi = lo + per < E ? lo + per : E;
  int r_sum = 0, p_sum = 0;
  for (int e = lo; e < hi; ++e) {
    r_sum += sh[e];
    p_sum += (sh[e] / 128 + 1) / 2;
  }
  int r_inc = r_sum, p_inc = p_sum;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int a = __shfl_up_sync(0xffffffffu, r_inc, o), b = __shfl_up_sync(0xffffffffu, p_inc, o);
    if (lane >= o) {
      r_inc += a;
      p_inc += b;
    }
  }
  if (lane == 31) {
    wr[warp] = r_inc;
    wp[warp] = p_inc;
  }
  __syncthreads();
  if (warp == 0) {
    int a = lane < nwarps ? wr[lane] : 0, b = lane < nwarps ? wp[lane] : 0;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int x = __shfl_up_sync(0xffffffffu, a, o), y = __shfl_up_sync(0xffffffffu, b, o);
      if (lane >= o) {
        a += x;
        b += y;
      }
    }
    wr[lane] = a;  // inclusive over warps
    wp[lane] = b;
  }
  __syncthreads();
  int r_run = r_inc - r_sum + (warp > 0 ? wr[warp - 1] : 0);
  int p_run = p_inc - p_sum + (warp > 0 ? wp[warp - 1] : 0);
  for (int e = lo; e < hi; ++e) {
    rows_off[e] = r_run;
    pair_off[e] = p_run;
    seg_off[e] = r_run;
    r_run += sh[e];
    p_run += (sh[e] / 128 + 1) / 2;
  }
  if (tid == blockDim.x - 1) {  // the last thread's running totals are the grand totals
    rows_off[E] = r_run;
    pair_off[E] = p_run;
    seg_off[E] = r_run;
    int nt = r_run / 128;
    *num_m_tiles = nt > max_tiles ? max_tiles : nt;
    if (num_pair_tiles != nullptr) *num_pair_tiles = p_run > max_pairs ? max_pairs : p_run;
  }
  __syncthreads();
  for (int e = warp; e < E; e += nwarps) {
    const int t0 = rows_off[e] / 128, t1 = rows_off[e + 1] / 128;
    for (int t = t0 + lane; t < t1 && t < max_tiles; t += 32) tile_expert[t] = e;
    if (pair_tiles != nullptr) {
      const int p0 = pair_off[e], np = pair_off[e + 1] - p0, n128 = t1 - t0;
      for (int i = lane; i < np; i += 32) {
        if (p0 + i < max_pairs) {
          const int halves = (2 * i + 2 <= n128) ? 2 : 1;
          pair_tiles[2 * (p0 + i)] = (t0 + 2 * i) * 128;
          pair_tiles[2 * (p0 + i) + 1] = e | (halves << 16);
        }
      }
    }
  }
}

// One warp per chunk walks its entries in order; rank within (chunk, expert) from match/popc.
__global__ void plan_scatter_kernel(const int* __restrict__ idx, int n, int E, const int* __restrict__ block_off,
                                    const int* __restrict__ seg_off, int* __restrict__ pos,
                                    int* __restrict__ row_slot, int capacity, int* __restrict__ row_tok, int K) {
  extern __shared__ int cnt[];  // [E] running count inside this chunk
  const int lane = threadIdx.x;
  for (int e = lane; e < E; e += 32) cnt[e] = 0;
  __syncwarp();
  const int base = blockIdx.x * PLAN_CHUNK;
  for (int i = 0; i < PLAN_CHUNK; i += 32) {
    const int g = base + i + lane;
    int e = -1;
    if (g < n) {
      e = idx[g];
      if (e < 0 || e >= E) e = -1;
    }
    const unsigned peers = __match_any_sync(0xffffffffu, e);
    const int rank = __popc(peers & ((1u << lane) - 1u));
    int start = 0;
    if (e >= 0) start = cnt[e];
    __syncwarp();
    if (e >= 0 && rank == 0) cnt[e] = start + __popc(peers);
    __syncwarp();
    if (e >= 0) {
      const int p = seg_off[e] + block_off[static_cast<size_t>(blockIdx.x) * E + e] + start + rank;
      if (p < capacity) {
        pos[g] = p;
        row_slot[p] = g;
        if (row_tok != nullptr) row_tok[p] = g / K;
      } else {
        pos[g] = -1;
      }
    } else if (g < n) {
      pos[g] = -1;
    }
  }
}

// xs[r] = x[row_slot[r] / K] for live rows, 0 for padding rows; rows past the live region untouched.
__global__ void moe_gather_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ row_slot,
                                  const int* __restrict__ seg_off, int E, int K, int H,
                                  __nv_bfloat16* __restrict__ xs, int capacity) {
  int live = seg_off[E];
  if (live > capacity) live = capacity;
  const int nch = H >> 3;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
  for (int r = blockIdx.x * wpb + warp; r < live; r += gridDim.x * wpb) {
    const int s = row_slot[r];
    uint4* dst = reinterpret_cast<uint4*>(xs + static_cast<size_t>(r) * H);
    if (s >= 0) {
      const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<size_t>(s / K) * H);
      for (int c = lane; c < nch; c += 32) dst[c] = src[c];
    } else {
      for (int c = lane; c < nch; c += 32) dst[c] = make_uint4(0, 0, 0, 0);
    }
  }
}

// out[t] = sum_k w[t,k] * ys[pos[t,k]] (+ res[t]);  w == null -> plain sum.  Fixed k order.
// pos == null: slot (t, k) reads row t*K + k.  wait_flags != null: rows of `ys` are being stored by
// peer GPUs; every block first waits (bounded) until all `wait_n` flag words reach the epoch.
__global__ void moe_combine_kernel(const __nv_bfloat16* __restrict__ ys, const int* __restrict__ pos,
                                   const float* __restrict__ w, const __nv_bfloat16* __restrict__ res, int T, int K,
                                   int H, __nv_bfloat16* __restrict__ out, const int* wait_flags, int wait_n,
                                   const int* epoch_base, int epoch_off, int* status) {
  const int nch = H >> 3;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
  if (wait_flags != nullptr) {
    __shared__ int ok_s;
    if (threadIdx.x == 0) {
      const int epoch = *epoch_base + epoch_off;
      int ok = 1;
      for (int r = 0; r < wait_n && ok; ++r) ok = wait_flag_ge(wait_flags + r, epoch, 10000000000ull) ? 1 : 0;
      if (!ok) report(status, ST_TIMEOUT_PEER);
      ok_s = ok;
    }
    __syncthreads();
    if (!ok_s) return;
  }
  for (int t = blockIdx.x * wpb + warp; t < T; t += gridDim.x * wpb) {
    for (int c = lane; c < nch; c += 32) {
      float acc[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
      if (res) {
        const uint4 q = *reinterpret_cast<const uint4*>(res + static_cast<size_t>(t) * H + c * 8);
        const uint32_t u[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = unpack_bf16x2(u[j]);
          acc[2 * j] = f.x;
          acc[2 * j + 1] = f.y;
        }
      }
      for (int k = 0; k < K; ++k) {
        const int p = pos ? pos[static_cast<size_t>(t) * K + k] : t * K + k;
        if (p < 0) continue;
        const float wk = w ? w[static_cast<size_t>(t) * K + k] : 1.f;
        // rows may have been written by a peer a moment ago: read them past L1
        const uint4 q = __ldcg(reinterpret_cast<const uint4*>(ys + static_cast<size_t>(p) * H + c * 8));
        const uint32_t u[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = unpack_bf16x2(u[j]);
          acc[2 * j] += wk * f.x;
          acc[2 * j + 1] += wk * f.y;
        }
      }
      *reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * H + c * 8) =
          make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]), pack_bf16x2(acc[4], acc[5]),
                     pack_bf16x2(acc[6], acc[7]));
    }
  }
}

// Backward of the weighted combine, per sorted row r (slot s = row_slot[r], token t = s / K):
//   dys[r] = w[s] * dout[t]        dw[s] = <dout[t], ys[r]>        padding rows -> 0
__global__ void moe_combine_bwd_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ ys,
                                       const int* __restrict__ row_slot, const int* __restrict__ seg_off,
                                       const float* __restrict__ w, int E, int K, int H,
                                       __nv_bfloat16* __restrict__ dys, float* __restrict__ dw, int capacity) {
  int live = seg_off[E];
  if (live > capacity) live = capacity;
  const int nch = H >> 3;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
  for (int r = blockIdx.x * wpb + warp; r < live; r += gridDim.x * wpb) {
    const int s = row_slot[r];
    uint4* dst = reinterpret_cast<uint4*>(dys + static_cast<size_t>(r) * H);
    if (s < 0) {
      for (int c = lane; c < nch; c += 32) dst[c] = make_uint4(0, 0, 0, 0);
      continue;
    }
    const float wk = w[s];
    const uint4* g = reinterpret_cast<const uint4*>(dout + static_cast<size_t>(s / K) * H);
    const uint4* y = reinterpret_cast<const uint4*>(ys + static_cast<size_t>(r) * H);
    float dot = 0.f;
    for (int c = lane; c < nch; c += 32) {
      const uint4 gq = g[c], yq = y[c];
      const uint32_t gu[4] = {gq.x, gq.y, gq.z, gq.w}, yu[4] = {yq.x, yq.y, yq.z, yq.w};
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 gf = unpack_bf16x2(gu[j]), yf = unpack_bf16x2(yu[j]);
        dot += gf.x * yf.x + gf.y * yf.y;
        o[j] = pack_bf16x2(wk * gf.x, wk * gf.y);
      }
      dst[c] = make_uint4(o[0], o[1], o[2], o[3]);
    }
    dot = warp_sum(dot);
    if (lane == 0) dw[s] = dot;
  }
}

// dw[t, k] = <dout[t], y[t * K + k]>: gradient of the routing weights when the expert outputs are laid out by
// (token, slot), as the expert-parallel return buffer is.  One warp per (token, slot), fixed summation order.
__global__ void moe_slot_dot_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ y, int n,
                                    int K, int H, float* __restrict__ dw) {
  const int nch = H >> 3;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
  for (int i = blockIdx.x * wpb + warp; i < n; i += gridDim.x * wpb) {
    const uint4* g = reinterpret_cast<const uint4*>(dout + static_cast<size_t>(i / K) * H);
    const uint4* r = reinterpret_cast<const uint4*>(y + static_cast<size_t>(i) * H);
    float dot = 0.f;
    for (int c = lane; c < nch; c += 32) {
      const uint4 gq = g[c], yq = __ldcg(r + c);
      const uint32_t gu[4] = {gq.x, gq.y, gq.z, gq.w}, yu[4] = {yq.x, yq.y, yq.z, yq.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 gf = unpack_bf16x2(gu[j]), yf = unpack_bf16x2(yu[j]);
        dot += gf.x * yf.x + gf.y * yf.y;
      }
    }
    dot = warp_sum(dot);
    if (lane == 0) dw[i] = dot;
  }
}

// dw[slot(r)] = sum over the n_tiles partial dot products the SwiGLU-backward epilogue left for sorted row r.
__global__ void moe_row_dot_reduce_kernel(const float* __restrict__ row_dot, const int* __restrict__ row_slot,
                                          const int* __restrict__ seg_off, int E, int n_tiles, int capacity,
                                          float* __restrict__ dw) {
  int live = seg_off[E];
  if (live > capacity) live = capacity;
  for (int r = blockIdx.x * blockDim.x + threadIdx.x; r < live; r += gridDim.x * blockDim.x) {
    const int s = row_slot[r];
    if (s < 0) continue;
    float a = 0.f;
    for (int n = 0; n < n_tiles; ++n) a += row_dot[static_cast<size_t>(r) * n_tiles + n];
    dw[s] = a;
  }
}

}  // namespace b200

using namespace b200;

extern "C" int b200_moe_row_dot_reduce(const float* row_dot, const int* row_slot, const int* seg_off, int E,
                                       int n_tiles, int capacity, float* dw, cudaStream_t stream) {
  if (n_tiles <= 0 || capacity <= 0) return -1;
  moe_row_dot_reduce_kernel<<<296, 256, 0, stream>>>(row_dot, row_slot, seg_off, E, n_tiles, capacity, dw);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int b200_moe_slot_dot(const void* dout, const void* y, int T, int K, int H, float* dw, cudaStream_t stream) {
  if (H % 8 != 0) return -1;
  if (T <= 0 || K <= 0) return 0;
  int grid = (T * K + 7) / 8;
  if (grid > 1184) grid = 1184;
  moe_slot_dot_kernel<<<grid, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(dout),
                                                reinterpret_cast<const __nv_bfloat16*>(y), T * K, K, H, dw);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int b200_moe_plan_blocks(int n) { return (n + PLAN_CHUNK - 1) / PLAN_CHUNK; }

// scratch: int32[plan_blocks(n) * E].  row_slot must hold `capacity` ints; it is reset to -1 here.
extern "C" int b200_moe_plan(const int* idx, int n, int E, int* scratch, int* counts, int* seg_off, int* tile_expert,
                             int* num_m_tiles, int* pos, int* row_slot, int capacity, int* pair_tiles, int max_pairs,
                             int* num_pair_tiles, int* row_tok, int K, cudaStream_t stream) {
  if (n <= 0 || E <= 0 || E > 65535 || capacity % 128 != 0) return -1;
  const size_t scan_sm = (3 * static_cast<size_t>(E) + 2) * sizeof(int);
  if (static_cast<size_t>(E) * sizeof(int) > 48 * 1024 || scan_sm > 200 * 1024) return -1;
  if (scan_sm > 48 * 1024) {
    static bool raised = false;
    if (!raised) {
      if (cudaFuncSetAttribute(plan_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess)
        return -3;
      raised = true;
    }
  }
  const int nb = b200_moe_plan_blocks(n);
  const size_t sm = static_cast<size_t>(E) * sizeof(int);
  cudaMemsetAsync(row_slot, 0xff, static_cast<size_t>(capacity) * sizeof(int), stream);
  // source token of every sorted row, for operand gathers; padding rows keep an index outside any tensor
  if (row_tok != nullptr) cudaMemsetAsync(row_tok, 0x7f, static_cast<size_t>(capacity) * sizeof(int), stream);
  plan_hist_kernel<<<nb, 256, sm, stream>>>(idx, n, E, scratch);
  plan_scan_kernel<<<1, 1024, scan_sm, stream>>>(
      scratch, nb, E, counts, seg_off, tile_expert, capacity / 128, num_m_tiles, pair_tiles, max_pairs,
      num_pair_tiles);
  plan_scatter_kernel<<<nb, 32, sm, stream>>>(idx, n, E, scratch, seg_off, pos, row_slot, capacity, row_tok,
                                              K > 0 ? K : 1);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int b200_moe_gather(const void* x, const int* row_slot, const int* seg_off, int E, int K, int H, void* xs,
                               int capacity, cudaStream_t stream) {
  if (H % 8 != 0) return -1;
  moe_gather_kernel<<<1184, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(x), row_slot, seg_off, E, K, H,
                                              reinterpret_cast<__nv_bfloat16*>(xs), capacity);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int b200_moe_combine(const void* ys, const int* pos, const float* w, const void* res, int T, int K, int H,
                                void* out, const int* wait_flags, int wait_n, const int* epoch_base, int epoch_off,
                                int* status, cudaStream_t stream) {
  if (H % 8 != 0) return -1;
  if (T <= 0) return 0;
  int grid = (T + 7) / 8;
  if (grid > 1184) grid = 1184;
  moe_combine_kernel<<<grid, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(ys), pos, w,
                                               reinterpret_cast<const __nv_bfloat16*>(res), T, K, H,
                                               reinterpret_cast<__nv_bfloat16*>(out), wait_flags, wait_n, epoch_base,
                                               epoch_off, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int b200_moe_combine_bwd(const void* dout, const void* ys, const int* row_slot, const int* seg_off,
                                    const float* w, int E, int K, int H, void* dys, float* dw, int capacity,
                                    cudaStream_t stream) {
  if (H % 8 != 0) return -1;
  moe_combine_bwd_kernel<<<1184, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(dout),
                                                   reinterpret_cast<const __nv_bfloat16*>(ys), row_slot, seg_off, w,
                                                   E, K, H, reinterpret_cast<__nv_bfloat16*>(dys), dw, capacity);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
