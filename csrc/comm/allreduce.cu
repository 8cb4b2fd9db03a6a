// Gradient all-reduce over NVLink peer memory, fused with the data-parallel average and with the
// squared-norm partials that gradient clipping needs.
//
// Every rank's flat fp32 gradient buffer lives in symmetric memory (all ranks have every peer's
// buffer mapped).  One launch per bucket:
//   1. arrive barrier : flag words in the peers' signal area tell everybody that this rank's
//                       gradients for the bucket are complete (they were written by earlier kernels
//                       on the same stream);
//   2. two-shot reduce: rank r owns slice r of the bucket: it loads that slice from every peer
//                       (plain peer loads, or one multimem.ld_reduce through the NVSwitch), scales
//                       by 1/world, accumulates sum(v^2), and stores the result into every rank's
//                       buffer (peer stores, or one multimem.st);
//   3. done barrier   : the last block to finish posts "done" to all peers and waits for theirs, so
//                       kernel completion on this stream means the whole bucket is final locally.
// All waits are bounded; a wait that runs out records ST_TIMEOUT_PEER and the kernel returns.
// No TMA is involved: cross-GPU traffic is ordinary ld/st (or multimem) from inside the kernel.
#include "../common/ptx.cuh"
#include "../ops_api.h"

namespace b200 {

constexpr int AR_THREADS = 256;  // 256 x ~120 registers: fits next to a resident GEMM CTA on the same SM
constexpr int AR_UNROLL = 2;

struct ArPeers {
  float* buf[B200_MAX_RANKS];   // flat gradient buffers (same layout on every rank)
  int* flags[B200_MAX_RANKS];   // int[2 * B200_MAX_RANKS] per rank: arrive[src], done[src]
  float* norm[B200_MAX_RANKS];  // float[B200_MAX_RANKS] per rank: squared-norm partial of each source rank
};

__device__ __forceinline__ float4 ld_peer_f4(const float* p) {
  float4 v;
  asm volatile("ld.volatile.global.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ void st_peer_f4(float* p, float4 v) {
  asm volatile("st.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}
__device__ __forceinline__ float4 multimem_ld_reduce_f4(const float* mc) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(mc)
               : "memory");
  return v;
}
__device__ __forceinline__ void multimem_st_f4(float* mc, float4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc), "f"(v.x), "f"(v.y), "f"(v.z),
               "f"(v.w)
               : "memory");
}

// state: local scratch, int[2] + float[2 + 148]: {blocks finished, unused} / {unused, running sum of the step,
// one partial sum of squares per block}
template <bool MULTIMEM>
__global__ void __launch_bounds__(AR_THREADS)
allreduce_kernel(ArPeers peers, float* mc_buf, int rank, int world, long long off, long long n, float scale,
                 const int* epoch_base, int epoch_off, int final_bucket, int publish, int* state_i, float* state_f,
                 int* status, unsigned long long limit_ns) {
  __shared__ float sh[AR_THREADS / 32];
  __shared__ int sh_ok;
  int* my_flags = peers.flags[rank];
  // epochs grow monotonically; the base lives in device memory so that a captured graph can be replayed
  const int epoch = *epoch_base + epoch_off;
  // ---- 1. arrive
  if (blockIdx.x == 0 && threadIdx.x < world) st_release_sys(peers.flags[threadIdx.x] + rank, epoch);
  if (threadIdx.x == 0) {
    int ok = 1;
    for (int r = 0; r < world && ok; ++r) ok = wait_flag_ge(my_flags + r, epoch, limit_ns) ? 1 : 0;
    sh_ok = ok;
  }
  __syncthreads();
  float ss = 0.f;
  if (sh_ok) {
    // ---- 2. reduce my slice, publish it everywhere
    const long long n4 = n >> 2;  // bucket sizes are multiples of 4 floats
    const long long per = (n4 + world - 1) / world;
    const long long lo = per * rank, hi = (lo + per < n4) ? lo + per : n4;
    // AR_UNROLL independent 16-byte accesses per thread and peer are in flight at once: NVLink
    // round trips take microseconds, so bandwidth comes from memory-level parallelism
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i0 = lo + static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i0 < hi;
         i0 += stride * AR_UNROLL) {
      float4 acc[AR_UNROLL];
#pragma unroll
      for (int u = 0; u < AR_UNROLL; ++u) acc[u] = make_float4(0.f, 0.f, 0.f, 0.f);
      if constexpr (MULTIMEM) {
#pragma unroll
        for (int u = 0; u < AR_UNROLL; ++u) {
          const long long i = i0 + u * stride;
          if (i < hi) acc[u] = multimem_ld_reduce_f4(mc_buf + off + (i << 2));
        }
      } else {
        // issue the loads of every peer before the first add, so that all of them are in flight together
        float4 v[B200_MAX_RANKS][AR_UNROLL];
#pragma unroll
        for (int r = 0; r < B200_MAX_RANKS; ++r) {
          if (r < world) {
            const float* src = peers.buf[(rank + r) % world] + off;  // stagger the peers
#pragma unroll
            for (int u = 0; u < AR_UNROLL; ++u) {
              const long long i = i0 + u * stride;
              v[r][u] = i < hi ? ld_peer_f4(src + (i << 2)) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
          }
        }
#pragma unroll
        for (int r = 0; r < B200_MAX_RANKS; ++r) {
          if (r < world) {
#pragma unroll
            for (int u = 0; u < AR_UNROLL; ++u) {
              acc[u].x += v[r][u].x; acc[u].y += v[r][u].y; acc[u].z += v[r][u].z; acc[u].w += v[r][u].w;
            }
          }
        }
      }
#pragma unroll
      for (int u = 0; u < AR_UNROLL; ++u) {
        acc[u].x *= scale; acc[u].y *= scale; acc[u].z *= scale; acc[u].w *= scale;
        const long long i = i0 + u * stride;
        if (i < hi) ss += acc[u].x * acc[u].x + acc[u].y * acc[u].y + acc[u].z * acc[u].z + acc[u].w * acc[u].w;
      }
      if (!publish) {
        // reduce-scatter: only the owner keeps its slice (sharded optimizer state)
        float* dst = peers.buf[rank] + off;
#pragma unroll
        for (int u = 0; u < AR_UNROLL; ++u) {
          const long long i = i0 + u * stride;
          if (i < hi) st_peer_f4(dst + (i << 2), acc[u]);
        }
      } else if constexpr (MULTIMEM) {
#pragma unroll
        for (int u = 0; u < AR_UNROLL; ++u) {
          const long long i = i0 + u * stride;
          if (i < hi) multimem_st_f4(mc_buf + off + (i << 2), acc[u]);
        }
      } else {
        for (int r = 0; r < world; ++r) {
          float* dst = peers.buf[(rank + r) % world] + off;
#pragma unroll
          for (int u = 0; u < AR_UNROLL; ++u) {
            const long long i = i0 + u * stride;
            if (i < hi) st_peer_f4(dst + (i << 2), acc[u]);
          }
        }
      }
    }
  } else if (threadIdx.x == 0) {
    report(status, ST_TIMEOUT_PEER);
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = ss;
  __syncthreads();
  // ---- 3. done: last block of this rank posts and waits
  if (threadIdx.x == 0) {
    float s = 0.f;
    for (int i = 0; i < AR_THREADS / 32; ++i) s += sh[i];
    // per-block slots summed in block order by the last block: the same data always give the same
    // bits, whatever order the blocks finish in (an atomic running sum would not)
    state_f[2 + blockIdx.x] = s;
    __threadfence_system();
    const int ticket = atomicAdd(&state_i[0], 1);
    if (ticket == static_cast<int>(gridDim.x) - 1) {
      __threadfence();
      float bucket = 0.f;
      for (unsigned b = 0; b < gridDim.x; ++b) bucket += *(reinterpret_cast<volatile float*>(state_f) + 2 + b);
      const float total = state_f[1] + bucket;
      state_f[1] = final_bucket ? 0.f : total;
      state_i[0] = 0;
      if (final_bucket)
        for (int r = 0; r < world; ++r) peers.norm[r][rank] = total;  // peer store of this rank's partial
      __threadfence_system();
      for (int r = 0; r < world; ++r) st_release_sys(peers.flags[r] + B200_MAX_RANKS + rank, epoch);
      bool ok = true;
      for (int r = 0; r < world && ok; ++r) ok = wait_flag_ge(my_flags + B200_MAX_RANKS + r, epoch, limit_ns);
      if (!ok) report(status, ST_TIMEOUT_PEER);
    }
  }
}

// coef[0] = min(1, max_norm / (norm + 1e-6)), coef[1] = norm, norm^2 = sum of the ranks' partials
__global__ void clip_coef_multi_kernel(const float* __restrict__ parts, int world, float max_norm,
                                       float* __restrict__ coef) {
  float s = 0.f;
  for (int r = 0; r < world; ++r) s += parts[r];
  const float norm = sqrtf(s);
  coef[0] = max_norm > 0.f ? fminf(1.f, max_norm / (norm + 1e-6f)) : 1.f;
  coef[1] = norm;
}

// Post flag word `index` (= channel * B200_MAX_RANKS + rank) on every rank and wait for all ranks' words of
// that channel.  One thread; used after kernels that stored into peers' memory (parameter publish).
__global__ void peer_barrier_kernel(ArPeers peers, int rank, int world, int chan, const int* epoch_base, int epoch_off,
                                    int* status, unsigned long long limit_ns) {
  const int epoch = *epoch_base + epoch_off;
  __threadfence_system();
  for (int r = 0; r < world; ++r) st_release_sys(peers.flags[r] + chan * B200_MAX_RANKS + rank, epoch);
  bool ok = true;
  for (int r = 0; r < world && ok; ++r)
    ok = wait_flag_ge(peers.flags[rank] + chan * B200_MAX_RANKS + r, epoch, limit_ns);
  if (!ok) report(status, ST_TIMEOUT_PEER);
}

// Parameter all-gather for sharded parameters: every rank keeps `per` bf16 elements of a unit at the same
// offset of its shard buffer (symmetric memory); this rank pulls all ranks' pieces with plain 16-byte peer
// loads (no TMA, no waits: the pieces are stable between two optimizer steps) into a LOCAL staging buffer,
// which is what the GEMMs' TMA then reads.  dst[r * per + i] = shard_r[i], clipped to `n` elements.
struct AgPeers {
  const uint4* shard[B200_MAX_RANKS];
};
__global__ void __launch_bounds__(512)
allgather_bf16_kernel(AgPeers peers, int world, long long per16, long long n16, uint4* __restrict__ dst) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  constexpr int U = 4;
  for (int r0 = 0; r0 < world; ++r0) {
    const int r = (r0 + blockIdx.x) % world;  // blocks start on different peers
    const uint4* src = peers.shard[r];
    const long long base = static_cast<long long>(r) * per16;
    long long len = n16 - base;
    if (len > per16) len = per16;
    for (long long i0 = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i0 < len; i0 += stride * U) {
      uint4 v[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = i0 + u * stride;
        if (i < len)
          asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                       : "=r"(v[u].x), "=r"(v[u].y), "=r"(v[u].z), "=r"(v[u].w)
                       : "l"(src + i));
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = i0 + u * stride;
        if (i < len) dst[base + i] = v[u];
      }
    }
  }
}

}  // namespace b200

using namespace b200;

// shards: every rank's pointer to the unit's piece (bf16, 16-byte aligned); per / n in elements, multiples of 8
extern "C" int b200_allgather_bf16(const void* const* shards, int world, long long per, long long n, void* dst,
                                   int blocks, cudaStream_t stream) {
  if (world < 1 || world > B200_MAX_RANKS || (per & 7) != 0 || (n & 7) != 0) return -1;
  if (n <= 0) return 0;
  AgPeers ap;
  for (int r = 0; r < B200_MAX_RANKS; ++r) ap.shard[r] = r < world ? reinterpret_cast<const uint4*>(shards[r]) : nullptr;
  if (blocks < 1) blocks = 1;
  if (blocks > 296) blocks = 296;
  allgather_bf16_kernel<<<blocks, 512, 0, stream>>>(ap, world, per >> 3, n >> 3, reinterpret_cast<uint4*>(dst));
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int b200_allreduce(const B200Peers* p, int rank, int world, long long off, long long n, float scale,
                              const int* epoch_base, int epoch_off, int final_bucket, int publish, int use_multimem,
                              int blocks, int* state_i, float* state_f, int* status, unsigned long long limit_ns,
                              cudaStream_t stream) {
  if (world < 1 || world > B200_MAX_RANKS || rank < 0 || rank >= world) return -1;
  if (n <= 0) return 0;
  if ((n & 3) != 0 || (off & 3) != 0) return -1;
  if (use_multimem && p->mc_buf == nullptr) return -1;
  ArPeers ap;
  for (int r = 0; r < B200_MAX_RANKS; ++r) {
    ap.buf[r] = reinterpret_cast<float*>(p->buf[r]);
    ap.flags[r] = reinterpret_cast<int*>(p->flags[r]);
    ap.norm[r] = reinterpret_cast<float*>(p->norm[r]);
  }
  if (blocks < 1) blocks = 1;
  if (blocks > 148) blocks = 148;
  if (limit_ns == 0) limit_ns = 10000000000ull;  // ten seconds: peers may be busy with compute
  float* mc = reinterpret_cast<float*>(p->mc_buf);
  if (use_multimem)
    allreduce_kernel<true><<<blocks, AR_THREADS, 0, stream>>>(ap, mc, rank, world, off, n, scale, epoch_base, epoch_off,
                                                               final_bucket, publish, state_i, state_f, status,
                                                               limit_ns);
  else
    allreduce_kernel<false><<<blocks, AR_THREADS, 0, stream>>>(ap, mc, rank, world, off, n, scale, epoch_base, epoch_off,
                                                                final_bucket, publish, state_i, state_f, status,
                                                                limit_ns);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int b200_clip_coef_multi(const float* parts, int world, float max_norm, float* coef, cudaStream_t stream) {
  clip_coef_multi_kernel<<<1, 1, 0, stream>>>(parts, world, max_norm, coef);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int b200_peer_barrier(const B200Peers* p, int rank, int world, int chan, const int* epoch_base, int epoch_off,
                                 int* status, unsigned long long limit_ns, cudaStream_t stream) {
  if (world < 1 || world > B200_MAX_RANKS || rank < 0 || rank >= world || chan < 0 || chan > 3) return -1;
  ArPeers ap;
  for (int r = 0; r < B200_MAX_RANKS; ++r) {
    ap.buf[r] = nullptr;
    ap.norm[r] = nullptr;
    ap.flags[r] = reinterpret_cast<int*>(p->flags[r]);
  }
  if (limit_ns == 0) limit_ns = 10000000000ull;
  peer_barrier_kernel<<<1, 1, 0, stream>>>(ap, rank, world, chan, epoch_base, epoch_off, status, limit_ns);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
