// Expert parallelism over NVLink peer memory: count exchange + receive layout, and the row push
// (dispatch) from token owners into expert owners' receive buffers.  The matching pieces on the
// compute side live in the GEMM kernel itself: its producer warp waits for the senders' flags before
// the first TMA load of the (local) receive buffer, and its scatter epilogue stores result rows
// straight into the token owners' return buffers and then posts completion flags.
//
// Protocol per layer and direction (all buffers symmetric, all flags monotonic epochs):
//   ep_exchange : every rank writes its per-expert counts into every peer's count matrix, posts
//                 flag CH_COUNTS, waits for all peers, then derives (identically on every rank)
//                 each owner's padded segment layout, its own send bases, its receive tile map,
//                 and zeroes the padding rows of its receive buffer.
//   ep_dispatch : one warp per (token, slot): copies the row (optionally scaled) into the owner's
//                 receive buffer at send_base[e] + rank-in-expert, records (source rank, slot) for
//                 the way back, and the last block posts flag CH_DISPATCH to every owner.
// Cross-GPU traffic is plain st.global to peer addresses; TMA only ever reads local memory.
#include "../common/ptx.cuh"
#include "../ops_api.h"

namespace b200 {

struct EpPeers {
  void* p[B200_MAX_RANKS];
};

__device__ __forceinline__ bool wait_all_flags(const int* flags, int n, int epoch, unsigned long long limit_ns) {
  for (int r = 0; r < n; ++r)
    if (!wait_flag_ge(flags + r, epoch, limit_ns)) return false;
  return true;
}

// counts[E] (this rank's assignments per global expert) -> layout.  One block.
__global__ void __launch_bounds__(1024)
ep_exchange_kernel(const int* __restrict__ counts, EpPeers cmat /* int [W][E] per rank */, EpPeers flags, int chan,
                   const int* epoch_base, int epoch_off, int rank, int world, int E, int H, int capacity,
                   int* __restrict__ send_base /* [E] */, int* __restrict__ recv_seg_off /* [El+1] */,
                   int* __restrict__ recv_tile_expert, int* __restrict__ recv_num_m_tiles,
                   __nv_bfloat16* __restrict__ recv_buf, int* __restrict__ recv_meta, int* status,
                   unsigned long long limit_ns, int* __restrict__ recv_pair_tiles, int max_pairs,
                   int* __restrict__ recv_num_pair_tiles) {
  extern __shared__ int sm[];  // [E] segment offsets of every expert inside its owner's buffer, then [E] totals
  int* seg = sm;
  int* tot = sm + E;
  __shared__ int ok_s;
  const int epoch = *epoch_base + epoch_off;
  const int El = E / world;
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    const int c = counts[e];
    for (int r = 0; r < world; ++r) reinterpret_cast<int*>(cmat.p[r])[rank * E + e] = c;
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int r = 0; r < world; ++r)
      st_release_sys(reinterpret_cast<int*>(flags.p[r]) + chan * B200_MAX_RANKS + rank, epoch);
    ok_s = wait_all_flags(reinterpret_cast<int*>(flags.p[rank]) + chan * B200_MAX_RANKS, world, epoch, limit_ns) ? 1 : 0;
    if (!ok_s) report(status, ST_TIMEOUT_PEER);
  }
  __syncthreads();
  if (!ok_s) {
    if (threadIdx.x == 0) {
      *recv_num_m_tiles = 0;
      if (recv_num_pair_tiles != nullptr) *recv_num_pair_tiles = 0;
    }
    return;
  }
  const int* cm = reinterpret_cast<const int*>(cmat.p[rank]);
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int t = 0;
    for (int s = 0; s < world; ++s) t += ld_relaxed_sys(cm + s * E + e);
    tot[e] = t;
  }
  __syncthreads();
  if (threadIdx.x < world) {  // one thread per owner: padded prefix over its experts
    const int o = threadIdx.x;
    int run = 0;
    for (int el = 0; el < El; ++el) {
      const int e = o * El + el;
      seg[e] = run;
      run += (tot[e] + 127) / 128 * 128;
    }
    if (o == rank) {
      recv_seg_off[El] = run;
      int nt = run / 128;
      if (run > capacity) {  // more rows routed here than the buffer holds: refuse, do not overrun
        report(status, ST_BAD_ARGUMENT);
        nt = 0;
      }
      *recv_num_m_tiles = nt;
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int before = 0;
    for (int s = 0; s < rank; ++s) before += ld_relaxed_sys(cm + s * E + e);
    send_base[e] = seg[e] + before;
  }
  const int total_rows = recv_seg_off[El] <= capacity ? recv_seg_off[El] : 0;
  for (int el = threadIdx.x; el < El; el += blockDim.x) {
    const int e = rank * El + el;
    recv_seg_off[el] = seg[e];
    const int t0 = seg[e] / 128, t1 = (seg[e] + (tot[e] + 127) / 128 * 128) / 128;
    for (int t = t0; t < t1 && t * 128 < total_rows; ++t) recv_tile_expert[t] = el;
  }
  // the same rows as pair tiles for the pair-tile GEMM kernel: two 128-row tiles of one expert, or its last one
  if (recv_pair_tiles != nullptr && threadIdx.x == 0) {
    int np = 0;
    for (int el = 0; el < El && total_rows > 0; ++el) {
      const int e = rank * El + el;
      const int t0 = seg[e] / 128, n128 = (tot[e] + 127) / 128;
      for (int i = 0; 2 * i < n128 && np < max_pairs; ++i, ++np) {
        recv_pair_tiles[2 * np] = (t0 + 2 * i) * 128;
        recv_pair_tiles[2 * np + 1] = el | ((2 * i + 2 <= n128 ? 2 : 1) << 16);
      }
    }
    *recv_num_pair_tiles = np;
  }
}

// Zero the padding rows of every local expert segment (they enter the weight-gradient contraction) and mark them
// as sourceless.  One block per local expert: the ranges are rebuilt from the (by now complete) count matrix, so
// the layout kernel above, which is a single block on the critical path, does not have to touch the rows.
__global__ void ep_pad_zero_kernel(const int* __restrict__ cm /* this rank's int [W][E] */,
                                   const int* __restrict__ recv_seg_off, int rank, int world, int E, int H,
                                   int capacity, __nv_bfloat16* __restrict__ recv_buf, int* __restrict__ recv_meta) {
  const int El = E / world;
  const int el = blockIdx.x;
  if (el >= El || recv_seg_off[El] > capacity) return;  // refused step: nothing will be read
  const int e = rank * El + el;
  int tot = 0;
  for (int s = 0; s < world; ++s) tot += ld_relaxed_sys(cm + s * E + e);
  const int lo = recv_seg_off[el] + tot, hi = recv_seg_off[el] + (tot + 127) / 128 * 128;
  if (lo < 0 || hi > capacity) return;
  const int nch = H >> 3;
  for (int i = threadIdx.x; i < (hi - lo) * nch; i += blockDim.x) {
    const int r = lo + i / nch, c = i - (i / nch) * nch;
    reinterpret_cast<uint4*>(recv_buf + static_cast<size_t>(r) * H)[c] = make_uint4(0, 0, 0, 0);
  }
  for (int r = lo + threadIdx.x; r < hi; r += blockDim.x) recv_meta[r] = -1;
}

// Push rows to their expert owners.  src row of assignment i is rows[i / K] (scaled by scale[i] if given).
__global__ void ep_dispatch_kernel(const __nv_bfloat16* __restrict__ rows, const float* __restrict__ scale,
                                   const int* __restrict__ idx, const int* __restrict__ pos,
                                   const int* __restrict__ local_seg_off, const int* __restrict__ send_base,
                                   EpPeers recv_buf, EpPeers recv_meta, EpPeers flags, int chan, const int* epoch_base,
                                   int epoch_off, int rank, int world, int E, int n, int K, int H, int capacity,
                                   int* counter) {
  const int El = E / world;
  const int nch = H >> 3;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
  for (int i = blockIdx.x * wpb + warp; i < n; i += gridDim.x * wpb) {
    const int e = idx[i];
    const int p = pos[i];
    if (e < 0 || e >= E || p < 0) continue;
    const int o = e / El;
    const int row = send_base[e] + (p - local_seg_off[e]);
    if (row >= capacity) continue;  // the owner has already refused this step (status set there)
    const uint4* src = reinterpret_cast<const uint4*>(rows + static_cast<size_t>(i / K) * H);
    uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(recv_buf.p[o]) + static_cast<size_t>(row) * H);
    if (scale) {
      const float s = scale[i];
      for (int c = lane; c < nch; c += 32) {
        const uint4 q = src[c];
        const uint32_t u[4] = {q.x, q.y, q.z, q.w};
        uint32_t w[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = unpack_bf16x2(u[j]);
          w[j] = pack_bf16x2(s * f.x, s * f.y);
        }
        dst[c] = make_uint4(w[0], w[1], w[2], w[3]);
      }
    } else {
      for (int c = lane; c < nch; c += 32) dst[c] = src[c];
    }
    if (lane == 0) reinterpret_cast<int*>(recv_meta.p[o])[row] = (rank << 28) | i;
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int ticket = atomicAdd(counter, 1);
    if (ticket == static_cast<int>(gridDim.x) - 1) {
      *counter = 0;
      __threadfence_system();
      const int epoch = *epoch_base + epoch_off;
      for (int r = 0; r < world; ++r)
        st_release_sys(reinterpret_cast<int*>(flags.p[r]) + chan * B200_MAX_RANKS + rank, epoch);
    }
  }
}

}  // namespace b200

using namespace b200;

static EpPeers to_peers(void* const* p) {
  EpPeers e;
  for (int r = 0; r < B200_MAX_RANKS; ++r) e.p[r] = p[r];
  return e;
}

extern "C" int b200_ep_exchange(const int* counts, void* const* cmat, void* const* flags, int chan, const int* epoch_base,
                                int epoch_off, int rank, int world, int E, int H, int capacity, int* send_base,
                                int* recv_seg_off, int* recv_tile_expert, int* recv_num_m_tiles, void* recv_buf,
                                int* recv_meta, int* status, unsigned long long limit_ns, int* recv_pair_tiles,
                                int max_pairs, int* recv_num_pair_tiles, cudaStream_t stream) {
  if (world < 1 || world > B200_MAX_RANKS || E % world != 0 || H % 8 != 0 || capacity % 128 != 0) return -1;
  const size_t smem = 2 * static_cast<size_t>(E) * sizeof(int);
  if (smem > 200 * 1024) return -1;
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(ep_exchange_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (limit_ns == 0) limit_ns = 10000000000ull;
  ep_exchange_kernel<<<1, 1024, smem, stream>>>(counts, to_peers(cmat), to_peers(flags), chan, epoch_base, epoch_off,
                                                rank, world, E, H, capacity, send_base, recv_seg_off, recv_tile_expert,
                                                recv_num_m_tiles, reinterpret_cast<__nv_bfloat16*>(recv_buf), recv_meta,
                                                status, limit_ns, recv_pair_tiles, max_pairs, recv_num_pair_tiles);
  ep_pad_zero_kernel<<<E / world, 256, 0, stream>>>(reinterpret_cast<const int*>(cmat[rank]), recv_seg_off, rank, world,
                                                   E, H, capacity, reinterpret_cast<__nv_bfloat16*>(recv_buf),
                                                   recv_meta);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int b200_ep_dispatch(const void* rows, const float* scale, const int* idx, const int* pos,
                                const int* local_seg_off, const int* send_base, void* const* recv_buf,
                                void* const* recv_meta, void* const* flags, int chan, const int* epoch_base,
                                int epoch_off, int rank, int world, int E, int n, int K, int H, int capacity,
                                int* counter, cudaStream_t stream) {
  if (world < 1 || world > B200_MAX_RANKS || E % world != 0 || H % 8 != 0 || n <= 0) return -1;
  int grid = (n + 7) / 8;
  if (grid > 592) grid = 592;
  ep_dispatch_kernel<<<grid, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(rows), scale, idx, pos,
                                               local_seg_off, send_base, to_peers(recv_buf), to_peers(recv_meta),
                                               to_peers(flags), chan, epoch_base, epoch_off, rank, world, E, n, K, H,
                                               capacity, counter);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
