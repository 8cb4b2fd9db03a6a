// Causal grouped-query flash attention, backward, for sm_100a (head_dim 128).  Three kernels:
//
//   delta : Dsc[b,h,s] = softmax_scale * sum_d dO[b,s,h,d] * O[b,s,h,d]
//   dQ    : work item = (batch, query head, 128 query rows); loops over key tiles j <= query tile:
//             S = Q K_j^T, dP = dO V_j^T                       (both operands in shared memory)
//             P = exp2(S*c - lse2), dS = P * (dP*scale - Dsc)   (one query row per pair of threads)
//             dQ += dS K_j                                      (dS from TMEM, K_j read MN-major)
//   dK/dV : work item = (batch, key/value head, 128 key rows); loops over the query heads of the group
//           and their query tiles i >= key tile:
//             S^T = K_j Q_i^T, dP^T = V_j dO_i^T                (TMEM lanes = key rows)
//             P^T, dS^T as above with per-column statistics read from shared memory
//             dV += P^T dO_i, dK += dS^T Q_i                    (P^T, dS^T from TMEM; dO_i, Q_i MN-major)
//           so the sum over the query heads of a group happens in the TMEM accumulators.
//
// Roles as in the forward kernel: warp 0 TMA producer, warp 1 MMA issuer (owns the 512 TMEM columns),
// warps 2..9 element-wise (TMEM lane quarter = warp % 4).
//
// dQ kernel: 128 x 128 score tiles, the score buffer double-buffered in TMEM (S[2], dP, dQ = 512 columns).
// Of a tile, warps 2..5 take columns 0..63 and warps 6..9 columns 64..127; a thread writes its 64 dS values
// (bf16 pairs, tcgen05.st) over the first 32 of the score columns it has just read, and dQ += dS K_j takes
// them as its A operand from TMEM.  Issue order: S(0) dP(0) S(1) | dQ(0) dP(1) S(2) | dQ(1) dP(2) S(3) | ...
// (MMAs of one thread execute in issue order, so S(j+2) may overwrite the columns dS(j) was read from).
// dP(j+1) stays behind dQ(j) although the dP columns are free earlier: with the threads of tile j+1 reading
// TMEM while the dQ(j) MMAs (TMEM operand) run, the kernel took 350 us instead of about 220 us.  Folding the
// delta pre-pass into this kernel (per-row dot product at the start of a work item) cost 30 us more than
// the separate 46 us kernel saves, so delta stays a kernel of its own.
// K_j is one ring slot that is read K-major by the score MMA and MN-major by the gradient MMA.
//
// dK/dV kernel: all 512 TMEM columns would be live with 128-wide score tiles (S^T, dP^T, dV, dK) and
// nothing could overlap, so this loop advances in SUB-TILES of 64 query rows: score tiles are 128 x 64 and
// double-buffered, the score MMAs of sub-tile u+1 run while the threads work on sub-tile u.  Warps 2..5
// take columns 0..31 of a sub-tile, warps 6..9 columns 32..63; P^T and dS^T go over the first 16 of the 32
// score columns a thread has read.  A ring slot holds the 64 rows of Q_i and dO_i of one sub-tile.
//
// Measured MMA issue rates that shaped this (clock64 trace of one CTA): a 128x64x16 MMA with both
// operands in shared memory takes about 74 cycles, a 128x128x16 MMA with its A operand in TMEM about 128
// (twice the 64 of the shared-memory form), so both kernels are bound by the tensor pipe's operand paths,
// not by the element-wise threads (about 800 cycles per sub-tile, idle most of the time).
#include "../common/ptx.cuh"
#include "../common/tma_host.h"
#include "attn_api.h"

namespace b200 {

constexpr int FB_THREADS = 320;
constexpr int FB_TILE = 32768;  // 128 x 128 bf16
constexpr int FB_SMEM = 232448;
constexpr unsigned long long FB_LIMIT_NS = 2000000000ull;

struct FbArgs {
  const float* lse2;  // [B, nh, S]
  const float* dsc;   // [B, nh, S]
  __nv_bfloat16* dq;  // [B, S, nh, 128]
  __nv_bfloat16* dk;  // [B, S, nkv, 128]
  __nv_bfloat16* dv;
  int B, S, nh, nkv;
  int items;
  float scale, scale_log2;
  int* status;
};

__device__ __forceinline__ int fb_sched(int round, int cta, int ctas) {
  return round * ctas + ((round & 1) ? ctas - 1 - cta : cta);
}

// ----------------------------------------------------------------------------------------- delta
template <int HD>
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o,
                                  float* __restrict__ dsc, int B, int S, int nh, float scale) {
  // HD / 8 lanes per (b, s, h): 8 elements per lane (one 16-byte load from each tensor)
  constexpr int LPR = HD / 8;
  const long long w = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) / LPR;
  const int l16 = threadIdx.x & (LPR - 1);
  const long long total = static_cast<long long>(B) * S * nh;
  const bool live = w < total;
  float s = 0.f;
  if (live) {
    const uint4 a = reinterpret_cast<const uint4*>(o + w * HD)[l16];
    const uint4 b = reinterpret_cast<const uint4*>(d_o + w * HD)[l16];
    const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 af = unpack_bf16x2(aw[e]), bf = unpack_bf16x2(bw[e]);
      s = fmaf(af.x, bf.x, s);
      s = fmaf(af.y, bf.y, s);
    }
  }
#pragma unroll
  for (int off = LPR / 2; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
  if (live && l16 == 0) {
    const long long bs = w / nh;
    const int h = static_cast<int>(w - bs * nh);
    const long long b_ = bs / S;
    const int s_ = static_cast<int>(bs - b_ * S);
    dsc[(b_ * nh + h) * S + s_] = s * scale;
  }
}

// -------------------------------------------------------------------------------------------- dQ
constexpr int DQ_RING = 5;

template <int HD>
__global__ void __launch_bounds__(FB_THREADS, 1)
flash_bwd_dq_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapK,
                    const __grid_constant__ CUtensorMap mapV, const __grid_constant__ CUtensorMap mapDO,
                    const FbArgs args) {
  extern __shared__ uint8_t smem_raw[];
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = base;
  uint8_t* sDO = base + FB_TILE;
  uint8_t* sR = base + 2 * FB_TILE;  // K_j at even ring entries, V_j at odd ones
  uint64_t* bars = reinterpret_cast<uint64_t*>(base + 7 * FB_TILE);
  uint64_t& bar_q_full = bars[0];
  uint64_t& bar_q_empty = bars[1];
  uint64_t* bar_r_full = bars + 2;    // [DQ_RING]
  uint64_t* bar_r_empty = bars + 7;   // [DQ_RING]
  uint64_t* bar_s_full = bars + 12;   // [2]
  uint64_t& bar_dp_full = bars[14];
  uint64_t& bar_ds_full = bars[15];
  uint64_t& bar_dq_full = bars[16];
  uint64_t& bar_drain = bars[17];
  uint32_t& tmem_base_slot = *reinterpret_cast<uint32_t*>(bars + 18);
  int& go = *reinterpret_cast<int*>(bars + 19);

  if (threadIdx.x == 0) {
    go = 1;
    if (base + 7 * FB_TILE + 256 > smem_raw + FB_SMEM) {
      report(args.status, ST_BAD_ARGUMENT);
      go = 0;
    }
    tma_prefetch_desc(&mapQ);
    tma_prefetch_desc(&mapK);
    tma_prefetch_desc(&mapV);
    tma_prefetch_desc(&mapDO);
    mbar_init(&bar_q_full, 1);
    mbar_init(&bar_q_empty, 1);
    for (int s = 0; s < DQ_RING; ++s) {
      mbar_init(&bar_r_full[s], 1);
      mbar_init(&bar_r_empty[s], 1);
    }
    mbar_init(&bar_s_full[0], 1);
    mbar_init(&bar_s_full[1], 1);
    mbar_init(&bar_dp_full, 1);
    mbar_init(&bar_ds_full, 8);
    mbar_init(&bar_dq_full, 1);
    mbar_init(&bar_drain, 1);
    fence_mbar_init();
  }
  __syncthreads();
  if (!go) return;
  if (warp == 1) {
    tmem_alloc(&tmem_base_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_slot;
  // TMEM columns: S[0] 0, S[1] 128, dP 256, dQ 384
  constexpr int KC = HD / 64;               // 64-column chunks of a head
  constexpr int TILE_BYTES = 128 * HD * 2;  // bytes of one Q / dO / K / V tile
  const int group = args.nh / args.nkv;
  const int per_qt = args.B * args.nh;
  const int n_qt = args.S >> 7;

  if (warp == 0) {
    if (lane == 0) {
      bool ok = true;
      uint32_t load = 0;
      int it_count = 0;
      for (int t; (t = fb_sched(it_count, blockIdx.x, gridDim.x)) < args.items && ok; ++it_count) {
        if (*reinterpret_cast<volatile int*>(args.status) != 0) break;
        const int qt = n_qt - 1 - t / per_qt, r = t % per_qt, b = r / args.nh, h = r % args.nh, hk = h / group;
        if (!mbar_wait_ns(&bar_q_empty, (it_count & 1) ^ 1u, FB_LIMIT_NS)) {
          ok = false;
          break;
        }
        mbar_expect_tx(&bar_q_full, 2 * TILE_BYTES);
#pragma unroll
        for (int kc = 0; kc < KC; ++kc) {
          tma_load_3d(sQ + kc * 16384, &mapQ, &bar_q_full, h * HD + kc * 64, qt * 128, b);
          tma_load_3d(sDO + kc * 16384, &mapDO, &bar_q_full, h * HD + kc * 64, qt * 128, b);
        }
        for (int j = 0; j <= qt && ok; ++j) {
          for (int kv = 0; kv < 2; ++kv) {
            const int slot = load % DQ_RING;
            if (!mbar_wait_ns(&bar_r_empty[slot], ((load / DQ_RING) & 1) ^ 1u, FB_LIMIT_NS)) {
              ok = false;
              break;
            }
            mbar_expect_tx(&bar_r_full[slot], TILE_BYTES);
            uint8_t* dst = sR + slot * FB_TILE;
            const CUtensorMap* m = kv ? &mapV : &mapK;
#pragma unroll
            for (int kc = 0; kc < KC; ++kc)
              tma_load_3d(dst + kc * 16384, m, &bar_r_full[slot], hk * HD + kc * 64, j * 128, b);
            ++load;
          }
        }
      }
      if (!ok) report(args.status, ST_TIMEOUT_PRODUCER);
      for (uint32_t i = load > DQ_RING ? load - DQ_RING : 0; i < load; ++i)
        (void)mbar_wait_ns(&bar_r_full[i % DQ_RING], (i / DQ_RING) & 1, FB_LIMIT_NS);
      if (it_count > 0) (void)mbar_wait_ns(&bar_q_full, (it_count - 1) & 1, FB_LIMIT_NS);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_kk = make_idesc_bf16(128, 128, 0, 0);  // both operands K-major
      constexpr uint32_t idesc_mn = make_idesc_bf16(128, HD, 0, 1);  // B MN-major
      bool ok = true;
      uint32_t load = 0, g = 0;
      int it_count = 0;
      const uint32_t q_addr = smem_u32(sQ), do_addr = smem_u32(sDO);
      auto ring_wait = [&](uint32_t idx) -> bool {
        const bool r = mbar_wait_ns(&bar_r_full[idx % DQ_RING], (idx / DQ_RING) & 1, FB_LIMIT_NS);
        tc_fence_after();
        return r;
      };
      auto issue_kk = [&](uint32_t d_col, uint32_t a_addr, uint32_t b_addr) {
#pragma unroll
        for (int kc = 0; kc < KC; ++kc)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_bf16(tmem + d_col, make_smem_desc(a_addr + kc * 16384 + k * 32, 16, 1024),
                      make_smem_desc(b_addr + kc * 16384 + k * 32, 16, 1024), idesc_kk, (kc | k) != 0 ? 1u : 0u);
      };
      for (int t; (t = fb_sched(it_count, blockIdx.x, gridDim.x)) < args.items && ok; ++it_count) {
        const int qt = n_qt - 1 - t / per_qt;
        const int n = qt + 1;
        auto k_slot = [&](int j) { return smem_u32(sR + ((load + 2 * j) % DQ_RING) * FB_TILE); };
        auto v_slot = [&](int j) { return smem_u32(sR + ((load + 2 * j + 1) % DQ_RING) * FB_TILE); };
        ok = mbar_wait_ns(&bar_q_full, it_count & 1, FB_LIMIT_NS);
        if (!ok) break;
        tc_fence_after();
        // S(0), dP(0), S(1)
        if (!ring_wait(load)) { ok = false; break; }
        issue_kk(((g + 0) & 1) * 128, q_addr, k_slot(0));
        umma_commit(&bar_s_full[(g + 0) & 1]);
        if (!ring_wait(load + 1)) { ok = false; break; }
        issue_kk(256, do_addr, v_slot(0));
        umma_commit(&bar_r_empty[(load + 1) % DQ_RING]);
        umma_commit(&bar_dp_full);
        if (n == 1) umma_commit(&bar_q_empty);
        if (n > 1) {
          if (!ring_wait(load + 2)) { ok = false; break; }
          issue_kk(((g + 1) & 1) * 128, q_addr, k_slot(1));
          umma_commit(&bar_s_full[(g + 1) & 1]);
        }
        for (int j = 0; j < n; ++j) {
          if (!mbar_wait_ns(&bar_ds_full, (g + j) & 1, FB_LIMIT_NS)) { ok = false; break; }
          tc_fence_after();
          // dQ += dS K_j : A = dS in TMEM (k-steps 0..3 at score columns 0..31, 4..7 at columns 64..95)
          const uint32_t kj = k_slot(j);
          const uint32_t ds_col = ((g + j) & 1) * 128;
#pragma unroll
          for (int ks = 0; ks < 8; ++ks)
            umma_bf16_ts(tmem + 384, tmem + ds_col + (ks < 4 ? ks * 8 : 64 + (ks - 4) * 8),
                         make_smem_desc(kj + ks * 2048, 16384, 1024), idesc_mn, (j | ks) != 0 ? 1u : 0u);
          umma_commit(&bar_r_empty[(load + 2 * j) % DQ_RING]);
          umma_commit(&bar_dq_full);
          // the threads are done with dP(j): the next dP goes first so that they can start on tile j+1
          // while dQ(j) runs (dS(j) sits in the score buffer of tile j, not in the dP columns)
          if (j + 1 < n) {
            if (!ring_wait(load + 2 * (j + 1) + 1)) { ok = false; break; }
            issue_kk(256, do_addr, v_slot(j + 1));
            umma_commit(&bar_r_empty[(load + 2 * (j + 1) + 1) % DQ_RING]);
            umma_commit(&bar_dp_full);
            if (j + 1 == n - 1) umma_commit(&bar_q_empty);
          }
          if (j + 2 < n) {
            if (!ring_wait(load + 2 * (j + 2))) { ok = false; break; }
            issue_kk(((g + j + 2) & 1) * 128, q_addr, k_slot(j + 2));
            umma_commit(&bar_s_full[(g + j + 2) & 1]);
          }
        }
        load += 2 * n;
        g += n;
      }
      if (!ok) report(args.status, ST_TIMEOUT_MMA);
      umma_commit(&bar_drain);
      (void)mbar_wait_ns(&bar_drain, 0, FB_LIMIT_NS);
    }
  } else {
    const int q4 = warp & 3;
    const int half = (warp - 2) >> 2;
    const int row_l = q4 * 32 + lane;
    const uint32_t t_row = tmem + (static_cast<uint32_t>(q4 * 32) << 16);
    const float sl2 = args.scale_log2, scale = args.scale;
    bool ok = true;
    uint32_t g = 0;
    int it_count = 0;
    for (int t; (t = fb_sched(it_count, blockIdx.x, gridDim.x)) < args.items && ok; ++it_count) {
      const int qt = n_qt - 1 - t / per_qt, r = t % per_qt, b = r / args.nh, h = r % args.nh;
      const int n = qt + 1;
      const long long stat = (static_cast<long long>(b) * args.nh + h) * args.S + qt * 128 + row_l;
      const float lse2 = args.lse2[stat], dsc = args.dsc[stat];
      for (int j = 0; j < n; ++j, ++g) {
        if (!mbar_wait_ns(&bar_s_full[g & 1], (g >> 1) & 1, FB_LIMIT_NS) ||
            !mbar_wait_ns(&bar_dp_full, g & 1, FB_LIMIT_NS)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const bool diag = j == n - 1;
        uint32_t pk[32];
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t s[32], dp[32];
          tmem_ld_32x32(t_row + (g & 1) * 128 + half * 64 + c * 32, s);
          tmem_ld_32x32(t_row + 256 + half * 64 + c * 32, dp);
          tmem_ld_wait();
          float ds[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float x = fmaf(__uint_as_float(s[i]), sl2, -lse2);
            const float p = (i & 3) == 3 ? ex2_poly(x) : ex2_approx(x);
            ds[i] = p * fmaf(__uint_as_float(dp[i]), scale, -dsc);
            if (diag && half * 64 + c * 32 + i > row_l) ds[i] = 0.f;
          }
#pragma unroll
          for (int i = 0; i < 16; ++i) pk[c * 16 + i] = pack_bf16x2(ds[2 * i], ds[2 * i + 1]);
        }
        tmem_st_32x32(t_row + (g & 1) * 128 + half * 64, pk);  // over this thread's own score columns
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bar_ds_full);
      }
      if (!ok) break;
      if (!mbar_wait_ns(&bar_dq_full, (g - 1) & 1, FB_LIMIT_NS)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const long long row_g = static_cast<long long>(b) * args.S + qt * 128 + row_l;
      uint4* dst = reinterpret_cast<uint4*>(args.dq + (row_g * args.nh + h) * HD + half * (HD / 2));
#pragma unroll
      for (int hh = 0; hh < HD / 64; ++hh) {
        uint32_t rr[32];
        tmem_ld_32x32(t_row + 384 + half * (HD / 2) + hh * 32, rr);
        tmem_ld_wait();
#pragma unroll
        for (int c8 = 0; c8 < 4; ++c8)
          dst[hh * 4 + c8] = make_uint4(
              pack_bf16x2(__uint_as_float(rr[c8 * 8]), __uint_as_float(rr[c8 * 8 + 1])),
              pack_bf16x2(__uint_as_float(rr[c8 * 8 + 2]), __uint_as_float(rr[c8 * 8 + 3])),
              pack_bf16x2(__uint_as_float(rr[c8 * 8 + 4]), __uint_as_float(rr[c8 * 8 + 5])),
              pack_bf16x2(__uint_as_float(rr[c8 * 8 + 6]), __uint_as_float(rr[c8 * 8 + 7])));
      }
      tc_fence_before();
    }
    if (!ok) report(args.status, ST_TIMEOUT_EPILOGUE);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}


constexpr int FB_RING = 5;        // dK/dV ring slots, one sub-tile each: two half tiles of 64 rows (2 x 16 KB)
constexpr int FB_SLOT = 32768;
constexpr int FB_HALF = 16384;    // 64 rows x 128 columns bf16: [hd chunk 0: 64 rows x 128 B][hd chunk 1]

__device__ __forceinline__ uint32_t fb_a_col(int ks) { return ks < 2 ? ks * 8 : 32 + (ks - 2) * 8; }

// ----------------------------------------------------------------------------------------- dK, dV
template <int HD>
__global__ void __launch_bounds__(FB_THREADS, 1)
flash_bwd_dkv_kernel(const __grid_constant__ CUtensorMap mapQ64, const __grid_constant__ CUtensorMap mapK,
                     const __grid_constant__ CUtensorMap mapV, const __grid_constant__ CUtensorMap mapDO64,
                     const FbArgs args) {
  extern __shared__ uint8_t smem_raw[];
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = base;
  uint8_t* sV = base + FB_TILE;
  uint8_t* sR = base + 2 * FB_TILE;  // slot: {64 rows of Q_i, 64 rows of dO_i}
  float* sStat = reinterpret_cast<float*>(base + 7 * FB_TILE);  // [slot][lse2 x 64 | dsc x 64]
  uint64_t* bars = reinterpret_cast<uint64_t*>(base + 7 * FB_TILE + FB_RING * 512);
  uint64_t& bar_kv_full = bars[0];
  uint64_t& bar_kv_empty = bars[1];
  uint64_t* bar_r_full = bars + 2;    // [FB_RING]
  uint64_t* bar_r_empty = bars + 7;   // [FB_RING]
  uint64_t* bar_s_full = bars + 12;   // [2]
  uint64_t* bar_ds_full = bars + 14;  // [2]
  uint64_t& bar_acc_full = bars[16];
  uint64_t& bar_drain = bars[17];
  uint32_t& tmem_base_slot = *reinterpret_cast<uint32_t*>(bars + 18);
  int& go = *reinterpret_cast<int*>(bars + 19);

  if (threadIdx.x == 0) {
    go = 1;
    if (base + 7 * FB_TILE + FB_RING * 512 + 256 > smem_raw + FB_SMEM) {
      report(args.status, ST_BAD_ARGUMENT);
      go = 0;
    }
    tma_prefetch_desc(&mapQ64);
    tma_prefetch_desc(&mapK);
    tma_prefetch_desc(&mapV);
    tma_prefetch_desc(&mapDO64);
    mbar_init(&bar_kv_full, 1);
    mbar_init(&bar_kv_empty, 1);
    for (int s = 0; s < FB_RING; ++s) {
      mbar_init(&bar_r_full[s], 1);
      mbar_init(&bar_r_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bar_s_full[s], 1);
      mbar_init(&bar_ds_full[s], 8);
    }
    mbar_init(&bar_acc_full, 1);
    mbar_init(&bar_drain, 1);
    fence_mbar_init();
  }
  __syncthreads();
  if (!go) return;
  if (warp == 1) {
    tmem_alloc(&tmem_base_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_slot;
  // TMEM columns: S^T[2] at 0 / 64, dP^T[2] at 128 / 192, dV at 256, dK at 384
  constexpr int KC = HD / 64;
  constexpr int TILE_BYTES = 128 * HD * 2;
  const int group = args.nh / args.nkv;
  const int per_j = args.B * args.nkv;
  const int n_qt = args.S >> 7;
  // item t: key tile j = t / per_j (small j = many query tiles = heavy, first), then (batch, key/value head)

  if (warp == 0) {
    if (lane == 0) {
      bool ok = true;
      uint32_t u = 0;
      int it_count = 0;
      for (int t; (t = fb_sched(it_count, blockIdx.x, gridDim.x)) < args.items && ok; ++it_count) {
        if (*reinterpret_cast<volatile int*>(args.status) != 0) break;
        const int j = t / per_j, r = t % per_j, b = r / args.nkv, hk = r % args.nkv;
        if (!mbar_wait_ns(&bar_kv_empty, (it_count & 1) ^ 1u, FB_LIMIT_NS)) {
          ok = false;
          break;
        }
        mbar_expect_tx(&bar_kv_full, 2 * TILE_BYTES);
#pragma unroll
        for (int kc = 0; kc < KC; ++kc) {
          tma_load_3d(sK + kc * 16384, &mapK, &bar_kv_full, hk * HD + kc * 64, j * 128, b);
          tma_load_3d(sV + kc * 16384, &mapV, &bar_kv_full, hk * HD + kc * 64, j * 128, b);
        }
        for (int gi = 0; gi < group && ok; ++gi) {
          const int h = hk * group + gi;
          for (int row0 = j * 128; row0 < args.S; row0 += 64, ++u) {  // query rows of this sub-tile
            const int slot = u % FB_RING;
            if (!mbar_wait_ns(&bar_r_empty[slot], ((u / FB_RING) & 1) ^ 1u, FB_LIMIT_NS)) {
              ok = false;
              break;
            }
            mbar_expect_tx(&bar_r_full[slot], TILE_BYTES + 512);  // 64 rows of Q and of dO, two statistics rows
            uint8_t* dst = sR + slot * FB_SLOT;
#pragma unroll
            for (int kc = 0; kc < KC; ++kc) {
              tma_load_3d(dst + kc * 8192, &mapQ64, &bar_r_full[slot], h * HD + kc * 64, row0, b);
              tma_load_3d(dst + FB_HALF + kc * 8192, &mapDO64, &bar_r_full[slot], h * HD + kc * 64, row0, b);
            }
            const long long so = (static_cast<long long>(b) * args.nh + h) * args.S + row0;
            bulk_load_1d(sStat + slot * 128, args.lse2 + so, 256, &bar_r_full[slot]);
            bulk_load_1d(sStat + slot * 128 + 64, args.dsc + so, 256, &bar_r_full[slot]);
          }
        }
      }
      if (!ok) report(args.status, ST_TIMEOUT_PRODUCER);
      for (uint32_t i = u > FB_RING ? u - FB_RING : 0; i < u; ++i)
        (void)mbar_wait_ns(&bar_r_full[i % FB_RING], (i / FB_RING) & 1, FB_LIMIT_NS);
      if (it_count > 0) (void)mbar_wait_ns(&bar_kv_full, (it_count - 1) & 1, FB_LIMIT_NS);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(128, 64, 0, 0);
      constexpr uint32_t idesc_g = make_idesc_bf16(128, HD, 0, 1);
      bool ok = true;
      uint32_t u0 = 0;
      int it_count = 0;
      const uint32_t k_addr = smem_u32(sK), v_addr = smem_u32(sV);
      auto slot_addr = [&](uint32_t u) { return smem_u32(sR + (u % FB_RING) * FB_SLOT); };
      auto ring_wait = [&](uint32_t u) -> bool {
        const bool r = mbar_wait_ns(&bar_r_full[u % FB_RING], (u / FB_RING) & 1, FB_LIMIT_NS);
        tc_fence_after();
        return r;
      };
      auto mma1 = [&](uint32_t u) {  // S^T = K_j Q_sub^T, dP^T = V_j dO_sub^T
        const uint32_t buf = u & 1, qq = slot_addr(u), dd = qq + FB_HALF;
#pragma unroll
        for (int kc = 0; kc < KC; ++kc)
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            umma_bf16(tmem + buf * 64, make_smem_desc(k_addr + kc * 16384 + k * 32, 16, 1024),
                      make_smem_desc(qq + kc * 8192 + k * 32, 16, 1024), idesc_s, (kc | k) != 0 ? 1u : 0u);
            umma_bf16(tmem + 128 + buf * 64, make_smem_desc(v_addr + kc * 16384 + k * 32, 16, 1024),
                      make_smem_desc(dd + kc * 8192 + k * 32, 16, 1024), idesc_s, (kc | k) != 0 ? 1u : 0u);
          }
        umma_commit(&bar_s_full[buf]);
      };
      for (int t; (t = fb_sched(it_count, blockIdx.x, gridDim.x)) < args.items && ok; ++it_count) {
        const int j = t / per_j;
        const int subs = group * 2 * (n_qt - j);
        ok = mbar_wait_ns(&bar_kv_full, it_count & 1, FB_LIMIT_NS);
        if (!ok) break;
        tc_fence_after();
        if (!ring_wait(u0) || !ring_wait(u0 + 1)) { ok = false; break; }
        mma1(u0);
        mma1(u0 + 1);
        for (int m = 0; m < subs; ++m) {
          const uint32_t u = u0 + m, buf = u & 1;
          if (!mbar_wait_ns(&bar_ds_full[buf], (u >> 1) & 1, FB_LIMIT_NS)) { ok = false; break; }
          tc_fence_after();
          const uint32_t qq = slot_addr(u), dd = qq + FB_HALF;
          // dV += P^T dO_sub, dK += dS^T Q_sub : A from TMEM, B = the 64 query rows read MN-major
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) {
            umma_bf16_ts(tmem + 256, tmem + buf * 64 + fb_a_col(ks), make_smem_desc(dd + ks * 2048, 8192, 1024),
                         idesc_g, (m | ks) != 0 ? 1u : 0u);
            umma_bf16_ts(tmem + 384, tmem + 128 + buf * 64 + fb_a_col(ks), make_smem_desc(qq + ks * 2048, 8192, 1024),
                         idesc_g, (m | ks) != 0 ? 1u : 0u);
          }
          umma_commit(&bar_r_empty[u % FB_RING]);
          if (m == subs - 1) {
            umma_commit(&bar_acc_full);
            umma_commit(&bar_kv_empty);
          }
          if (m + 2 < subs) {
            if (!ring_wait(u + 2)) { ok = false; break; }
            mma1(u + 2);
          }
        }
        u0 += subs;
      }
      if (!ok) report(args.status, ST_TIMEOUT_MMA);
      umma_commit(&bar_drain);
      (void)mbar_wait_ns(&bar_drain, 0, FB_LIMIT_NS);
    }
  } else {
    const int q4 = warp & 3;
    const int half = (warp - 2) >> 2;
    const int row_l = q4 * 32 + lane;  // key row inside the tile
    const uint32_t t_row = tmem + (static_cast<uint32_t>(q4 * 32) << 16);
    const float sl2 = args.scale_log2, scale = args.scale;
    bool ok = true;
    uint32_t u = 0;
    int it_count = 0;
    for (int t; (t = fb_sched(it_count, blockIdx.x, gridDim.x)) < args.items && ok; ++it_count) {
      const int j = t / per_j, r = t % per_j, b = r / args.nkv, hk = r % args.nkv;
      const int per_head = 2 * (n_qt - j), subs = group * per_head;
      for (int m = 0; m < subs; ++m, ++u) {
        const uint32_t buf = u & 1;
        if (!mbar_wait_ns(&bar_s_full[buf], (u >> 1) & 1, FB_LIMIT_NS)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const float* stat = sStat + (u % FB_RING) * 128 + half * 32;
        // query tile == key tile (the first two sub-tiles of every head): query index must be >= key index
        const int mh = m % per_head;
        const int col0 = mh < 2 ? mh * 64 + half * 32 : 1024;
        uint32_t s[32], dp[32];
        tmem_ld_32x32(t_row + buf * 64 + half * 32, s);
        tmem_ld_32x32(t_row + 128 + buf * 64 + half * 32, dp);
        tmem_ld_wait();
        uint32_t pp[16], pd[16];
#pragma unroll
        for (int i4 = 0; i4 < 8; ++i4) {
          const float4 l4 = *reinterpret_cast<const float4*>(stat + i4 * 4);
          const float4 d4 = *reinterpret_cast<const float4*>(stat + 64 + i4 * 4);
          const float lv[4] = {l4.x, l4.y, l4.z, l4.w}, dv_[4] = {d4.x, d4.y, d4.z, d4.w};
          float pe[4], de[4];
#pragma unroll
          for (int e4 = 0; e4 < 4; ++e4) {
            const int c = i4 * 4 + e4;
            const float x = fmaf(__uint_as_float(s[c]), sl2, -lv[e4]);
            float p = e4 == 3 ? ex2_poly(x) : ex2_approx(x);
            if (col0 + c < row_l) p = 0.f;
            pe[e4] = p;
            de[e4] = p * fmaf(__uint_as_float(dp[c]), scale, -dv_[e4]);
          }
          pp[i4 * 2] = pack_bf16x2(pe[0], pe[1]);
          pp[i4 * 2 + 1] = pack_bf16x2(pe[2], pe[3]);
          pd[i4 * 2] = pack_bf16x2(de[0], de[1]);
          pd[i4 * 2 + 1] = pack_bf16x2(de[2], de[3]);
        }
        tmem_st_32x16(t_row + buf * 64 + half * 32, pp);
        tmem_st_32x16(t_row + 128 + buf * 64 + half * 32, pd);
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bar_ds_full[buf]);
      }
      if (!ok) break;
      if (!mbar_wait_ns(&bar_acc_full, it_count & 1, FB_LIMIT_NS)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const long long row_g = static_cast<long long>(b) * args.S + j * 128 + row_l;
      const long long off = (row_g * args.nkv + hk) * HD + half * (HD / 2);
#pragma unroll
      for (int which = 0; which < 2; ++which) {
        uint4* dst = reinterpret_cast<uint4*>((which ? args.dk : args.dv) + off);
#pragma unroll
        for (int hh = 0; hh < HD / 64; ++hh) {
          uint32_t rr[32];
          tmem_ld_32x32(t_row + 256 + which * 128 + half * (HD / 2) + hh * 32, rr);
          tmem_ld_wait();
#pragma unroll
          for (int c8 = 0; c8 < 4; ++c8)
            dst[hh * 4 + c8] = make_uint4(
                pack_bf16x2(__uint_as_float(rr[c8 * 8]), __uint_as_float(rr[c8 * 8 + 1])),
                pack_bf16x2(__uint_as_float(rr[c8 * 8 + 2]), __uint_as_float(rr[c8 * 8 + 3])),
                pack_bf16x2(__uint_as_float(rr[c8 * 8 + 4]), __uint_as_float(rr[c8 * 8 + 5])),
                pack_bf16x2(__uint_as_float(rr[c8 * 8 + 6]), __uint_as_float(rr[c8 * 8 + 7])));
        }
      }
      tc_fence_before();
    }
    if (!ok) report(args.status, ST_TIMEOUT_EPILOGUE);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

}  // namespace b200

using namespace b200;

template <int HD>
static int launch_flash_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o,
                            const float* lse, float* delta, void* dq, void* dk, void* dv, int B, int S, int nh,
                            int nkv, long long ldq, long long ldk, long long ldv, float softmax_scale, int* status,
                            cudaStream_t stream) {
  CUtensorMap mq, mk, mv, mdo, mq64, mdo64;
  const uint64_t qrow = static_cast<uint64_t>(nh) * HD, krow = static_cast<uint64_t>(nkv) * HD;
  const uint64_t pq = (ldq > 0 ? ldq : qrow) * 2, pk = (ldk > 0 ? ldk : krow) * 2, pv = (ldv > 0 ? ldv : krow) * 2;
  // a failing map is reported as -(100 + 10 * its position + the encoder's code)
  int rc = make_map(&mq, q, qrow, S, B, pq, pq * S, 64, 128);
  if (rc != 0) return rc - 100;
  rc = make_map(&mdo, d_o, qrow, S, B, qrow * 2, qrow * 2 * S, 64, 128);
  if (rc != 0) return rc - 110;
  rc = make_map(&mk, k, krow, S, B, pk, pk * S, 64, 128);
  if (rc != 0) return rc - 120;
  rc = make_map(&mv, v, krow, S, B, pv, pv * S, 64, 128);
  if (rc != 0) return rc - 130;
  rc = make_map(&mq64, q, qrow, S, B, pq, pq * S, 64, 64);
  if (rc != 0) return rc - 140;
  rc = make_map(&mdo64, d_o, qrow, S, B, qrow * 2, qrow * 2 * S, 64, 64);
  if (rc != 0) return rc - 150;
  static bool configured = false;
  static int sms = 0;
  if (!configured) {
    if (cudaFuncSetAttribute(flash_bwd_dq_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, FB_SMEM) !=
            cudaSuccess ||
        cudaFuncSetAttribute(flash_bwd_dkv_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, FB_SMEM) !=
            cudaSuccess)
      return -10;
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    configured = true;
  }
  const long long rows = static_cast<long long>(B) * S * nh;
  attn_delta_kernel<HD><<<static_cast<unsigned>((rows * (HD / 8) + 255) / 256), 256, 0, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(o), reinterpret_cast<const __nv_bfloat16*>(d_o), delta, B, S, nh,
      softmax_scale);
  FbArgs a;
  a.lse2 = lse;
  a.dsc = delta;
  a.dq = reinterpret_cast<__nv_bfloat16*>(dq);
  a.dk = reinterpret_cast<__nv_bfloat16*>(dk);
  a.dv = reinterpret_cast<__nv_bfloat16*>(dv);
  a.B = B; a.S = S; a.nh = nh; a.nkv = nkv;
  a.scale = softmax_scale;
  a.scale_log2 = softmax_scale * 1.4426950408889634f;
  a.status = status;
  a.items = B * nh * (S / 128);
  flash_bwd_dq_kernel<HD><<<a.items < sms ? a.items : sms, FB_THREADS, FB_SMEM, stream>>>(mq, mk, mv, mdo, a);
  a.items = B * nkv * (S / 128);
  flash_bwd_dkv_kernel<HD><<<a.items < sms ? a.items : sms, FB_THREADS, FB_SMEM, stream>>>(mq64, mk, mv, mdo64, a);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

extern "C" int b200_flash_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o,
                              const float* lse, float* delta, void* dq, void* dk, void* dv, int B, int S, int nh,
                              int nkv, int head_dim, long long ldq, long long ldk, long long ldv, float softmax_scale,
                              int* status, cudaStream_t stream) {
  if (B <= 0 || S <= 0 || (S & 127) != 0 || nh <= 0 || nkv <= 0 || nh % nkv != 0) return -1;
  if (head_dim == 128)
    return launch_flash_bwd<128>(q, k, v, o, d_o, lse, delta, dq, dk, dv, B, S, nh, nkv, ldq, ldk, ldv, softmax_scale, status,
                                 stream);
  if (head_dim == 64)
    return launch_flash_bwd<64>(q, k, v, o, d_o, lse, delta, dq, dk, dv, B, S, nh, nkv, ldq, ldk, ldv, softmax_scale, status,
                                stream);
  return -3;
}
