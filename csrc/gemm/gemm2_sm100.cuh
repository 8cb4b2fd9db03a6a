// Pair-tile member of the GEMM family: two CTAs on neighbouring SMs (a cluster of two) share one
// 256 x BN output tile through `tcgen05.mma.cta_group::2`.
//
//   * each CTA loads ITS half of both operands (128 rows of A, BN/2 rows or columns of B) with its own
//     ordinary TMA loads - no multicast anywhere - so a k-block costs every SM 32 KB of shared-memory
//     fill instead of 48 KB, and the tensor core reads half the B bytes per MMA;
//   * one thread of the even CTA issues the MMAs for the pair; each CTA ends up with its 128
//     accumulator rows in its own TMEM (2 x BN columns, double buffered);
//   * the epilogue warps of both CTAs convert their rows, stage 32-row pieces in 128-byte-swizzled
//     shared memory and write them with TMA stores (fp32 accumulation: TMA add), so global memory sees
//     full 128-byte lines instead of one row fragment per lane.
//
// Same warp roles, tile order, modes and epilogue semantics as `gemm_sm100_kernel`; the grouped-by-rows
// mode walks a list of pair tiles (start row, expert, 1 or 2 live halves) so that the 128-row padding of
// the expert-sorted layout stays as it is.
#pragma once
#include "gemm_sm100.cuh"

namespace b200 {

constexpr int GEMM2_BM = 256;  // rows of a pair tile

template <int BN, int EPI>
struct Gemm2Cfg {
  static constexpr int A_BYTES = 128 * GEMM_BK * 2;
  static constexpr int B_BYTES = (BN / 2) * GEMM_BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  // 4 KB staging buffers (32 rows x 128 B) per epilogue warp.  The SwiGLU backward also stages its INPUT
  // (the stored pre-activations) through shared memory: two double-buffered 4 KB tiles (gate, up) that TMA
  // fetches one 64-column piece ahead, plus two output tiles.
  static constexpr int RING = (EPI == EPI_SWIGLU) ? 3 : (EPI == EPI_SWIGLU_BWD) ? 6 : (EPI == EPI_QKROPE) ? 4 : 2;
  static constexpr int EPI_BYTES = 4 * RING * 4096;
  static constexpr int STAGES_FIT = (232448 - 1024 - 512 - EPI_BYTES) / STAGE_BYTES;
  static constexpr int STAGES = STAGES_FIT > 8 ? 8 : STAGES_FIT;
  static constexpr int TMEM_COLS = 2 * BN;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + EPI_BYTES + 1024;
};

struct Tile2 {
  int m0, n_idx, e, k0, num_kb, halves;
};

__device__ __forceinline__ void decode_tile2(const GemmArgs& a, int t, int m_tiles, int n_tiles, Tile2& ti) {
  int r = t;
  ti.e = 0;
  ti.halves = 2;
  if (a.mode == MODE_GROUPED_K) {
    const int per = m_tiles * n_tiles;
    ti.e = t / per;
    r = t - ti.e * per;
  }
  int m_idx, n_idx;
  if (a.m_fast) {
    n_idx = r / m_tiles;
    m_idx = r - n_idx * m_tiles;
  } else {
    m_idx = r / n_tiles;
    n_idx = r - m_idx * n_tiles;
  }
  ti.m0 = m_idx * GEMM2_BM;
  ti.n_idx = n_idx;
  if (a.mode == MODE_GROUPED_K) {
    ti.k0 = a.seg_off[ti.e];
    ti.num_kb = (a.seg_off[ti.e + 1] - ti.k0) / GEMM_BK;
  } else {
    ti.k0 = 0;
    ti.num_kb = (a.K + GEMM_BK - 1) / GEMM_BK;
    if (a.mode == MODE_GROUPED_M) {
      const int2 p = reinterpret_cast<const int2*>(a.pair_tiles)[m_idx];
      ti.m0 = p.x;
      ti.e = p.y & 0xffff;
      ti.halves = p.y >> 16;
    }
  }
}

// lane r of an epilogue warp owns row r of a 32-row x 128-byte staging buffer (1024-byte aligned);
// 16-byte chunk c of the row sits at position c ^ (r & 7): the layout TMA expects for SWIZZLE_128B.
__device__ __forceinline__ void stage_write(uint8_t* buf, int lane, int chunk, uint4 v) {
  *reinterpret_cast<uint4*>(buf + lane * 128 + ((chunk ^ (lane & 7)) << 4)) = v;
}

template <int BN, bool A_MN, bool B_MN, int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GEMM_THREADS, 1)
gemm2_sm100_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
                   const __grid_constant__ CUtensorMap mapC, const __grid_constant__ CUtensorMap mapX,
                   const GemmArgs args) {
  using Cfg = Gemm2Cfg<BN, EPI>;
  constexpr int STAGES = Cfg::STAGES;
  constexpr int RING = Cfg::RING;
  constexpr int BN_OUT = (EPI == EPI_SWIGLU) ? BN / 2 : BN;  // output columns per tile
  constexpr int BH = BN / 2;                                 // B rows (or columns) loaded by one CTA

  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t bar_full[STAGES];   // used in the even CTA: both CTAs' loads of a stage have landed
  __shared__ uint64_t bar_empty[STAGES];  // in each CTA: the pair's MMAs have consumed the stage
  __shared__ uint64_t bar_tfull[2];       // in each CTA: accumulator buffer complete
  __shared__ uint64_t bar_tempty[2];      // used in the even CTA: all 8 epilogue warps of the pair have drained it
  __shared__ uint64_t bar_in[4][3];       // SwiGLU backward: per epilogue warp and buffer, pre-activation tile landed
  __shared__ uint32_t tmem_base_slot;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* epi_smem = tiles + STAGES * Cfg::STAGE_BYTES;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&mapA);
    tma_prefetch_desc(&mapB);
    tma_prefetch_desc(&mapC);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&bar_full[s], 1);
      mbar_init(&bar_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bar_tfull[s], 1);
      mbar_init(&bar_tempty[s], 8);
    }
    for (int s = 0; s < 12; ++s) mbar_init(&bar_in[s / 3][s % 3], 1);
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc2(&tmem_base_slot, Cfg::TMEM_COLS);
    tmem_relinquish2();
  }
  tc_fence_before();
  __syncthreads();
  // barrier initialisation and TMEM allocation of both CTAs are visible to both before any remote arrive
  cluster_arrive();
  cluster_wait();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;

  int m_tiles;
  if (args.mode == MODE_GROUPED_M) {
    m_tiles = *args.num_m_tiles;
    const int cap = args.max_pair_tiles;
    m_tiles = m_tiles < 0 ? 0 : (m_tiles > cap ? cap : m_tiles);
  } else {
    m_tiles = (args.M + GEMM2_BM - 1) / GEMM2_BM;
  }
  const int n_tiles = (args.N + BN_OUT - 1) / BN_OUT;
  const int total = (args.mode == MODE_GROUPED_K ? args.num_experts : 1) * m_tiles * n_tiles;
  const int first = blockIdx.x >> 1;
  const int step = gridDim.x >> 1;

  if (warp == 0 && (args.a_gather != nullptr || args.b_gather != nullptr)) {
    // ------------------------------------------------ producer with gathered operand rows (both CTAs)
    // All 32 lanes issue: a 128-row operand tile is 32 gather4 copies of four rows each, one per lane.
    const uint32_t full0 = mapa_shared(smem_u32(&bar_full[0]), 0);
    constexpr int OOB = 0x7f7f7f7f;
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    if (args.ep.wait_flags != nullptr && first < total) {
      if (lane == 0) {
        const int epoch = *args.ep.epoch_base + args.ep.wait_epoch_off;
        for (int r = 0; r < args.ep.wait_n && ok; ++r) ok = wait_flag_ge(args.ep.wait_flags + r, epoch, args.ep.limit_ns);
        if (!ok) report(args.status, ST_TIMEOUT_PEER);
      }
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      asm volatile("fence.proxy.async;" ::: "memory");
    }
    for (int t = first; t < total && ok; t += step) {
      Tile2 ti;
      decode_tile2(args, t, m_tiles, n_tiles, ti);
      const int eb = (args.mode == MODE_GROUPED_K) ? 0 : ti.e;
      const int n0 = ti.n_idx * BN_OUT;
      const int am0 = ti.m0 + static_cast<int>(rank) * 128;
      int4 aidx = make_int4(OOB, OOB, OOB, OOB);
      if constexpr (!A_MN) {
        if (args.a_gather != nullptr && am0 + lane * 4 + 3 < args.M)
          aidx = *reinterpret_cast<const int4*>(args.a_gather + am0 + lane * 4);
      }
      for (int kb = 0; kb < ti.num_kb; ++kb) {
        if (!mbar_wait(&bar_empty[stage], phase ^ 1u)) {
          if (lane == 0) report(args.status, ST_TIMEOUT_PRODUCER);
          ok = false;
          break;
        }
        if (leader && lane == 0) mbar_expect_tx(&bar_full[stage], 2 * Cfg::STAGE_BYTES);
        const uint32_t fb = full0 + static_cast<uint32_t>(stage) * 8u;
        uint8_t* sa = tiles + stage * Cfg::STAGE_BYTES;
        uint8_t* sb = sa + Cfg::A_BYTES;
        const int kk = ti.k0 + kb * GEMM_BK;
        if (args.a_gather != nullptr) {
          if constexpr (!A_MN) {  // K-major A: 128 rows of 64 contraction elements, rows named by output row
            tma2_gather4(sa + lane * 512, &mapA, fb, kk, aidx.x, aidx.y, aidx.z, aidx.w);
          } else {  // MN-major A: two sub-tiles of 64 contraction rows x 64 columns, rows named by contraction row
            const int j = lane >> 4, l16 = lane & 15;
            const int4 kidx = *reinterpret_cast<const int4*>(args.a_gather + kk + l16 * 4);
            tma2_gather4(sa + j * 8192 + l16 * 512, &mapA, fb, am0 + 64 * j, kidx.x, kidx.y, kidx.z, kidx.w);
          }
        } else if (lane == 0) {
          if constexpr (!A_MN) {
            tma2_load_2d(sa, &mapA, fb, kk, am0);
          } else {
            tma2_load_2d(sa, &mapA, fb, am0, kk);
            tma2_load_2d(sa + 8192, &mapA, fb, am0 + 64, kk);
          }
        }
        if (args.b_gather != nullptr) {
          // MN-major B: BH / 64 sub-tiles of 64 contraction rows x 64 columns; 16 lanes per sub-tile
          if constexpr (B_MN && BH == 128) {
            const int j = lane >> 4, l16 = lane & 15;
            const int4 bidx = *reinterpret_cast<const int4*>(args.b_gather + kk + l16 * 4);
            tma2_gather4(sb + j * 8192 + l16 * 512, &mapB, fb, n0 + static_cast<int>(rank) * BH + 64 * j, bidx.x,
                         bidx.y, bidx.z, bidx.w);
          }
        } else if (lane == 0) {
          if constexpr (!B_MN) {
            int brow;
            if constexpr (EPI == EPI_SWIGLU) {
              brow = leader ? n0 : args.n_half + n0;
            } else {
              brow = n0 + static_cast<int>(rank) * BH;
            }
            tma2_load_3d(sb, &mapB, fb, kk, brow, eb);
          } else {
#pragma unroll
            for (int j = 0; j < BH / 64; ++j)
              tma2_load_3d(sb + j * 8192, &mapB, fb, n0 + static_cast<int>(rank) * BH + 64 * j, kk, eb);
          }
        }
        __syncwarp();
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
    for (int i = 0; i < STAGES; ++i) {
      (void)mbar_wait(&bar_empty[stage], phase ^ 1u);
      if (++stage == STAGES) {
        stage = 0;
        phase ^= 1u;
      }
    }
  } else if (warp == 0) {
    // ------------------------------------------------------------ producer (both CTAs)
    if (lane == 0) {
      const uint32_t full0 = mapa_shared(smem_u32(&bar_full[0]), 0);  // the even CTA's bar_full[0]
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      if (args.ep.wait_flags != nullptr && first < total) {
        const int epoch = *args.ep.epoch_base + args.ep.wait_epoch_off;
        for (int r = 0; r < args.ep.wait_n && ok; ++r) ok = wait_flag_ge(args.ep.wait_flags + r, epoch, args.ep.limit_ns);
        if (!ok) report(args.status, ST_TIMEOUT_PEER);
        asm volatile("fence.proxy.async;" ::: "memory");
      }
      for (int t = first; t < total && ok; t += step) {
        Tile2 ti;
        decode_tile2(args, t, m_tiles, n_tiles, ti);
        const int eb = (args.mode == MODE_GROUPED_K) ? 0 : ti.e;
        const int n0 = ti.n_idx * BN_OUT;
        const int am0 = ti.m0 + static_cast<int>(rank) * 128;
        for (int kb = 0; kb < ti.num_kb; ++kb) {
          if (!mbar_wait(&bar_empty[stage], phase ^ 1u)) {
            report(args.status, ST_TIMEOUT_PRODUCER);
            ok = false;
            break;
          }
          if (leader) mbar_expect_tx(&bar_full[stage], 2 * Cfg::STAGE_BYTES);
          const uint32_t fb = full0 + static_cast<uint32_t>(stage) * 8u;
          uint8_t* sa = tiles + stage * Cfg::STAGE_BYTES;
          uint8_t* sb = sa + Cfg::A_BYTES;
          const int kk = ti.k0 + kb * GEMM_BK;
          if constexpr (!A_MN) {
            tma2_load_2d(sa, &mapA, fb, kk, am0);
          } else {
            tma2_load_2d(sa, &mapA, fb, am0, kk);
            tma2_load_2d(sa + 8192, &mapA, fb, am0 + 64, kk);
          }
          if constexpr (!B_MN) {
            int brow;
            if constexpr (EPI == EPI_SWIGLU) {
              brow = leader ? n0 : args.n_half + n0;  // even CTA: gate rows, odd CTA: up rows
            } else {
              brow = n0 + static_cast<int>(rank) * BH;
            }
            tma2_load_3d(sb, &mapB, fb, kk, brow, eb);
          } else {
#pragma unroll
            for (int j = 0; j < BH / 64; ++j)
              tma2_load_3d(sb + j * 8192, &mapB, fb, n0 + static_cast<int>(rank) * BH + 64 * j, kk, eb);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      // Stay until the pair's MMAs have released every stage: their completion arrives on this CTA's
      // barriers from the other CTA, and copies in flight must have landed before shared memory goes away.
      for (int i = 0; i < STAGES; ++i) {
        (void)mbar_wait(&bar_empty[stage], phase ^ 1u);
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------- MMA issuer (even CTA only)
    if (lane == 0 && leader) {
      constexpr uint32_t idesc = make_idesc_bf16(GEMM2_BM, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      const uint32_t empty_own = smem_u32(&bar_empty[0]);
      const uint32_t empty_peer = mapa_shared(empty_own, 1);
      const uint32_t tfull_own = smem_u32(&bar_tfull[0]);
      const uint32_t tfull_peer = mapa_shared(tfull_own, 1);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = first; t < total && ok; t += step) {
        Tile2 ti;
        decode_tile2(args, t, m_tiles, n_tiles, ti);
        if (!mbar_wait(&bar_tempty[acc], acc_phase ^ 1u)) {
          report(args.status, ST_TIMEOUT_MMA);
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BN);
        for (int kb = 0; kb < ti.num_kb; ++kb) {
          if (!mbar_wait(&bar_full[stage], phase)) {
            report(args.status, ST_TIMEOUT_MMA);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(tiles + stage * Cfg::STAGE_BYTES);
          const uint32_t b_addr = a_addr + Cfg::A_BYTES;
#pragma unroll
          for (int k = 0; k < GEMM_BK / 16; ++k) {
            const uint64_t adesc =
                A_MN ? make_smem_desc(a_addr + k * 2048, 8192, 1024) : make_smem_desc(a_addr + k * 32, 16, 1024);
            const uint64_t bdesc =
                B_MN ? make_smem_desc(b_addr + k * 2048, 8192, 1024) : make_smem_desc(b_addr + k * 32, 16, 1024);
            umma2_bf16(d_tmem, adesc, bdesc, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma2_commit(empty_own + static_cast<uint32_t>(stage) * 8u);
          umma2_commit(empty_peer + static_cast<uint32_t>(stage) * 8u);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        umma2_commit(tfull_own + static_cast<uint32_t>(acc) * 8u);
        umma2_commit(tfull_peer + static_cast<uint32_t>(acc) * 8u);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (both CTAs)
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    const uint32_t lane_base = static_cast<uint32_t>(q * 32) << 16;
    const uint32_t tempty0 = mapa_shared(smem_u32(&bar_tempty[0]), 0);
    uint8_t* ring = epi_smem + q * (RING * 4096);
    int slot = 0;
    int acc = 0;
    uint32_t acc_phase = 0;
    int in_buf = 0;            // SwiGLU backward: buffer the next pre-activation piece goes to
    uint32_t in_phase = 0;     // bit b = parity of the next completion of bar_in[q][b]
    for (int t = first; t < total; t += step) {
      Tile2 ti;
      decode_tile2(args, t, m_tiles, n_tiles, ti);
      const int row0 = ti.m0 + static_cast<int>(rank) * 128 + q * 32;  // first row of this warp's piece
      const long long row_g = static_cast<long long>(row0) + lane;
      // grouped by rows: the odd CTA's half of a pair tile may lie past the expert's segment
      const bool live = leader || ti.halves == 2;
      const bool row_ok = live && row_g < args.M;
      const int n0 = ti.n_idx * BN_OUT;
      if constexpr (EPI == EPI_SWIGLU_BWD) {
        // fetch the first 64-column piece of the stored pre-activations while the MMAs of the tile still run
        if (live && n0 < args.N && lane == 0) {
          uint64_t* b = &bar_in[q][in_buf];
          bulk_wait_read<1>();  // the store that last read this buffer (three pieces ago) is done with it
          mbar_expect_tx(b, 8192);
          tma_load_3d(ring + in_buf * 8192, &mapC, b, n0, row0, 0);         // gate columns
          tma_load_3d(ring + in_buf * 8192 + 4096, &mapC, b, n0, row0, 1);  // up columns
        }
      }
      if (!mbar_wait(&bar_tfull[acc], acc_phase)) {
        report(args.status, ST_TIMEOUT_EPILOGUE);
        break;
      }
      tc_fence_after();
      const uint32_t t_acc = tmem_base + lane_base + static_cast<uint32_t>(acc * BN);

      if constexpr (EPI == EPI_BF16 || EPI == EPI_LSE) {
        float run_max = -INFINITY, run_sum = 0.f;
#pragma unroll 1
        for (int c = 0; c < BN / 64; ++c) {
          const int cbase = n0 + c * 64;
          if (cbase >= args.N) break;
          uint8_t* buf = ring + slot * 4096;
          if (live) {
            if (lane == 0) bulk_wait_read<RING - 1>();
            __syncwarp();
          }
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int col0 = cbase + h * 32;
            if (col0 >= args.N) break;
            uint32_t r[32];
            tmem_ld_32x32(t_acc + c * 64 + h * 32, r);
            tmem_ld_wait();
            uint32_t p[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) p[j] = pack_bf16x2(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
            if constexpr (EPI == EPI_LSE) {
              // statistics of the bf16-rounded logits, valid columns only
              constexpr float kLog2e = 1.4426950408889634f;
              if (col0 + 32 <= args.N) {
                // two values per issue slot (f32x2) and four independent partial sums
                float cmax = -INFINITY;
                uint64_t v2[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                  const float2 f = unpack_bf16x2(p[j]);
                  v2[j] = pack2(f.x, f.y);
                  cmax = fmax3(cmax, f.x, f.y);
                }
                const float new_max = fmaxf(run_max, cmax);
                const float nm = -new_max * kLog2e;
                const uint64_t l2 = pack2(kLog2e, kLog2e), nm2 = pack2(nm, nm);
                uint64_t acc2[4] = {0ull, 0ull, 0ull, 0ull};
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                  float xl, xh;
                  unpack2(fma2(v2[j], l2, nm2), xl, xh);
                  acc2[j & 3] = add2(acc2[j & 3], pack2(ex2_approx(xl), ex2_approx(xh)));
                }
                float a0, a1, a2, a3, a4, a5, a6, a7;
                unpack2(acc2[0], a0, a1);
                unpack2(acc2[1], a2, a3);
                unpack2(acc2[2], a4, a5);
                unpack2(acc2[3], a6, a7);
                const float ssum = ((a0 + a1) + (a2 + a3)) + ((a4 + a5) + (a6 + a7));
                run_sum = run_sum * ex2_approx((run_max - new_max) * kLog2e) + ssum;
                run_max = new_max;
              } else {
                float v[32];
                float cmax = -INFINITY;
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                  const float2 f = unpack_bf16x2(p[j]);
                  v[2 * j] = (col0 + 2 * j < args.N) ? f.x : -INFINITY;
                  v[2 * j + 1] = (col0 + 2 * j + 1 < args.N) ? f.y : -INFINITY;
                  cmax = fmax3(cmax, v[2 * j], v[2 * j + 1]);
                }
                const float new_max = fmaxf(run_max, cmax);
                const float nm = -new_max * kLog2e;
                float ssum = 0.f;
#pragma unroll
                for (int j = 0; j < 32; ++j) ssum += ex2_approx(fmaf(v[j], kLog2e, nm));
                run_sum = run_sum * ex2_approx((run_max - new_max) * kLog2e) + ssum;
                run_max = new_max;
              }
            }
            if (live) {
#pragma unroll
              for (int j = 0; j < 4; ++j)
                stage_write(buf, lane, h * 4 + j, make_uint4(p[4 * j], p[4 * j + 1], p[4 * j + 2], p[4 * j + 3]));
            }
          }
          if (live) {
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              tma_store_3d(&mapC, buf, cbase, row0, 0);
              bulk_commit();
            }
            slot = (slot + 1 == RING) ? 0 : slot + 1;
          }
        }
        if constexpr (EPI == EPI_LSE) {
          if (row_ok) {
            float2* part = reinterpret_cast<float2*>(args.aux0);
            part[row_g * n_tiles + ti.n_idx] = make_float2(run_max, run_sum);
          }
        }
      } else if constexpr (EPI == EPI_QKROPE) {
        // A 256-column tile is two heads of 128.  Per head: (a) the raw projection goes out as in the bf16 epilogue
        // while the sum of squares of the stored (bf16-rounded) values is taken; (b) for q and k heads the columns
        // are read from TMEM again in rotate-half pairs (i, i + 64), normalised, weighted and rotated, and the
        // result is stored to the second output; v heads are copied there from the same staging buffers.
        const int nqk = args.rope_nh + args.rope_nkv;
        const int pos = row_ok ? static_cast<int>(row_g % args.rope_S) : 0;
#pragma unroll 1
        for (int hh = 0; hh < BN / 128; ++hh) {
          const int cb = n0 + hh * 128;
          if (cb >= args.N) break;
          const int head = cb >> 7;
          const bool is_v = head >= nqk;
          float ss = 0.f;
#pragma unroll 1
          for (int half = 0; half < 2; ++half) {
            uint8_t* buf = ring + slot * 4096;
            if (live) {
              if (lane == 0) bulk_wait_read<RING - 1>();
              __syncwarp();
            }
#pragma unroll
            for (int c2 = 0; c2 < 2; ++c2) {
              uint32_t r[32];
              tmem_ld_32x32(t_acc + hh * 128 + half * 64 + c2 * 32, r);
              tmem_ld_wait();
              uint32_t p[16];
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                p[j] = pack_bf16x2(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
                const float2 f = unpack_bf16x2(p[j]);
                ss = fmaf(f.x, f.x, ss);
                ss = fmaf(f.y, f.y, ss);
              }
              if (live) {
#pragma unroll
                for (int j = 0; j < 4; ++j)
                  stage_write(buf, lane, c2 * 4 + j, make_uint4(p[4 * j], p[4 * j + 1], p[4 * j + 2], p[4 * j + 3]));
              }
            }
            if (live) {
              fence_proxy_async_smem();
              __syncwarp();
              if (lane == 0) {
                tma_store_3d(&mapC, buf, cb + half * 64, row0, 0);
                if (is_v) tma_store_3d(&mapX, buf, cb + half * 64, row0, 0);
                bulk_commit();
              }
              slot = (slot + 1 == RING) ? 0 : slot + 1;
            }
          }
          if (is_v) continue;
          const float rstd = rsqrtf(ss * (1.0f / 128.0f) + args.rope_eps);
          if (row_ok) args.rope_rstd[row_g * nqk + head] = rstd;
          const float* wv = head < args.rope_nh ? args.rope_w : args.rope_kw;
          const float* csr = args.rope_cs + static_cast<size_t>(pos) * 128;  // 64 (cos, sin) pairs
          uint8_t* buf_lo = ring + slot * 4096;
          const int slot_hi = (slot + 1 == RING) ? 0 : slot + 1;
          uint8_t* buf_hi = ring + slot_hi * 4096;
          if (live) {
            if (lane == 0) bulk_wait_read<RING - 2>();
            __syncwarp();
          }
#pragma unroll 1
          for (int c = 0; c < 2; ++c) {
            uint32_t lo[32], hi[32];
            tmem_ld_32x32(t_acc + hh * 128 + c * 32, lo);
            tmem_ld_32x32(t_acc + hh * 128 + 64 + c * 32, hi);
            tmem_ld_wait();
            uint32_t plo[16], phi[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int i = c * 32 + 2 * j;  // frequency index of the pair's first element
              // values as stored (bf16), normalised and rounded again, then weighted: the unfused module sequence
              const float2 xl = unpack_bf16x2(pack_bf16x2(__uint_as_float(lo[2 * j]), __uint_as_float(lo[2 * j + 1])));
              const float2 xh = unpack_bf16x2(pack_bf16x2(__uint_as_float(hi[2 * j]), __uint_as_float(hi[2 * j + 1])));
              const float2 nl = unpack_bf16x2(pack_bf16x2(xl.x * rstd, xl.y * rstd));
              const float2 nh2 = unpack_bf16x2(pack_bf16x2(xh.x * rstd, xh.y * rstd));
              const float2 wl = *reinterpret_cast<const float2*>(wv + i);
              const float2 wh = *reinterpret_cast<const float2*>(wv + 64 + i);
              const float4 cs4 = *reinterpret_cast<const float4*>(csr + 2 * i);  // cos_i, sin_i, cos_i+1, sin_i+1
              const float l0 = nl.x * wl.x, l1 = nl.y * wl.y, h0 = nh2.x * wh.x, h1 = nh2.y * wh.y;
              plo[j] = pack_bf16x2(l0 * cs4.x - h0 * cs4.y, l1 * cs4.z - h1 * cs4.w);
              phi[j] = pack_bf16x2(h0 * cs4.x + l0 * cs4.y, h1 * cs4.z + l1 * cs4.w);
            }
            if (live) {
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                stage_write(buf_lo, lane, c * 4 + j, make_uint4(plo[4 * j], plo[4 * j + 1], plo[4 * j + 2], plo[4 * j + 3]));
                stage_write(buf_hi, lane, c * 4 + j, make_uint4(phi[4 * j], phi[4 * j + 1], phi[4 * j + 2], phi[4 * j + 3]));
              }
            }
          }
          if (live) {
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              tma_store_3d(&mapX, buf_lo, cb, row0, 0);
              bulk_commit();
              tma_store_3d(&mapX, buf_hi, cb + 64, row0, 0);
              bulk_commit();
            }
            slot = (slot_hi + 1 == RING) ? 0 : slot_hi + 1;
          }
        }
      } else if constexpr (EPI == EPI_F32) {
        const bool empty_acc = ti.num_kb == 0;
        if (live && !(empty_acc && args.beta)) {
#pragma unroll 1
          for (int c = 0; c < BN / 32; ++c) {
            const int col0 = n0 + c * 32;
            if (col0 >= args.N) break;
            uint32_t r[32];
            tmem_ld_32x32(t_acc + c * 32, r);
            tmem_ld_wait();
            if (empty_acc) {
#pragma unroll
              for (int j = 0; j < 32; ++j) r[j] = 0u;
            }
            uint8_t* buf = ring + slot * 4096;
            if (lane == 0) bulk_wait_read<RING - 1>();
            __syncwarp();
#pragma unroll
            for (int j = 0; j < 8; ++j) stage_write(buf, lane, j, make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]));
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              if (args.beta)
                tma_reduce_add_3d(&mapC, buf, col0, row0, ti.e);
              else
                tma_store_3d(&mapC, buf, col0, row0, ti.e);
              bulk_commit();
            }
            slot = (slot + 1 == RING) ? 0 : slot + 1;
          }
        }
      } else if constexpr (EPI == EPI_SWIGLU) {
        // accumulator columns [0, BN/2) = gate, [BN/2, BN) = up, for output columns n0 .. n0+BN/2.
        // Three staging buffers (activation, gate, up) are filled over two 32-column halves.
        float wr = 1.f;  // routing weight of this lane's row, folded into the stored activation when given
        if (args.row_w != nullptr) {
          wr = 0.f;
          if (row_ok) {
            const int sl = args.row_slot[row_g];
            if (sl >= 0) wr = args.row_w[sl];
          }
        }
#pragma unroll 1
        for (int c = 0; c < BN / 128; ++c) {
          const int cbase = n0 + c * 64;
          if (cbase >= args.N) break;
          if (live) {
            if (lane == 0) bulk_wait_read<0>();
            __syncwarp();
          }
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int col0 = cbase + h * 32;
            if (col0 >= args.N) break;
            uint32_t g[32], u[32];
            tmem_ld_32x32(t_acc + c * 64 + h * 32, g);
            tmem_ld_32x32(t_acc + BN / 2 + c * 64 + h * 32, u);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint32_t pg[4], pu[4], pa[4];
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                pg[i] = pack_bf16x2(__uint_as_float(g[8 * j + 2 * i]), __uint_as_float(g[8 * j + 2 * i + 1]));
                pu[i] = pack_bf16x2(__uint_as_float(u[8 * j + 2 * i]), __uint_as_float(u[8 * j + 2 * i + 1]));
                // activation from the bf16-rounded pre-activations, so that backward sees the same values
                const float2 gf = unpack_bf16x2(pg[i]);
                const float2 uf = unpack_bf16x2(pu[i]);
                pa[i] = pack_bf16x2(wr * gf.x * sigmoidf_fast(gf.x) * uf.x, wr * gf.y * sigmoidf_fast(gf.y) * uf.y);
              }
              if (live) {
                stage_write(ring, lane, h * 4 + j, make_uint4(pa[0], pa[1], pa[2], pa[3]));
                stage_write(ring + 4096, lane, h * 4 + j, make_uint4(pg[0], pg[1], pg[2], pg[3]));
                stage_write(ring + 8192, lane, h * 4 + j, make_uint4(pu[0], pu[1], pu[2], pu[3]));
              }
            }
          }
          if (live) {
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              tma_store_3d(&mapC, ring, cbase, row0, 0);         // activation [rows, I]
              tma_store_3d(&mapX, ring + 4096, cbase, row0, 0);  // pre-activations [2][rows][I]: gate
              tma_store_3d(&mapX, ring + 8192, cbase, row0, 1);  // up
              bulk_commit();
            }
          }
        }
      } else if constexpr (EPI == EPI_SWIGLU_BWD) {
        // ring of this warp: three buffers [gate 32 x 128 B][up 32 x 128 B].  A piece is loaded into a buffer, its
        // gradients are written over it in place (every thread overwrites exactly the chunks it has read) and
        // stored from there, so a buffer is free again once the store issued three pieces ago has read it:
        // neither the load of the next piece nor the stores ever wait for each other.
        bool ok_in = true;
        float wr = 1.f, rdot = 0.f;
        if (args.row_w != nullptr) {
          wr = 0.f;
          if (row_ok) {
            const int sl = args.row_slot[row_g];
            if (sl >= 0) wr = args.row_w[sl];
          }
        }
#pragma unroll 1
        for (int c = 0; c < BN / 64 && ok_in; ++c) {
          const int cbase = n0 + c * 64;
          if (cbase >= args.N) break;
          uint8_t* inb = ring + in_buf * 8192;
          const int nxt = in_buf == 2 ? 0 : in_buf + 1;
          if (live) {
            __syncwarp();
            if (lane == 0 && c + 1 < BN / 64 && cbase + 64 < args.N) {  // next piece of this tile
              uint64_t* b = &bar_in[q][nxt];
              bulk_wait_read<1>();  // all stores but the latest have read their buffers: `nxt` is free
              mbar_expect_tx(b, 8192);
              tma_load_3d(ring + nxt * 8192, &mapC, b, cbase + 64, row0, 0);
              tma_load_3d(ring + nxt * 8192 + 4096, &mapC, b, cbase + 64, row0, 1);
            }
            ok_in = mbar_wait(&bar_in[q][in_buf], (in_phase >> in_buf) & 1u);
            in_phase ^= 1u << in_buf;
            __syncwarp();
            if (!ok_in) {
              report(args.status, ST_TIMEOUT_EPILOGUE);
              break;
            }
          }
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int col0 = cbase + h * 32;
            if (col0 >= args.N) break;
            uint32_t r[32];
            tmem_ld_32x32(t_acc + c * 64 + h * 32, r);
            tmem_ld_wait();
            if (live) {
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const int pos = ((h * 4 + j) ^ (lane & 7)) << 4;
                const uint4 gq = *reinterpret_cast<const uint4*>(inb + lane * 128 + pos);
                const uint4 uq = *reinterpret_cast<const uint4*>(inb + 4096 + lane * 128 + pos);
                const uint32_t gw[4] = {gq.x, gq.y, gq.z, gq.w};
                const uint32_t uw[4] = {uq.x, uq.y, uq.z, uq.w};
                uint32_t og[4], ou[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  const float2 gf = unpack_bf16x2(gw[i]);
                  const float2 uf = unpack_bf16x2(uw[i]);
                  float d0 = __uint_as_float(r[8 * j + 2 * i]);
                  float d1 = __uint_as_float(r[8 * j + 2 * i + 1]);
                  const float s0 = sigmoidf_fast(gf.x), s1 = sigmoidf_fast(gf.y);
                  // gradient of the routing weight: <d(weighted activation), activation> (columns < N only)
                  if (col0 + 8 * j + 2 * i < args.N) rdot += d0 * gf.x * s0 * uf.x + d1 * gf.y * s1 * uf.y;
                  d0 *= wr;
                  d1 *= wr;
                  og[i] = pack_bf16x2(d0 * uf.x * s0 * (1.f + gf.x * (1.f - s0)),
                                      d1 * uf.y * s1 * (1.f + gf.y * (1.f - s1)));
                  ou[i] = pack_bf16x2(d0 * gf.x * s0, d1 * gf.y * s1);
                }
                stage_write(inb, lane, h * 4 + j, make_uint4(og[0], og[1], og[2], og[3]));
                stage_write(inb + 4096, lane, h * 4 + j, make_uint4(ou[0], ou[1], ou[2], ou[3]));
              }
            }
          }
          if (live) {
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              tma_store_3d(&mapX, inb, cbase, row0, 0);         // d(pre-activations) [2][rows][I]: gate
              tma_store_3d(&mapX, inb + 4096, cbase, row0, 1);  // up
              bulk_commit();
            }
            in_buf = nxt;
          }
        }
        if (args.row_dot != nullptr && row_ok) args.row_dot[row_g * n_tiles + ti.n_idx] = rdot;
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(tempty0 + static_cast<uint32_t>(acc) * 8u);
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
    // the staging buffers must have been read before shared memory goes away
    if (lane == 0) bulk_wait_read<0>();
    __syncwarp();
    if (args.ep.counter != nullptr) {
      // everything this CTA stored is ordered before its ticket; the last CTA of the grid tells every
      // rank that this rank's rows have been delivered
      if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
      __threadfence_system();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (threadIdx.x == 64) {
        const int ticket = atomicAdd(args.ep.counter, 1);
        if (ticket == static_cast<int>(gridDim.x) - 1) {
          *args.ep.counter = 0;
          __threadfence_system();
          const int epoch = *args.ep.epoch_base + args.ep.post_epoch_off;
          for (int r = 0; r < args.ep.world; ++r) st_release_sys(args.ep.post_flags[r] + args.ep.post_index, epoch);
        }
      }
    }
  }

  // Neither CTA may leave (or free TMEM) while the other can still arrive on its barriers or run MMAs
  // that write its TMEM.
  tc_fence_before();
  __syncthreads();
  cluster_arrive();
  cluster_wait();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc2(tmem_base, Cfg::TMEM_COLS);
  }
}

}  // namespace b200
