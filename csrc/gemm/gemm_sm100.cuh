// Persistent, warp-specialised bf16 GEMM family for sm_100a.
//
//   warp 0      : TMA producer (one lane) - global -> 128B-swizzled shared tiles, mbarrier completion
//   warp 1      : tcgen05.mma issuer (one lane) + TMEM owner; accumulators double-buffered in TMEM
//   warps 2..5  : epilogue - tcgen05.ld -> registers -> fused epilogue -> global
//
// One template covers dense, grouped-by-rows (ragged expert segments padded to 128 rows) and
// grouped-by-contraction (per-expert weight gradients) problems; operands may be K-major or
// MN-major so that forward, input-gradient and weight-gradient GEMMs read the same tensors with
// no transposed copies.
#pragma once
#include "../common/ptx.cuh"

namespace b200 {

constexpr int GEMM_BM = 128;
constexpr int GEMM_BK = 64;
constexpr int GEMM_THREADS = 192;

enum GemmMode : int { MODE_DENSE = 0, MODE_GROUPED_M = 1, MODE_GROUPED_K = 2 };
enum GemmEpi : int {
  EPI_BF16 = 0,        // C bf16 = acc
  EPI_F32 = 1,         // C fp32 (+)= acc            (beta selects accumulate)
  EPI_SWIGLU = 2,      // acc = [gate | up]; C = silu(gate)*up, aux0 = pre-activations
  EPI_SWIGLU_BWD = 3,  // acc = d(act); aux0 = pre-activations; aux1 = d(pre-activations)
  EPI_LSE = 4,         // C bf16 = acc, aux0 = per (row, n-tile) (max, sum exp) partials
  EPI_BF16_SCATTER = 5,  // bf16 rows stored into peers' buffers: row r -> scatter_dst[src(r)] + slot(r) * ldc
  EPI_QKROPE = 6,        // C bf16 = acc (raw QKV projection); aux0 = q / k heads RMS-normalised + rotated, v copied
};

// Expert-parallel hooks (all optional; null pointers switch them off).
struct GemmEp {
  const int* wait_flags;  // local flag words the producer waits on (>= epoch) before its first load
  int wait_n;
  const int* epoch_base;  // device scalar; epochs are epoch_base + offset so that graph replays keep counting
  int wait_epoch_off;
  void* scatter_dst[8];     // EPI_BF16_SCATTER: every rank's return buffer
  const int* scatter_meta;  // per row: (source rank << 28) | slot, or -1 for a padding row
  int* post_flags[8];       // completion flag words on every rank, set by the last CTA to finish
  int post_index;
  int post_epoch_off;
  int world;
  int* counter;             // local ticket counter, zero between launches
  unsigned long long limit_ns;
};

struct GemmArgs {
  int mode;
  int M, N, K;      // dense: problem; grouped_m: M = padded row capacity; grouped_k: M,N of one expert's output
  int num_experts;  // grouped_k
  int m_fast;       // 1: consecutive tiles walk the M dimension first
  int beta;         // EPI_F32: 1 = accumulate into C
  int n_half;       // EPI_SWIGLU*: row/column offset of the "up" half (= intermediate size)
  const int* tile_expert;  // grouped_m: expert of each 128-row tile
  const int* num_m_tiles;  // grouped_m: device scalar, number of live 128-row tiles
  const int* seg_off;      // grouped_k: [E+1] padded row offsets (multiples of 128)
  const int* pair_tiles;   // grouped_m, pair-tile kernel: per tile (first row, expert | live halves << 16)
  int max_pair_tiles;      // capacity of pair_tiles; num_m_tiles then counts pair tiles
  // pair-tile kernel: operand rows fetched by index (TMA gather) instead of from a materialised sorted copy.
  // a_gather[r] = source row of A row r (K-major A); b_gather[k] = source row of contraction row k (MN-major B,
  // grouped by contraction).  An index outside the source tensor gives a zero row.
  const int* a_gather;
  const int* b_gather;
  // pair-tile SwiGLU epilogues, optional routing-weight folding: the weight of sorted row r is
  // row_w[row_slot[r]] (0 for padding rows, row_slot < 0).  Forward: the stored activation is multiplied by it
  // (so the down projection yields weighted expert outputs and the combine is a plain sum).  Backward: the
  // incoming d(weighted activation) is multiplied by it, and row_dot[r * n_tiles + n] receives this tile's part
  // of <d(weighted activation)[r], activation[r]> = the gradient of the routing weight.
  const int* row_slot;
  const float* row_w;
  float* row_dot;
  // EPI_QKROPE (head_dim 128): cos/sin table [S, 64, 2], norm weights [128] of q and of k, reciprocal RMS out
  // [M, nh + nkv]; row r sits at position r % rope_S
  const float* rope_cs;
  const float* rope_w;
  const float* rope_kw;
  float* rope_rstd;
  int rope_S, rope_nh, rope_nkv;
  float rope_eps;
  void* C;
  long long ldc;
  long long c_expert_stride;  // grouped_k: elements between experts in C
  void* aux0;
  long long ld_aux0;
  void* aux1;
  long long ld_aux1;
  int* status;
  GemmEp ep;
};

struct TileInfo {
  int m0, n_idx, e, k0, num_kb;
};

template <int BN>
struct GemmCfg {
  static constexpr int STAGES = (BN == 256) ? 4 : (BN == 128) ? 6 : 8;
  static constexpr int A_BYTES = GEMM_BM * GEMM_BK * 2;
  static constexpr int B_BYTES = BN * GEMM_BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int TMEM_COLS = (2 * BN < 32) ? 32 : 2 * BN;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024;
  // the row-scatter epilogue stages 32 rows x 256 bytes per epilogue warp behind the operand ring
  static constexpr int SMEM_BYTES_SCATTER = SMEM_BYTES + 4 * 8192;
};

__device__ __forceinline__ void decode_tile(const GemmArgs& a, int t, int m_tiles, int n_tiles, TileInfo& ti) {
  int r = t;
  ti.e = 0;
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
  ti.m0 = m_idx * GEMM_BM;
  ti.n_idx = n_idx;
  if (a.mode == MODE_GROUPED_K) {
    ti.k0 = a.seg_off[ti.e];
    ti.num_kb = (a.seg_off[ti.e + 1] - ti.k0) / GEMM_BK;
  } else {
    ti.k0 = 0;
    ti.num_kb = (a.K + GEMM_BK - 1) / GEMM_BK;
    if (a.mode == MODE_GROUPED_M) ti.e = a.tile_expert[m_idx];
  }
}

// sigmoid(x) = 0.5 tanh(x / 2) + 0.5: one MUFU instruction (tanh.approx, relative error about 2^-11) where
// 1 / (1 + exp(-x)) takes an exponential, a reciprocal and the division's refinement steps.  The SwiGLU epilogues
// are bound by instruction issue, and their results are rounded to bf16 (2^-9) anyway.
__device__ __forceinline__ float sigmoidf_fast(float x) {
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.5f * x));
  return fmaf(t, 0.5f, 0.5f);
}

template <int BN, bool A_MN, bool B_MN, int EPI>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_sm100_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
                  const GemmArgs args) {
  using Cfg = GemmCfg<BN>;
  constexpr int STAGES = Cfg::STAGES;
  // output columns produced per tile
  constexpr int BN_OUT = (EPI == EPI_SWIGLU) ? BN / 2 : BN;

  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t bar_full[STAGES];
  __shared__ uint64_t bar_empty[STAGES];
  __shared__ uint64_t bar_tfull[2];
  __shared__ uint64_t bar_tempty[2];
  __shared__ uint64_t bar_drain;
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;  // set by a warp role that gave up, so that the others stop waiting at once

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

  if (threadIdx.x == 0) {
    abort_flag = 0;
    tma_prefetch_desc(&mapA);
    tma_prefetch_desc(&mapB);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&bar_full[s], 1);
      mbar_init(&bar_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bar_tfull[s], 1);
      mbar_init(&bar_tempty[s], 4);
    }
    mbar_init(&bar_drain, 1);
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(&tmem_base_slot, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;

  int m_tiles;
  if (args.mode == MODE_GROUPED_M) {
    m_tiles = *args.num_m_tiles;
    const int cap = args.M / GEMM_BM;
    m_tiles = m_tiles < 0 ? 0 : (m_tiles > cap ? cap : m_tiles);
  } else {
    m_tiles = (args.M + GEMM_BM - 1) / GEMM_BM;
  }
  const int n_tiles = (args.N + BN_OUT - 1) / BN_OUT;
  const int total = (args.mode == MODE_GROUPED_K ? args.num_experts : 1) * m_tiles * n_tiles;

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int issued = 0;
      bool ok = true;
      if (args.ep.wait_flags != nullptr && blockIdx.x < total) {
        // rows of the A operand are being pushed into local memory by peer GPUs: wait for their flags,
        // then order the (generic-proxy) acquire before the async-proxy TMA reads
        const int epoch = *args.ep.epoch_base + args.ep.wait_epoch_off;
        for (int r = 0; r < args.ep.wait_n && ok; ++r) ok = wait_flag_ge(args.ep.wait_flags + r, epoch, args.ep.limit_ns);
        if (!ok) {
          report(args.status, ST_TIMEOUT_PEER);
          *reinterpret_cast<volatile int*>(&abort_flag) = 1;
        }
        asm volatile("fence.proxy.async;" ::: "memory");
      }
      for (int t = blockIdx.x; t < total && ok; t += gridDim.x) {
        TileInfo ti;
        decode_tile(args, t, m_tiles, n_tiles, ti);
        const int eb = (args.mode == MODE_GROUPED_K) ? 0 : ti.e;
        const int n0 = ti.n_idx * BN_OUT;
        for (int kb = 0; kb < ti.num_kb; ++kb) {
          if (!mbar_wait(&bar_empty[stage], phase ^ 1u)) {
            report(args.status, ST_TIMEOUT_PRODUCER);
            ok = false;
            break;
          }
          uint64_t* fb = &bar_full[stage];
          mbar_expect_tx(fb, Cfg::STAGE_BYTES);
          uint8_t* sa = tiles + stage * Cfg::STAGE_BYTES;
          uint8_t* sb = sa + Cfg::A_BYTES;
          const int kk = ti.k0 + kb * GEMM_BK;
          if constexpr (!A_MN) {
            tma_load_2d(sa, &mapA, fb, kk, ti.m0);
          } else {
            tma_load_2d(sa, &mapA, fb, ti.m0, kk);
            tma_load_2d(sa + 8192, &mapA, fb, ti.m0 + 64, kk);
          }
          if constexpr (!B_MN) {
            if constexpr (EPI == EPI_SWIGLU) {
              tma_load_3d(sb, &mapB, fb, kk, n0, eb);
              tma_load_3d(sb + (BN / 2) * 128, &mapB, fb, kk, args.n_half + n0, eb);
            } else {
              tma_load_3d(sb, &mapB, fb, kk, n0, eb);
            }
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) tma_load_3d(sb + j * 8192, &mapB, fb, n0 + 64 * j, kk, eb);
          }
          ++issued;
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (!ok) {
        // Leave only after the copies already issued have landed (bounded): walk the
        // stages still in flight, oldest first.
        int pend = issued < STAGES ? issued : STAGES;
        int s = stage;
        uint32_t ph = phase;
        for (int i = 0; i < pend; ++i) {
          if (--s < 0) {
            s = STAGES - 1;
            ph ^= 1u;
          }
          (void)mbar_wait(&bar_full[s], ph);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(GEMM_BM, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total && ok; t += gridDim.x) {
        TileInfo ti;
        decode_tile(args, t, m_tiles, n_tiles, ti);
        if (!mbar_wait_abortable(&bar_tempty[acc], acc_phase ^ 1u, &abort_flag)) {
          report(args.status, ST_TIMEOUT_MMA);
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BN);
        for (int kb = 0; kb < ti.num_kb; ++kb) {
          if (!mbar_wait_abortable(&bar_full[stage], phase, &abort_flag)) {
            report(args.status, ST_TIMEOUT_MMA);
            *reinterpret_cast<volatile int*>(&abort_flag) = 1;
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
            umma_bf16(d_tmem, adesc, bdesc, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(&bar_empty[stage]);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        umma_commit(&bar_tfull[acc]);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
      if (!ok) {
        // all tensor-core work issued so far must retire before TMEM is freed
        umma_commit(&bar_drain);
        (void)mbar_wait(&bar_drain, 0);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    const int row_l = q * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(q * 32) << 16;
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int t = blockIdx.x; t < total; t += gridDim.x) {
      TileInfo ti;
      decode_tile(args, t, m_tiles, n_tiles, ti);
      if (!mbar_wait_abortable(&bar_tfull[acc], acc_phase, &abort_flag)) {
        report(args.status, ST_TIMEOUT_EPILOGUE);
        break;
      }
      tc_fence_after();
      const uint32_t t_acc = tmem_base + lane_base + static_cast<uint32_t>(acc * BN);
      const long long row_g = static_cast<long long>(ti.m0) + row_l;
      const bool row_ok = row_g < args.M;
      const int n0 = ti.n_idx * BN_OUT;

      if constexpr (EPI == EPI_BF16_SCATTER) {
        // result rows go straight to the rank that owns the token (plain peer stores)
        int meta = -1;
        if (row_ok) meta = args.ep.scatter_meta[row_g];
        const bool live = meta >= 0;
        __nv_bfloat16* crow = nullptr;
        if (live)
          crow = reinterpret_cast<__nv_bfloat16*>(args.ep.scatter_dst[(meta >> 28) & 7]) +
                 static_cast<long long>(meta & 0x0fffffff) * args.ldc;
        if ((args.N & 127) == 0) {
          // Whole-row pieces: the warp's 32 rows x 128 columns are staged in shared memory (lane = row on the way in),
          // then every store instruction writes two rows' 256 contiguous bytes (16 lanes x 16 B per row), so a peer
          // receives 256-byte runs instead of one 16-byte fragment per lane and row.
          uint8_t* stg = tiles + STAGES * Cfg::STAGE_BYTES + q * 8192;
          const unsigned long long cptr = reinterpret_cast<unsigned long long>(crow);
#pragma unroll 1
          for (int g = 0; g < BN / 128; ++g) {
            const int colg = n0 + g * 128;
            if (colg >= args.N) break;
#pragma unroll
            for (int c4 = 0; c4 < 4; ++c4) {
              uint32_t r[32];
              tmem_ld_32x32(t_acc + g * 128 + c4 * 32, r);
              tmem_ld_wait();
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const int k = c4 * 4 + j;  // 16-byte chunk of the row, swizzled by the row so that lanes spread over banks
                *reinterpret_cast<uint4*>(stg + lane * 256 + ((k ^ (lane & 15)) << 4)) =
                    make_uint4(pack_bf16x2(__uint_as_float(r[8 * j]), __uint_as_float(r[8 * j + 1])),
                               pack_bf16x2(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3])),
                               pack_bf16x2(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5])),
                               pack_bf16x2(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7])));
              }
            }
            __syncwarp();
            const int k = lane & 15;
#pragma unroll 4
            for (int i = 0; i < 16; ++i) {
              const int row = 2 * i + (lane >> 4);
              const unsigned long long base = __shfl_sync(0xffffffffu, cptr, row);
              const uint4 v = *reinterpret_cast<const uint4*>(stg + row * 256 + ((k ^ (row & 15)) << 4));
              if (base != 0ull) reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(base) + colg)[k] = v;
            }
            __syncwarp();  // the staging buffer is rewritten by the next group
          }
        } else {
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          const int col0 = n0 + c * 32;
          if (col0 >= args.N) break;
          uint32_t r[32];
          tmem_ld_32x32(t_acc + c * 32, r);
          tmem_ld_wait();
          if (live) {
            if (col0 + 32 <= args.N) {
              uint4* dst = reinterpret_cast<uint4*>(crow + col0);
#pragma unroll
              for (int j = 0; j < 4; ++j)
                dst[j] = make_uint4(pack_bf16x2(__uint_as_float(r[8 * j]), __uint_as_float(r[8 * j + 1])),
                                    pack_bf16x2(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3])),
                                    pack_bf16x2(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5])),
                                    pack_bf16x2(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7])));
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (col0 + j < args.N) crow[col0 + j] = __float2bfloat16(__uint_as_float(r[j]));
            }
          }
        }
        }
      } else if constexpr (EPI == EPI_BF16 || EPI == EPI_LSE) {
        __nv_bfloat16* crow = reinterpret_cast<__nv_bfloat16*>(args.C) + row_g * args.ldc;
        float run_max = -INFINITY, run_sum = 0.f;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          const int col0 = n0 + c * 32;
          if (col0 >= args.N) break;
          uint32_t r[32];
          tmem_ld_32x32(t_acc + c * 32, r);
          tmem_ld_wait();
          uint32_t p[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) p[j] = pack_bf16x2(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
          const bool full = col0 + 32 <= args.N;
          if constexpr (EPI == EPI_LSE) {
            // statistics of the bf16-rounded logits, valid columns only
            if (full) {
              // two values per issue slot (f32x2) and four independent partial sums: this epilogue runs on
              // one warp per scheduler and a serial chain of 32 adds per chunk was its longest dependency
              constexpr float kLog2e = 1.4426950408889634f;
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
              uint64_t acc[4] = {0ull, 0ull, 0ull, 0ull};
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                float xl, xh;
                unpack2(fma2(v2[j], l2, nm2), xl, xh);
                acc[j & 3] = add2(acc[j & 3], pack2(ex2_approx(xl), ex2_approx(xh)));
              }
              float a0, a1, a2, a3, a4, a5, a6, a7;
              unpack2(acc[0], a0, a1);
              unpack2(acc[1], a2, a3);
              unpack2(acc[2], a4, a5);
              unpack2(acc[3], a6, a7);
              const float ssum = ((a0 + a1) + (a2 + a3)) + ((a4 + a5) + (a6 + a7));
              run_sum = run_sum * ex2_approx((run_max - new_max) * kLog2e) + ssum;
              run_max = new_max;
            } else {
            float cmax = -INFINITY;
            float v[32];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              float2 f = unpack_bf16x2(p[j]);
              v[2 * j] = (col0 + 2 * j < args.N) ? f.x : -INFINITY;
              v[2 * j + 1] = (col0 + 2 * j + 1 < args.N) ? f.y : -INFINITY;
              cmax = fmaxf(cmax, fmaxf(v[2 * j], v[2 * j + 1]));
            }
            const float new_max = fmaxf(run_max, cmax);
            float s = 0.f;
#pragma unroll
            for (int j = 0; j < 32; ++j) s += __expf(v[j] - new_max);
            run_sum = run_sum * __expf(run_max - new_max) + s;
            run_max = new_max;
            }
          }
          if (row_ok) {
            if (full) {
              uint4* dst = reinterpret_cast<uint4*>(crow + col0);
#pragma unroll
              for (int j = 0; j < 4; ++j) dst[j] = make_uint4(p[4 * j], p[4 * j + 1], p[4 * j + 2], p[4 * j + 3]);
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (col0 + j < args.N) crow[col0 + j] = __float2bfloat16(__uint_as_float(r[j]));
            }
          }
        }
        if constexpr (EPI == EPI_LSE) {
          if (row_ok) {
            float2* part = reinterpret_cast<float2*>(args.aux0);
            part[row_g * n_tiles + ti.n_idx] = make_float2(run_max, run_sum);
          }
        }
      } else if constexpr (EPI == EPI_F32) {
        float* crow = reinterpret_cast<float*>(args.C) + static_cast<long long>(ti.e) * args.c_expert_stride +
                      row_g * args.ldc;
        const bool empty_acc = ti.num_kb == 0;
        if (!(empty_acc && args.beta)) {
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
            if (row_ok) {
              if (col0 + 32 <= args.N) {
                float4* dst = reinterpret_cast<float4*>(crow + col0);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                  float4 v = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                         __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
                  if (args.beta) {
                    const float4 o = dst[j];
                    v.x += o.x;
                    v.y += o.y;
                    v.z += o.z;
                    v.w += o.w;
                  }
                  dst[j] = v;
                }
              } else {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                  if (col0 + j < args.N) {
                    const float v = __uint_as_float(r[j]);
                    crow[col0 + j] = args.beta ? crow[col0 + j] + v : v;
                  }
              }
            }
          }
        }
      } else if constexpr (EPI == EPI_SWIGLU) {
        // accumulator columns [0, BN/2) = gate, [BN/2, BN) = up, for output columns n0 .. n0+BN/2
        __nv_bfloat16* crow = reinterpret_cast<__nv_bfloat16*>(args.C) + row_g * args.ldc;
        __nv_bfloat16* gurow = reinterpret_cast<__nv_bfloat16*>(args.aux0) + row_g * args.ld_aux0;
#pragma unroll 1
        for (int c = 0; c < BN / 64; ++c) {
          const int col0 = n0 + c * 32;
          if (col0 >= args.N) break;
          uint32_t g[32], u[32];
          tmem_ld_32x32(t_acc + c * 32, g);
          tmem_ld_32x32(t_acc + BN / 2 + c * 32, u);
          tmem_ld_wait();
          uint32_t pg[16], pu[16], pa[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            pg[j] = pack_bf16x2(__uint_as_float(g[2 * j]), __uint_as_float(g[2 * j + 1]));
            pu[j] = pack_bf16x2(__uint_as_float(u[2 * j]), __uint_as_float(u[2 * j + 1]));
            // activation from the bf16-rounded pre-activations, so that backward sees the same values
            const float2 gf = unpack_bf16x2(pg[j]);
            const float2 uf = unpack_bf16x2(pu[j]);
            pa[j] = pack_bf16x2(gf.x * sigmoidf_fast(gf.x) * uf.x, gf.y * sigmoidf_fast(gf.y) * uf.y);
          }
          if (row_ok) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              if (col0 + 8 * j < args.N) {  // N is a multiple of 8
                *reinterpret_cast<uint4*>(crow + col0 + 8 * j) =
                    make_uint4(pa[4 * j], pa[4 * j + 1], pa[4 * j + 2], pa[4 * j + 3]);
                *reinterpret_cast<uint4*>(gurow + col0 + 8 * j) =
                    make_uint4(pg[4 * j], pg[4 * j + 1], pg[4 * j + 2], pg[4 * j + 3]);
                *reinterpret_cast<uint4*>(gurow + args.n_half + col0 + 8 * j) =
                    make_uint4(pu[4 * j], pu[4 * j + 1], pu[4 * j + 2], pu[4 * j + 3]);
              }
            }
          }
        }
      } else if constexpr (EPI == EPI_SWIGLU_BWD) {
        const __nv_bfloat16* gurow = reinterpret_cast<const __nv_bfloat16*>(args.aux0) + row_g * args.ld_aux0;
        __nv_bfloat16* drow = reinterpret_cast<__nv_bfloat16*>(args.aux1) + row_g * args.ld_aux1;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          const int col0 = n0 + c * 32;
          if (col0 >= args.N) break;
          uint32_t r[32];
          tmem_ld_32x32(t_acc + c * 32, r);
          tmem_ld_wait();
          if (row_ok) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              if (col0 + 8 * j < args.N) {
                const uint4 gq = *reinterpret_cast<const uint4*>(gurow + col0 + 8 * j);
                const uint4 uq = *reinterpret_cast<const uint4*>(gurow + args.n_half + col0 + 8 * j);
                const uint32_t gw[4] = {gq.x, gq.y, gq.z, gq.w};
                const uint32_t uw[4] = {uq.x, uq.y, uq.z, uq.w};
                uint32_t og[4], ou[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  const float2 gf = unpack_bf16x2(gw[i]);
                  const float2 uf = unpack_bf16x2(uw[i]);
                  const float d0 = __uint_as_float(r[8 * j + 2 * i]);
                  const float d1 = __uint_as_float(r[8 * j + 2 * i + 1]);
                  const float s0 = sigmoidf_fast(gf.x), s1 = sigmoidf_fast(gf.y);
                  og[i] = pack_bf16x2(d0 * uf.x * s0 * (1.f + gf.x * (1.f - s0)),
                                      d1 * uf.y * s1 * (1.f + gf.y * (1.f - s1)));
                  ou[i] = pack_bf16x2(d0 * gf.x * s0, d1 * gf.y * s1);
                }
                *reinterpret_cast<uint4*>(drow + col0 + 8 * j) = make_uint4(og[0], og[1], og[2], og[3]);
                *reinterpret_cast<uint4*>(drow + args.n_half + col0 + 8 * j) = make_uint4(ou[0], ou[1], ou[2], ou[3]);
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar_tempty[acc]);
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
    if (args.ep.counter != nullptr) {
      // everything this CTA stored (possibly into peers' memory) is ordered before its ticket; the
      // last CTA of the grid tells every rank that this rank's rows have been delivered
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

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

}  // namespace b200
