// Causal grouped-query flash attention, forward, for sm_100a (head_dim 128 or 64: template parameter HD).
//
// Persistent CTAs (one per SM).  A work item is (batch, pair of query heads that share one key/value head,
// 128 query rows); key/value tiles of 128 rows stream through a 5-slot TMA ring (K0, V0, K1, V1, ...) and
// every tile that is loaded feeds four MMAs (scores and P*V of both heads).
//
//   warp 0      : TMA producer (one lane); runs ahead across work items
//   warp 1      : tcgen05.mma issuer (one lane), owns the 512 TMEM columns
//   warps 2..5  : softmax of head A, one query row per thread (TMEM lane quarter = warp % 4)
//   warps 6..9  : softmax of head B
//
// TMEM: S_A, S_B (scores) and O_A, O_B (output accumulators), 128 columns each.  The probabilities never
// touch shared memory: the thread that owns a row writes them (bf16 pairs, tcgen05.st) over the first 64
// columns of its own score row and the P*V MMA takes its A operand from TMEM.  A 128x128x16 MMA with both
// operands in shared memory reads 8 KB per 64 cycles, i.e. all of the SM's shared-memory bandwidth; with
// P in TMEM the tensor pipe, the TMA writes and nothing else share that bandwidth.
// The probabilities are scaled by a reference maximum that follows the true running maximum lazily (only
// when it has grown by more than 2^8), so an accumulator is rescaled in TMEM only a few times per row.
// Issue order on the tensor pipe (MMAs of one thread execute in issue order, so S(j+1) may overwrite the
// columns P(j) was read from):
//   S_A(0) S_B(0) | U_A(0) S_A(1) U_B(0) S_B(1) | U_A(1) S_A(2) U_B(1) S_B(2) | ...
// so while one head's softmax runs the tensor pipe works for the other head.
//
// Shared-memory operands use the same 128-byte-swizzled tile shapes as the GEMM family: Q and K are
// K-major [128 rows x 64] chunks, V is MN-major ([64 key rows x 64] boxes) so that it is read as stored.
#include "../common/ptx.cuh"
#include "../common/tma_host.h"
#include "attn_api.h"

namespace b200 {

constexpr int FA_THREADS = 320;
constexpr int FA_TILE = 32768;   // slot size: 128 x 128 bf16 (head_dim 64 fills half of a slot)
constexpr int FA_RING = 5;       // K/V slots
constexpr int FA_EXTRA = 256;    // barriers
constexpr int FA_SMEM = 232448;  // everything a CTA may have; the seven tiles alone take 224 KB
constexpr unsigned long long FA_LIMIT_NS = 2000000000ull;  // nothing here waits on another GPU

struct FaFwdArgs {
  __nv_bfloat16* O;
  float* lse;
  int B, S, nh, nkv;
  int items;
  float scale_log2;
  int* status;
};

struct FaItem {
  int b, pair, qt, n;
};

__device__ __forceinline__ FaItem fa_item(const FaFwdArgs& a, int t) {
  // heaviest query tiles first
  const int per_qt = a.B * (a.nh >> 1);
  FaItem it;
  it.qt = (a.S >> 7) - 1 - t / per_qt;
  const int r = t % per_qt;
  it.b = r / (a.nh >> 1);
  it.pair = r % (a.nh >> 1);
  it.n = it.qt + 1;
  return it;
}

// Items are sorted heaviest first; CTA c takes item c of every round, the rounds alternating in direction
// ("snake") so that every CTA gets nearly the same number of key tiles.
__device__ __forceinline__ int fa_sched(int round, int cta, int ctas) {
  return round * ctas + ((round & 1) ? ctas - 1 - cta : cta);
}

template <int HD>
__global__ void __launch_bounds__(FA_THREADS, 1)
flash_fwd_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapK,
                 const __grid_constant__ CUtensorMap mapV, const FaFwdArgs args) {
  // no static shared memory: the operand tiles leave 3 KB, laid out by hand behind them
  extern __shared__ uint8_t smem_raw[];
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = base;                // [2 heads]
  uint8_t* sR = base + 2 * FA_TILE;  // ring
  uint64_t* bars = reinterpret_cast<uint64_t*>(base + 7 * FA_TILE);
  uint64_t* bar_q_full = bars;         // [2]
  uint64_t* bar_q_empty = bars + 2;    // [2]
  uint64_t* bar_r_full = bars + 4;     // [FA_RING]
  uint64_t* bar_r_empty = bars + 9;    // [FA_RING]
  uint64_t* bar_s_full = bars + 14;    // [2]
  uint64_t* bar_p_full = bars + 16;    // [2]
  uint64_t* bar_u_full = bars + 18;    // [2]
  uint64_t& bar_drain = bars[20];
  uint32_t& tmem_base_slot = *reinterpret_cast<uint32_t*>(bars + 21);
  int& go = *reinterpret_cast<int*>(bars + 22);

  if (threadIdx.x == 0) {
    go = 1;
    if (base + 7 * FA_TILE + FA_EXTRA > smem_raw + FA_SMEM) {  // alignment slack larger than planned
      report(args.status, ST_BAD_ARGUMENT);
      go = 0;
    }
    tma_prefetch_desc(&mapQ);
    tma_prefetch_desc(&mapK);
    tma_prefetch_desc(&mapV);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bar_q_full[s], 1);
      mbar_init(&bar_q_empty[s], 1);
      mbar_init(&bar_s_full[s], 1);
      mbar_init(&bar_p_full[s], 4);
      mbar_init(&bar_u_full[s], 1);
    }
    for (int s = 0; s < FA_RING; ++s) {
      mbar_init(&bar_r_full[s], 1);
      mbar_init(&bar_r_empty[s], 1);
    }
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
  const int group = args.nh / args.nkv;
  constexpr int KC = HD / 64;              // 64-column chunks of a head
  constexpr int TILE_BYTES = 128 * HD * 2;  // bytes that one Q, K or V tile brings in

  if (warp == 0) {
    if (lane == 0) {
      bool ok = true;
      uint32_t load = 0;  // ring loads issued so far
      uint32_t q_loads = 0;
      int it_count = 0;
      for (int t; (t = fa_sched(it_count, blockIdx.x, gridDim.x)) < args.items && ok; ++it_count) {
        if (*reinterpret_cast<volatile int*>(args.status) != 0) break;  // somebody gave up: stop feeding
        const FaItem it = fa_item(args, t);
        const int hk = (2 * it.pair) / group;
        for (int x = 0; x < 2 && ok; ++x) {
          if (!mbar_wait_ns(&bar_q_empty[x], (it_count & 1) ^ 1u, FA_LIMIT_NS)) {
            ok = false;
            break;
          }
          mbar_expect_tx(&bar_q_full[x], TILE_BYTES);
#pragma unroll
          for (int kc = 0; kc < KC; ++kc)
            tma_load_3d(sQ + x * FA_TILE + kc * 16384, &mapQ, &bar_q_full[x], (2 * it.pair + x) * HD + kc * 64,
                        it.qt * 128, it.b);
          ++q_loads;
        }
        for (int j = 0; j < it.n && ok; ++j) {
          {
            const int slot = load % FA_RING;
            if (!mbar_wait_ns(&bar_r_empty[slot], ((load / FA_RING) & 1) ^ 1u, FA_LIMIT_NS)) {
              ok = false;
              break;
            }
            mbar_expect_tx(&bar_r_full[slot], TILE_BYTES);
            uint8_t* dst = sR + slot * FA_TILE;
#pragma unroll
            for (int kc = 0; kc < KC; ++kc)
              tma_load_3d(dst + kc * 16384, &mapK, &bar_r_full[slot], hk * HD + kc * 64, j * 128, it.b);
            ++load;
          }
          {
            const int slot = load % FA_RING;
            if (!mbar_wait_ns(&bar_r_empty[slot], ((load / FA_RING) & 1) ^ 1u, FA_LIMIT_NS)) {
              ok = false;
              break;
            }
            mbar_expect_tx(&bar_r_full[slot], TILE_BYTES);
            uint8_t* dst = sR + slot * FA_TILE;
#pragma unroll
            for (int kh = 0; kh < 2; ++kh)
#pragma unroll
              for (int jn = 0; jn < KC; ++jn)
                tma_load_3d(dst + kh * (KC * 8192) + jn * 8192, &mapV, &bar_r_full[slot], hk * HD + jn * 64,
                            j * 128 + kh * 64, it.b);
            ++load;
          }
        }
      }
      if (!ok) report(args.status, ST_TIMEOUT_PRODUCER);
      // copies already issued must land before the CTA may exit (normally the consumers have seen them all)
      for (uint32_t i = load > FA_RING ? load - FA_RING : 0; i < load; ++i)
        (void)mbar_wait_ns(&bar_r_full[i % FA_RING], (i / FA_RING) & 1, FA_LIMIT_NS);
      for (uint32_t i = q_loads > 2 ? q_loads - 2 : 0; i < q_loads; ++i)
        (void)mbar_wait_ns(&bar_q_full[i & 1], ((i >> 1) & 1), FA_LIMIT_NS);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(128, 128, 0, 0);
      constexpr uint32_t idesc_u = make_idesc_bf16(128, HD, 0, 1);
      bool ok = true;
      uint32_t load = 0;  // ring entries consumed before this item
      uint32_t g = 0;     // key tiles processed before this item (phase of the per-tile barriers)
      int it_count = 0;

      auto ring_wait = [&](uint32_t idx) -> bool {
        const bool r = mbar_wait_ns(&bar_r_full[idx % FA_RING], (idx / FA_RING) & 1, FA_LIMIT_NS);
        tc_fence_after();
        return r;
      };
      auto issue_s = [&](int x, uint32_t k_idx) {
        const uint32_t q_addr = smem_u32(sQ + x * FA_TILE);
        const uint32_t k_addr = smem_u32(sR + (k_idx % FA_RING) * FA_TILE);
#pragma unroll
        for (int kc = 0; kc < KC; ++kc)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_bf16(tmem + x * 128, make_smem_desc(q_addr + kc * 16384 + k * 32, 16, 1024),
                      make_smem_desc(k_addr + kc * 16384 + k * 32, 16, 1024), idesc_s, (kc | k) != 0 ? 1u : 0u);
        umma_commit(&bar_s_full[x]);
      };
      auto issue_u = [&](int x, uint32_t v_idx, bool acc) {
        const uint32_t v_addr = smem_u32(sR + (v_idx % FA_RING) * FA_TILE);
#pragma unroll
        for (int kc = 0; kc < 2; ++kc)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_bf16_ts(tmem + 256 + x * 128, tmem + x * 128 + (kc * 4 + k) * 8,
                         make_smem_desc(v_addr + kc * (KC * 8192) + k * 2048, 8192, 1024), idesc_u,
                         (acc || (kc | k) != 0) ? 1u : 0u);
        umma_commit(&bar_u_full[x]);
      };

      for (int t; (t = fa_sched(it_count, blockIdx.x, gridDim.x)) < args.items && ok; ++it_count) {
        const FaItem it = fa_item(args, t);
        const int n = it.n;
        // ring entries of this item: K_j = load + 2j, V_j = load + 2j + 1
        ok = mbar_wait_ns(&bar_q_full[0], it_count & 1, FA_LIMIT_NS) &&
             mbar_wait_ns(&bar_q_full[1], it_count & 1, FA_LIMIT_NS) && ring_wait(load);
        if (!ok) break;
        issue_s(0, load);
        if (n == 1) umma_commit(&bar_q_empty[0]);
        issue_s(1, load);
        if (n == 1) umma_commit(&bar_q_empty[1]);
        umma_commit(&bar_r_empty[load % FA_RING]);
        for (int j = 0; j < n; ++j) {
          const uint32_t v_idx = load + 2 * j + 1, k_next = load + 2 * j + 2;
          const bool more = j + 1 < n, last_s = j + 1 == n - 1;
          const uint32_t ph = (g + j) & 1;
          if (!ring_wait(v_idx) || !mbar_wait_ns(&bar_p_full[0], ph, FA_LIMIT_NS)) {
            ok = false;
            break;
          }
          tc_fence_after();
          issue_u(0, v_idx, j > 0);
          if (more) {
            if (!ring_wait(k_next)) {
              ok = false;
              break;
            }
            issue_s(0, k_next);
            if (last_s) umma_commit(&bar_q_empty[0]);
          }
          if (!mbar_wait_ns(&bar_p_full[1], ph, FA_LIMIT_NS)) {
            ok = false;
            break;
          }
          tc_fence_after();
          issue_u(1, v_idx, j > 0);
          umma_commit(&bar_r_empty[v_idx % FA_RING]);
          if (more) {
            issue_s(1, k_next);
            if (last_s) umma_commit(&bar_q_empty[1]);
            umma_commit(&bar_r_empty[k_next % FA_RING]);
          }
        }
        load += 2 * n;
        g += n;
      }
      if (!ok) report(args.status, ST_TIMEOUT_MMA);
      umma_commit(&bar_drain);  // everything issued must retire before TMEM is freed
      (void)mbar_wait_ns(&bar_drain, 0, FA_LIMIT_NS);
    }
  } else {
    const int q4 = warp & 3;
    const int x = (warp - 2) >> 2;  // head of the pair
    const int row_l = q4 * 32 + lane;
    const uint32_t t_row = tmem + (static_cast<uint32_t>(q4 * 32) << 16);
    const uint32_t t_s = t_row + x * 128;
    const uint32_t t_o = t_row + 256 + x * 128;
    const float sl2 = args.scale_log2;
    bool ok = true;
    uint32_t g = 0;
    int it_count = 0;

    for (int t; (t = fa_sched(it_count, blockIdx.x, gridDim.x)) < args.items && ok; ++it_count) {
      const FaItem it = fa_item(args, t);
      const int n = it.n;
      // m_ref: the reference the probabilities are scaled by (lags the true maximum by at most 2^8)
      float m_ref = -INFINITY, l_run = 0.f;
      for (int j = 0; j < n; ++j, ++g) {
        if (!mbar_wait_ns(&bar_s_full[x], g & 1, FA_LIMIT_NS)) {
          ok = false;
          break;
        }
        tc_fence_after();
        // pass 1: row maximum (the scores are read from TMEM again for the exponentials, which keeps
        // the live registers at 64 instead of 128)
        const bool diag = j == n - 1;  // diagonal tile: key index may not exceed the query index
        float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          uint32_t r0[32], r1[32];
          tmem_ld_32x32(t_s + hh * 64, r0);
          tmem_ld_32x32(t_s + hh * 64 + 32, r1);
          tmem_ld_wait();
          if (diag) {
#pragma unroll
            for (int c = 0; c < 32; ++c) {
              if (hh * 64 + c > row_l) r0[c] = 0xff800000u;
              if (hh * 64 + 32 + c > row_l) r1[c] = 0xff800000u;
            }
          }
#pragma unroll
          for (int c = 0; c < 32; c += 4) {
            mx0 = fmax3(mx0, __uint_as_float(r0[c]), __uint_as_float(r1[c]));
            mx1 = fmax3(mx1, __uint_as_float(r0[c + 1]), __uint_as_float(r1[c + 1]));
            mx2 = fmax3(mx2, __uint_as_float(r0[c + 2]), __uint_as_float(r1[c + 2]));
            mx3 = fmax3(mx3, __uint_as_float(r0[c + 3]), __uint_as_float(r1[c + 3]));
          }
        }
        const float m_new = fmaxf(fmax3(mx0, mx1, mx2), mx3);
        if (j == 0) {
          m_ref = m_new;  // nothing accumulated yet
        } else {
          const bool grow = (m_new - m_ref) * sl2 > 8.0f;
          if (__any_sync(0xffffffffu, grow)) {
            // rescale this row of the accumulator: the previous P*V must have retired first
            if (!mbar_wait_ns(&bar_u_full[x], (g - 1) & 1, FA_LIMIT_NS)) {
              ok = false;
              break;
            }
            tc_fence_after();
            const float a = grow ? ex2_approx((m_ref - m_new) * sl2) : 1.0f;
#pragma unroll
            for (int hh = 0; hh < HD / 32; ++hh) {
              uint32_t r[32];
              tmem_ld_32x32(t_o + hh * 32, r);
              tmem_ld_wait();
#pragma unroll
              for (int c = 0; c < 32; ++c) r[c] = __float_as_uint(__uint_as_float(r[c]) * a);
              tmem_st_32x32(t_o + hh * 32, r);
            }
            tmem_st_wait();
            l_run *= a;
            if (grow) m_ref = m_new;
          }
        }
        // pass 2: exponentials -> P as bf16 pairs over the first 64 columns of this row's scores.  Columns
        // [32 hh, 32 hh + 32) are written after score columns [64 hh, 64 hh + 64) have been read.
        const float mb = m_ref * sl2;
        float rs0 = 0.f, rs1 = 0.f, rs2 = 0.f, rs3 = 0.f;
        uint64_t acc2[4] = {0ull, 0ull, 0ull, 0ull};
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          uint32_t r[64];
          {
            uint32_t r0[32], r1[32];
            tmem_ld_32x32(t_s + hh * 64, r0);
            tmem_ld_32x32(t_s + hh * 64 + 32, r1);
            tmem_ld_wait();
#pragma unroll
            for (int c = 0; c < 32; ++c) {
              r[c] = r0[c];
              r[32 + c] = r1[c];
            }
          }
          if (diag) {
#pragma unroll
            for (int c = 0; c < 64; ++c)
              if (hh * 64 + c > row_l) r[c] = 0xff800000u;
          }
          uint32_t pk[32];
          if (diag) {
#pragma unroll
            for (int c8 = 0; c8 < 8; ++c8) {
              float p[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) p[i] = ex2_approx(fmaf(__uint_as_float(r[c8 * 8 + i]), sl2, -mb));
              rs0 += p[0] + p[4];
              rs1 += p[1] + p[5];
              rs2 += p[2] + p[6];
              rs3 += p[3] + p[7];
#pragma unroll
              for (int i = 0; i < 4; ++i) pk[c8 * 4 + i] = pack_bf16x2(p[2 * i], p[2 * i + 1]);
            }
          } else {
            // two values per issue slot (f32x2) for the scale and the sums: this loop is bound by issue slots
            const uint64_t sl2_2 = pack2(sl2, sl2), nmb2 = pack2(-mb, -mb);
#pragma unroll
            for (int c8 = 0; c8 < 8; ++c8) {
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                const float lo = __uint_as_float(r[c8 * 8 + 2 * k]), hi = __uint_as_float(r[c8 * 8 + 2 * k + 1]);
                float xl, xh;
                unpack2(fma2(pack2(lo, hi), sl2_2, nmb2), xl, xh);
                const uint64_t p2 = pack2(ex2_approx(xl), ex2_approx(xh));
                acc2[k] = add2(acc2[k], p2);
                float pl, ph;
                unpack2(p2, pl, ph);
                pk[c8 * 4 + k] = pack_bf16x2(pl, ph);
              }
            }
          }
          tmem_st_32x32(t_s + hh * 32, pk);
        }
        tmem_st_wait();
        {
          float a0, a1, a2, a3, a4, a5, a6, a7;
          unpack2(acc2[0], a0, a1);
          unpack2(acc2[1], a2, a3);
          unpack2(acc2[2], a4, a5);
          unpack2(acc2[3], a6, a7);
          l_run += ((rs0 + rs1) + (rs2 + rs3)) + (((a0 + a1) + (a2 + a3)) + ((a4 + a5) + (a6 + a7)));
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bar_p_full[x]);
      }
      if (!ok) break;
      // epilogue of the item: the last P*V must have retired
      if (!mbar_wait_ns(&bar_u_full[x], (g - 1) & 1, FA_LIMIT_NS)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const float inv = 1.0f / l_run;
      const int h = 2 * it.pair + x;
      const long long row_g = static_cast<long long>(it.b) * args.S + it.qt * 128 + row_l;
      uint4* dst = reinterpret_cast<uint4*>(args.O + (row_g * args.nh + h) * HD);
#pragma unroll
      for (int hh = 0; hh < HD / 32; ++hh) {
        uint32_t r[32];
        tmem_ld_32x32(t_o + hh * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int c8 = 0; c8 < 4; ++c8)
          dst[hh * 4 + c8] = make_uint4(
              pack_bf16x2(__uint_as_float(r[c8 * 8]) * inv, __uint_as_float(r[c8 * 8 + 1]) * inv),
              pack_bf16x2(__uint_as_float(r[c8 * 8 + 2]) * inv, __uint_as_float(r[c8 * 8 + 3]) * inv),
              pack_bf16x2(__uint_as_float(r[c8 * 8 + 4]) * inv, __uint_as_float(r[c8 * 8 + 5]) * inv),
              pack_bf16x2(__uint_as_float(r[c8 * 8 + 6]) * inv, __uint_as_float(r[c8 * 8 + 7]) * inv));
      }
      args.lse[(static_cast<long long>(it.b) * args.nh + h) * args.S + it.qt * 128 + row_l] =
          m_ref * sl2 + log2f(l_run);
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
static int launch_flash_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int B, int S, int nh,
                            int nkv, long long ldq, long long ldk, long long ldv, float softmax_scale, int* status,
                            cudaStream_t stream) {
  CUtensorMap mq, mk, mv;
  const uint64_t qrow = static_cast<uint64_t>(nh) * HD, krow = static_cast<uint64_t>(nkv) * HD;
  // row pitch of each operand in bytes (a token's heads are contiguous; tokens may be further apart)
  const uint64_t pq = (ldq > 0 ? ldq : qrow) * 2, pk = (ldk > 0 ? ldk : krow) * 2, pv = (ldv > 0 ? ldv : krow) * 2;
  int rc = make_map(&mq, q, qrow, S, B, pq, pq * S, 64, 128);
  if (rc == 0) rc = make_map(&mk, k, krow, S, B, pk, pk * S, 64, 128);
  if (rc == 0) rc = make_map(&mv, v, krow, S, B, pv, pv * S, 64, 64);
  if (rc != 0) return rc - 100;
  static bool configured = false;
  static int sms = 0;
  if (!configured) {
    if (cudaFuncSetAttribute(flash_fwd_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, FA_SMEM) !=
        cudaSuccess)
      return -10;
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    configured = true;
  }
  FaFwdArgs a;
  a.O = reinterpret_cast<__nv_bfloat16*>(o);
  a.lse = lse;
  a.B = B; a.S = S; a.nh = nh; a.nkv = nkv;
  a.items = B * (nh / 2) * (S / 128);
  a.scale_log2 = softmax_scale * 1.4426950408889634f;
  a.status = status;
  const int grid = a.items < sms ? a.items : sms;
  flash_fwd_kernel<HD><<<grid, FA_THREADS, FA_SMEM, stream>>>(mq, mk, mv, a);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

extern "C" int b200_flash_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int B, int S, int nh,
                              int nkv, int head_dim, long long ldq, long long ldk, long long ldv, float softmax_scale,
                              int* status, cudaStream_t stream) {
  if (B <= 0 || S <= 0 || (S & 127) != 0 || nh <= 0 || nkv <= 0 || nh % nkv != 0) return -1;
  if (((nh / nkv) & 1) != 0) return -2;  // two query heads of one CTA must share their key/value head
  if (head_dim == 128) return launch_flash_fwd<128>(q, k, v, o, lse, B, S, nh, nkv, ldq, ldk, ldv, softmax_scale, status, stream);
  if (head_dim == 64) return launch_flash_fwd<64>(q, k, v, o, lse, B, S, nh, nkv, ldq, ldk, ldv, softmax_scale, status, stream);
  return -3;
}
