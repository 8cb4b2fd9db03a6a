// Host side of the tcgen05 GEMM family: tensor-map construction and kernel dispatch.
#include "gemm_api.h"
#include "gemm_sm100.cuh"
#include "gemm2_sm100.cuh"
#include "../common/tma_host.h"

#include <cudaTypedefs.h>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <unordered_map>

namespace b200 {

static PFN_cuTensorMapEncodeTiled_v12000 encode_fn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
  });
  return fn;
}

struct MapKey {
  const void* base;
  uint64_t d0, d1, d2, s1, s2;
  uint32_t b0, b1;
  bool operator==(const MapKey& o) const { return std::memcmp(this, &o, sizeof(MapKey)) == 0; }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    const uint64_t* p = reinterpret_cast<const uint64_t*>(&k);
    uint64_t h = 1469598103934665603ull;
    for (size_t i = 0; i < sizeof(MapKey) / 8; ++i) h = (h ^ p[i]) * 1099511628211ull;
    return static_cast<size_t>(h);
  }
};

// bf16 tensor, up to 3 dims (inner first), 128B swizzle, zero fill out of bounds.
static int g_last_encode_result = 0;
int tma_last_encode_result() { return g_last_encode_result; }

int make_map(CUtensorMap* out, const void* base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t s1_bytes,
                    uint64_t s2_bytes, uint32_t b0, uint32_t b1) {
  static std::mutex mu;
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  MapKey key;
  std::memset(&key, 0, sizeof(key));
  key.base = base;
  key.d0 = d0; key.d1 = d1; key.d2 = d2; key.s1 = s1_bytes; key.s2 = s2_bytes; key.b0 = b0; key.b1 = b1;
  {
    std::lock_guard<std::mutex> g(mu);
    auto it = cache.find(key);
    if (it != cache.end()) {
      *out = it->second;
      return 0;
    }
  }
  auto fn = encode_fn();
  if (fn == nullptr) return -1;
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0 || (s1_bytes & 15u) != 0 || (s2_bytes & 15u) != 0) return -2;
  const int rank = d2 > 0 ? 3 : 2;
  cuuint64_t dims[3] = {d0, d1, d2 > 0 ? d2 : 1};
  cuuint64_t strides[2] = {s1_bytes, s2_bytes};
  cuuint32_t box[3] = {b0, b1, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  auto encode = [&] {
    return fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rank, const_cast<void*>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  };
  CUresult r = encode();
  if (r == CUDA_ERROR_INVALID_CONTEXT) {
    // The encoder is a driver call and wants a current context; a thread that has not made a runtime call yet (an
    // autograd worker whose first node lands here) has none bound.  Any runtime call binds the primary context.
    (void)cudaFree(nullptr);
    r = encode();
  }
  if (r != CUDA_SUCCESS) {
    g_last_encode_result = static_cast<int>(r);
    return -3;
  }
  std::lock_guard<std::mutex> g(mu);
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, *out);
  return 0;
}

// Store-side map: 3-D tensor {d0 inner, d1, d2} of 2- or 4-byte elements, box {b0, b1, 1}, 128-byte swizzle.
int make_store_map(CUtensorMap* out, int elem_bytes, const void* base, uint64_t d0, uint64_t d1, uint64_t d2,
                   uint64_t s1_bytes, uint64_t s2_bytes, uint32_t b0, uint32_t b1) {
  static std::mutex mu;
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  MapKey key;
  std::memset(&key, 0, sizeof(key));
  key.base = base;
  key.d0 = d0; key.d1 = d1; key.d2 = d2; key.s1 = s1_bytes; key.s2 = s2_bytes; key.b0 = b0;
  key.b1 = b1 | (static_cast<uint32_t>(elem_bytes) << 16);
  {
    std::lock_guard<std::mutex> g(mu);
    auto it = cache.find(key);
    if (it != cache.end()) {
      *out = it->second;
      return 0;
    }
  }
  auto fn = encode_fn();
  if (fn == nullptr) return -1;
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0 || (s1_bytes & 15u) != 0 || (s2_bytes & 15u) != 0) return -2;
  if (b0 * static_cast<uint32_t>(elem_bytes) != 128u) return -2;
  cuuint64_t dims[3] = {d0, d1, d2 > 0 ? d2 : 1};
  cuuint64_t strides[2] = {s1_bytes, s2_bytes > 0 ? s2_bytes : s1_bytes * d1};
  cuuint32_t box[3] = {b0, b1, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  auto encode = [&] {
    return fn(out, elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3,
              const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  };
  CUresult r = encode();
  if (r == CUDA_ERROR_INVALID_CONTEXT) {  // see make_map
    (void)cudaFree(nullptr);
    r = encode();
  }
  if (r != CUDA_SUCCESS) {
    g_last_encode_result = static_cast<int>(r);
    return -3;
  }
  std::lock_guard<std::mutex> g(mu);
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, *out);
  return 0;
}

static int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  }
  return n;
}

template <int BN, bool A_MN, bool B_MN, int EPI>
static int launch_one(const CUtensorMap& ma, const CUtensorMap& mb, const GemmArgs& args, int grid,
                      cudaStream_t stream) {
  auto kern = gemm_sm100_kernel<BN, A_MN, B_MN, EPI>;
  constexpr int smem = EPI == EPI_BF16_SCATTER ? GemmCfg<BN>::SMEM_BYTES_SCATTER : GemmCfg<BN>::SMEM_BYTES;
  static_assert(smem <= 232448, "dynamic shared memory of one CTA");
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -10;
    configured = true;
  }
  kern<<<grid, GEMM_THREADS, smem, stream>>>(ma, mb, args);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// number of CTA pairs that can be resident at once (queried once per kernel variant)
template <int BN, bool A_MN, bool B_MN, int EPI>
static int launch_pair(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mc, const CUtensorMap& mx,
                       const GemmArgs& args, long long pair_tiles, cudaStream_t stream) {
  auto kern = gemm2_sm100_kernel<BN, A_MN, B_MN, EPI>;
  using Cfg = Gemm2Cfg<BN, EPI>;
  static int max_pairs = 0;
  if (max_pairs == 0) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES) != cudaSuccess)
      return -10;
    cudaLaunchConfig_t cfg;
    std::memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(static_cast<unsigned>(sm_count() / 2 * 2));
    cfg.blockDim = dim3(GEMM_THREADS);
    cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
    cudaLaunchAttribute at;
    at.id = cudaLaunchAttributeClusterDimension;
    at.val.clusterDim.x = 2;
    at.val.clusterDim.y = 1;
    at.val.clusterDim.z = 1;
    cfg.attrs = &at;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) {
      (void)cudaGetLastError();
      n = sm_count() / 2;
    }
    max_pairs = n < sm_count() / 2 ? n : sm_count() / 2;
  }
  long long pairs = pair_tiles < max_pairs ? pair_tiles : max_pairs;
  if (pairs <= 0) return 0;
  kern<<<static_cast<unsigned>(2 * pairs), GEMM_THREADS, Cfg::SMEM_BYTES, stream>>>(ma, mb, mc, mx, args);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

}  // namespace b200

using namespace b200;

extern "C" int b200_gemm(const B200GemmDesc* d, cudaStream_t stream) {
  const int bn = d->bn;
  if (bn != 256 && bn != 128 && bn != 64) return -20;
  GemmArgs a;
  a.mode = d->mode;
  a.M = d->M; a.N = d->N; a.K = d->K;
  a.num_experts = d->num_experts;
  a.m_fast = d->m_fast;
  a.beta = d->beta;
  a.n_half = d->n_half;
  a.tile_expert = d->tile_expert;
  a.num_m_tiles = d->num_m_tiles;
  a.seg_off = d->seg_off;
  a.pair_tiles = d->pair_tiles;
  a.max_pair_tiles = d->max_pair_tiles;
  a.a_gather = d->a_gather;
  a.b_gather = d->b_gather;
  a.row_slot = d->row_slot;
  a.row_w = d->row_w;
  a.row_dot = d->row_dot;
  a.rope_cs = d->rope_cs;
  a.rope_w = d->rope_w;
  a.rope_kw = d->rope_kw;
  a.rope_rstd = d->rope_rstd;
  a.rope_S = d->rope_S;
  a.rope_nh = d->rope_nh;
  a.rope_nkv = d->rope_nkv;
  a.rope_eps = d->rope_eps;
  if (d->epi == EPI_QKROPE) {
    if (!d->cta2 || d->bn != 256 || d->a_mn || d->b_mn || d->mode != MODE_DENSE) return -24;
    if (!d->rope_cs || !d->rope_w || !d->rope_kw || !d->rope_rstd || !d->aux0 || d->rope_S <= 0) return -24;
    if (d->N != (d->rope_nh + 2 * d->rope_nkv) * 128) return -24;
  }
  if ((a.a_gather || a.b_gather || a.row_w || a.row_dot) && !d->cta2) return -23;
  if ((a.row_w != nullptr) != (a.row_slot != nullptr)) return -23;
  a.C = d->C; a.ldc = d->ldc; a.c_expert_stride = d->c_expert_stride;
  a.aux0 = d->aux0; a.ld_aux0 = d->ld_aux0;
  a.aux1 = d->aux1; a.ld_aux1 = d->ld_aux1;
  a.status = d->status;
  a.ep.wait_flags = d->ep_wait_flags;
  a.ep.wait_n = d->ep_wait_n;
  a.ep.epoch_base = d->ep_epoch_base;
  a.ep.wait_epoch_off = d->ep_wait_epoch_off;
  for (int r = 0; r < 8; ++r) {
    a.ep.scatter_dst[r] = d->ep_scatter_dst[r];
    a.ep.post_flags[r] = d->ep_post_flags[r];
  }
  a.ep.scatter_meta = d->ep_scatter_meta;
  a.ep.post_index = d->ep_post_index;
  a.ep.post_epoch_off = d->ep_post_epoch_off;
  a.ep.world = d->ep_world;
  a.ep.counter = d->ep_counter;
  a.ep.limit_ns = d->ep_limit_ns ? d->ep_limit_ns : 10000000000ull;
  if ((a.ep.wait_flags || a.ep.counter) && a.ep.epoch_base == nullptr) return -22;
  if (d->epi == EPI_BF16_SCATTER && a.ep.scatter_meta == nullptr) return -22;

  CUtensorMap ma, mb;
  int rc;
  // A: 2-D. K-major: dims {K, rows}; MN-major: dims {M extent, contraction rows}.
  if (d->a_gather != nullptr) {
    if (d->a_mn && d->mode != MODE_GROUPED_K) return -23;
    rc = make_map(&ma, d->A, d->a_inner, d->a_rows, 0, static_cast<uint64_t>(d->lda) * 2, 0, 64, 1);  // gather box
  } else {
    rc = make_map(&ma, d->A, d->a_inner, d->a_rows, 0, static_cast<uint64_t>(d->lda) * 2, 0, 64, d->a_mn ? 64 : 128);
  }
  if (rc) return rc;
  if (d->cta2) {
    // ---- pair-tile kernel: each CTA loads bn/2 rows (or columns) of B; C and the SwiGLU side tensors
    // are written through TMA store maps
    if (bn != 256 && bn != 128) return -20;
    if (d->epi == EPI_BF16_SCATTER) return -21;
    if (d->mode == MODE_GROUPED_M && (d->pair_tiles == nullptr || d->max_pair_tiles <= 0)) return -22;
    if (d->b_gather != nullptr) {
      if (!d->b_mn || bn != 256 || d->mode != MODE_GROUPED_K) return -23;
      rc = make_map(&mb, d->B, d->b_inner, d->b_rows, 0, static_cast<uint64_t>(d->ldb) * 2, 0, 64, 1);  // gather box
    } else {
      rc = make_map(&mb, d->B, d->b_inner, d->b_rows, d->b_experts > 0 ? d->b_experts : 1,
                    static_cast<uint64_t>(d->ldb) * 2,
                    static_cast<uint64_t>(d->b_expert_stride > 0 ? d->b_expert_stride : d->ldb * (long long)d->b_rows) * 2,
                    64, d->b_mn ? 64u : static_cast<uint32_t>(bn / 2));
    }
    if (rc) return rc - 3;
    CUtensorMap mc, mx;
    const bool f32 = d->epi == EPI_F32;
    const int bn_out2 = d->epi == EPI_SWIGLU ? bn / 2 : bn;
    const uint64_t c_rows = d->mode == MODE_GROUPED_K ? static_cast<uint64_t>(d->M) : static_cast<uint64_t>(d->M);
    if (d->epi == EPI_SWIGLU_BWD) {
      // the epilogue reads the stored pre-activations through TMA: [2][rows][I] view of aux0 (gate, up planes)
      if (d->aux0 == nullptr) return -22;
      rc = make_store_map(&mc, 2, d->aux0, static_cast<uint64_t>(d->N), static_cast<uint64_t>(d->M), 2,
                          static_cast<uint64_t>(d->ld_aux0) * 2, static_cast<uint64_t>(d->n_half) * 2, 64, 32);
      if (rc) return rc - 6;
    } else {
      rc = make_store_map(&mc, f32 ? 4 : 2, d->C, static_cast<uint64_t>(d->N), c_rows,
                          d->mode == MODE_GROUPED_K ? static_cast<uint64_t>(d->num_experts) : 1,
                          static_cast<uint64_t>(d->ldc) * (f32 ? 4 : 2),
                          static_cast<uint64_t>(d->c_expert_stride) * (f32 ? 4 : 2), f32 ? 32 : 64, 32);
      if (rc) return rc - 6;
    }
    if (d->epi == EPI_QKROPE) {
      rc = make_store_map(&mx, 2, d->aux0, static_cast<uint64_t>(d->N), static_cast<uint64_t>(d->M), 1,
                          static_cast<uint64_t>(d->ld_aux0) * 2, static_cast<uint64_t>(d->ld_aux0) * 2 * d->M, 64, 32);
      if (rc) return rc - 9;
    } else if (d->epi == EPI_SWIGLU || d->epi == EPI_SWIGLU_BWD) {
      // [2][rows][I] view of the pre-activation tensor: plane 0 = gate columns, plane 1 = up columns
      void* xb = d->epi == EPI_SWIGLU ? d->aux0 : d->aux1;
      const long long ldx = d->epi == EPI_SWIGLU ? d->ld_aux0 : d->ld_aux1;
      if (xb == nullptr || (d->epi == EPI_SWIGLU_BWD && d->aux0 == nullptr)) return -22;
      rc = make_store_map(&mx, 2, xb, static_cast<uint64_t>(d->N), static_cast<uint64_t>(d->M), 2,
                          static_cast<uint64_t>(ldx) * 2, static_cast<uint64_t>(d->n_half) * 2, 64, 32);
      if (rc) return rc - 9;
    } else {
      mx = mc;
    }
    long long ptiles;
    if (d->mode == MODE_GROUPED_M)
      ptiles = static_cast<long long>(d->max_pair_tiles) * ((d->N + bn_out2 - 1) / bn_out2);
    else
      ptiles = static_cast<long long>((d->M + GEMM2_BM - 1) / GEMM2_BM) * ((d->N + bn_out2 - 1) / bn_out2) *
               (d->mode == MODE_GROUPED_K ? d->num_experts : 1);
#define B200_CASE2(BN_, AMN_, BMN_, EPI_)                                                   \
  if (bn == BN_ && d->a_mn == AMN_ && d->b_mn == BMN_ && d->epi == EPI_)                    \
    return launch_pair<BN_, AMN_ != 0, BMN_ != 0, EPI_>(ma, mb, mc, mx, a, ptiles, stream);
    B200_CASE2(256, 0, 0, EPI_BF16)
    B200_CASE2(128, 0, 0, EPI_BF16)
    B200_CASE2(256, 0, 1, EPI_BF16)
    B200_CASE2(128, 0, 1, EPI_BF16)
    B200_CASE2(256, 1, 1, EPI_F32)
    B200_CASE2(128, 1, 1, EPI_F32)
    B200_CASE2(256, 0, 0, EPI_F32)
    B200_CASE2(256, 0, 0, EPI_SWIGLU)
    B200_CASE2(256, 0, 1, EPI_SWIGLU_BWD)
    B200_CASE2(256, 0, 0, EPI_LSE)
    B200_CASE2(256, 0, 0, EPI_QKROPE)
#undef B200_CASE2
    return -21;
  }
  const uint32_t b_box_rows = d->b_mn ? 64u : (d->epi == EPI_SWIGLU ? bn / 2 : bn);
  rc = make_map(&mb, d->B, d->b_inner, d->b_rows, d->b_experts > 0 ? d->b_experts : 1,
                static_cast<uint64_t>(d->ldb) * 2,
                static_cast<uint64_t>(d->b_expert_stride > 0 ? d->b_expert_stride : d->ldb * (long long)d->b_rows) * 2,
                64, b_box_rows);
  if (rc) return rc - 3;

  const int bn_out = d->epi == EPI_SWIGLU ? bn / 2 : bn;
  long long tiles = static_cast<long long>((d->M + GEMM_BM - 1) / GEMM_BM) * ((d->N + bn_out - 1) / bn_out);
  if (d->mode == MODE_GROUPED_K) tiles *= d->num_experts;
  int grid = sm_count();
  if (tiles < grid) grid = static_cast<int>(tiles);
  if (grid <= 0) return 0;

#define B200_CASE(BN_, AMN_, BMN_, EPI_)                                                     \
  if (bn == BN_ && d->a_mn == AMN_ && d->b_mn == BMN_ && d->epi == EPI_)                    \
    return launch_one<BN_, AMN_ != 0, BMN_ != 0, EPI_>(ma, mb, a, grid, stream);
  B200_CASE(256, 0, 0, EPI_BF16)
  B200_CASE(128, 0, 0, EPI_BF16)
  B200_CASE(64, 0, 0, EPI_BF16)
  B200_CASE(256, 0, 1, EPI_BF16)
  B200_CASE(128, 0, 1, EPI_BF16)
  B200_CASE(256, 1, 1, EPI_F32)
  B200_CASE(128, 1, 1, EPI_F32)
  B200_CASE(256, 0, 0, EPI_F32)
  B200_CASE(128, 0, 0, EPI_F32)
  B200_CASE(64, 0, 0, EPI_F32)
  B200_CASE(256, 0, 0, EPI_SWIGLU)
  B200_CASE(128, 0, 0, EPI_SWIGLU)
  B200_CASE(256, 0, 1, EPI_SWIGLU_BWD)
  B200_CASE(128, 0, 1, EPI_SWIGLU_BWD)
  B200_CASE(256, 0, 0, EPI_LSE)
  B200_CASE(256, 0, 0, EPI_BF16_SCATTER)
  B200_CASE(128, 0, 0, EPI_BF16_SCATTER)
  B200_CASE(256, 0, 1, EPI_BF16_SCATTER)
  B200_CASE(128, 0, 1, EPI_BF16_SCATTER)
#undef B200_CASE
  return -21;
}
