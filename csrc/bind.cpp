// Python bindings: thin wrappers that unpack torch tensors and call the C launchers.
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include "gemm/gemm_api.h"
#include "ops_api.h"

#include <cstring>
#include <vector>

namespace {

using torch::Tensor;
using OptT = c10::optional<Tensor>;

cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

template <typename T>
T* ptr_or_null(const OptT& t) {
  return t.has_value() && t->defined() ? reinterpret_cast<T*>(t->data_ptr()) : nullptr;
}

void check_cuda(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
}

int64_t gemm(int64_t mode, int64_t epi, int64_t bn, int64_t a_mn, int64_t b_mn, int64_t M, int64_t N, int64_t K,
             int64_t num_experts, int64_t m_fast, int64_t beta, int64_t n_half, const Tensor& A, int64_t lda,
             int64_t a_inner, int64_t a_rows, const Tensor& B, int64_t ldb, int64_t b_expert_stride, int64_t b_inner,
             int64_t b_rows, int64_t b_experts, const OptT& tile_expert, const OptT& num_m_tiles,
             const OptT& seg_off, const Tensor& C, int64_t ldc, int64_t c_expert_stride, const OptT& aux0,
             int64_t ld_aux0, const OptT& aux1, int64_t ld_aux1, const Tensor& status, const OptT& ep_wait_flags,
             int64_t ep_wait_n, const OptT& ep_epoch_base, int64_t ep_wait_epoch_off,
             const std::vector<int64_t>& ep_scatter_dst, const OptT& ep_scatter_meta,
             const std::vector<int64_t>& ep_post_flags, int64_t ep_post_index, int64_t ep_post_epoch_off,
             int64_t ep_world, const OptT& ep_counter, int64_t cta2, const OptT& pair_tiles,
             int64_t ep_limit_ns, const OptT& a_gather, const OptT& b_gather, const OptT& row_slot,
             const OptT& row_w, const OptT& row_dot, const OptT& rope_cs, const OptT& rope_w, const OptT& rope_kw,
             const OptT& rope_rstd,
             int64_t rope_S, int64_t rope_nh, int64_t rope_nkv, double rope_eps) {
  check_cuda(A, "A");
  check_cuda(B, "B");
  check_cuda(C, "C");
  TORCH_CHECK(A.scalar_type() == at::kBFloat16 && B.scalar_type() == at::kBFloat16, "A and B must be bf16");
  c10::cuda::CUDAGuard guard(A.device());
  B200GemmDesc d;
  std::memset(&d, 0, sizeof(d));
  d.mode = (int)mode; d.epi = (int)epi; d.bn = (int)bn; d.a_mn = (int)a_mn; d.b_mn = (int)b_mn;
  d.M = (int)M; d.N = (int)N; d.K = (int)K;
  d.num_experts = (int)num_experts; d.m_fast = (int)m_fast; d.beta = (int)beta; d.n_half = (int)n_half;
  d.A = A.data_ptr(); d.lda = lda; d.a_inner = a_inner; d.a_rows = a_rows;
  d.B = B.data_ptr(); d.ldb = ldb; d.b_expert_stride = b_expert_stride; d.b_inner = b_inner; d.b_rows = b_rows;
  d.b_experts = (int)b_experts;
  d.tile_expert = ptr_or_null<const int>(tile_expert);
  d.num_m_tiles = ptr_or_null<const int>(num_m_tiles);
  d.seg_off = ptr_or_null<const int>(seg_off);
  d.C = C.data_ptr(); d.ldc = ldc; d.c_expert_stride = c_expert_stride;
  d.aux0 = ptr_or_null<void>(aux0); d.ld_aux0 = ld_aux0;
  d.aux1 = ptr_or_null<void>(aux1); d.ld_aux1 = ld_aux1;
  d.status = reinterpret_cast<int*>(status.data_ptr());
  d.ep_wait_flags = ptr_or_null<const int>(ep_wait_flags);
  d.ep_wait_n = (int)ep_wait_n;
  d.ep_epoch_base = ptr_or_null<const int>(ep_epoch_base);
  d.ep_wait_epoch_off = (int)ep_wait_epoch_off;
  for (size_t r = 0; r < ep_scatter_dst.size() && r < 8; ++r) d.ep_scatter_dst[r] = reinterpret_cast<void*>(ep_scatter_dst[r]);
  d.ep_scatter_meta = ptr_or_null<const int>(ep_scatter_meta);
  for (size_t r = 0; r < ep_post_flags.size() && r < 8; ++r) d.ep_post_flags[r] = reinterpret_cast<int*>(ep_post_flags[r]);
  d.ep_post_index = (int)ep_post_index;
  d.ep_post_epoch_off = (int)ep_post_epoch_off;
  d.ep_world = (int)ep_world;
  d.ep_counter = ptr_or_null<int>(ep_counter);
  d.ep_limit_ns = (unsigned long long)ep_limit_ns;
  d.a_gather = ptr_or_null<const int>(a_gather);
  d.b_gather = ptr_or_null<const int>(b_gather);
  if (d.a_gather != nullptr)
    TORCH_CHECK(a_gather->scalar_type() == at::kInt && (mode == 2 || a_gather->numel() >= M),
                "a_gather: int32, one entry per A row");
  if (d.b_gather != nullptr) TORCH_CHECK(b_gather->scalar_type() == at::kInt, "b_gather must be int32");
  d.row_slot = ptr_or_null<const int>(row_slot);
  d.row_w = ptr_or_null<const float>(row_w);
  d.row_dot = ptr_or_null<float>(row_dot);
  if (d.row_slot != nullptr)
    TORCH_CHECK(row_slot->scalar_type() == at::kInt && row_slot->numel() >= M, "row_slot: int32, one entry per row");
  if (d.row_w != nullptr) TORCH_CHECK(row_w->scalar_type() == at::kFloat, "row_w must be fp32");
  if (d.row_dot != nullptr) TORCH_CHECK(row_dot->scalar_type() == at::kFloat, "row_dot must be fp32");
  d.rope_cs = ptr_or_null<const float>(rope_cs);
  d.rope_w = ptr_or_null<const float>(rope_w);
  d.rope_kw = ptr_or_null<const float>(rope_kw);
  d.rope_rstd = ptr_or_null<float>(rope_rstd);
  d.rope_S = (int)rope_S; d.rope_nh = (int)rope_nh; d.rope_nkv = (int)rope_nkv; d.rope_eps = (float)rope_eps;
  if (epi == 6) {
    TORCH_CHECK(d.rope_cs && d.rope_w && d.rope_kw && d.rope_rstd,
                "fused QKV epilogue: rope_cs, rope_w, rope_kw and rope_rstd are required");
    TORCH_CHECK(rope_cs->scalar_type() == at::kFloat && rope_cs->numel() >= rope_S * 128 &&
                    rope_w->scalar_type() == at::kFloat && rope_w->numel() >= 128 &&
                    rope_kw->scalar_type() == at::kFloat && rope_kw->numel() >= 128 &&
                    rope_rstd->scalar_type() == at::kFloat && rope_rstd->numel() >= M * (rope_nh + rope_nkv),
                "fused QKV epilogue: fp32 table [S,64,2], weights [128] each, rstd [M, nh+nkv]");
  }
  d.cta2 = (int)cta2;
  d.pair_tiles = ptr_or_null<const int>(pair_tiles);
  d.max_pair_tiles = pair_tiles.has_value() && pair_tiles->defined() ? (int)(pair_tiles->numel() / 2) : 0;
  const int rc = b200_gemm(&d, cur_stream());
  TORCH_CHECK(rc == 0, "b200_gemm failed with host code ", rc);
  return rc;
}

}  // namespace

void bind_ops(pybind11::module_& m);  // bind_ops.cpp

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  namespace py = pybind11;
  m.def("gemm", &gemm, "tcgen05 GEMM family (dense / grouped)", py::arg("mode"), py::arg("epi"), py::arg("bn"),
        py::arg("a_mn"), py::arg("b_mn"), py::arg("M"), py::arg("N"), py::arg("K"), py::arg("num_experts"),
        py::arg("m_fast"), py::arg("beta"), py::arg("n_half"), py::arg("A"), py::arg("lda"), py::arg("a_inner"),
        py::arg("a_rows"), py::arg("B"), py::arg("ldb"), py::arg("b_expert_stride"), py::arg("b_inner"),
        py::arg("b_rows"), py::arg("b_experts"), py::arg("tile_expert"), py::arg("num_m_tiles"), py::arg("seg_off"),
        py::arg("C"), py::arg("ldc"), py::arg("c_expert_stride"), py::arg("aux0"), py::arg("ld_aux0"),
        py::arg("aux1"), py::arg("ld_aux1"), py::arg("status"), py::arg("ep_wait_flags") = py::none(),
        py::arg("ep_wait_n") = 0, py::arg("ep_epoch_base") = py::none(), py::arg("ep_wait_epoch_off") = 0,
        py::arg("ep_scatter_dst") = std::vector<int64_t>(), py::arg("ep_scatter_meta") = py::none(),
        py::arg("ep_post_flags") = std::vector<int64_t>(), py::arg("ep_post_index") = 0,
        py::arg("ep_post_epoch_off") = 0, py::arg("ep_world") = 0, py::arg("ep_counter") = py::none(),
        py::arg("cta2") = 0, py::arg("pair_tiles") = py::none(), py::arg("ep_limit_ns") = 0,
        py::arg("a_gather") = py::none(), py::arg("b_gather") = py::none(), py::arg("row_slot") = py::none(),
        py::arg("row_w") = py::none(), py::arg("row_dot") = py::none(), py::arg("rope_cs") = py::none(),
        py::arg("rope_w") = py::none(), py::arg("rope_kw") = py::none(), py::arg("rope_rstd") = py::none(),
        py::arg("rope_S") = 0,
        py::arg("rope_nh") = 0, py::arg("rope_nkv") = 0, py::arg("rope_eps") = 0.0);
  bind_ops(m);
}
