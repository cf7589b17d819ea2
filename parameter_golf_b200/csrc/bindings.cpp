// pybind11 bindings: torch tensors in, raw pointers + the current CUDA stream out to the kernel library.
#include <ATen/cuda/CUDAContext.h>
#include <pybind11/numpy.h>
#include <pybind11/stl.h>
#include <torch/extension.h>

#include "artifact.h"
#include "loader.h"
#include "pgb.h"

namespace {

cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

void check_bf16(const torch::Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(t.scalar_type() == torch::kBFloat16, name, " must be bfloat16");
}

int* status_ptr(const c10::optional<torch::Tensor>& status) {
  if (!status.has_value()) return nullptr;
  TORCH_CHECK(status->is_cuda() && status->scalar_type() == torch::kInt32 && status->numel() >= 4, "status must be int32[4] on CUDA");
  return status->data_ptr<int>();
}

// Operands are 2-D ([rows, cols]) or 3-D ([batch, rows, cols]) with a contiguous last dim.
// a_kmajor: A is [.., M, K]; otherwise A is [.., K, M]. Same for B with N.
void gemm(torch::Tensor A, torch::Tensor B, torch::Tensor D, bool a_kmajor, bool b_kmajor, int64_t epi, double alpha, double beta,
          double slope, c10::optional<torch::Tensor> aux, c10::optional<torch::Tensor> colscale, c10::optional<torch::Tensor> D2,
          int64_t splits, c10::optional<torch::Tensor> status, c10::optional<torch::Tensor> wait_flag, int64_t wait_value,
          int64_t seg_row0, c10::optional<torch::Tensor> seg_D0, int64_t seg_row1, c10::optional<torch::Tensor> seg_D1,
          c10::optional<torch::Tensor> batch_sumsq, int64_t sumsq_pow) {
  check_bf16(A, "A");
  check_bf16(B, "B");
  TORCH_CHECK(A.dim() == B.dim() && A.dim() == D.dim() && (A.dim() == 2 || A.dim() == 3), "gemm: operands must all be 2-D or all 3-D");
  TORCH_CHECK(A.stride(-1) == 1 && B.stride(-1) == 1 && D.stride(-1) == 1, "gemm: last dim must be contiguous");
  const int nd = A.dim();
  pgb::GemmArgs g;
  g.batch = nd == 3 ? (int)A.size(0) : 1;
  g.a_kmajor = a_kmajor;
  g.b_kmajor = b_kmajor;
  g.M = (int)(a_kmajor ? A.size(-2) : A.size(-1));
  g.K = (int)(a_kmajor ? A.size(-1) : A.size(-2));
  g.N = (int)(b_kmajor ? B.size(-2) : B.size(-1));
  const int kb = (int)(b_kmajor ? B.size(-1) : B.size(-2));
  TORCH_CHECK(kb == g.K, "gemm: reduction dims differ: ", g.K, " vs ", kb);
  const bool segmented = seg_D0.has_value();
  TORCH_CHECK(D.size(-1) == g.N && (segmented ? D.size(-2) == seg_row0 : D.size(-2) == g.M), "gemm: D must be [M, N]");
  if (segmented) {
    // rows [0, seg_row0) -> D, [seg_row0, seg_row1) -> seg_D0, [seg_row1, M) -> seg_D1 (when given)
    const int64_t end0 = seg_D1.has_value() ? seg_row1 : g.M;
    TORCH_CHECK(seg_row0 > 0 && seg_D0->scalar_type() == torch::kFloat32 && seg_D0->is_cuda() && seg_D0->dim() == nd && seg_D0->size(-1) == g.N &&
                    seg_D0->size(-2) == end0 - seg_row0 && seg_D0->stride(-2) == D.stride(-2) && seg_D0->stride(-1) == 1,
                "gemm: first row segment must be fp32 [rows, N] with D's row stride");
    g.seg_rows[0] = (int)seg_row0;
    g.seg_D[0] = seg_D0->data_ptr<float>();
    if (seg_D1.has_value()) {
      TORCH_CHECK(seg_row1 > seg_row0 && seg_D1->scalar_type() == torch::kFloat32 && seg_D1->is_cuda() && seg_D1->dim() == nd &&
                      seg_D1->size(-1) == g.N && seg_D1->size(-2) == g.M - seg_row1 && seg_D1->stride(-2) == D.stride(-2) && seg_D1->stride(-1) == 1,
                  "gemm: second row segment must be fp32 [rows, N] with D's row stride");
      g.seg_rows[1] = (int)seg_row1;
      g.seg_D[1] = seg_D1->data_ptr<float>();
    }
    TORCH_CHECK(nd == 2, "gemm: row segments are for un-batched products");
  }
  if (nd == 3) TORCH_CHECK(B.size(0) == g.batch && D.size(0) == g.batch, "gemm: batch sizes differ");
  g.A = A.data_ptr();
  g.B = B.data_ptr();
  g.D = D.data_ptr();
  g.lda = A.stride(-2);
  g.ldb = B.stride(-2);
  g.ldd = D.stride(-2);
  g.stride_a = nd == 3 ? A.stride(0) : 0;
  g.stride_b = nd == 3 ? B.stride(0) : 0;
  g.stride_d = nd == 3 ? D.stride(0) : 0;
  g.epi = (int)epi;
  const bool f32_out = (epi == pgb::EPI_F32 || epi == pgb::EPI_F32_ATOMIC);
  TORCH_CHECK(D.scalar_type() == (f32_out ? torch::kFloat32 : torch::kBFloat16), "gemm: D dtype does not match the epilogue");
  if (aux.has_value()) {
    check_bf16(*aux, "aux");
    TORCH_CHECK(aux->dim() == nd && aux->size(-2) == g.M && aux->size(-1) == g.N && aux->stride(-1) == 1, "gemm: aux must be [M, N]");
    g.aux = aux->data_ptr();
    g.ld_aux = aux->stride(-2);
    g.stride_aux = nd == 3 ? aux->stride(0) : 0;
  }
  if (epi == pgb::EPI_AXPBY_BF16 || epi == pgb::EPI_RESID_BF16 || epi == pgb::EPI_MUL_ACTGRAD)
    TORCH_CHECK(g.aux != nullptr, "gemm: this epilogue needs aux");
  if (colscale.has_value()) {
    TORCH_CHECK(colscale->is_cuda() && colscale->scalar_type() == torch::kFloat32 && colscale->numel() == g.N && colscale->is_contiguous(),
                "gemm: colscale must be fp32[N]");
    g.colscale = colscale->data_ptr<float>();
  }
  if (epi == pgb::EPI_RESID_BF16) TORCH_CHECK(g.colscale != nullptr, "gemm: residual epilogue needs colscale");
  if (D2.has_value()) {
    check_bf16(*D2, "D2");
    TORCH_CHECK(D2->sizes() == D.sizes() && D2->strides() == D.strides(), "gemm: D2 must match D");
    g.D2 = D2->data_ptr();
  }
  if (epi == pgb::EPI_ACT_SQ) TORCH_CHECK(g.D2 != nullptr, "gemm: activation epilogue needs D2");
  g.alpha = (float)alpha;
  g.beta = (float)beta;
  g.slope = (float)slope;
  g.splits = (int)splits;
  g.status = status_ptr(status);
  if (wait_flag.has_value()) {
    TORCH_CHECK(wait_flag->is_cuda() && wait_flag->scalar_type() == torch::kInt32, "wait_flag must be a CUDA int32 tensor");
    g.wait_flag = wait_flag->data_ptr<int>();
    g.wait_value = (int)wait_value;
  }
  if (batch_sumsq.has_value()) {
    TORCH_CHECK(batch_sumsq->is_cuda() && batch_sumsq->scalar_type() == torch::kFloat32 && batch_sumsq->is_contiguous() && batch_sumsq->numel() >= g.batch &&
                    (sumsq_pow == 1 || sumsq_pow == 2) && !f32_out,
                "gemm: batch_sumsq must be fp32[batch] (power 1 or 2) with a bf16 epilogue");
    g.batch_sumsq = batch_sumsq->data_ptr<float>();
    g.sumsq_pow = (int)sumsq_pow;
  }
  pgb::gemm_bf16(g, cur_stream());
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("gemm", &gemm, "tcgen05 bf16 GEMM with fused epilogue");
  // ---- host-side artifact primitives (artifact.cpp) -----------------------------------------------------------------
  m.def("pack_bits", [](py::buffer q, int bits) {
    py::buffer_info info = q.request();
    TORCH_CHECK(info.itemsize == 1, "pack_bits expects int8 codes");
    std::string out;
    {
      py::gil_scoped_release nogil;
      out = pgb::pack_bits(static_cast<const int8_t*>(info.ptr), (size_t)info.size, bits);
    }
    return py::bytes(out);
  });
  m.def("unpack_bits", [](py::bytes data, size_t count, int bits) {
    const std::string d = data;
    py::array_t<int8_t> out((py::ssize_t)count);
    pgb::unpack_bits(reinterpret_cast<const uint8_t*>(d.data()), d.size(), count, bits, out.mutable_data());
    return out;
  });
  m.def("crc32", [](py::bytes data) {
    const std::string d = data;
    return pgb::crc32_ieee(reinterpret_cast<const uint8_t*>(d.data()), d.size());
  });
  m.def("write_pgrs", [](const std::vector<std::tuple<std::string, std::vector<uint32_t>, int, py::bytes>>& tensors, const std::string& metadata) {
    std::vector<pgb::PgrsTensor> ts;
    ts.reserve(tensors.size());
    for (const auto& t : tensors) {
      pgb::PgrsTensor r;
      r.name = std::get<0>(t);
      r.dims = std::get<1>(t);
      r.dtype = (uint8_t)std::get<2>(t);
      r.data = std::get<3>(t);
      ts.push_back(std::move(r));
    }
    return py::bytes(pgb::write_pgrs(ts, metadata));
  });
  m.def("read_pgrs", [](py::bytes buf) {
    std::string meta;
    const std::vector<pgb::PgrsTensor> ts = pgb::read_pgrs(buf, &meta);
    py::list out;
    for (const auto& t : ts) out.append(py::make_tuple(t.name, t.dims, (int)t.dtype, py::bytes(t.data)));
    return py::make_tuple(out, meta);
  });
#include "bindings_more.inc"
}
