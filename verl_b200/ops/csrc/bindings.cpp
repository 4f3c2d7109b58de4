// torch.ops.verl_b200.* bindings: tensors in, raw pointers + current stream out to the C launchers.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include "launchers.h"

namespace {

inline cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

#define CHECK_CUDA_CONTIG(x) TORCH_CHECK((x).is_cuda() && (x).is_contiguous(), #x " must be a contiguous CUDA tensor")

// D = A * B^T (+bias).  a: [M,K] (or [K,M] when a_mn), b: [N,K] (or [K,N] when b_mn). Rows may be strided views
// (stride(1) == 1).
at::Tensor gemm(const at::Tensor& a, const at::Tensor& b, const c10::optional<at::Tensor>& bias,
                const c10::optional<at::Tensor>& out, bool a_mn, bool b_mn, bool out_f32, bool accumulate,
                int64_t max_ctas) {
  TORCH_CHECK(a.is_cuda() && b.is_cuda(), "gemm: CUDA tensors required");
  TORCH_CHECK(a.scalar_type() == at::kBFloat16 && b.scalar_type() == at::kBFloat16, "gemm: bf16 operands required");
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && a.stride(1) == 1 && b.stride(1) == 1, "gemm: 2-D row-major operands");
  const c10::cuda::CUDAGuard guard(a.device());
  const int64_t M = a_mn ? a.size(1) : a.size(0);
  const int64_t K = a_mn ? a.size(0) : a.size(1);
  const int64_t N = b_mn ? b.size(1) : b.size(0);
  const int64_t Kb = b_mn ? b.size(0) : b.size(1);
  TORCH_CHECK(K == Kb, "gemm: contraction mismatch ", K, " vs ", Kb);
  at::Tensor d;
  if (out.has_value()) {
    d = *out;
    TORCH_CHECK(d.dim() == 2 && d.size(0) == M && d.size(1) == N && d.stride(1) == 1, "gemm: bad out shape");
    TORCH_CHECK(d.scalar_type() == (out_f32 ? at::kFloat : at::kBFloat16), "gemm: bad out dtype");
  } else {
    TORCH_CHECK(!accumulate, "gemm: accumulate needs out");
    d = at::empty({M, N}, a.options().dtype(out_f32 ? at::kFloat : at::kBFloat16));
  }
  const void* bias_ptr = nullptr;
  if (bias.has_value()) {
    TORCH_CHECK(bias->scalar_type() == at::kBFloat16 && bias->numel() == N && bias->is_contiguous(), "gemm: bad bias");
    bias_ptr = bias->data_ptr();
  }
  if (M == 0 || N == 0) return d;
  const int rc = vb_gemm_bf16(a.data_ptr(), b.data_ptr(), d.data_ptr(), bias_ptr, (int)M, (int)N, (int)K, a.stride(0),
                              b.stride(0), d.stride(0), a_mn, b_mn, out_f32, accumulate, (int)max_ctas, cur_stream());
  TORCH_CHECK(rc == 0, "vb_gemm_bf16 failed with code ", rc, " (M=", M, " N=", N, " K=", K, ")");
  return d;
}

int64_t gemm_status() { return vb_gemm_status(); }

}  // namespace

TORCH_LIBRARY(verl_b200, m) {
  m.def("gemm", &gemm);
  m.def("gemm_status", &gemm_status);
}
