// torch.ops.verl_b200.* bindings: tensors in, raw pointers + current stream out to the C launchers.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include "launchers.h"

#include <algorithm>
#include <atomic>
#include <cstdlib>
#include <vector>

namespace {

// Number of kernels of this library launched (or captured into a CUDA graph) by this process.
std::atomic<int64_t> g_launches{0};
inline void count(int64_t n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
int64_t launch_count() { return g_launches.load(std::memory_order_relaxed); }
void add_launches(int64_t n) { count(n); }

using at::Tensor;
using OptTensor = c10::optional<at::Tensor>;

inline cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }
inline const void* optr(const OptTensor& t) { return t.has_value() ? t->data_ptr() : nullptr; }
inline const float* fptr(const OptTensor& t) { return t.has_value() ? t->data_ptr<float>() : nullptr; }

#define CHECK_BF16(x) TORCH_CHECK((x).is_cuda() && (x).scalar_type() == at::kBFloat16, #x " must be a CUDA bf16 tensor")
#define CHECK_F32(x) TORCH_CHECK((x).is_cuda() && (x).scalar_type() == at::kFloat, #x " must be a CUDA fp32 tensor")
#define CHECK_RC(rc, what) TORCH_CHECK((rc) == 0, what " failed with code ", (rc))

// VERL_B200_SKINNY_GEMM=0 routes GEMMs with few tokens through the general kernel (read once per process).
static bool skinny_enabled() {
  static const bool on = [] { const char* v = getenv("VERL_B200_SKINNY_GEMM"); return v == nullptr || v[0] != '0'; }();
  return on;
}

// Row ranges of one weight matrix against few tokens in one launch: out[:, c_s : c_s + rows_s] = a @ w[w0_s : w0_s + rows_s]^T
// (+ bias[w0_s : ...]) with the ranges' outputs side by side. ranges: flat list (w0, rows, w0, rows, ...), at most four ranges,
// rows multiples of 8. Returns false (and does nothing) when the shape is not served: the caller then runs one GEMM per range.
bool gemm_row_ranges_(const Tensor& a, const Tensor& w, const OptTensor& bias, std::vector<int64_t> ranges, Tensor out) {
  if (!skinny_enabled() || !a.is_cuda() || a.scalar_type() != at::kBFloat16 || w.scalar_type() != at::kBFloat16) return false;
  const int64_t M = a.size(0), K = a.size(1);
  const int nseg = (int)(ranges.size() / 2);
  if (a.dim() != 2 || w.dim() != 2 || w.size(1) != K || a.stride(1) != 1 || w.stride(1) != 1 || M < 1 || M > 1024 || nseg < 1 || nseg > 4 ||
      K % 8 || a.stride(0) % 8 || w.stride(0) % 8 || out.stride(0) % 4 || out.stride(1) != 1 || out.scalar_type() != at::kBFloat16 ||
      reinterpret_cast<uintptr_t>(out.data_ptr()) % 8 || reinterpret_cast<uintptr_t>(a.data_ptr()) % 16 ||
      reinterpret_cast<uintptr_t>(w.data_ptr()) % 16)
    return false;
  int w0[4], rows[4];
  int64_t N = 0;
  for (int s = 0; s < nseg; ++s) {
    w0[s] = (int)ranges[2 * s];
    rows[s] = (int)ranges[2 * s + 1];
    if (rows[s] <= 0 || rows[s] % 8 || w0[s] < 0 || w0[s] + rows[s] > w.size(0)) return false;
    N += rows[s];
  }
  TORCH_CHECK(out.dim() == 2 && out.size(0) == M && out.size(1) == N, "gemm_row_ranges_: out must be [M, sum of the ranges' rows]");
  const void* bias_ptr = nullptr;
  if (bias.has_value()) {
    TORCH_CHECK(bias->scalar_type() == at::kBFloat16 && bias->numel() == w.size(0) && bias->is_contiguous(), "gemm_row_ranges_: bias per row of w");
    bias_ptr = bias->data_ptr();
  }
  const c10::cuda::CUDAGuard guard(a.device());
  const int s = vb_gemm_skinny_seg_splits((int)M, (int)K, nseg, w0, rows);
  if (s < 1) return false;
  Tensor ws;
  if (s > 1) ws = at::empty({s, M, N}, a.options().dtype(at::kFloat));
  count(1);
  const int rc = vb_gemm_skinny_seg(a.data_ptr(), w.data_ptr(), out.data_ptr(), bias_ptr, (int)M, (int)K, (int)w.size(0), a.stride(0),
                                    w.stride(0), out.stride(0), nseg, w0, rows, s, s > 1 ? ws.data_ptr<float>() : nullptr, (int)M, 0,
                                    cur_stream());
  TORCH_CHECK(rc == 0, "vb_gemm_skinny_seg failed with code ", rc, " (M=", M, " N=", N, " K=", K, ")");
  return true;
}

// D = A * B^T (+bias).  a: [M,K] (or [K,M] when a_mn), b: [N,K] (or [K,N] when b_mn); rows may be strided.
Tensor gemm(const Tensor& a, const Tensor& b, const OptTensor& bias, const OptTensor& out, bool a_mn, bool b_mn,
            bool out_f32, bool accumulate, int64_t max_ctas) {
  CHECK_BF16(a);
  CHECK_BF16(b);
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && a.stride(1) == 1 && b.stride(1) == 1, "gemm: 2-D row-major operands");
  const c10::cuda::CUDAGuard guard(a.device());
  const int64_t M = a_mn ? a.size(1) : a.size(0);
  const int64_t K = a_mn ? a.size(0) : a.size(1);
  const int64_t N = b_mn ? b.size(1) : b.size(0);
  const int64_t Kb = b_mn ? b.size(0) : b.size(1);
  TORCH_CHECK(K == Kb, "gemm: contraction mismatch ", K, " vs ", Kb);
  Tensor d;
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
  if (skinny_enabled() && M <= 1024 && !a_mn && !b_mn && !out_f32 && !accumulate && max_ctas == 0 && N % 8 == 0 && K % 8 == 0 &&
      a.stride(0) % 8 == 0 && b.stride(0) % 8 == 0 && d.stride(0) % 4 == 0 && reinterpret_cast<uintptr_t>(d.data_ptr()) % 8 == 0 &&
      reinterpret_cast<uintptr_t>(a.data_ptr()) % 16 == 0 && reinterpret_cast<uintptr_t>(b.data_ptr()) % 16 == 0) {
    // few tokens: the transposed kernel (128 weight rows x up to 512 tokens per CTA, K split with the fold inside the launch)
    const int s = vb_gemm_skinny_splits((int)M, (int)N, (int)K);
    if (s >= 1) {
      Tensor ws;
      if (s > 1) ws = at::empty({s, M, N}, a.options().dtype(at::kFloat));
      count(1);
      const int rc = vb_gemm_skinny(a.data_ptr(), b.data_ptr(), d.data_ptr(), bias_ptr, (int)M, (int)N, (int)K, a.stride(0), b.stride(0),
                                    d.stride(0), s, s > 1 ? ws.data_ptr<float>() : nullptr, (int)M, 0, cur_stream());
      TORCH_CHECK(rc == 0, "vb_gemm_skinny failed with code ", rc, " (M=", M, " N=", N, " K=", K, ")");
      return d;
    }
  }
  // skinny GEMMs (decode: few output tiles, deep K) are split along K so that every SM streams weights
  const int splits = (max_ctas == 0) ? vb_gemm_suggest_splits((int)M, (int)N, (int)K) : 1;
  Tensor ws;
  if (splits > 1) ws = at::empty({splits, M, N}, a.options().dtype(at::kFloat));
  count((splits > 1 && !vb_gemm_fold_in_kernel()) ? 2 : 1);  // GEMM (+ the reduce launch of a K-split one)
  const int rc = vb_gemm_bf16_ex(a.data_ptr(), b.data_ptr(), d.data_ptr(), bias_ptr, (int)M, (int)N, (int)K, a.stride(0),
                                 b.stride(0), d.stride(0), a_mn, b_mn, out_f32, accumulate, (int)max_ctas, splits,
                                 splits > 1 ? ws.data_ptr<float>() : nullptr, cur_stream());
  TORCH_CHECK(rc == 0, "vb_gemm_bf16 failed with code ", rc, " (M=", M, " N=", N, " K=", K, ")");
  return d;
}

// act = silu(a W_gate^T) * (a W_up^T) for the stacked weight w = [W_gate; W_up] ([2I, K]); with want_gu the pre-activation
// [M, 2I] is returned as well (else an empty tensor).
std::tuple<Tensor, Tensor> gemm_swiglu(const Tensor& a, const Tensor& w, bool want_gu) {
  CHECK_BF16(a);
  CHECK_BF16(w);
  TORCH_CHECK(a.dim() == 2 && w.dim() == 2 && a.stride(1) == 1 && w.stride(1) == 1 && a.size(1) == w.size(1) && w.size(0) % 2 == 0,
              "gemm_swiglu: a [M, K], w [2I, K]");
  const c10::cuda::CUDAGuard guard(a.device());
  const int64_t M = a.size(0), K = a.size(1), I = w.size(0) / 2;
  Tensor act = at::empty({M, I}, a.options());
  Tensor gu = want_gu ? at::empty({M, 2 * I}, a.options()) : at::empty({0}, a.options());
  if (M == 0) return {act, gu};
  count(1);
  const int rc = vb_gemm_bf16_swiglu(a.data_ptr(), w.data_ptr(), act.data_ptr(), want_gu ? gu.data_ptr() : nullptr, (int)M, (int)I, (int)K,
                                     a.stride(0), w.stride(0), act.stride(0), 2 * I, cur_stream());
  TORCH_CHECK(rc == 0, "vb_gemm_bf16_swiglu failed with code ", rc, " (M=", M, " I=", I, " K=", K, ")");
  return {act, gu};
}

int64_t gemm_status() {
  int a = vb_gemm_status();
  if (a == 0) a = vb_gemm_skinny_status();
  int b = vb_attn_status();
  if (b == 0) b = vb_attn_bwd_status();
  if (b == 0) b = vb_fp8_status();
  const int c = vb_pd_status();
  return a != 0 ? a : (b != 0 ? 100 + b : (c != 0 ? 200 + c : 0));
}

// Causal GQA attention over packed sequences. q [T, nh, hd], k/v [T, nkv, hd] (strided views), cu_seqlens int32 [B+1].
// Returns (out [T, nh, hd] bf16, lse [nh, T] fp32).
std::tuple<Tensor, Tensor> attn_fwd(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& cu_seqlens,
                                    double scale) {
  CHECK_BF16(q);
  CHECK_BF16(k);
  CHECK_BF16(v);
  TORCH_CHECK(q.dim() == 3 && k.dim() == 3 && q.stride(2) == 1 && q.stride(1) == q.size(2) && k.stride(1) == k.size(2) &&
              v.stride(1) == v.size(2), "attn_fwd: [T, heads, hd] views with packed heads");
  TORCH_CHECK(cu_seqlens.is_cuda() && cu_seqlens.scalar_type() == at::kInt && cu_seqlens.is_contiguous());
  const c10::cuda::CUDAGuard guard(q.device());
  const int64_t T = q.size(0), nh = q.size(1), hd = q.size(2), nkv = k.size(1);
  Tensor out = at::empty({T, nh, hd}, q.options());
  Tensor lse = at::empty({nh, T}, q.options().dtype(at::kFloat));
  count(1);
  const int rc = vb_attn_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), q.stride(0), k.stride(0), v.stride(0),
                             cu_seqlens.data_ptr<int>(), (int)cu_seqlens.numel() - 1, (int)T, (int)nh, (int)nkv, (int)hd,
                             (float)scale, out.data_ptr(), out.stride(0), lse.data_ptr<float>(), cur_stream());
  CHECK_RC(rc, "vb_attn_fwd");
  return {out, lse};
}

// (dq, dk, dv) of causal varlen GQA attention; q/out/dout: [T, nh, hd] views, k/v: [T, nkv, hd] views, lse [nh, T].
std::tuple<Tensor, Tensor, Tensor> attn_bwd(const Tensor& dout, const Tensor& q, const Tensor& k, const Tensor& v,
                                            const Tensor& out, const Tensor& lse, const Tensor& cu_seqlens, int64_t max_seqlen,
                                            double scale) {
  CHECK_BF16(q);
  CHECK_BF16(k);
  CHECK_BF16(v);
  CHECK_BF16(out);
  CHECK_BF16(dout);
  CHECK_F32(lse);
  auto packed = [](const Tensor& t) { return t.dim() == 3 && t.stride(2) == 1 && t.stride(1) == t.size(2); };
  TORCH_CHECK(packed(q) && packed(k) && packed(v) && packed(out) && packed(dout), "attn_bwd: [T, heads, hd] views with packed heads");
  TORCH_CHECK(cu_seqlens.is_cuda() && cu_seqlens.scalar_type() == at::kInt && cu_seqlens.is_contiguous() && lse.is_contiguous());
  const c10::cuda::CUDAGuard guard(q.device());
  const int64_t T = q.size(0), nh = q.size(1), hd = q.size(2), nkv = k.size(1);
  Tensor dq = at::empty({T, nh, hd}, q.options());
  Tensor dk = at::empty({T, nkv, hd}, q.options());
  Tensor dv = at::empty({T, nkv, hd}, q.options());
  if (T == 0) return {dq, dk, dv};
  auto fo = q.options().dtype(at::kFloat);
  Tensor delta = at::empty({nh, T}, fo);
  Tensor dq32 = at::empty({T, nh * hd}, fo);
  count(4);
  const int rc = vb_attn_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), dout.data_ptr(), q.stride(0), k.stride(0),
                             v.stride(0), out.stride(0), dout.stride(0), lse.data_ptr<float>(), cu_seqlens.data_ptr<int>(),
                             (int)cu_seqlens.numel() - 1, (int)T, (int)nh, (int)nkv, (int)hd, (float)scale, dq.data_ptr(),
                             dk.data_ptr(), dv.data_ptr(), dq.stride(0), dk.stride(0), dv.stride(0), delta.data_ptr<float>(),
                             dq32.data_ptr<float>(), (int)max_seqlen, cur_stream());
  CHECK_RC(rc, "vb_attn_bwd");
  return {dq, dk, dv};
}

// (logprob, entropy, lse) of labels under softmax(hidden @ weight^T / temperature); [T,V] logits never exist.
std::tuple<Tensor, Tensor, Tensor> lmhead_fwd(const Tensor& hidden, const Tensor& weight, const Tensor& labels,
                                              double inv_temp) {
  CHECK_BF16(hidden);
  CHECK_BF16(weight);
  TORCH_CHECK(labels.is_cuda() && labels.scalar_type() == at::kLong && labels.is_contiguous(), "labels: int64");
  TORCH_CHECK(hidden.dim() == 2 && weight.dim() == 2 && hidden.stride(1) == 1 && weight.stride(1) == 1);
  const c10::cuda::CUDAGuard guard(hidden.device());
  const int64_t T = hidden.size(0), H = hidden.size(1), V = weight.size(0);
  TORCH_CHECK(weight.size(1) == H && labels.numel() == T);
  auto fo = hidden.options().dtype(at::kFloat);
  Tensor lp = at::empty({T}, fo), ent = at::empty({T}, fo), lse = at::empty({T}, fo);
  if (T == 0) return {lp, ent, lse};
  Tensor partial = at::empty({3, (int64_t)vb_lmhead_num_tiles((int)V), T}, fo);
  Tensor lab = at::zeros({T}, fo);
  count(2);
  const int rc = vb_lmhead_fwd(hidden.data_ptr(), weight.data_ptr(), reinterpret_cast<long long*>(labels.data_ptr()), (float)inv_temp,
                               partial.data_ptr<float>(), lab.data_ptr<float>(), lp.data_ptr<float>(),
                               ent.data_ptr<float>(), lse.data_ptr<float>(), (int)T, (int)V, (int)H, hidden.stride(0),
                               weight.stride(0), cur_stream());
  CHECK_RC(rc, "vb_lmhead_fwd");
  return {lp, ent, lse};
}

// d loss / d logits for vocabulary rows [v0, v0 + weight_chunk.size(0)) as bf16 [T, Vc].
Tensor lmhead_dlogits(const Tensor& hidden, const Tensor& weight_chunk, const Tensor& labels, int64_t v0,
                      double inv_temp, const Tensor& lse, const OptTensor& ex, const Tensor& g_lp,
                      const OptTensor& g_ent, const OptTensor& out) {
  CHECK_BF16(hidden);
  CHECK_BF16(weight_chunk);
  CHECK_F32(lse);
  CHECK_F32(g_lp);
  const c10::cuda::CUDAGuard guard(hidden.device());
  const int64_t T = hidden.size(0), H = hidden.size(1), Vc = weight_chunk.size(0);
  Tensor d = out.has_value() ? *out : at::empty({T, Vc}, hidden.options());
  TORCH_CHECK(d.size(0) == T && d.size(1) == Vc && d.stride(1) == 1);
  count(1);
  const int rc = vb_lmhead_dlogits(hidden.data_ptr(), weight_chunk.data_ptr(), reinterpret_cast<long long*>(labels.data_ptr()), (int)v0,
                                   (float)inv_temp, lse.data_ptr<float>(), fptr(ex), g_lp.data_ptr<float>(),
                                   fptr(g_ent), d.data_ptr(), (int)T, (int)Vc, (int)H, hidden.stride(0),
                                   weight_chunk.stride(0), d.stride(0), cur_stream());
  CHECK_RC(rc, "vb_lmhead_dlogits");
  return d;
}

// y = rmsnorm(x (+ residual)) * w. Returns (y, residual_out or x, rstd).
std::tuple<Tensor, Tensor, Tensor> rmsnorm_fwd(const Tensor& x, const OptTensor& residual, const Tensor& w,
                                               double eps) {
  CHECK_BF16(x);
  CHECK_BF16(w);
  TORCH_CHECK(x.is_contiguous() && w.is_contiguous());
  const c10::cuda::CUDAGuard guard(x.device());
  const int64_t H = x.size(-1), T = x.numel() / H;
  Tensor y = at::empty_like(x);
  Tensor rstd = at::empty({T}, x.options().dtype(at::kFloat));
  Tensor res_out = residual.has_value() ? at::empty_like(x) : x;
  if (residual.has_value()) TORCH_CHECK(residual->is_contiguous() && residual->sizes() == x.sizes());
  count(1);
  const int rc = vb_rmsnorm_fwd(x.data_ptr(), optr(residual), w.data_ptr(), y.data_ptr(),
                                residual.has_value() ? res_out.data_ptr() : nullptr, rstd.data_ptr<float>(), (int)T,
                                (int)H, (float)eps, cur_stream());
  CHECK_RC(rc, "vb_rmsnorm_fwd");
  return {y, res_out, rstd};
}

// dx = d/dx of rmsnorm (+ dres_in); dw accumulated into `dw` (fp32 [H]) when accumulate, else overwritten.
Tensor rmsnorm_bwd(const Tensor& dy, const Tensor& x, const Tensor& w, const Tensor& rstd, const OptTensor& dres_in,
                   Tensor dw, bool accumulate) {
  CHECK_BF16(dy);
  CHECK_BF16(x);
  CHECK_F32(dw);
  TORCH_CHECK(dy.is_contiguous() && x.is_contiguous());
  const c10::cuda::CUDAGuard guard(x.device());
  const int64_t H = x.size(-1), T = x.numel() / H;
  Tensor dx = at::empty_like(x);
  if (T == 0) return dx;
  Tensor scratch = at::empty({(int64_t)vb_rmsnorm_bwd_blocks((int)T), H}, x.options().dtype(at::kFloat));
  count(2);
  const int rc = vb_rmsnorm_bwd(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr<float>(), optr(dres_in),
                                dx.data_ptr(), dw.data_ptr<float>(), scratch.data_ptr<float>(), (int)T, (int)H,
                                accumulate, cur_stream());
  CHECK_RC(rc, "vb_rmsnorm_bwd");
  return dx;
}

// In-place rotary embedding on x [T, nheads, hd] (a view with row stride x.stride(0)).
void rope_(Tensor x, const Tensor& pos, const Tensor& cos_t, const Tensor& sin_t, bool backward) {
  CHECK_BF16(x);
  CHECK_F32(cos_t);
  TORCH_CHECK(x.dim() == 3 && x.stride(2) == 1 && x.stride(1) == x.size(2), "rope: [T, nheads, hd] with packed heads");
  TORCH_CHECK(pos.scalar_type() == at::kInt && pos.is_contiguous(), "rope: int32 positions");
  const c10::cuda::CUDAGuard guard(x.device());
  count(1);
  const int rc = vb_rope(x.data_ptr(), pos.data_ptr<int>(), cos_t.data_ptr<float>(), sin_t.data_ptr<float>(),
                         (int)x.size(0), (int)x.size(1), (int)x.size(2), x.stride(0), backward, cur_stream());
  CHECK_RC(rc, "vb_rope");
}

// qkv bf16 [T, (nh + 2 nkv) * hd] (projection output, row-contiguous); caches [num_blocks, block_size, nkv, hd]; slot int64 [T]
void rope_kv_append_(Tensor qkv, const Tensor& pos, const Tensor& cos_t, const Tensor& sin_t, const Tensor& slot, Tensor kc, Tensor vc,
                     int64_t nh, int64_t nkv, int64_t hd) {
  CHECK_BF16(qkv);
  CHECK_F32(cos_t);
  TORCH_CHECK(qkv.dim() == 2 && qkv.stride(1) == 1 && qkv.size(1) == (nh + 2 * nkv) * hd, "rope_kv_append: qkv [T, (nh + 2 nkv) * hd]");
  TORCH_CHECK(pos.scalar_type() == at::kInt && pos.is_contiguous() && slot.scalar_type() == at::kLong && slot.is_contiguous());
  TORCH_CHECK(kc.is_contiguous() && vc.is_contiguous() && kc.dim() == 4 && kc.size(2) == nkv && kc.size(3) == hd);
  const c10::cuda::CUDAGuard guard(qkv.device());
  count(1);
  CHECK_RC(vb_rope_kv_append(qkv.data_ptr(), qkv.stride(0), pos.data_ptr<int>(), cos_t.data_ptr<float>(), sin_t.data_ptr<float>(),
                             reinterpret_cast<long long*>(slot.data_ptr()), kc.data_ptr(), vc.data_ptr(), (int)qkv.size(0), (int)nh,
                             (int)nkv, (int)hd, cur_stream()),
           "vb_rope_kv_append");
}

Tensor swiglu_fwd(const Tensor& gu) {
  CHECK_BF16(gu);
  TORCH_CHECK(gu.is_contiguous() && gu.dim() == 2);
  const c10::cuda::CUDAGuard guard(gu.device());
  const int64_t T = gu.size(0), I = gu.size(1) / 2;
  Tensor out = at::empty({T, I}, gu.options());
  count(1);
  CHECK_RC(vb_swiglu_fwd(gu.data_ptr(), out.data_ptr(), T, (int)I, cur_stream()), "vb_swiglu_fwd");
  return out;
}
Tensor swiglu_bwd(const Tensor& dout, const Tensor& gu) {
  CHECK_BF16(gu);
  CHECK_BF16(dout);
  TORCH_CHECK(gu.is_contiguous() && dout.is_contiguous());
  const c10::cuda::CUDAGuard guard(gu.device());
  Tensor dgu = at::empty_like(gu);
  count(1);
  CHECK_RC(vb_swiglu_bwd(dout.data_ptr(), gu.data_ptr(), dgu.data_ptr(), gu.size(0), (int)(gu.size(1) / 2), cur_stream()),
           "vb_swiglu_bwd");
  return dgu;
}

Tensor embedding_fwd(const Tensor& ids, const Tensor& w) {
  CHECK_BF16(w);
  TORCH_CHECK(ids.is_cuda() && ids.scalar_type() == at::kLong && ids.is_contiguous() && w.is_contiguous());
  const c10::cuda::CUDAGuard guard(w.device());
  Tensor out = at::empty({ids.numel(), w.size(1)}, w.options());
  count(1);
  CHECK_RC(vb_embedding_fwd(reinterpret_cast<long long*>(ids.data_ptr()), w.data_ptr(), out.data_ptr(), (int)ids.numel(), (int)w.size(1),
                            (int)w.size(0), cur_stream()),
           "vb_embedding_fwd");
  return out;
}
void embedding_bwd_(const Tensor& ids, const Tensor& dout, Tensor dw) {
  CHECK_BF16(dout);
  CHECK_F32(dw);
  TORCH_CHECK(dout.is_contiguous() && dw.is_contiguous());
  const c10::cuda::CUDAGuard guard(dw.device());
  count(1);
  CHECK_RC(vb_embedding_bwd(reinterpret_cast<long long*>(ids.data_ptr()), dout.data_ptr(), dw.data_ptr<float>(), (int)ids.numel(),
                            (int)dw.size(1), (int)dw.size(0), cur_stream()),
           "vb_embedding_bwd");
}

void sumsq_(const Tensor& g, Tensor ctrl) {
  CHECK_F32(g);
  CHECK_F32(ctrl);
  TORCH_CHECK(g.is_contiguous());
  const c10::cuda::CUDAGuard guard(g.device());
  count(1);
  CHECK_RC(vb_sumsq(g.data_ptr<float>(), g.numel(), ctrl.data_ptr<float>(), cur_stream()), "vb_sumsq");
}
void clip_coef_(Tensor ctrl, double max_norm) {
  const c10::cuda::CUDAGuard guard(ctrl.device());
  count(1);
  CHECK_RC(vb_clip_coef(ctrl.data_ptr<float>(), (float)max_norm, cur_stream()), "vb_clip_coef");
}
void adamw_(Tensor master, Tensor grad, Tensor m, Tensor v, const OptTensor& out_bf16, const OptTensor& ctrl, double lr,
            double beta1, double beta2, double eps, double wd, int64_t step, double grad_scale, bool zero_grad) {
  CHECK_F32(master);
  CHECK_F32(grad);
  CHECK_F32(m);
  CHECK_F32(v);
  TORCH_CHECK(master.is_contiguous() && grad.is_contiguous() && m.is_contiguous() && v.is_contiguous());
  const c10::cuda::CUDAGuard guard(master.device());
  void* ob = out_bf16.has_value() ? out_bf16->data_ptr() : nullptr;
  count(1);
  CHECK_RC(vb_adamw(master.data_ptr<float>(), grad.data_ptr<float>(), m.data_ptr<float>(), v.data_ptr<float>(), ob,
                    master.numel(), fptr(ctrl), (float)lr, (float)beta1, (float)beta2, (float)eps, (float)wd, (int)step,
                    (float)grad_scale, zero_grad, cur_stream()),
           "vb_adamw");
}
void cast_f32_bf16_(const Tensor& in, Tensor out, double scale) {
  CHECK_F32(in);
  CHECK_BF16(out);
  const c10::cuda::CUDAGuard guard(in.device());
  count(1);
  CHECK_RC(vb_cast_f32_bf16(in.data_ptr<float>(), out.data_ptr(), in.numel(), (float)scale, cur_stream()), "vb_cast");
}
void accum_bf16_f32_(const Tensor& in, Tensor out, double scale, bool accumulate) {
  CHECK_BF16(in);
  CHECK_F32(out);
  const c10::cuda::CUDAGuard guard(in.device());
  count(1);
  CHECK_RC(vb_accum_bf16_f32(in.data_ptr(), out.data_ptr<float>(), in.numel(), (float)scale, accumulate, cur_stream()),
           "vb_accum");
}

// k, v: [T, nkv, hd] views (row stride = stride(0)); slot: int64 [T]; caches: [num_slots, nkv, hd]
void kv_append_(const Tensor& k, const Tensor& v, const Tensor& slot, Tensor kc, Tensor vc) {
  CHECK_BF16(k);
  CHECK_BF16(v);
  TORCH_CHECK(k.dim() == 3 && k.stride(2) == 1 && k.stride(1) == k.size(2) && v.stride(1) == v.size(2));
  TORCH_CHECK(slot.scalar_type() == at::kLong && slot.is_contiguous() && kc.is_contiguous() && vc.is_contiguous());
  const c10::cuda::CUDAGuard guard(k.device());
  count(1);
  CHECK_RC(vb_kv_append(k.data_ptr(), v.data_ptr(), k.stride(0), v.stride(0), reinterpret_cast<long long*>(slot.data_ptr()), kc.data_ptr(),
                        vc.data_ptr(), (int)k.size(0), (int)k.size(1), (int)k.size(2), cur_stream()),
           "vb_kv_append");
}

// Decode attention with grouped shared prefixes (see vb_paged_decode_grouped). members int32 [NG, 8], grp_pages int32 [NG],
// skip int32 [B]; workspace: fp32 tensor of at least B * nh * (psplit + nsplit) * (hd + 2) elements (kept by the caller so that a
// captured decode step allocates nothing).
Tensor paged_decode_grouped(const Tensor& q, const Tensor& kc, const Tensor& vc, const Tensor& block_table, const Tensor& ctx_len,
                            const Tensor& members, const Tensor& grp_pages, const Tensor& skip, double scale, int64_t psplit,
                            int64_t nsplit, Tensor workspace) {
  CHECK_BF16(q);
  CHECK_BF16(kc);
  TORCH_CHECK(q.dim() == 3 && q.stride(2) == 1 && q.stride(1) == q.size(2) && kc.dim() == 4 && kc.size(1) == 64);
  for (const Tensor* t : {&block_table, &ctx_len, &members, &grp_pages, &skip})
    TORCH_CHECK(t->scalar_type() == at::kInt && t->is_contiguous() && t->is_cuda(), "paged_decode_grouped: int32 contiguous CUDA index tensors");
  TORCH_CHECK(members.dim() == 2 && members.size(1) == 8 && grp_pages.numel() == members.size(0) && skip.numel() == q.size(0));
  const c10::cuda::CUDAGuard guard(q.device());
  const int64_t B = q.size(0), nh = q.size(1), hd = q.size(2), nkv = kc.size(2), slots = psplit + nsplit;
  TORCH_CHECK(workspace.scalar_type() == at::kFloat && workspace.is_contiguous() && workspace.numel() >= B * nh * slots * (hd + 2),
              "paged_decode_grouped: workspace too small");
  Tensor out = at::empty({B, nh, hd}, q.options());
  float* po = workspace.data_ptr<float>();
  float* pml = po + B * nh * slots * hd;
  count(3);
  CHECK_RC(vb_paged_decode_grouped(q.data_ptr(), q.stride(0), kc.data_ptr(), vc.data_ptr(), kc.size(0) * 64, block_table.data_ptr<int>(),
                                   (int)block_table.size(1), ctx_len.data_ptr<int>(), members.data_ptr<int>(), grp_pages.data_ptr<int>(),
                                   skip.data_ptr<int>(), (int)members.size(0), out.data_ptr(), out.stride(0), (int)B, (int)nh, (int)nkv,
                                   (int)hd, 64, (float)scale, (int)psplit, (int)nsplit, po, pml, cur_stream()),
           "vb_paged_decode_grouped");
  return out;
}

// q: [B, nh, hd] view; caches [num_blocks, block_size, nkv, hd]; block_table int32 [B, max_blocks]; ctx_len int32 [B]
Tensor paged_decode(const Tensor& q, const Tensor& kc, const Tensor& vc, const Tensor& block_table,
                    const Tensor& ctx_len, double scale) {
  CHECK_BF16(q);
  CHECK_BF16(kc);
  TORCH_CHECK(q.dim() == 3 && q.stride(2) == 1 && q.stride(1) == q.size(2) && kc.dim() == 4);
  TORCH_CHECK(block_table.scalar_type() == at::kInt && ctx_len.scalar_type() == at::kInt);
  TORCH_CHECK(block_table.is_contiguous() && ctx_len.is_contiguous() && kc.is_contiguous() && vc.is_contiguous());
  const c10::cuda::CUDAGuard guard(q.device());
  const int64_t B = q.size(0), nh = q.size(1), hd = q.size(2);
  Tensor out = at::empty({B, nh, hd}, q.options());
  const int64_t nkv = kc.size(2), bs = kc.size(1);
  if (bs == 64 && (hd == 64 || hd == 128) && nh / nkv <= 16) {
    // TMA + tensor-core kernel; split the KV range when the grid would not fill the GPU
    int64_t nsplit = 1;
    const int64_t ctas = B * nkv;
    if (ctas < 296) nsplit = std::min<int64_t>(8, (296 + ctas - 1) / ctas);
    Tensor po, pml;
    if (nsplit > 1) {
      po = at::empty({B, nh, nsplit, hd}, q.options().dtype(at::kFloat));
      pml = at::empty({B, nh, nsplit, 2}, q.options().dtype(at::kFloat));
    }
    count(nsplit > 1 ? 2 : 1);
    const int rc = vb_paged_decode_v2(q.data_ptr(), q.stride(0), kc.data_ptr(), vc.data_ptr(), kc.size(0) * bs,
                                      block_table.data_ptr<int>(), (int)block_table.size(1), ctx_len.data_ptr<int>(),
                                      out.data_ptr(), out.stride(0), (int)B, (int)nh, (int)nkv, (int)hd, (int)bs,
                                      (float)scale, (int)nsplit, nsplit > 1 ? po.data_ptr<float>() : nullptr,
                                      nsplit > 1 ? pml.data_ptr<float>() : nullptr, cur_stream());
    CHECK_RC(rc, "vb_paged_decode_v2");
    return out;
  }
  count(1);
  CHECK_RC(vb_paged_decode(q.data_ptr(), q.stride(0), kc.data_ptr(), vc.data_ptr(), block_table.data_ptr<int>(),
                           (int)block_table.size(1), ctx_len.data_ptr<int>(), out.data_ptr(), out.stride(0), (int)B,
                           (int)nh, (int)kc.size(2), (int)hd, (int)kc.size(1), (float)scale, cur_stream()),
           "vb_paged_decode");
  return out;
}

// logits bf16 [B, V]; seeds int64 [B]. Returns (tokens int64 [B], logprobs fp32 [B]).
std::tuple<Tensor, Tensor> sample(const Tensor& logits, int64_t valid_vocab, double inv_temp, const Tensor& seeds,
                                  int64_t step) {
  CHECK_BF16(logits);
  TORCH_CHECK(logits.dim() == 2 && logits.stride(1) == 1 && seeds.scalar_type() == at::kLong);
  const c10::cuda::CUDAGuard guard(logits.device());
  const int64_t B = logits.size(0);
  Tensor tok = at::empty({B}, logits.options().dtype(at::kLong));
  Tensor lp = at::empty({B}, logits.options().dtype(at::kFloat));
  count(1);
  CHECK_RC(vb_sample(logits.data_ptr(), logits.stride(0), (int)B, (int)logits.size(1), (int)valid_vocab,
                     (float)inv_temp, reinterpret_cast<long long*>(seeds.data_ptr()), step, reinterpret_cast<long long*>(tok.data_ptr()), lp.data_ptr<float>(),
                     cur_stream()),
           "vb_sample");
  return {tok, lp};
}

// Same with top-k (<= 0: off) and top-p (>= 1: off) filtering done inside the kernel (histogram selection, no sort).
std::tuple<Tensor, Tensor> sample_topkp(const Tensor& logits, int64_t valid_vocab, double inv_temp, int64_t top_k, double top_p,
                                        const Tensor& seeds, int64_t step) {
  CHECK_BF16(logits);
  TORCH_CHECK(logits.dim() == 2 && logits.stride(1) == 1 && seeds.scalar_type() == at::kLong);
  TORCH_CHECK(inv_temp > 0.0 && top_p > 0.0, "sample_topkp: sampling only (greedy decoding uses sample)");
  const c10::cuda::CUDAGuard guard(logits.device());
  const int64_t B = logits.size(0);
  Tensor tok = at::empty({B}, logits.options().dtype(at::kLong));
  Tensor lp = at::empty({B}, logits.options().dtype(at::kFloat));
  count(1);
  CHECK_RC(vb_sample_topkp(logits.data_ptr(), logits.stride(0), (int)B, (int)logits.size(1), (int)valid_vocab, (float)inv_temp,
                           (int)top_k, (float)top_p, reinterpret_cast<long long*>(seeds.data_ptr()), step,
                           reinterpret_cast<long long*>(tok.data_ptr()), lp.data_ptr<float>(), cur_stream()),
           "vb_sample_topkp");
  return {tok, lp};
}

// rewards/mask fp32 [B, L]; group int32 [B] in [0, num_groups). Returns (advantages [B,L], scores [B]).
std::tuple<Tensor, Tensor> grpo_advantage(const Tensor& rewards, const Tensor& mask, const Tensor& group,
                                          int64_t num_groups, double eps, bool norm_by_std) {
  CHECK_F32(rewards);
  CHECK_F32(mask);
  TORCH_CHECK(group.scalar_type() == at::kInt && rewards.is_contiguous() && mask.is_contiguous());
  const c10::cuda::CUDAGuard guard(rewards.device());
  const int64_t B = rewards.size(0), L = rewards.size(1);
  Tensor adv = at::empty_like(rewards);
  Tensor scores = at::empty({B}, rewards.options());
  Tensor stats = at::empty({num_groups, 3}, rewards.options());
  count(2);
  CHECK_RC(vb_grpo_advantage(rewards.data_ptr<float>(), mask.data_ptr<float>(), group.data_ptr<int>(), (int)B, (int)L,
                             (int)num_groups, (float)eps, norm_by_std, scores.data_ptr<float>(),
                             stats.data_ptr<float>(), adv.data_ptr<float>(), cur_stream()),
           "vb_grpo_advantage");
  return {adv, scores};
}

std::tuple<Tensor, Tensor> gae(const Tensor& rewards, const Tensor& values, const Tensor& mask, double gamma,
                               double lam, bool whiten) {
  CHECK_F32(rewards);
  CHECK_F32(values);
  CHECK_F32(mask);
  TORCH_CHECK(rewards.is_contiguous() && values.is_contiguous() && mask.is_contiguous());
  const c10::cuda::CUDAGuard guard(rewards.device());
  Tensor adv = at::empty_like(rewards), ret = at::empty_like(rewards);
  Tensor acc = at::empty({4}, rewards.options());
  count(3);
  CHECK_RC(vb_gae(rewards.data_ptr<float>(), values.data_ptr<float>(), mask.data_ptr<float>(), (int)rewards.size(0),
                  (int)rewards.size(1), (float)gamma, (float)lam, whiten, adv.data_ptr<float>(), ret.data_ptr<float>(),
                  acc.data_ptr<float>(), cur_stream()),
           "vb_gae");
  return {adv, ret};
}

// ---- peer-memory collectives. `ptrs`: int64 CPU tensor of device addresses, one per rank (symmetric buffers).
inline const unsigned long long* uptr(const Tensor& t) {
  TORCH_CHECK(!t.is_cuda() && t.scalar_type() == at::kLong && t.is_contiguous(), "pointer table: int64 CPU tensor");
  return reinterpret_cast<const unsigned long long*>(t.data_ptr());
}

void peer_barrier(const Tensor& pad_ptrs, int64_t rank, int64_t epoch, double limit_s, const c10::optional<Tensor>& poison) {
  count(1);
  float* pz = nullptr;
  if (poison.has_value()) {
    TORCH_CHECK(poison->is_cuda() && poison->scalar_type() == at::kFloat && poison->numel() >= 1, "poison: fp32 CUDA tensor");
    pz = poison->data_ptr<float>();
  }
  CHECK_RC(vb_peer_barrier(uptr(pad_ptrs), (int)rank, (int)pad_ptrs.numel(), (unsigned int)epoch, limit_s, pz, cur_stream()),
           "vb_peer_barrier");
}

void rs_sumsq_(const Tensor& grad_ptrs, int64_t mc_ptr, Tensor out, int64_t lo, int64_t rank, double scale, Tensor ctrl) {
  CHECK_F32(out);
  CHECK_F32(ctrl);
  const c10::cuda::CUDAGuard guard(out.device());
  count(1);
  CHECK_RC(vb_rs_sumsq(uptr(grad_ptrs), (unsigned long long)mc_ptr, out.data_ptr<float>(), lo, out.numel(),
                       (int)grad_ptrs.numel(), (int)rank, (float)scale, ctrl.data_ptr<float>(), cur_stream()),
           "vb_rs_sumsq");
}

void adamw_allgather_(Tensor master, const Tensor& grad, Tensor m, Tensor v, const Tensor& param_ptrs, int64_t mc_ptr,
                      int64_t lo, int64_t rank, const Tensor& ctrl, double lr, double beta1, double beta2, double eps,
                      double wd, int64_t step) {
  CHECK_F32(master);
  CHECK_F32(grad);
  const c10::cuda::CUDAGuard guard(master.device());
  count(1);
  CHECK_RC(vb_adamw_allgather(master.data_ptr<float>(), grad.data_ptr<float>(), m.data_ptr<float>(), v.data_ptr<float>(),
                              uptr(param_ptrs), (unsigned long long)mc_ptr, lo, master.numel(), (int)param_ptrs.numel(),
                              (int)rank, ctrl.data_ptr<float>(), (float)lr, (float)beta1, (float)beta2, (float)eps, (float)wd,
                              (int)step, cur_stream()),
           "vb_adamw_allgather");
}

void allreduce_peer_(const Tensor& buf_ptrs, Tensor out, int64_t rank) {
  CHECK_BF16(out);
  const c10::cuda::CUDAGuard guard(out.device());
  count(1);
  CHECK_RC(vb_allreduce_peer(uptr(buf_ptrs), out.data_ptr(), out.numel(), (int)buf_ptrs.numel(), (int)rank, cur_stream()),
           "vb_allreduce_peer");
}

// Row-parallel linear + all-reduce in one kernel: out[M,N] = sum over ranks of a_r[M,K_r] @ b_r[N,K_r]^T (+bias).
// part_ptrs / flag_ptrs: CPU int64 tensors [world] with every rank's partial buffer and flag array addresses.
Tensor gemm_allreduce(const Tensor& a, const Tensor& b, const OptTensor& bias, const Tensor& part_ptrs, const Tensor& flag_ptrs,
                      Tensor epoch, int64_t buf_elems, int64_t rank, double limit_s, const OptTensor& out,
                      const OptTensor& splitk_ws, bool b_mn, int64_t rs_rows) {
  CHECK_BF16(a);
  CHECK_BF16(b);
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && a.stride(1) == 1 && b.stride(1) == 1 && a.size(1) == (b_mn ? b.size(0) : b.size(1)),
              "gemm_allreduce: 2-D operands with equal K (b stored [N, K], or [K, N] with b_mn)");
  TORCH_CHECK(epoch.scalar_type() == at::kInt && epoch.numel() >= 2 && epoch.is_cuda(), "gemm_allreduce: int32 cuda epoch[2]");
  const c10::cuda::CUDAGuard guard(a.device());
  const int64_t M = a.size(0), K = a.size(1), N = b_mn ? b.size(1) : b.size(0);
  // rs_rows > 0: reduce-scatter over rows; the result is this rank's [rs_rows, N] slice (zero where the slice runs past M)
  const int64_t out_rows = rs_rows > 0 ? rs_rows : M;
  Tensor d = out.has_value() ? *out : (rs_rows > 0 ? at::zeros({out_rows, N}, a.options()) : at::empty({M, N}, a.options()));
  TORCH_CHECK(d.scalar_type() == at::kBFloat16 && d.size(0) == out_rows && d.size(1) == N && d.stride(1) == 1, "gemm_allreduce: bad out");
  const void* bias_ptr = nullptr;
  if (bias.has_value()) {
    TORCH_CHECK(bias->scalar_type() == at::kBFloat16 && bias->numel() == N && bias->is_contiguous(), "gemm_allreduce: bad bias");
    bias_ptr = bias->data_ptr();
  }
  if (M == 0) return d;
  // decode-sized calls (few output tiles, deep K): K-split GEMM over all SMs + one fused reduce / all-reduce kernel
  int splits = (splitk_ws.has_value() && !b_mn && rs_rows <= 0) ? vb_gemm_suggest_splits((int)M, (int)N, (int)K) : 1;
  int skinny = 0;
  if (splitk_ws.has_value() && !b_mn && rs_rows <= 0 && skinny_enabled() && M <= 1024 && K % 8 == 0 && a.stride(0) % 8 == 0 &&
      b.stride(0) % 8 == 0 && reinterpret_cast<uintptr_t>(a.data_ptr()) % 16 == 0 && reinterpret_cast<uintptr_t>(b.data_ptr()) % 16 == 0) {
    const int s = vb_gemm_skinny_splits((int)M, (int)N, (int)K);
    if (s > 1) {
      splits = s;
      skinny = 1;
    }
  }
  if (splits > 1 && splitk_ws->numel() >= splits * M * N) {
    CHECK_F32((*splitk_ws));
    count(2);
    const int rc2 = vb_gemm_bf16_splitk_allreduce(a.data_ptr(), b.data_ptr(), d.data_ptr(), bias_ptr, (int)M, (int)N, (int)K, a.stride(0),
                                                  b.stride(0), d.stride(0), uptr(part_ptrs), uptr(flag_ptrs),
                                                  reinterpret_cast<unsigned int*>(epoch.data_ptr<int>()), buf_elems,
                                                  (int)part_ptrs.numel(), (int)rank, limit_s, splits, splitk_ws->data_ptr<float>(),
                                                  skinny, cur_stream());
    TORCH_CHECK(rc2 == 0, "vb_gemm_bf16_splitk_allreduce failed with code ", rc2, " (M=", M, " N=", N, " K=", K, ")");
    return d;
  }
  count(1);
  const int rc = vb_gemm_bf16_allreduce_ex(a.data_ptr(), b.data_ptr(), d.data_ptr(), bias_ptr, (int)M, (int)N, (int)K, a.stride(0),
                                           b.stride(0), d.stride(0), b_mn ? 1 : 0, (int)rs_rows, uptr(part_ptrs), uptr(flag_ptrs),
                                           reinterpret_cast<unsigned int*>(epoch.data_ptr<int>()), buf_elems, (int)part_ptrs.numel(),
                                           (int)rank, limit_s, cur_stream());
  TORCH_CHECK(rc == 0, "vb_gemm_bf16_allreduce failed with code ", rc, " (M=", M, " N=", N, " K=", K, ")");
  return d;
}

// GEMM (same operand conventions as `gemm`) that also runs a staged all-gather: chunks [chunk_begin, chunk_end) of 16 KB of a
// byte range kept in equal slices on the ranks of a group (src_ptrs: int64 CPU tensor, peer-mapped slice addresses) are copied
// into `dst` (a local uint8 / bf16 buffer) by an extra warp of every CTA. b_off_bytes >= 0: `b` is the view of `dst` at that byte
// offset and is gathered by this launch itself; tiles wait for their rows (`panels`: int32 scratch, one word per column tile).
Tensor gemm_fetch(const Tensor& a, const Tensor& b, const OptTensor& bias, const OptTensor& out, bool a_mn, bool b_mn, bool out_f32,
                  bool accumulate, const Tensor& src_ptrs, Tensor dst, int64_t total_bytes, int64_t slice_bytes, int64_t chunk_begin,
                  int64_t chunk_end, int64_t b_off_bytes, const OptTensor& panels, double limit_s) {
  CHECK_BF16(a);
  CHECK_BF16(b);
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && a.stride(1) == 1 && b.stride(1) == 1, "gemm_fetch: 2-D row-major operands");
  TORCH_CHECK(dst.is_cuda() && dst.is_contiguous() && (int64_t)dst.nbytes() >= total_bytes, "gemm_fetch: dst too small");
  const c10::cuda::CUDAGuard guard(a.device());
  const int64_t M = a_mn ? a.size(1) : a.size(0);
  const int64_t K = a_mn ? a.size(0) : a.size(1);
  const int64_t N = b_mn ? b.size(1) : b.size(0);
  TORCH_CHECK(K == (b_mn ? b.size(0) : b.size(1)), "gemm_fetch: contraction mismatch");
  Tensor d;
  if (out.has_value()) {
    d = *out;
    TORCH_CHECK(d.dim() == 2 && d.size(0) == M && d.size(1) == N && d.stride(1) == 1, "gemm_fetch: bad out shape");
    TORCH_CHECK(d.scalar_type() == (out_f32 ? at::kFloat : at::kBFloat16), "gemm_fetch: bad out dtype");
  } else {
    TORCH_CHECK(!accumulate, "gemm_fetch: accumulate needs out");
    d = at::empty({M, N}, a.options().dtype(out_f32 ? at::kFloat : at::kBFloat16));
  }
  const void* bias_ptr = nullptr;
  if (bias.has_value()) {
    TORCH_CHECK(bias->scalar_type() == at::kBFloat16 && bias->numel() == N && bias->is_contiguous(), "gemm_fetch: bad bias");
    bias_ptr = bias->data_ptr();
  }
  unsigned int* pc = nullptr;
  if (b_off_bytes >= 0) {
    TORCH_CHECK(panels.has_value() && panels->is_cuda() && panels->scalar_type() == at::kInt && panels->numel() >= (N + 127) / 128,
                "gemm_fetch: panels: int32 CUDA tensor with one word per 128 output columns");
    pc = reinterpret_cast<unsigned int*>(panels->data_ptr<int>());
  }
  if (M == 0 || N == 0) return d;
  count(1);
  const int rc = vb_gemm_bf16_fetch(a.data_ptr(), b.data_ptr(), d.data_ptr(), bias_ptr, (int)M, (int)N, (int)K, a.stride(0), b.stride(0),
                                    d.stride(0), a_mn, b_mn, out_f32, accumulate, uptr(src_ptrs), (int)src_ptrs.numel(),
                                    reinterpret_cast<unsigned long long>(dst.data_ptr()), total_bytes, slice_bytes, (int)chunk_begin,
                                    (int)chunk_end, b_off_bytes, pc, limit_s, cur_stream());
  TORCH_CHECK(rc == 0, "vb_gemm_bf16_fetch failed with code ", rc, " (M=", M, " N=", N, " K=", K, ")");
  return d;
}

// jobs: int64 CUDA tensor [njobs, 6] = (dst address, src address, rows, row bytes, dst row stride, src row stride), all in bytes;
// block_start: int32 CUDA tensor [njobs + 1] (16 KB blocks per job, prefix sums). Destinations may be peer-mapped memory.
void scatter_copy_(const Tensor& jobs, const Tensor& block_start, int64_t total_blocks) {
  TORCH_CHECK(jobs.is_cuda() && jobs.scalar_type() == at::kLong && jobs.dim() == 2 && jobs.size(1) == 6 && jobs.is_contiguous());
  TORCH_CHECK(block_start.is_cuda() && block_start.scalar_type() == at::kInt && block_start.numel() == jobs.size(0) + 1);
  const c10::cuda::CUDAGuard guard(jobs.device());
  count(1);
  CHECK_RC(vb_scatter_copy(jobs.data_ptr(), block_start.data_ptr<int>(), (int)jobs.size(0), (int)total_blocks, cur_stream()), "vb_scatter_copy");
}

// Graph-safe all-gather of a few words per rank over peer memory: out[r, :n] = rank r's src. buf_ptrs / flag_ptrs: CPU int64 [world].
void peer_share_(const Tensor& buf_ptrs, const Tensor& flag_ptrs, Tensor epoch, const Tensor& src, Tensor out, int64_t cap, int64_t rank,
                 double limit_s) {
  TORCH_CHECK(src.is_cuda() && out.is_cuda() && src.scalar_type() == at::kInt && out.scalar_type() == at::kInt && src.is_contiguous() &&
              out.is_contiguous() && out.numel() == src.numel() * buf_ptrs.numel(), "peer_share_: int32 src [n], out [world, n]");
  TORCH_CHECK(epoch.is_cuda() && epoch.scalar_type() == at::kInt && epoch.numel() >= 1, "peer_share_: int32 cuda epoch");
  const c10::cuda::CUDAGuard guard(src.device());
  count(1);
  CHECK_RC(vb_peer_share(uptr(buf_ptrs), uptr(flag_ptrs), reinterpret_cast<unsigned int*>(epoch.data_ptr<int>()), src.data_ptr(), out.data_ptr(),
                         (int)src.numel(), (int)cap, (int)rank, (int)buf_ptrs.numel(), limit_s, cur_stream()), "vb_peer_share");
}

int64_t comm_status() { return vb_comm_status(); }

// ---- fp8 (e4m3) with 1x128 block scales
// x [R, C] bf16 -> (q [R, C] uint8 holding e4m3, scales [C/128, R] fp32)
// NVFP4 fake quantisation (e2m1 values, 1x16 blocks, e4m3 block scales in units of global_scale); out may be x itself.
void nvfp4_fake_quant_(const Tensor& x, Tensor out, double global_scale) {
  CHECK_BF16(x);
  CHECK_BF16(out);
  TORCH_CHECK(x.dim() == 2 && out.dim() == 2 && x.stride(1) == 1 && out.stride(1) == 1 && x.sizes() == out.sizes() &&
              x.size(1) % 16 == 0, "nvfp4_fake_quant_: [R, C] with C % 16 == 0");
  const c10::cuda::CUDAGuard guard(x.device());
  count(1);
  CHECK_RC(vb_nvfp4_fake_quant(x.data_ptr(), x.stride(0), out.data_ptr(), out.stride(0), x.size(0), (int)x.size(1),
                               (float)global_scale, cur_stream()), "vb_nvfp4_fake_quant");
}

std::tuple<Tensor, Tensor> fp8_quant_1x128(const Tensor& x) {
  CHECK_BF16(x);
  TORCH_CHECK(x.dim() == 2 && x.stride(1) == 1 && x.size(1) % 128 == 0, "fp8_quant_1x128: [R, C] with C % 128 == 0");
  const c10::cuda::CUDAGuard guard(x.device());
  const int64_t R = x.size(0), C = x.size(1);
  Tensor q = at::empty({R, C}, x.options().dtype(at::kByte));
  Tensor sc = at::empty({C / 128, R}, x.options().dtype(at::kFloat));
  count(1);
  CHECK_RC(vb_fp8_quant_1x128(x.data_ptr(), x.stride(0), q.data_ptr(), q.stride(0), sc.data_ptr<float>(), (int)R, (int)C, cur_stream()),
           "vb_fp8_quant_1x128");
  return {q, sc};
}

// out[M, N] bf16 = dequant(aq, sa) @ dequant(bq, sb)^T (+bias)
Tensor gemm_fp8_blockscale(const Tensor& aq, const Tensor& sa, const Tensor& bq, const Tensor& sb, const OptTensor& bias) {
  TORCH_CHECK(aq.scalar_type() == at::kByte && bq.scalar_type() == at::kByte && aq.is_cuda() && bq.is_cuda());
  TORCH_CHECK(aq.dim() == 2 && bq.dim() == 2 && aq.stride(1) == 1 && bq.stride(1) == 1 && aq.size(1) == bq.size(1));
  CHECK_F32(sa);
  CHECK_F32(sb);
  const int64_t M = aq.size(0), K = aq.size(1), N = bq.size(0);
  TORCH_CHECK(sa.is_contiguous() && sb.is_contiguous() && sa.size(0) == K / 128 && sa.size(1) == M && sb.size(0) == K / 128 && sb.size(1) == N,
              "gemm_fp8_blockscale: scales must be [K/128, M] and [K/128, N]");
  const c10::cuda::CUDAGuard guard(aq.device());
  Tensor d = at::empty({M, N}, aq.options().dtype(at::kBFloat16));
  const void* bias_ptr = nullptr;
  if (bias.has_value()) {
    TORCH_CHECK(bias->scalar_type() == at::kBFloat16 && bias->numel() == N && bias->is_contiguous());
    bias_ptr = bias->data_ptr();
  }
  if (M == 0) return d;
  count(1);
  CHECK_RC(vb_gemm_fp8_blockscale(aq.data_ptr(), sa.data_ptr<float>(), bq.data_ptr(), sb.data_ptr<float>(), d.data_ptr(), bias_ptr, (int)M,
                                  (int)N, (int)K, aq.stride(0), bq.stride(0), d.stride(0), cur_stream()), "vb_gemm_fp8_blockscale");
  return d;
}

// w [R, C] bf16 -> (q [R, C] uint8 holding e4m3, scale_inv [ceil(R/128), ceil(C/128)] fp32): 128 x 128 weight blocks
std::tuple<Tensor, Tensor> fp8_quant_128x128(const Tensor& w) {
  CHECK_BF16(w);
  TORCH_CHECK(w.dim() == 2 && w.stride(1) == 1 && w.size(1) % 4 == 0, "fp8_quant_128x128: [R, C] with C % 4 == 0");
  const c10::cuda::CUDAGuard guard(w.device());
  const int64_t R = w.size(0), C = w.size(1);
  Tensor q = at::empty({R, C}, w.options().dtype(at::kByte));
  Tensor sc = at::empty({(R + 127) / 128, (C + 127) / 128}, w.options().dtype(at::kFloat));
  count(1);
  CHECK_RC(vb_fp8_quant_128x128(w.data_ptr(), w.stride(0), q.data_ptr(), q.stride(0), sc.data_ptr<float>(), (int)R, (int)C, cur_stream()),
           "vb_fp8_quant_128x128");
  return {q, sc};
}

// Grouped block-scaled fp8 GEMM of a mixture-of-experts layer: aq [rows_cap, K] (rows grouped by expert, 128-row aligned),
// bq [E * N, K]; scales [K/128, rows_cap] and [K/128, E * N]. Rows of tiles beyond num_mtiles are left as allocated (zeroed).
Tensor gemm_fp8_blockscale_grouped(const Tensor& aq, const Tensor& sa, const Tensor& bq, const Tensor& sb, int64_t N,
                                   const Tensor& tile_expert, const Tensor& num_mtiles) {
  TORCH_CHECK(aq.scalar_type() == at::kByte && bq.scalar_type() == at::kByte && aq.is_cuda() && bq.is_cuda());
  TORCH_CHECK(aq.dim() == 2 && bq.dim() == 2 && aq.stride(1) == 1 && bq.stride(1) == 1 && aq.size(1) == bq.size(1));
  CHECK_F32(sa);
  CHECK_F32(sb);
  const int64_t rows = aq.size(0), K = aq.size(1), EN = bq.size(0);
  TORCH_CHECK(N > 0 && EN % N == 0 && rows % 128 == 0, "gemm_fp8_blockscale_grouped: bq must hold E stacked [N, K] matrices");
  TORCH_CHECK(sa.is_contiguous() && sb.is_contiguous() && sa.size(0) == K / 128 && sa.size(1) == rows && sb.size(0) == K / 128 &&
              sb.size(1) == EN, "gemm_fp8_blockscale_grouped: scales must be [K/128, rows] and [K/128, E*N]");
  TORCH_CHECK(tile_expert.scalar_type() == at::kInt && tile_expert.is_cuda() && tile_expert.numel() >= rows / 128 &&
              num_mtiles.scalar_type() == at::kInt && num_mtiles.is_cuda());
  const c10::cuda::CUDAGuard guard(aq.device());
  Tensor d = at::zeros({rows, N}, aq.options().dtype(at::kBFloat16));
  count(1);
  CHECK_RC(vb_gemm_fp8_blockscale_grouped(aq.data_ptr(), sa.data_ptr<float>(), bq.data_ptr(), sb.data_ptr<float>(), d.data_ptr(), (int)rows,
                                          (int)N, (int)K, (int)(EN / N), aq.stride(0), bq.stride(0), d.stride(0),
                                          tile_expert.data_ptr<int>(), num_mtiles.data_ptr<int>(), cur_stream()),
           "vb_gemm_fp8_blockscale_grouped");
  return d;
}

// ---- mixture of experts
// (weights [T,k] fp32, experts [T,k] int32, counts [E] int32) from router logits [T, E]
std::tuple<Tensor, Tensor, Tensor> moe_route_topk(const Tensor& logits, int64_t k, bool renorm) {
  CHECK_BF16(logits);
  TORCH_CHECK(logits.dim() == 2 && logits.stride(1) == 1);
  const c10::cuda::CUDAGuard guard(logits.device());
  const int64_t T = logits.size(0), E = logits.size(1);
  Tensor w = at::empty({T, k}, logits.options().dtype(at::kFloat));
  Tensor idx = at::empty({T, k}, logits.options().dtype(at::kInt));
  Tensor counts = at::zeros({E}, logits.options().dtype(at::kInt));
  count(1);
  CHECK_RC(vb_moe_route_topk(logits.data_ptr(), logits.stride(0), (int)T, (int)E, (int)k, renorm, w.data_ptr<float>(),
                             idx.data_ptr<int>(), counts.data_ptr<int>(), cur_stream()), "vb_moe_route_topk");
  return {w, idx, counts};
}

// dst[r] = src[map[r]] (* scale[r]) or zeros where map[r] < 0
Tensor moe_gather_rows(const Tensor& src, const Tensor& map, const OptTensor& scale) {
  CHECK_BF16(src);
  TORCH_CHECK(src.dim() == 2 && src.stride(1) == 1 && map.scalar_type() == at::kInt && map.is_contiguous() && map.is_cuda());
  const c10::cuda::CUDAGuard guard(src.device());
  const int64_t rows = map.numel(), H = src.size(1);
  Tensor dst = at::empty({rows, H}, src.options());
  const float* sc = nullptr;
  if (scale.has_value()) {
    TORCH_CHECK(scale->scalar_type() == at::kFloat && scale->numel() == rows && scale->is_contiguous());
    sc = scale->data_ptr<float>();
  }
  count(1);
  CHECK_RC(vb_moe_gather_rows(src.data_ptr(), src.stride(0), map.data_ptr<int>(), sc, dst.data_ptr(), dst.stride(0), (int)rows,
                              (int)H, cur_stream()), "vb_moe_gather_rows");
  return dst;
}

// out[t] = sum_j w[t,j] * y[slot[t,j]]   (w optional: plain sum)
Tensor moe_combine(const Tensor& y, const Tensor& slot, const OptTensor& w) {
  CHECK_BF16(y);
  TORCH_CHECK(y.dim() == 2 && y.stride(1) == 1 && slot.dim() == 2 && slot.scalar_type() == at::kInt && slot.is_contiguous());
  const c10::cuda::CUDAGuard guard(y.device());
  const int64_t T = slot.size(0), k = slot.size(1), H = y.size(1);
  Tensor out = at::empty({T, H}, y.options());
  const float* wp = nullptr;
  if (w.has_value()) {
    TORCH_CHECK(w->scalar_type() == at::kFloat && w->numel() == T * k && w->is_contiguous());
    wp = w->data_ptr<float>();
  }
  count(1);
  CHECK_RC(vb_moe_combine(y.data_ptr(), y.stride(0), slot.data_ptr<int>(), wp, out.data_ptr(), out.stride(0), (int)T, (int)H, (int)k,
                          cur_stream()), "vb_moe_combine");
  return out;
}

Tensor moe_combine_bwd_w(const Tensor& g, const Tensor& y, const Tensor& slot) {
  CHECK_BF16(g);
  CHECK_BF16(y);
  TORCH_CHECK(g.stride(1) == 1 && y.stride(1) == 1 && slot.scalar_type() == at::kInt && slot.is_contiguous());
  const c10::cuda::CUDAGuard guard(y.device());
  const int64_t T = slot.size(0), k = slot.size(1), H = y.size(1);
  Tensor gw = at::empty({T, k}, y.options().dtype(at::kFloat));
  count(1);
  CHECK_RC(vb_moe_combine_bwd_w(g.data_ptr(), g.stride(0), y.data_ptr(), y.stride(0), slot.data_ptr<int>(), gw.data_ptr<float>(),
                                (int)T, (int)H, (int)k, cur_stream()), "vb_moe_combine_bwd_w");
  return gw;
}

// pointer tables for the peer kernels live on the device: int64 CUDA tensors
inline const unsigned long long* dptr(const Tensor& t) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kLong && t.is_contiguous(), "pointer table: int64 CUDA tensor");
  return reinterpret_cast<const unsigned long long*>(t.data_ptr());
}

void moe_dispatch_peer_(const Tensor& src, const Tensor& dst_ptrs, const Tensor& dest_rank, const Tensor& dest_row, int64_t k) {
  CHECK_BF16(src);
  TORCH_CHECK(src.dim() == 2 && src.stride(1) == 1 && dest_rank.scalar_type() == at::kInt && dest_row.scalar_type() == at::kInt);
  const c10::cuda::CUDAGuard guard(src.device());
  count(1);
  CHECK_RC(vb_moe_dispatch_peer(src.data_ptr(), src.stride(0), dptr(dst_ptrs), dest_rank.data_ptr<int>(), dest_row.data_ptr<int>(),
                                (int)dest_row.numel(), (int)k, (int)src.size(1), cur_stream()), "vb_moe_dispatch_peer");
}

Tensor moe_combine_peer(const Tensor& y_ptrs, const Tensor& src_rank, const Tensor& src_row, const OptTensor& w, int64_t H,
                        const Tensor& like) {
  TORCH_CHECK(src_rank.scalar_type() == at::kInt && src_row.scalar_type() == at::kInt && src_row.dim() == 2);
  const c10::cuda::CUDAGuard guard(like.device());
  const int64_t T = src_row.size(0), k = src_row.size(1);
  Tensor out = at::empty({T, H}, like.options().dtype(at::kBFloat16));
  const float* wp = nullptr;
  if (w.has_value()) {
    TORCH_CHECK(w->scalar_type() == at::kFloat && w->numel() == T * k && w->is_contiguous());
    wp = w->data_ptr<float>();
  }
  count(1);
  CHECK_RC(vb_moe_combine_peer(dptr(y_ptrs), src_rank.data_ptr<int>(), src_row.data_ptr<int>(), wp, out.data_ptr(), out.stride(0), (int)T,
                               (int)H, (int)k, cur_stream()), "vb_moe_combine_peer");
  return out;
}

void moe_publish_counts_(const Tensor& counts, const Tensor& table_ptrs, int64_t rank) {
  TORCH_CHECK(counts.scalar_type() == at::kInt && counts.is_cuda() && counts.is_contiguous());
  const c10::cuda::CUDAGuard guard(counts.device());
  count(1);
  CHECK_RC(vb_moe_publish_counts(counts.data_ptr<int>(), dptr(table_ptrs), (int)table_ptrs.numel(), (int)rank, (int)counts.numel(),
                                 cur_stream()), "vb_moe_publish_counts");
}

// mode 1: out[rows, N] = a[rows, K] @ W_e^T per 128-row tile (w: [E, N, K], or [E, K, N] when b_mn)
Tensor gemm_grouped_rows(const Tensor& a, const Tensor& w, bool b_mn, const Tensor& tile_expert, const Tensor& num_mtiles) {
  CHECK_BF16(a);
  CHECK_BF16(w);
  TORCH_CHECK(a.dim() == 2 && a.stride(1) == 1 && w.dim() == 3 && w.is_contiguous() && a.size(0) % 128 == 0);
  TORCH_CHECK(tile_expert.scalar_type() == at::kInt && tile_expert.is_cuda() && num_mtiles.scalar_type() == at::kInt && num_mtiles.is_cuda());
  const c10::cuda::CUDAGuard guard(a.device());
  const int64_t rows = a.size(0), K = a.size(1), E = w.size(0);
  const int64_t N = b_mn ? w.size(2) : w.size(1);
  TORCH_CHECK((b_mn ? w.size(1) : w.size(2)) == K, "gemm_grouped_rows: contraction mismatch");
  Tensor d = at::empty({rows, N}, a.options());
  if (rows == 0) return d;
  count(1);
  CHECK_RC(vb_gemm_grouped(1, a.data_ptr(), w.data_ptr(), d.data_ptr(), (int)rows, (int)rows, (int)N, (int)K, a.stride(0), w.stride(1),
                           d.stride(0), b_mn, 0, (int)E, tile_expert.data_ptr<int>(), num_mtiles.data_ptr<int>(), nullptr, cur_stream()),
           "vb_gemm_grouped(rows)");
  return d;
}

// mode 2: out[e] (+)= dy[seg_e]^T @ x[seg_e]   (out: fp32 [E, M, N])
void gemm_grouped_wgrad_(const Tensor& dy, const Tensor& x, Tensor out, const Tensor& seg_start, bool accumulate) {
  CHECK_BF16(dy);
  CHECK_BF16(x);
  CHECK_F32(out);
  TORCH_CHECK(dy.stride(1) == 1 && x.stride(1) == 1 && out.dim() == 3 && out.is_contiguous() && dy.size(0) == x.size(0) && dy.size(0) % 128 == 0);
  TORCH_CHECK(seg_start.scalar_type() == at::kInt && seg_start.is_cuda() && seg_start.numel() == out.size(0) + 1);
  const c10::cuda::CUDAGuard guard(dy.device());
  if (dy.size(0) == 0) return;
  if (!accumulate) out.zero_();
  count(1);
  CHECK_RC(vb_gemm_grouped(2, dy.data_ptr(), x.data_ptr(), out.data_ptr(), (int)dy.size(0), (int)out.size(1), (int)out.size(2), 0,
                           dy.stride(0), x.stride(0), out.stride(1), 1, 1, (int)out.size(0), nullptr, nullptr, seg_start.data_ptr<int>(),
                           cur_stream()), "vb_gemm_grouped(wgrad)");
}

}  // namespace

TORCH_LIBRARY(verl_b200, m) {
  m.def("peer_barrier", &peer_barrier);
  m.def("rs_sumsq_", &rs_sumsq_);
  m.def("adamw_allgather_", &adamw_allgather_);
  m.def("allreduce_peer_", &allreduce_peer_);
  m.def("gemm_allreduce", &gemm_allreduce);
  m.def("gemm_fetch", &gemm_fetch);
  m.def("gemm_skinny_splits", [](int64_t M, int64_t N, int64_t K) {
    return (int64_t)((skinny_enabled() && M <= 1024) ? vb_gemm_skinny_splits((int)M, (int)N, (int)K) : 0);
  });
  m.def("gemm_fold_in_kernel", []() { return (int64_t)vb_gemm_fold_in_kernel(); });
  m.def("gemm_suggest_splits", [](int64_t M, int64_t N, int64_t K) { return (int64_t)vb_gemm_suggest_splits((int)M, (int)N, (int)K); });
  m.def("scatter_copy_", &scatter_copy_);
  m.def("peer_share_", &peer_share_);
  m.def("comm_status", &comm_status);
  m.def("fp8_quant_1x128", &fp8_quant_1x128);
  m.def("fp8_quant_128x128", &fp8_quant_128x128);
  m.def("gemm_fp8_blockscale_grouped", &gemm_fp8_blockscale_grouped);
  m.def("nvfp4_fake_quant_", &nvfp4_fake_quant_);
  m.def("gemm_fp8_blockscale", &gemm_fp8_blockscale);
  m.def("moe_route_topk", &moe_route_topk);
  m.def("moe_gather_rows", &moe_gather_rows);
  m.def("moe_combine", &moe_combine);
  m.def("moe_combine_bwd_w", &moe_combine_bwd_w);
  m.def("moe_dispatch_peer_", &moe_dispatch_peer_);
  m.def("moe_combine_peer", &moe_combine_peer);
  m.def("moe_publish_counts_", &moe_publish_counts_);
  m.def("gemm_grouped_rows", &gemm_grouped_rows);
  m.def("gemm_grouped_wgrad_", &gemm_grouped_wgrad_);
  m.def("gemm", &gemm);
  m.def("gemm_status", &gemm_status);
  m.def("gemm_swiglu", &gemm_swiglu);
  m.def("gemm_row_ranges_", &gemm_row_ranges_);
  m.def("launch_count", &launch_count);
  m.def("add_launches", &add_launches);
  m.def("attn_fwd", &attn_fwd);
  m.def("attn_bwd", &attn_bwd);
  m.def("lmhead_fwd", &lmhead_fwd);
  m.def("lmhead_dlogits", &lmhead_dlogits);
  m.def("rmsnorm_fwd", &rmsnorm_fwd);
  m.def("rmsnorm_bwd", &rmsnorm_bwd);
  m.def("rope_", &rope_);
  m.def("swiglu_fwd", &swiglu_fwd);
  m.def("swiglu_bwd", &swiglu_bwd);
  m.def("embedding_fwd", &embedding_fwd);
  m.def("embedding_bwd_", &embedding_bwd_);
  m.def("sumsq_", &sumsq_);
  m.def("clip_coef_", &clip_coef_);
  m.def("adamw_", &adamw_);
  m.def("cast_f32_bf16_", &cast_f32_bf16_);
  m.def("accum_bf16_f32_", &accum_bf16_f32_);
  m.def("kv_append_", &kv_append_);
  m.def("paged_decode", &paged_decode);
  m.def("paged_decode_grouped", &paged_decode_grouped);
  m.def("rope_kv_append_", &rope_kv_append_);
  m.def("sample", &sample);
  m.def("sample_topkp", &sample_topkp);
  m.def("grpo_advantage", &grpo_advantage);
  m.def("gae", &gae);
}
