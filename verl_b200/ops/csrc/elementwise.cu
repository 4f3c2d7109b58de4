// Memory-bound fused kernels (bf16 activations, fp32 statistics): RMSNorm (+residual) fwd/bwd, RoPE,
// SwiGLU fwd/bwd, embedding fwd/bwd, fused AdamW (fp32 master -> bf16 working copy), gradient norm /
// clip coefficient, casts.  All use 16-byte vector accesses; every row length must be a multiple of 8.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

namespace vb {

struct alignas(16) bf16x8 {
  __nv_bfloat162 v[4];
};

__device__ __forceinline__ void unpack8(const bf16x8& p, float (&f)[8]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(p.v[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ bf16x8 pack8(const float (&f)[8]) {
  bf16x8 p;
#pragma unroll
  for (int i = 0; i < 4; ++i) p.v[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return p;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum; every thread receives the result. `red` must hold >= 32 floats.
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  const int nw = (blockDim.x + 31) >> 5;
  float t = (lane < nw) ? red[lane] : 0.f;
  t = warp_sum(t);
  return t;
}

// ------------------------------------------------------------------------------------------ RMSNorm
// y = x_eff * rstd * w, x_eff = x (+ residual); when residual != null, x_eff is written to res_out.
__global__ void rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ residual,
                                   const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                                   __nv_bfloat16* __restrict__ res_out, float* __restrict__ rstd_out, int H,
                                   float eps) {
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const bf16x8* xr = reinterpret_cast<const bf16x8*>(x + row * H);
  const bf16x8* rr = residual ? reinterpret_cast<const bf16x8*>(residual + row * H) : nullptr;
  bf16x8* ro = res_out ? reinterpret_cast<bf16x8*>(res_out + row * H) : nullptr;
  const int nv = H >> 3;
  float ss = 0.f;
  for (int i = threadIdx.x; i < nv; i += blockDim.x) {
    float f[8];
    unpack8(xr[i], f);
    if (rr) {
      float g[8];
      unpack8(rr[i], g);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] += g[j];
      bf16x8 h = pack8(f);
      ro[i] = h;
      unpack8(h, f);  // statistics on the rounded residual stream, as the next reader sees it
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) ss += f[j] * f[j];
  }
  ss = block_sum(ss, red);
  const float rstd = rsqrtf(ss / H + eps);
  if (threadIdx.x == 0 && rstd_out) rstd_out[row] = rstd;
  const bf16x8* src = rr ? reinterpret_cast<const bf16x8*>(res_out + row * H) : xr;
  const bf16x8* wv = reinterpret_cast<const bf16x8*>(w);
  bf16x8* yr = reinterpret_cast<bf16x8*>(y + row * H);
  for (int i = threadIdx.x; i < nv; i += blockDim.x) {
    float f[8], g[8];
    unpack8(src[i], f);
    unpack8(wv[i], g);
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = f[j] * rstd * g[j];
    yr[i] = pack8(f);
  }
}

// dx = rstd * (dy*w) - x * rstd^3 * mean(dy*w*x) (+ dres_in);  dw partial per block -> scratch[grid, H].
// Each block walks rows blockIdx.x, +gridDim.x, ...; each thread owns fixed column vectors so the dw
// partial stays in registers (H <= 8 * VEC_PER_THREAD * blockDim.x).
template <int VPT>
__global__ void rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                                   const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd,
                                   const __nv_bfloat16* __restrict__ dres_in, __nv_bfloat16* __restrict__ dx,
                                   float* __restrict__ dw_partial, int T, int H) {
  __shared__ float red[32];
  const int nv = H >> 3;
  float dwacc[VPT][8];
  float wreg[VPT][8];
#pragma unroll
  for (int v = 0; v < VPT; ++v) {
    const int i = threadIdx.x + v * blockDim.x;
#pragma unroll
    for (int j = 0; j < 8; ++j) dwacc[v][j] = 0.f;
    if (i < nv) unpack8(reinterpret_cast<const bf16x8*>(w)[i], wreg[v]);
  }
  for (long long row = blockIdx.x; row < T; row += gridDim.x) {
    const bf16x8* dyr = reinterpret_cast<const bf16x8*>(dy + row * H);
    const bf16x8* xr = reinterpret_cast<const bf16x8*>(x + row * H);
    const float rs = rstd[row];
    float dyv[VPT][8], xv[VPT][8];
    float dot = 0.f;
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      const int i = threadIdx.x + v * blockDim.x;
      if (i < nv) {
        unpack8(dyr[i], dyv[v]);
        unpack8(xr[i], xv[v]);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          dot += dyv[v][j] * wreg[v][j] * xv[v][j];
          dwacc[v][j] += dyv[v][j] * xv[v][j] * rs;
        }
      }
    }
    dot = block_sum(dot, red);
    const float c = dot * rs * rs * rs / H;
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      const int i = threadIdx.x + v * blockDim.x;
      if (i < nv) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = rs * dyv[v][j] * wreg[v][j] - xv[v][j] * c;
        if (dres_in) {
          float d[8];
          unpack8(reinterpret_cast<const bf16x8*>(dres_in + row * H)[i], d);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += d[j];
        }
        reinterpret_cast<bf16x8*>(dx + row * H)[i] = pack8(o);
      }
    }
  }
#pragma unroll
  for (int v = 0; v < VPT; ++v) {
    const int i = threadIdx.x + v * blockDim.x;
    if (i < nv) {
      float* dst = dw_partial + static_cast<long long>(blockIdx.x) * H + i * 8;
      *reinterpret_cast<float4*>(dst) = make_float4(dwacc[v][0], dwacc[v][1], dwacc[v][2], dwacc[v][3]);
      *reinterpret_cast<float4*>(dst + 4) = make_float4(dwacc[v][4], dwacc[v][5], dwacc[v][6], dwacc[v][7]);
    }
  }
}

// dw[h] (+)= sum_b partial[b, h]
__global__ void colsum_kernel(const float* __restrict__ partial, float* __restrict__ out, int B, int H,
                              int accumulate) {
  const int h = blockIdx.x * blockDim.x + threadIdx.x;
  if (h >= H) return;
  float s = 0.f;
  for (int b = 0; b < B; ++b) s += partial[static_cast<long long>(b) * H + h];
  out[h] = accumulate ? out[h] + s : s;
}

// ------------------------------------------------------------------------------------------ RoPE
// In place on x [T, nheads, hd] (row stride `ld` elements): HF rotate-half convention with a
// cos/sin table [max_pos, hd/2] (fp32).  sign = +1 forward, -1 backward (transpose of the rotation).
__global__ void rope_kernel(__nv_bfloat16* __restrict__ x, const int* __restrict__ pos,
                            const float* __restrict__ cos_t, const float* __restrict__ sin_t, int T, int nheads,
                            int hd, long long ld, float sign) {
  const int half = hd >> 1;
  const long long total = static_cast<long long>(T) * nheads * (half >> 1);  // two pairs per thread
  const long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (idx >= total) return;
  const int pairs = half >> 1;
  const int i2 = static_cast<int>(idx % pairs);
  const int h = static_cast<int>((idx / pairs) % nheads);
  const long long t = idx / (static_cast<long long>(pairs) * nheads);
  const int p = pos[t];
  const int i = i2 * 2;
  __nv_bfloat16* base = x + t * ld + static_cast<long long>(h) * hd;
  const float2 c = *reinterpret_cast<const float2*>(cos_t + static_cast<long long>(p) * half + i);
  float2 s = *reinterpret_cast<const float2*>(sin_t + static_cast<long long>(p) * half + i);
  s.x *= sign;
  s.y *= sign;
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(base + i));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(base + half + i));
  *reinterpret_cast<__nv_bfloat162*>(base + i) = __floats2bfloat162_rn(a.x * c.x - b.x * s.x, a.y * c.y - b.y * s.y);
  *reinterpret_cast<__nv_bfloat162*>(base + half + i) =
      __floats2bfloat162_rn(b.x * c.x + a.x * s.x, b.y * c.y + a.y * s.y);
}

// ------------------------------------------------------------------------------------------ SwiGLU
// gu [T, 2I]: gate = gu[:, :I], up = gu[:, I:].
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out,
                                  long long T, int I) {
  const int nv = I >> 3;
  const long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (idx >= T * nv) return;
  const long long t = idx / nv;
  const int i = static_cast<int>(idx % nv);
  float g[8], u[8];
  unpack8(reinterpret_cast<const bf16x8*>(gu + t * 2 * I)[i], g);
  unpack8(reinterpret_cast<const bf16x8*>(gu + t * 2 * I + I)[i], u);
#pragma unroll
  for (int j = 0; j < 8; ++j) g[j] = g[j] / (1.f + __expf(-g[j])) * u[j];
  reinterpret_cast<bf16x8*>(out + t * I)[i] = pack8(g);
}
__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ gu,
                                  __nv_bfloat16* __restrict__ dgu, long long T, int I) {
  const int nv = I >> 3;
  const long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (idx >= T * nv) return;
  const long long t = idx / nv;
  const int i = static_cast<int>(idx % nv);
  float g[8], u[8], d[8], dg[8], du[8];
  unpack8(reinterpret_cast<const bf16x8*>(gu + t * 2 * I)[i], g);
  unpack8(reinterpret_cast<const bf16x8*>(gu + t * 2 * I + I)[i], u);
  unpack8(reinterpret_cast<const bf16x8*>(dout + t * I)[i], d);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float sg = 1.f / (1.f + __expf(-g[j]));
    du[j] = d[j] * g[j] * sg;
    dg[j] = d[j] * u[j] * sg * (1.f + g[j] * (1.f - sg));
  }
  reinterpret_cast<bf16x8*>(dgu + t * 2 * I)[i] = pack8(dg);
  reinterpret_cast<bf16x8*>(dgu + t * 2 * I + I)[i] = pack8(du);
}

// ------------------------------------------------------------------------------------------ embedding
__global__ void embedding_fwd_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ w,
                                     __nv_bfloat16* __restrict__ out, int H, int V) {
  const long long t = blockIdx.x;
  long long id = ids[t];
  if (id < 0 || id >= V) id = 0;
  const bf16x8* src = reinterpret_cast<const bf16x8*>(w + id * H);
  bf16x8* dst = reinterpret_cast<bf16x8*>(out + t * H);
  for (int i = threadIdx.x; i < (H >> 3); i += blockDim.x) dst[i] = src[i];
}
__global__ void embedding_bwd_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ dout,
                                     float* __restrict__ dw, int H, int V) {
  const long long t = blockIdx.x;
  const long long id = ids[t];
  if (id < 0 || id >= V) return;
  for (int i = threadIdx.x; i < H; i += blockDim.x)
    atomicAdd(dw + id * H + i, __bfloat162float(dout[t * H + i]));
}

// ------------------------------------------------------------------------------------------ optimizer
// ctrl[0] = sum of squared gradients (accumulated by sumsq_kernel), ctrl[1] = clip coefficient,
// ctrl[2] = 1.0 when the step must be skipped (non-finite norm), ctrl[3] = grad norm.
constexpr int SUMSQ_MAX_BLOCKS = 148 * 8;
__device__ float g_sumsq_partial[SUMSQ_MAX_BLOCKS];  // scratch of the two-pass reduction (one call at a time per device)

__global__ void sumsq_kernel(const float* __restrict__ g, long long n, float* __restrict__ ctrl) {
  __shared__ float red[32];
  float s = 0.f;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long n4 = n >> 2;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n4; i += stride) {
    const float4 v = reinterpret_cast<const float4*>(g)[i];
    s += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  for (long long i = (n4 << 2) + blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n; i += stride)
    s += g[i] * g[i];
  s = block_sum(s, red);
  if (threadIdx.x == 0) g_sumsq_partial[blockIdx.x] = s;
}
// second pass: the block partials are folded in a fixed order (bitwise reproducible), then added to ctrl[0]
__global__ void sumsq_final_kernel(int blocks, float* __restrict__ ctrl) {
  __shared__ float red[32];
  float s = 0.f;
  for (int i = threadIdx.x; i < blocks; i += blockDim.x) s += g_sumsq_partial[i];
  s = block_sum(s, red);
  if (threadIdx.x == 0) ctrl[0] += s;
}
__global__ void clip_coef_kernel(float* __restrict__ ctrl, float max_norm) {
  const float norm = sqrtf(ctrl[0]);
  const bool finite = isfinite(norm);
  ctrl[3] = norm;
  ctrl[2] = finite ? 0.f : 1.f;
  ctrl[1] = (finite && max_norm > 0.f) ? fminf(1.f, max_norm / (norm + 1e-6f)) : 1.f;
}

// AdamW on a flat shard.  master (fp32) is updated in place; the bf16 working copy is refreshed in the
// same pass; the gradient is optionally zeroed for the next accumulation round.
__global__ void adamw_kernel(float* __restrict__ master, float* __restrict__ grad, float* __restrict__ m,
                             float* __restrict__ v, __nv_bfloat16* __restrict__ out_bf16, long long n,
                             const float* __restrict__ ctrl, float lr, float beta1, float beta2, float eps,
                             float wd, float bc1, float bc2_sqrt, float grad_scale, int zero_grad) {
  const long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (i >= n) return;
  const bool skip = ctrl && ctrl[2] != 0.f;
  const float coef = (ctrl ? ctrl[1] : 1.f) * grad_scale;
  if (!skip) {
    const float g = grad[i] * coef;
    float p = master[i];
    const float mi = beta1 * m[i] + (1.f - beta1) * g;
    const float vi = beta2 * v[i] + (1.f - beta2) * g * g;
    m[i] = mi;
    v[i] = vi;
    p *= (1.f - lr * wd);
    const float denom = sqrtf(vi) / bc2_sqrt + eps;
    p -= (lr / bc1) * (mi / denom);
    master[i] = p;
    if (out_bf16) out_bf16[i] = __float2bfloat16(p);
  }
  if (zero_grad) grad[i] = 0.f;
}

__global__ void cast_f32_bf16_kernel(const float* __restrict__ in, __nv_bfloat16* __restrict__ out, long long n,
                                     float scale) {
  const long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (i < n) out[i] = __float2bfloat16(in[i] * scale);
}

// out_f32[i] (+)= bf16 in[i] * scale
__global__ void accum_bf16_f32_kernel(const __nv_bfloat16* __restrict__ in, float* __restrict__ out, long long n,
                                      float scale, int accumulate) {
  const long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (i < n) {
    const float x = __bfloat162float(in[i]) * scale;
    out[i] = accumulate ? out[i] + x : x;
  }
}

}  // namespace vb

using namespace vb;

static inline int cdiv_ll(long long a, long long b) { return static_cast<int>((a + b - 1) / b); }

extern "C" {

int vb_rmsnorm_fwd(const void* x, const void* residual, const void* w, void* y, void* res_out, float* rstd, int T,
                   int H, float eps, cudaStream_t s) {
  if (T == 0) return 0;
  if (H % 8) return -1;
  const int threads = H >= 2048 ? 256 : 128;
  rmsnorm_fwd_kernel<<<T, threads, 0, s>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<const __nv_bfloat16*>(residual),
      reinterpret_cast<const __nv_bfloat16*>(w), reinterpret_cast<__nv_bfloat16*>(y),
      reinterpret_cast<__nv_bfloat16*>(res_out), rstd, H, eps);
  return static_cast<int>(cudaGetLastError());
}

// Number of partial rows the backward writes: scratch must hold rmsnorm_bwd_blocks(T) * H floats.
int vb_rmsnorm_bwd_blocks(int T) {
  const int cap = 148 * 4;
  return T < cap ? (T > 0 ? T : 1) : cap;
}

int vb_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, const void* dres_in, void* dx,
                   float* dw, float* scratch, int T, int H, int accumulate_dw, cudaStream_t s) {
  if (T == 0) return 0;
  if (H % 8) return -1;
  const int blocks = vb_rmsnorm_bwd_blocks(T);
  const int threads = 256;
  const int nv = H / 8;
  const int vpt = (nv + threads - 1) / threads;
#define VB_RB(V)                                                                                               \
  rmsnorm_bwd_kernel<V><<<blocks, threads, 0, s>>>(                                                             \
      reinterpret_cast<const __nv_bfloat16*>(dy), reinterpret_cast<const __nv_bfloat16*>(x),                   \
      reinterpret_cast<const __nv_bfloat16*>(w), rstd, reinterpret_cast<const __nv_bfloat16*>(dres_in),        \
      reinterpret_cast<__nv_bfloat16*>(dx), scratch, T, H)
  if (vpt <= 1) VB_RB(1);
  else if (vpt <= 2) VB_RB(2);
  else if (vpt <= 4) VB_RB(4);
  else return -2;  // H > 8192
#undef VB_RB
  colsum_kernel<<<cdiv_ll(H, 256), 256, 0, s>>>(scratch, dw, blocks, H, accumulate_dw);
  return static_cast<int>(cudaGetLastError());
}

int vb_rope(void* x, const int* pos, const float* cos_t, const float* sin_t, int T, int nheads, int hd, long long ld,
            int backward, cudaStream_t s) {
  if (T == 0) return 0;
  if (hd % 4) return -1;
  const long long total = static_cast<long long>(T) * nheads * (hd / 4);
  rope_kernel<<<cdiv_ll(total, 256), 256, 0, s>>>(reinterpret_cast<__nv_bfloat16*>(x), pos, cos_t, sin_t, T, nheads,
                                                  hd, ld, backward ? -1.f : 1.f);
  return static_cast<int>(cudaGetLastError());
}

int vb_swiglu_fwd(const void* gu, void* out, long long T, int I, cudaStream_t s) {
  if (T == 0) return 0;
  if (I % 8) return -1;
  swiglu_fwd_kernel<<<cdiv_ll(T * (I / 8), 256), 256, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(gu),
                                                            reinterpret_cast<__nv_bfloat16*>(out), T, I);
  return static_cast<int>(cudaGetLastError());
}
int vb_swiglu_bwd(const void* dout, const void* gu, void* dgu, long long T, int I, cudaStream_t s) {
  if (T == 0) return 0;
  if (I % 8) return -1;
  swiglu_bwd_kernel<<<cdiv_ll(T * (I / 8), 256), 256, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(dout),
                                                            reinterpret_cast<const __nv_bfloat16*>(gu),
                                                            reinterpret_cast<__nv_bfloat16*>(dgu), T, I);
  return static_cast<int>(cudaGetLastError());
}

int vb_embedding_fwd(const long long* ids, const void* w, void* out, int T, int H, int V, cudaStream_t s) {
  if (T == 0) return 0;
  if (H % 8) return -1;
  embedding_fwd_kernel<<<T, 128, 0, s>>>(ids, reinterpret_cast<const __nv_bfloat16*>(w),
                                         reinterpret_cast<__nv_bfloat16*>(out), H, V);
  return static_cast<int>(cudaGetLastError());
}
int vb_embedding_bwd(const long long* ids, const void* dout, float* dw, int T, int H, int V, cudaStream_t s) {
  if (T == 0) return 0;
  embedding_bwd_kernel<<<T, 256, 0, s>>>(ids, reinterpret_cast<const __nv_bfloat16*>(dout), dw, H, V);
  return static_cast<int>(cudaGetLastError());
}

int vb_sumsq(const float* g, long long n, float* ctrl, cudaStream_t s) {
  if (n == 0) return 0;
  long long blocks = (n / 4 + 255) / 256;
  if (blocks > SUMSQ_MAX_BLOCKS) blocks = SUMSQ_MAX_BLOCKS;
  if (blocks < 1) blocks = 1;
  sumsq_kernel<<<static_cast<int>(blocks), 256, 0, s>>>(g, n, ctrl);
  sumsq_final_kernel<<<1, 256, 0, s>>>(static_cast<int>(blocks), ctrl);
  return static_cast<int>(cudaGetLastError());
}
int vb_clip_coef(float* ctrl, float max_norm, cudaStream_t s) {
  clip_coef_kernel<<<1, 1, 0, s>>>(ctrl, max_norm);
  return static_cast<int>(cudaGetLastError());
}
int vb_adamw(float* master, float* grad, float* m, float* v, void* out_bf16, long long n, const float* ctrl, float lr,
             float beta1, float beta2, float eps, float wd, int step, float grad_scale, int zero_grad,
             cudaStream_t s) {
  if (n == 0) return 0;
  const float bc1 = 1.f - powf(beta1, static_cast<float>(step));
  const float bc2s = sqrtf(1.f - powf(beta2, static_cast<float>(step)));
  adamw_kernel<<<cdiv_ll(n, 256), 256, 0, s>>>(master, grad, m, v, reinterpret_cast<__nv_bfloat16*>(out_bf16), n, ctrl,
                                               lr, beta1, beta2, eps, wd, bc1, bc2s, grad_scale, zero_grad);
  return static_cast<int>(cudaGetLastError());
}
int vb_cast_f32_bf16(const float* in, void* out, long long n, float scale, cudaStream_t s) {
  if (n == 0) return 0;
  cast_f32_bf16_kernel<<<cdiv_ll(n, 256), 256, 0, s>>>(in, reinterpret_cast<__nv_bfloat16*>(out), n, scale);
  return static_cast<int>(cudaGetLastError());
}
int vb_accum_bf16_f32(const void* in, float* out, long long n, float scale, int accumulate, cudaStream_t s) {
  if (n == 0) return 0;
  accum_bf16_f32_kernel<<<cdiv_ll(n, 256), 256, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(in), out, n, scale,
                                                        accumulate);
  return static_cast<int>(cudaGetLastError());
}

}  // extern "C"
