// RMSNorm backward with its partial-sum buffer built into the module (see rmsnorm_bwd_static.h for who needs
// this and the rules of use).  Math, per row r with s = rstd[r]:
//   dx = s * (dy*w) - x * s^3 * mean_h(dy*w*x)  (+ dres_in),      dw[h] = sum_r dy[r,h] * x[r,h] * s
// Pass 1: one block per SM walks rows r = b, b+grid, ...; every thread keeps the dw partial of its own columns
// in registers and finally stores one full row of the buffer.  Pass 2 sums the rows of the buffer per column.
#include "rmsnorm_bwd_static.h"

#include <cuda_bf16.h>
#include <stdint.h>

#include <cstdint>
#include <mutex>

namespace {

constexpr int kMaxH = VB_RMSNORM_BWD_STATIC_MAX_H;
constexpr int kMaxBlocks = VB_RMSNORM_BWD_STATIC_MAX_BLOCKS;
constexpr int kThreads = 256;
constexpr int kMaxDevices = 64;

// 148 x 8192 fp32 = 4.625 MiB per device, reserved when the module loads.
static __device__ __align__(256) float g_partial[static_cast<size_t>(kMaxBlocks) * kMaxH];

struct alignas(16) Pack8 {
  __nv_bfloat162 v[4];
};

__device__ __forceinline__ void widen(const Pack8& p, float (&f)[8]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(p.v[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}

__device__ __forceinline__ float block_total(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();  // red may still be read by the previous row
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = lane < (kThreads >> 5) ? red[lane] : 0.f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  return t;
}

template <int VPT>
__global__ void __launch_bounds__(kThreads) bwd_rows_kernel(const __nv_bfloat16* __restrict__ dy,
                                                            const __nv_bfloat16* __restrict__ x,
                                                            const __nv_bfloat16* __restrict__ w,
                                                            const float* __restrict__ rstd,
                                                            const __nv_bfloat16* __restrict__ dres_in,
                                                            __nv_bfloat16* __restrict__ dx, float* __restrict__ partial,
                                                            int T, int H) {
  __shared__ float red[32];
  const int nvec = H >> 3;
  float acc[VPT][8], wv[VPT][8];
#pragma unroll
  for (int v = 0; v < VPT; ++v) {
    const int c = threadIdx.x + v * kThreads;
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[v][j] = 0.f, wv[v][j] = 0.f;
    if (c < nvec) widen(reinterpret_cast<const Pack8*>(w)[c], wv[v]);
  }
  for (long long r = blockIdx.x; r < T; r += gridDim.x) {
    const Pack8* dyr = reinterpret_cast<const Pack8*>(dy + r * H);
    const Pack8* xr = reinterpret_cast<const Pack8*>(x + r * H);
    const float s = rstd[r];
    float g[VPT][8], xx[VPT][8];
    float dot = 0.f;
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      const int c = threadIdx.x + v * kThreads;
      if (c < nvec) {
        widen(dyr[c], g[v]);
        widen(xr[c], xx[v]);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          dot += g[v][j] * wv[v][j] * xx[v][j];
          acc[v][j] += g[v][j] * xx[v][j] * s;
        }
      }
    }
    dot = block_total(dot, red);
    const float k = dot * s * s * s / static_cast<float>(H);
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      const int c = threadIdx.x + v * kThreads;
      if (c < nvec) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = s * g[v][j] * wv[v][j] - xx[v][j] * k;
        if (dres_in != nullptr) {
          float d[8];
          widen(reinterpret_cast<const Pack8*>(dres_in + r * H)[c], d);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += d[j];
        }
        Pack8 p;
#pragma unroll
        for (int j = 0; j < 4; ++j) p.v[j] = __floats2bfloat162_rn(o[2 * j], o[2 * j + 1]);
        reinterpret_cast<Pack8*>(dx + r * H)[c] = p;
      }
    }
  }
  // every block stores its whole row of the buffer (zeros when it saw no row), so pass 2 reads only fresh data
  float* row = partial + static_cast<long long>(blockIdx.x) * H;
#pragma unroll
  for (int v = 0; v < VPT; ++v) {
    const int c = threadIdx.x + v * kThreads;
    if (c < nvec) {
      reinterpret_cast<float4*>(row + c * 8)[0] = make_float4(acc[v][0], acc[v][1], acc[v][2], acc[v][3]);
      reinterpret_cast<float4*>(row + c * 8)[1] = make_float4(acc[v][4], acc[v][5], acc[v][6], acc[v][7]);
    }
  }
}

__global__ void sum_rows_kernel(const float* __restrict__ partial, float* __restrict__ dw, int rows, int H,
                                int accumulate) {
  const int h = blockIdx.x * blockDim.x + threadIdx.x;
  if (h >= H) return;
  float t = 0.f;
  for (int b = 0; b < rows; ++b) t += partial[static_cast<long long>(b) * H + h];
  dw[h] = accumulate ? dw[h] + t : t;
}

std::mutex g_mu;
float* g_addr[kMaxDevices] = {};

// Address of this device's copy of g_partial; looked up once per device, no allocation involved.
int buffer_for_current_device(float** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (dev < 0 || dev >= kMaxDevices) return -4;
  std::lock_guard<std::mutex> lock(g_mu);
  if (g_addr[dev] == nullptr) {
    float* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_partial);
    if (e != cudaSuccess) return static_cast<int>(e);
    g_addr[dev] = p;
  }
  *out = g_addr[dev];
  return 0;
}

}  // namespace

extern "C" int vb_rmsnorm_bwd_static(const void* dy, const void* x, const void* w, const float* rstd,
                                     const void* dres_in, void* dx, float* dw, int T, int H, int accumulate_dw,
                                     cudaStream_t stream) {
  if (T < 0) return -3;
  if (H <= 0 || (H % 8) != 0) return -1;
  if (H > kMaxH) return -2;
  // every row is read and written in 16-byte packets: a null or unaligned pointer would fault on the device, so it is
  // turned away here, before anything is launched
  if (dy == nullptr || x == nullptr || w == nullptr || rstd == nullptr || dx == nullptr || dw == nullptr) return -5;
  const auto misaligned = [](const void* p, uintptr_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) != 0; };
  if (misaligned(dy, 16) || misaligned(x, 16) || misaligned(w, 16) || misaligned(dx, 16) ||
      (dres_in != nullptr && misaligned(dres_in, 16)) || misaligned(rstd, 4) || misaligned(dw, 4))
    return -6;
  float* partial = nullptr;
  const int rc = buffer_for_current_device(&partial);
  if (rc != 0) return rc;
  if (T == 0) {
    // no rows: the weight gradient of this call is zero; "overwritten" still has to hold
    if (!accumulate_dw) return static_cast<int>(cudaMemsetAsync(dw, 0, static_cast<size_t>(H) * sizeof(float), stream));
    return 0;
  }
  const int blocks = T < kMaxBlocks ? T : kMaxBlocks;
  const int vpt = (H / 8 + kThreads - 1) / kThreads;
  const auto* dy_ = static_cast<const __nv_bfloat16*>(dy);
  const auto* x_ = static_cast<const __nv_bfloat16*>(x);
  const auto* w_ = static_cast<const __nv_bfloat16*>(w);
  const auto* dr_ = static_cast<const __nv_bfloat16*>(dres_in);
  auto* dx_ = static_cast<__nv_bfloat16*>(dx);
  if (vpt <= 1) bwd_rows_kernel<1><<<blocks, kThreads, 0, stream>>>(dy_, x_, w_, rstd, dr_, dx_, partial, T, H);
  else if (vpt <= 2) bwd_rows_kernel<2><<<blocks, kThreads, 0, stream>>>(dy_, x_, w_, rstd, dr_, dx_, partial, T, H);
  else bwd_rows_kernel<4><<<blocks, kThreads, 0, stream>>>(dy_, x_, w_, rstd, dr_, dx_, partial, T, H);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return static_cast<int>(e);
  sum_rows_kernel<<<(H + 255) / 256, 256, 0, stream>>>(partial, dw, blocks, H, accumulate_dw);
  return static_cast<int>(cudaGetLastError());
}

extern "C" const char* vb_rmsnorm_bwd_static_strerror(int code) {
  switch (code) {
    case 0: return "ok";
    case -1: return "vb_rmsnorm_bwd_static: row length H must be a positive multiple of 8";
    case -2: return "vb_rmsnorm_bwd_static: row length H exceeds the built-in buffer (max 8192); use vb_rmsnorm_bwd with your own scratch";
    case -3: return "vb_rmsnorm_bwd_static: negative row count";
    case -4: return "vb_rmsnorm_bwd_static: device ordinal beyond the per-device table (64)";
    case -5: return "vb_rmsnorm_bwd_static: dy, x, w, rstd, dx and dw must not be null";
    case -6: return "vb_rmsnorm_bwd_static: dy, x, w, dx and dres_in must be 16-byte aligned (rstd and dw 4-byte aligned)";
    default: return code > 0 ? cudaGetErrorString(static_cast<cudaError_t>(code)) : "vb_rmsnorm_bwd_static: unknown code";
  }
}
