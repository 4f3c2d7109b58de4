// NVFP4 fake quantisation for quantisation-aware training: y = dequant(quant(x)) with e2m1 values in blocks of 16 along
// the row, one e4m3 scale per block expressed in units of a per-tensor fp32 scale.
//
//   block_scale = e4m3(amax_block / (6 * global_scale)) * global_scale        (1.0 when that underflows)
//   y           = sign(x) * round_e2m1(|x| / block_scale) * block_scale       e2m1 grid {0, .5, 1, 1.5, 2, 3, 4, 6},
//                                                                              ties to the even mantissa
// One thread owns one block: two 16-byte loads, 16 values in registers, two 16-byte stores. Purely memory bound.
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace vb {

__device__ __forceinline__ float e2m1_round(float a) {
  // thresholds are the midpoints of the grid; "<=" where the tie goes to the lower (even-mantissa) value
  return a <= 0.25f ? 0.f : a < 0.75f ? 0.5f : a <= 1.25f ? 1.f : a < 1.75f ? 1.5f : a <= 2.5f ? 2.f : a < 3.5f ? 3.f : a <= 5.f ? 4.f : 6.f;
}

__global__ void nvfp4_fake_quant_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, __nv_bfloat16* __restrict__ y,
                                        long long ldy, long long rows, int blocks_per_row, float global_scale) {
  const long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (i >= rows * blocks_per_row) return;
  const long long r = i / blocks_per_row;
  const int c = static_cast<int>(i % blocks_per_row) * 16;
  const uint4* src = reinterpret_cast<const uint4*>(x + r * ldx + c);
  uint4 raw[2] = {src[0], src[1]};
  const __nv_bfloat16* h = reinterpret_cast<const __nv_bfloat16*>(raw);
  float v[16];
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    v[j] = __bfloat162float(h[j]);
    amax = fmaxf(amax, fabsf(v[j]));
  }
  const float gs = global_scale > 0.f ? global_scale : 1e-12f;
  const float want = fminf(amax / (6.f * gs), 448.f);
  const __nv_fp8_storage_t s8 = __nv_cvt_float_to_fp8(want, __NV_SATFINITE, __NV_E4M3);
  float scale = __half2float(__half(__nv_cvt_fp8_to_halfraw(s8, __NV_E4M3))) * global_scale;
  if (!(scale >= 1e-5f)) scale = 1.f;
  const float inv = 1.f / scale;
  uint4 out[2];
  __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(out);
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    const float q = e2m1_round(fabsf(v[j]) * inv) * scale;
    o[j] = __float2bfloat16(v[j] >= 0.f ? q : -q);
  }
  uint4* dst = reinterpret_cast<uint4*>(y + r * ldy + c);
  dst[0] = out[0];
  dst[1] = out[1];
}

}  // namespace vb

// x, y: bf16 [rows, cols] with row strides ldx / ldy (elements); cols % 16 == 0, rows 16-byte aligned. y may alias x.
extern "C" int vb_nvfp4_fake_quant(const void* x, long long ldx, void* y, long long ldy, long long rows, int cols,
                                   float global_scale, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return 0;
  if ((cols % 16) || (ldx % 8) || (ldy % 8)) return -1;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15) return -2;
  const int bpr = cols / 16;
  const long long n = rows * bpr;
  const int threads = 256;
  vb::nvfp4_fake_quant_kernel<<<static_cast<unsigned int>((n + threads - 1) / threads), threads, 0, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), ldx, reinterpret_cast<__nv_bfloat16*>(y), ldy, rows, bpr, global_scale);
  return static_cast<int>(cudaGetLastError());
}
