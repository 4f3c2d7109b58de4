// fp8 (e4m3) GEMM with 1x128 block scaling on both operands, and the quantiser that produces such operands.
//
//   D[M,N] (bf16) = sum over 128-wide K blocks kb of  sa[kb, m] * sb[kb, n] * ( Aq[m, kb] . Bq[n, kb] )
//
// Aq [M, K], Bq [N, K] are e4m3, K-major, K % 128 == 0. Scales are fp32 and stored block-major: sa [K/128, M],
// sb [K/128, N], so the 128 scales a tile needs for one K block are contiguous.
//
// One CTA per 128 x 128 output tile:
//   warp 0      TMA: A and B tiles of one K block (128 rows x 128 bytes, 128B swizzle) through a 4-stage ring
//   warp 1      MMA: four tcgen05.mma kind::f8f6f4 (K = 32 each) per K block into one of two TMEM buffers (fresh
//               accumulation per block, because the block's scale factors differ per row and column)
//   warps 2..5  thread == output row: tcgen05.ld the block's 128 partial sums, multiply by sa[m] * sb[n], accumulate in
//               registers; after the last block store the row as bf16
#include "tcgen05_common.cuh"

#include <cuda_fp8.h>
#include <math.h>

namespace vb {

constexpr int F8_BM = 128, F8_BN = 128, F8_BK = 128, F8_STAGES = 4, F8_THREADS = 192;

struct Fp8GemmParams {
  int M, N, K;
  const float* sa;  // [K/128, M]
  const float* sb;  // [K/128, N]
  __nv_bfloat16* D;
  long long ldd;
  const __nv_bfloat16* bias;
  int* status;
  // grouped (mixture-of-experts) mode: A rows are grouped by expert in 128-row aligned segments, B holds E stacked [N, K]
  // matrices and sb E stacked column-scale rows; the 128-row tile i belongs to expert grp_tile_expert[i]
  const int* grp_tile_expert;  // nullptr = plain GEMM
  const int* grp_num_mtiles;   // device scalar: tiles in use (tiles beyond it return at once)
  long long ldsb;              // row stride of sb (N, or E * N when grouped)
};

struct Fp8Smem {
  static constexpr int TILE = F8_BM * F8_BK;  // 16 KB (one byte per element)
  static constexpr int OFF_B = F8_STAGES * TILE;
  static constexpr int OFF_SB = 2 * F8_STAGES * TILE;              // per epilogue warp: [2][128] fp32 column scales
  static constexpr int OFF_BAR = OFF_SB + 4 * 2 * F8_BN * 4;
  static constexpr int TOTAL = OFF_BAR + 256 + 1024;
};

__global__ void __launch_bounds__(F8_THREADS, 1)
gemm_fp8_blockscale_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                           const Fp8GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem + Fp8Smem::OFF_B;
  float* s_sb = reinterpret_cast<float*>(smem + Fp8Smem::OFF_SB);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Fp8Smem::OFF_BAR);
  uint64_t* full_bar = bars;                       // [STAGES]
  uint64_t* empty_bar = bars + F8_STAGES;          // [STAGES]
  uint64_t* acc_full = bars + 2 * F8_STAGES;       // [2]
  uint64_t* acc_empty = bars + 2 * F8_STAGES + 2;  // [2]
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 2 * F8_STAGES + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * F8_BN, m0 = blockIdx.y * F8_BM;
  const int num_kb = p.K / F8_BK;
  int b_row0 = n0;  // first row of the B operand (and column of sb) of this tile
  if (p.grp_tile_expert != nullptr) {
    if (static_cast<int>(blockIdx.y) >= *p.grp_num_mtiles) return;  // uniform over the CTA; nothing allocated yet
    b_row0 = p.grp_tile_expert[blockIdx.y] * p.N + n0;
  }

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tma_a);
    tma_prefetch_desc(&tma_b);
    for (int s = 0; s < F8_STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 4);
    }
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_holder, 2 * F8_BN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    if (lane == 0) {
      for (int kb = 0; kb < num_kb; ++kb) {
        const int st = kb % F8_STAGES;
        if (!mbar_wait(&empty_bar[st], ((kb / F8_STAGES) & 1) ^ 1)) {
          atomicExch(p.status, ST_TIMEOUT_PRODUCER);
          break;
        }
        mbar_expect_tx(&full_bar[st], 2 * Fp8Smem::TILE);
        tma_load_2d(smem_a + st * Fp8Smem::TILE, &tma_a, &full_bar[st], kb * F8_BK, m0);
        tma_load_2d(smem_b + st * Fp8Smem::TILE, &tma_b, &full_bar[st], kb * F8_BK, b_row0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_e4m3(F8_BM, F8_BN);
      bool ok = true;
      for (int kb = 0; kb < num_kb && ok; ++kb) {
        const int st = kb % F8_STAGES, buf = kb & 1;
        if (!mbar_wait(&acc_empty[buf], ((kb >> 1) & 1) ^ 1) || !mbar_wait(&full_bar[st], (kb / F8_STAGES) & 1)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t sa = smem_u32(smem_a + st * Fp8Smem::TILE), sb = smem_u32(smem_b + st * Fp8Smem::TILE);
#pragma unroll
        for (int k = 0; k < F8_BK / 32; ++k) {
          const uint64_t da = make_smem_desc_sw128(sa + k * 32, 16, 1024);
          const uint64_t db = make_smem_desc_sw128(sb + k * 32, 16, 1024);
          tc_mma_f8_ss(tmem_base + buf * F8_BN, da, db, idesc, k > 0 ? 1u : 0u);
        }
        tc_commit(&empty_bar[st]);
        tc_commit(&acc_full[buf]);
      }
      if (!ok) atomicExch(p.status, ST_TIMEOUT_MMA);
    }
  } else {
    const int q = warp & 3;
    const int row = m0 + q * 32 + lane;
    const bool row_ok = row < p.M;
    const uint32_t lane_off = static_cast<uint32_t>(q * 32) << 16;
    float* my_sb = s_sb + q * (2 * F8_BN);
    float acc[F8_BN];
#pragma unroll
    for (int j = 0; j < F8_BN; ++j) acc[j] = 0.f;
    bool ok = true;
    for (int kb = 0; kb < num_kb; ++kb) {
      const int buf = kb & 1;
      // column scales of this K block (each warp keeps its own copy: no barrier across warps)
      float* csb = my_sb + buf * F8_BN;
#pragma unroll
      for (int u = 0; u < F8_BN / 32; ++u) {
        const int n = n0 + lane + 32 * u;
        csb[lane + 32 * u] = n < p.N ? p.sb[static_cast<long long>(kb) * p.ldsb + (b_row0 - n0) + n] : 0.f;
      }
      const float ra = row_ok ? p.sa[static_cast<long long>(kb) * p.M + row] : 0.f;
      __syncwarp();
      if (!mbar_wait(&acc_full[buf], (kb >> 1) & 1)) {
        ok = false;
        break;
      }
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < F8_BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(tmem_base + buf * F8_BN + c * 32 + lane_off, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) acc[c * 32 + j] = fmaf(__uint_as_float(r[j]), ra * csb[c * 32 + j], acc[c * 32 + j]);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);
    }
    if (!ok) {
      if (lane == 0) atomicExch(p.status, ST_TIMEOUT_EPILOGUE);
    } else if (row_ok) {
      __nv_bfloat16* out = p.D + static_cast<long long>(row) * p.ldd + n0;
#pragma unroll
      for (int j = 0; j < F8_BN; j += 8) {
        if (n0 + j < p.N) {
          float b[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
          if (p.bias != nullptr) {
#pragma unroll
            for (int u = 0; u < 8; ++u) b[u] = __bfloat162float(p.bias[n0 + j + u]);
          }
          uint4 v;
          v.x = pack_bf16x2(acc[j] + b[0], acc[j + 1] + b[1]);
          v.y = pack_bf16x2(acc[j + 2] + b[2], acc[j + 3] + b[3]);
          v.z = pack_bf16x2(acc[j + 4] + b[4], acc[j + 5] + b[5]);
          v.w = pack_bf16x2(acc[j + 6] + b[6], acc[j + 7] + b[7]);
          *reinterpret_cast<uint4*>(out + j) = v;
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * F8_BN);
  }
}

// x [R, C] bf16 -> q [R, C] e4m3 and scales [C/128, R] fp32 with  x ~= q * scale,  scale = amax(block) / 448.
// One warp per (row, 128-column block): 4 elements per lane.
__global__ void fp8_quant_1x128_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, uint8_t* __restrict__ q, long long ldq,
                                       float* __restrict__ scales, int R, int C) {
  const long long w = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int nblk = C / 128;
  if (w >= static_cast<long long>(R) * nblk) return;
  const int r = static_cast<int>(w / nblk), b = static_cast<int>(w % nblk);
  const __nv_bfloat16* src = x + static_cast<long long>(r) * ldx + b * 128 + lane * 4;
  const uint2 raw = *reinterpret_cast<const uint2*>(src);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
  const float2 a = __bfloat1622float2(h[0]), c = __bfloat1622float2(h[1]);
  float amax = fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(c.x), fabsf(c.y)));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const float scale = fmaxf(amax, 1e-12f) / 448.f;
  const float inv = 1.f / scale;
  __nv_fp8x4_e4m3 packed(make_float4(a.x * inv, a.y * inv, c.x * inv, c.y * inv));
  *reinterpret_cast<uint32_t*>(q + static_cast<long long>(r) * ldq + b * 128 + lane * 4) = *reinterpret_cast<uint32_t*>(&packed);
  if (lane == 0) scales[static_cast<long long>(b) * R + r] = scale;
}

// w [R, C] bf16 -> q [R, C] e4m3 and scale_inv [ceil(R/128), ceil(C/128)] fp32: one scale per 128 x 128 block
// (w ~= q * scale_inv, scale_inv = amax(block) / 448), the weight format of block-scaled fp8 checkpoints.
// One CTA of 256 threads per block: pass 1 reduces |w| over the block, pass 2 converts.
__global__ void fp8_quant_128x128_kernel(const __nv_bfloat16* __restrict__ w, long long ldw, uint8_t* __restrict__ q, long long ldq,
                                         float* __restrict__ scale_inv, int R, int C) {
  __shared__ float s_red[8];
  __shared__ float s_scale;
  const int bc = blockIdx.x, br = blockIdx.y;
  const int r0 = br * 128, c0 = bc * 128;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // thread t covers columns (t % 32) * 4 .. +3 of rows (t / 32) + 8 * i
  const int col = c0 + (tid & 31) * 4;
  float amax = 0.f;
  float4 vals[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const int row = r0 + (tid >> 5) + 8 * i;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (row < R && col < C) {  // C % 4 == 0: a 4-vector is inside or outside as a whole
      const uint2 raw = *reinterpret_cast<const uint2*>(w + static_cast<long long>(row) * ldw + col);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
      const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
      v = make_float4(a.x, a.y, b.x, b.y);
    }
    vals[i] = v;
    amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if (lane == 0) s_red[warp] = amax;
  __syncthreads();
  if (tid == 0) {
    float m = s_red[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) m = fmaxf(m, s_red[i]);
    const float sc = fmaxf(m, 1e-12f) / 448.f;
    s_scale = sc;
    scale_inv[static_cast<long long>(br) * gridDim.x + bc] = sc;
  }
  __syncthreads();
  const float inv = 1.f / s_scale;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const int row = r0 + (tid >> 5) + 8 * i;
    if (row < R && col < C) {
      const float4 v = vals[i];
      __nv_fp8x4_e4m3 packed(make_float4(v.x * inv, v.y * inv, v.z * inv, v.w * inv));
      *reinterpret_cast<uint32_t*>(q + static_cast<long long>(row) * ldq + col) = *reinterpret_cast<uint32_t*>(&packed);
    }
  }
}

__device__ int g_fp8_status[4];

}  // namespace vb

using namespace vb;

extern "C" int vb_fp8_quant_1x128(const void* x, long long ldx, void* q, long long ldq, float* scales, int R, int C, cudaStream_t s) {
  if (R <= 0 || C <= 0) return 0;
  if ((C % 128) || (ldx % 4) || (ldq % 4)) return -1;
  const long long threads = static_cast<long long>(R) * (C / 128) * 32;
  fp8_quant_1x128_kernel<<<static_cast<int>((threads + 255) / 256), 256, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(x), ldx,
                                                                                 reinterpret_cast<uint8_t*>(q), ldq, scales, R, C);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int vb_fp8_quant_128x128(const void* w, long long ldw, void* q, long long ldq, float* scale_inv, int R, int C, cudaStream_t s) {
  if (R <= 0 || C <= 0) return 0;
  if ((C % 4) || (ldw % 4) || (ldq % 4)) return -1;
  dim3 grid((C + 127) / 128, (R + 127) / 128);
  fp8_quant_128x128_kernel<<<grid, 256, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(w), ldw, reinterpret_cast<uint8_t*>(q), ldq,
                                                scale_inv, R, C);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int vb_gemm_fp8_blockscale(const void* Aq, const float* sa, const void* Bq, const float* sb, void* D, const void* bias, int M,
                                      int N, int K, long long lda, long long ldb, long long ldd, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((K % 128) || (N % 8) || (lda % 16) || (ldb % 16) || (ldd % 8)) return -1;
  if ((reinterpret_cast<uintptr_t>(Aq) | reinterpret_cast<uintptr_t>(Bq) | reinterpret_cast<uintptr_t>(D)) & 15) return -2;
  CUtensorMap ta, tb;
  if (!make_tmap_2d(&ta, Aq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, M, K, lda, F8_BK, F8_BM, CU_TENSOR_MAP_SWIZZLE_128B)) return -3;
  if (!make_tmap_2d(&tb, Bq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, N, K, ldb, F8_BK, F8_BN, CU_TENSOR_MAP_SWIZZLE_128B)) return -3;
  static int* status = nullptr;
  if (status == nullptr) cudaGetSymbolAddress(reinterpret_cast<void**>(&status), g_fp8_status);
  Fp8GemmParams p{};
  p.M = M; p.N = N; p.K = K; p.sa = sa; p.sb = sb; p.D = reinterpret_cast<__nv_bfloat16*>(D); p.ldd = ldd;
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias); p.status = status;
  p.ldsb = N;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_fp8_blockscale_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Fp8Smem::TOTAL);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  dim3 grid((N + F8_BN - 1) / F8_BN, (M + F8_BM - 1) / F8_BM);
  gemm_fp8_blockscale_kernel<<<grid, F8_THREADS, Fp8Smem::TOTAL, stream>>>(ta, tb, p);
  return static_cast<int>(cudaGetLastError());
}

// Grouped variant for mixture-of-experts layers: D[rows, N] = A[rows, K] * B_e^T for the expert e of each 128-row tile.
//  Aq [rows_cap, K] e4m3 with scales sa [K/128, rows_cap]; Bq [E * N, K] e4m3 with scales sb [K/128, E * N];
//  tile_expert[i] = expert of tile i, num_mtiles (device scalar) = tiles in use. Rows of unused tiles are not written.
extern "C" int vb_gemm_fp8_blockscale_grouped(const void* Aq, const float* sa, const void* Bq, const float* sb, void* D, int rows_cap,
                                              int N, int K, int E, long long lda, long long ldb, long long ldd, const int* tile_expert,
                                              const int* num_mtiles, cudaStream_t stream) {
  if (rows_cap <= 0 || N <= 0 || K <= 0 || E <= 0) return 0;
  if ((K % 128) || (N % 8) || (rows_cap % F8_BM) || (lda % 16) || (ldb % 16) || (ldd % 8)) return -1;
  if ((reinterpret_cast<uintptr_t>(Aq) | reinterpret_cast<uintptr_t>(Bq) | reinterpret_cast<uintptr_t>(D)) & 15) return -2;
  CUtensorMap ta, tb;
  if (!make_tmap_2d(&ta, Aq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, rows_cap, K, lda, F8_BK, F8_BM, CU_TENSOR_MAP_SWIZZLE_128B)) return -3;
  if (!make_tmap_2d(&tb, Bq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, static_cast<uint64_t>(E) * N, K, ldb, F8_BK, F8_BN, CU_TENSOR_MAP_SWIZZLE_128B)) return -3;
  static int* status = nullptr;
  if (status == nullptr) cudaGetSymbolAddress(reinterpret_cast<void**>(&status), g_fp8_status);
  Fp8GemmParams p{};
  p.M = rows_cap; p.N = N; p.K = K; p.sa = sa; p.sb = sb; p.D = reinterpret_cast<__nv_bfloat16*>(D); p.ldd = ldd;
  p.bias = nullptr; p.status = status;
  p.grp_tile_expert = tile_expert; p.grp_num_mtiles = num_mtiles; p.ldsb = static_cast<long long>(E) * N;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_fp8_blockscale_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Fp8Smem::TOTAL);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  dim3 grid((N + F8_BN - 1) / F8_BN, rows_cap / F8_BM);
  gemm_fp8_blockscale_kernel<<<grid, F8_THREADS, Fp8Smem::TOTAL, stream>>>(ta, tb, p);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int vb_fp8_status() {
  int h[4] = {0, 0, 0, 0};
  if (cudaMemcpyFromSymbol(h, g_fp8_status, sizeof(h)) != cudaSuccess) return -1;
  if (h[0] != 0) {
    int z[4] = {0, 0, 0, 0};
    cudaMemcpyToSymbol(g_fp8_status, z, sizeof(z));
  }
  return h[0];
}
