// Persistent warp-specialised bf16 GEMM for sm_100a.
//
//   D[M,N] = A[M,K] * B[N,K]^T (+ bias[N])           fp32 accumulation in TMEM
//
// Operand layouts (row-major storage in global memory):
//   A "K-major":  stored [M, K]  (K contiguous)        A "MN-major": stored [K, M]  (M contiguous)
//   B "K-major":  stored [N, K]  (K contiguous)        B "MN-major": stored [K, N]  (N contiguous)
// so the three GEMMs of a linear layer need no transposes:
//   forward  Y  = X  W^T : A = X  (K-major),  B = W  (K-major)
//   dgrad    dX = dY W   : A = dY (K-major),  B = W  (MN-major, stored [N_w, K_w])
//   wgrad    dW = dY^T X : A = dY (MN-major), B = X  (MN-major)     (fp32 output, optional +=)
//
// Structure per CTA (192 threads, one CTA per SM, persistent over tiles):
//   warp 0      TMA producer: cp.async.bulk.tensor (128B swizzle) into a STAGES-deep smem ring
//   warp 1      MMA issuer: one elected thread issues tcgen05.mma (128 x BN x 16) into one of two
//               TMEM accumulators; tcgen05.commit releases smem stages / publishes the accumulator
//   warps 2..5  epilogue: tcgen05.ld (32 lanes x 32 columns per warp) -> bias -> bf16/fp32 -> global
// The epilogue of tile i overlaps the main loop of tile i+1 through the double-buffered accumulator.
#include "tcgen05_common.cuh"

#include <stdio.h>

namespace vb {

// --------------------------------------------------------------------------- kernel
constexpr int BM = 128;
constexpr int BK = 64;  // 64 bf16 = 128 bytes = one swizzle row
constexpr int GEMM_THREADS = 192;

struct GemmParams {
  int M, N, K;
  void* D;
  long long ldd;
  const __nv_bfloat16* bias;
  int out_f32;
  int accumulate;
  int* status;
};

__device__ int g_gemm_status[4];

template <int BN, int STAGES>
struct GemmSmem {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int RING = STAGES * (A_BYTES + B_BYTES);
  static constexpr int TOTAL = RING + 256 + 1024;  // barriers + alignment slack
};

template <int BN, bool A_MN, bool B_MN, int STAGES>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                 const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  constexpr int A_BYTES = GemmSmem<BN, STAGES>::A_BYTES;
  constexpr int B_BYTES = GemmSmem<BN, STAGES>::B_BYTES;
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem + STAGES * A_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + GemmSmem<BN, STAGES>::RING);
  uint64_t* full_bar = bars;                   // [STAGES]
  uint64_t* empty_bar = bars + STAGES;         // [STAGES]
  uint64_t* acc_full = bars + 2 * STAGES;      // [2]
  uint64_t* acc_empty = bars + 2 * STAGES + 2; // [2]
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const int num_m = (p.M + BM - 1) / BM;
  const int num_n = (p.N + BN - 1) / BN;
  const int num_tiles = num_m * num_n;
  const int num_kb = (p.K + BK - 1) / BK;
  constexpr int GROUP_M = 8;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tma_a);
    tma_prefetch_desc(&tma_b);
    for (int s = 0; s < STAGES; ++s) {
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
    tmem_alloc(tmem_holder, 2 * BN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  auto tile_coords = [&](int t, int& m_idx, int& n_idx) {
    const int per_group = GROUP_M * num_n;
    const int g = t / per_group;
    const int first_m = g * GROUP_M;
    const int gsize = min(num_m - first_m, GROUP_M);
    const int r = t - g * per_group;
    m_idx = first_m + (r % gsize);
    n_idx = r / gsize;
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int m_idx, n_idx;
        tile_coords(t, m_idx, n_idx);
        const int m0 = m_idx * BM, n0 = n_idx * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1)) {
            atomicExch(p.status, ST_TIMEOUT_PRODUCER);
            ok = false;
            break;
          }
          mbar_expect_tx(&full_bar[stage], A_BYTES + B_BYTES);
          uint8_t* sa = smem_a + stage * A_BYTES;
          uint8_t* sb = smem_b + stage * B_BYTES;
          const int k0 = kb * BK;
          if constexpr (!A_MN) {
            tma_load_2d(sa, &tma_a, &full_bar[stage], k0, m0);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_2d(sa + j * (BK * 128), &tma_a, &full_bar[stage], m0 + 64 * j, k0);
          }
          if constexpr (!B_MN) {
            tma_load_2d(sb, &tma_b, &full_bar[stage], k0, n0);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) tma_load_2d(sb + j * (BK * 128), &tma_b, &full_bar[stage], n0 + 64 * j, k0);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_f16(BM, BN, A_MN, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1)) {
          atomicExch(p.status, ST_TIMEOUT_MMA);
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase)) {
            atomicExch(p.status, ST_TIMEOUT_MMA);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem_a + stage * A_BYTES);
          const uint32_t sb = smem_u32(smem_b + stage * B_BYTES);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t da = A_MN ? make_smem_desc_sw128(sa + k * 2048, BK * 128, 1024)
                                     : make_smem_desc_sw128(sa + k * 32, 16, 1024);
            const uint64_t db = B_MN ? make_smem_desc_sw128(sb + k * 2048, BK * 128, 1024)
                                     : make_smem_desc_sw128(sb + k * 32, 16, 1024);
            tc_mma_f16_ss(d_tmem, da, db, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          tc_commit(&empty_bar[stage]);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        tc_commit(&acc_full[acc]);
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1;
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;  // TMEM lane quarter this warp may access
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
      int m_idx, n_idx;
      tile_coords(t, m_idx, n_idx);
      const int m0 = m_idx * BM, n0 = n_idx * BN;
      if (!mbar_wait(&acc_full[acc], acc_phase)) {
        if (lane == 0) atomicExch(p.status, ST_TIMEOUT_EPILOGUE);
        ok = false;
        break;
      }
      tc_fence_after();
      const int row = m0 + q * 32 + lane;
      const bool row_ok = row < p.M;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        const int col0 = n0 + c * 32;
        if (col0 >= p.N) break;  // uniform across the warp
        uint32_t r[32];
        tmem_ld_32x32(tmem_base + acc * BN + c * 32 + (static_cast<uint32_t>(q * 32) << 16), r);
        tmem_ld_wait();
        if (row_ok) {
          const int ncols = min(32, p.N - col0);  // multiple of 8
          if (p.bias != nullptr) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              if (j < ncols) r[j] = __float_as_uint(__uint_as_float(r[j]) + __bfloat162float(p.bias[col0 + j]));
            }
          }
          if (p.out_f32) {
            float* out = reinterpret_cast<float*>(p.D) + static_cast<long long>(row) * p.ldd + col0;
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              if (j < ncols) {
                float4 v = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]),
                                       __uint_as_float(r[j + 3]));
                if (p.accumulate) {
                  const float4 o = *reinterpret_cast<const float4*>(out + j);
                  v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
                }
                *reinterpret_cast<float4*>(out + j) = v;
              }
            }
          } else {
            __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.D) + static_cast<long long>(row) * p.ldd + col0;
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              if (j < ncols) {
                uint4 v;
                v.x = pack_bf16x2(__uint_as_float(r[j]), __uint_as_float(r[j + 1]));
                v.y = pack_bf16x2(__uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
                v.z = pack_bf16x2(__uint_as_float(r[j + 4]), __uint_as_float(r[j + 5]));
                v.w = pack_bf16x2(__uint_as_float(r[j + 6]), __uint_as_float(r[j + 7]));
                *reinterpret_cast<uint4*>(out + j) = v;
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[acc]);
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * BN);
  }
}

// --------------------------------------------------------------------------- launcher
template <int BN, bool A_MN, bool B_MN, int STAGES>
static cudaError_t launch_variant(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int sms,
                                  cudaStream_t stream) {
  auto kern = gemm_bf16_kernel<BN, A_MN, B_MN, STAGES>;
  constexpr int smem = GemmSmem<BN, STAGES>::TOTAL;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    configured = true;
  }
  const int tiles = ((p.M + BM - 1) / BM) * ((p.N + BN - 1) / BN);
  const int grid = tiles < sms ? tiles : sms;
  kern<<<grid, GEMM_THREADS, smem, stream>>>(ta, tb, p);
  return cudaGetLastError();
}

}  // namespace vb

using namespace vb;

// Returns 0 on success, a negative code for bad arguments, a positive cudaError_t otherwise.
//  a_mn / b_mn: operand is stored [K, M|N] (MN contiguous) instead of [M|N, K].
//  lda / ldb / ldd: row stride in elements of the stored matrix.
extern "C" int vb_gemm_bf16(const void* A, const void* B, void* D, const void* bias, int M, int N, int K,
                            long long lda, long long ldb, long long ldd, int a_mn, int b_mn, int out_f32,
                            int accumulate, int max_ctas, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((N % 8) || (K % 8) || (lda % 8) || (ldb % 8) || (ldd % (out_f32 ? 4 : 8))) return -1;
  if (a_mn && (M % 8)) return -1;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(D)) & 15) return -2;
  int sms = num_sms();
  if (max_ctas > 0 && max_ctas < sms) sms = max_ctas;
  const bool wide = N > 128;
  const int BN = wide ? 256 : 128;
  CUtensorMap ta, tb;
  bool ok;
  if (!a_mn) ok = make_tmap_2d(&ta, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, K, lda, BK, BM, CU_TENSOR_MAP_SWIZZLE_128B);
  else       ok = make_tmap_2d(&ta, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, M, lda, 64, BK, CU_TENSOR_MAP_SWIZZLE_128B);
  if (!ok) return -3;
  if (!b_mn) ok = make_tmap_2d(&tb, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, K, ldb, BK, BN, CU_TENSOR_MAP_SWIZZLE_128B);
  else       ok = make_tmap_2d(&tb, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, N, ldb, 64, BK, CU_TENSOR_MAP_SWIZZLE_128B);
  if (!ok) return -3;
  int* status = nullptr;
  cudaGetSymbolAddress(reinterpret_cast<void**>(&status), g_gemm_status);
  GemmParams p{M, N, K, D, ldd, reinterpret_cast<const __nv_bfloat16*>(bias), out_f32, accumulate, status};
  cudaError_t e;
#define VB_LAUNCH(BN_, AM, BMJ, ST) e = launch_variant<BN_, AM, BMJ, ST>(ta, tb, p, sms, stream)
  if (wide) {
    if (!a_mn && !b_mn) VB_LAUNCH(256, false, false, 4);
    else if (!a_mn && b_mn) VB_LAUNCH(256, false, true, 4);
    else if (a_mn && b_mn) VB_LAUNCH(256, true, true, 4);
    else VB_LAUNCH(256, true, false, 4);
  } else {
    if (!a_mn && !b_mn) VB_LAUNCH(128, false, false, 6);
    else if (!a_mn && b_mn) VB_LAUNCH(128, false, true, 6);
    else if (a_mn && b_mn) VB_LAUNCH(128, true, true, 6);
    else VB_LAUNCH(128, true, false, 6);
  }
#undef VB_LAUNCH
  return static_cast<int>(e);
}

// Reads (and clears) the GEMM status word of the current device. Synchronises the device.
extern "C" int vb_gemm_status() {
  int h[4] = {0, 0, 0, 0};
  if (cudaMemcpyFromSymbol(h, g_gemm_status, sizeof(h)) != cudaSuccess) return -1;
  if (h[0] != 0) {
    int z[4] = {0, 0, 0, 0};
    cudaMemcpyToSymbol(g_gemm_status, z, sizeof(z));
  }
  return h[0];
}
