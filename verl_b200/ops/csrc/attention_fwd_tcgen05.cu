// Causal GQA attention forward over packed (varlen) sequences on tcgen05 tensor cores.
//
// One CTA = one (sequence, 128-row query tile, query head).  Two CTAs are co-resident per SM (<= 113 KB shared
// memory and 256 TMEM columns each), so the softmax of one tile overlaps the MMAs of the other.
//
//   warp 0      TMA: Q tile once, then K/V tiles of 64 keys through a 2-stage ring (128B swizzle)
//   warp 1      MMA: S_j = Q K_j^T into one of two TMEM S buffers (issued one block ahead), O += P_j V_j
//   warps 2..5  softmax: thread == query row.  tcgen05.ld S -> scale, causal mask, online max/sum in the exp2
//               domain -> P (bf16) written to shared memory in the K-major 128B-swizzle layout the MMA reads;
//               O in TMEM is rescaled (tcgen05.ld / tcgen05.st) only when some row maximum of the warp moved.
// Epilogue: O / l -> bf16 [T, nh, hd]; LSE (natural log) -> [nh, T] for the backward pass.
#include "tcgen05_common.cuh"

#include <math.h>

namespace vb {

constexpr int ATT_BQ = 128;
constexpr int ATT_BKV = 64;
constexpr int ATT_THREADS = 192;

struct AttnFwdParams {
  const int* cu_seqlens;  // [B+1]
  int num_seqs;
  int nh, nkv;
  __nv_bfloat16* out;  // [T, nh, hd]
  long long ldo;
  float* lse;  // [nh, T]
  int total_tokens;
  float scale_log2;
  int* status;
};

template <int HD>
struct AttnSmem {
  static constexpr int Q_BYTES = ATT_BQ * HD * 2;
  static constexpr int KV_BYTES = ATT_BKV * HD * 2;  // one of K or V, one stage
  static constexpr int P_BYTES = ATT_BQ * ATT_BKV * 2;
  static constexpr int OFF_K = Q_BYTES;
  static constexpr int OFF_V = OFF_K + 2 * KV_BYTES;
  static constexpr int OFF_P = OFF_V + 2 * KV_BYTES;
  static constexpr int OFF_BAR = OFF_P + P_BYTES;
  // No alignment slack and no static shared memory: two CTAs (2 x (TOTAL + 1 KB reserved)) must fit the 228 KB of an
  // SM; the dynamic window then starts 1024-byte aligned, which the kernel verifies before touching it.
  static constexpr int TOTAL = OFF_BAR + 128;
};

template <int HD>
__global__ void __launch_bounds__(ATT_THREADS, 2)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                const __grid_constant__ CUtensorMap tm_v, const AttnFwdParams p) {
  using L = AttnSmem<HD>;
  constexpr int PANELS = HD / 64;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  if ((smem_u32(smem) & 1023u) != 0u) {  // the swizzled TMA/MMA layouts need 1024-byte aligned tiles
    if (threadIdx.x == 0) atomicExch(p.status, 9);
    return;
  }
  uint8_t* sQ = smem;
  uint8_t* sK = smem + L::OFF_K;
  uint8_t* sV = smem + L::OFF_V;
  uint8_t* sP = smem + L::OFF_P;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::OFF_BAR);
  uint64_t* q_full = bars;         // 1
  uint64_t* kv_full = bars + 1;    // 2
  uint64_t* kv_empty = bars + 3;   // 2
  uint64_t* bar_s = bars + 5;      // 2
  uint64_t* bar_p = bars + 7;      // 1
  uint64_t* bar_o = bars + 8;      // 1
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 9);
  int* s_tile = reinterpret_cast<int*>(bars + 10);  // seq start token, q0, seqlen, valid

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head = blockIdx.y;
  const int kvh = head / (p.nh / p.nkv);

  if (threadIdx.x == 0) {
    // locate (sequence, query block) of this CTA: tiles are enumerated sequence by sequence
    int t = blockIdx.x, found = 0, start = 0, q0 = 0, len = 0;
    for (int s = 0; s < p.num_seqs; ++s) {
      const int a = p.cu_seqlens[s], b = p.cu_seqlens[s + 1];
      const int nt = (b - a + ATT_BQ - 1) / ATT_BQ;
      if (t < nt) {
        // heavy (late) query blocks first: they have the most key blocks
        start = a; len = b - a; q0 = (nt - 1 - t) * ATT_BQ; found = 1;
        break;
      }
      t -= nt;
    }
    s_tile[0] = start; s_tile[1] = q0; s_tile[2] = len; s_tile[3] = found;
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], 1);
      mbar_init(&bar_s[i], 1);
    }
    mbar_init(bar_p, 4);
    mbar_init(bar_o, 1);
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_holder, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  const int seq_start = s_tile[0], q0 = s_tile[1], seqlen = s_tile[2];
  const bool valid_tile = s_tile[3] != 0;
  const int kv_end = min(q0 + ATT_BQ, seqlen);
  const int nblk = valid_tile ? (kv_end + ATT_BKV - 1) / ATT_BKV : 0;
  constexpr uint32_t TM_S0 = 0, TM_O = 128;

  if (warp == 0) {
    if (lane == 0 && valid_tile) {
      mbar_expect_tx(q_full, L::Q_BYTES);
#pragma unroll
      for (int c = 0; c < PANELS; ++c) tma_load_2d(sQ + c * (ATT_BQ * 128), &tm_q, q_full, head * HD + 64 * c, seq_start + q0);
      for (int j = 0; j < nblk; ++j) {
        const int st = j & 1;
        if (!mbar_wait(&kv_empty[st], ((j >> 1) & 1) ^ 1)) {
          atomicExch(p.status, ST_TIMEOUT_PRODUCER);
          break;
        }
        mbar_expect_tx(&kv_full[st], 2 * L::KV_BYTES);
#pragma unroll
        for (int c = 0; c < PANELS; ++c) {
          tma_load_2d(sK + st * L::KV_BYTES + c * (ATT_BKV * 128), &tm_k, &kv_full[st], kvh * HD + 64 * c, seq_start + j * ATT_BKV);
          tma_load_2d(sV + st * L::KV_BYTES + c * (ATT_BKV * 128), &tm_v, &kv_full[st], kvh * HD + 64 * c, seq_start + j * ATT_BKV);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && valid_tile) {
      constexpr uint32_t idesc_s = make_idesc_f16(ATT_BQ, ATT_BKV, false, false);
      constexpr uint32_t idesc_o = make_idesc_f16(ATT_BQ, HD, false, true);
      bool ok = mbar_wait(q_full, 0);
      auto issue_s = [&](int j) {
        const int st = j & 1;
        if (!mbar_wait(&kv_full[st], (j >> 1) & 1)) return false;
        tc_fence_after();
        const uint32_t aq = smem_u32(sQ), bk = smem_u32(sK + st * L::KV_BYTES);
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint64_t da = make_smem_desc_sw128(aq + (k >> 2) * (ATT_BQ * 128) + (k & 3) * 32, 16, 1024);
          const uint64_t db = make_smem_desc_sw128(bk + (k >> 2) * (ATT_BKV * 128) + (k & 3) * 32, 16, 1024);
          tc_mma_f16_ss(tmem_base + TM_S0 + (j & 1) * ATT_BKV, da, db, idesc_s, k > 0 ? 1u : 0u);
        }
        tc_commit(&bar_s[j & 1]);
        return true;
      };
      if (ok) ok = issue_s(0);
      for (int j = 0; j < nblk && ok; ++j) {
        if (j + 1 < nblk) ok = issue_s(j + 1);
        if (!ok) break;
        if (!mbar_wait(bar_p, j & 1)) { ok = false; break; }
        tc_fence_after();
        const int st = j & 1;
        const uint32_t ap = smem_u32(sP), bv = smem_u32(sV + st * L::KV_BYTES);
#pragma unroll
        for (int k = 0; k < ATT_BKV / 16; ++k) {
          const uint64_t da = make_smem_desc_sw128(ap + k * 32, 16, 1024);
          const uint64_t db = make_smem_desc_sw128(bv + k * 2048, ATT_BKV * 128, 1024);
          tc_mma_f16_ss(tmem_base + TM_O, da, db, idesc_o, (j > 0 || k > 0) ? 1u : 0u);
        }
        tc_commit(&kv_empty[st]);
        tc_commit(bar_o);
      }
      if (!ok) atomicExch(p.status, ST_TIMEOUT_MMA);
    }
  } else if (valid_tile) {
    // ------------------------------------------------------------------ softmax / epilogue
    const int q = warp & 3;
    const int r = q * 32 + lane;          // row inside the tile
    const int row = q0 + r;               // row inside the sequence
    const uint32_t lane_off = static_cast<uint32_t>(q * 32) << 16;
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    for (int j = 0; j < nblk; ++j) {
      if (!mbar_wait(&bar_s[j & 1], (j >> 1) & 1)) { ok = false; break; }
      tc_fence_after();
      uint32_t x0[32], x1[32];
      tmem_ld_32x32(tmem_base + TM_S0 + (j & 1) * ATT_BKV + lane_off, x0);
      tmem_ld_32x32(tmem_base + TM_S0 + (j & 1) * ATT_BKV + 32 + lane_off, x1);
      tmem_ld_wait();
      const int col0 = j * ATT_BKV;
      const bool need_mask = col0 + ATT_BKV - 1 > q0;  // block touches the diagonal of some row of the tile
      float mx = -INFINITY;
#pragma unroll
      for (int c = 0; c < 32; ++c) {
        float a = __uint_as_float(x0[c]) * p.scale_log2, b = __uint_as_float(x1[c]) * p.scale_log2;
        if (need_mask) {
          if (col0 + c > row) a = -INFINITY;
          if (col0 + 32 + c > row) b = -INFINITY;
        }
        x0[c] = __float_as_uint(a);
        x1[c] = __float_as_uint(b);
        mx = fmaxf(mx, fmaxf(a, b));
      }
      const float m_new = fmaxf(m_run, mx);
      const float alpha = (m_new == -INFINITY) ? 1.f : exp2f(m_run - m_new);
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
      float sum = 0.f;
      uint32_t pk[32];
#pragma unroll
      for (int c = 0; c < 32; c += 2) {
        const float a0 = exp2f(__uint_as_float(x0[c]) - m_use), a1 = exp2f(__uint_as_float(x0[c + 1]) - m_use);
        const float b0 = exp2f(__uint_as_float(x1[c]) - m_use), b1 = exp2f(__uint_as_float(x1[c + 1]) - m_use);
        sum += (a0 + a1) + (b0 + b1);
        pk[c >> 1] = pack_bf16x2(a0, a1);
        pk[16 + (c >> 1)] = pack_bf16x2(b0, b1);
      }
      l_run = l_run * alpha + sum;
      m_run = m_new;
      if (j > 0) {
        // P and O are in use by the previous block's P*V until bar_o
        if (!mbar_wait(bar_o, (j - 1) & 1)) { ok = false; break; }
        tc_fence_after();
        if (__any_sync(0xffffffffu, alpha < 1.f)) {
#pragma unroll 1
          for (int c = 0; c < HD / 32; ++c) {
            uint32_t o[32];
            tmem_ld_32x32(tmem_base + TM_O + c * 32 + lane_off, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_32x32(tmem_base + TM_O + c * 32 + lane_off, o);
          }
          tmem_st_wait();
        }
      }
      // P row r: 64 bf16 = 8 chunks of 16 bytes, chunk index XOR (r & 7) (128B swizzle)
      uint8_t* prow = sP + r * 128;
#pragma unroll
      for (int ch = 0; ch < 8; ++ch) {
        const uint4 v = make_uint4(pk[ch * 4], pk[ch * 4 + 1], pk[ch * 4 + 2], pk[ch * 4 + 3]);
        *reinterpret_cast<uint4*>(prow + ((ch ^ (r & 7)) << 4)) = v;
      }
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_p);
    }
    if (ok && nblk > 0) ok = mbar_wait(bar_o, (nblk - 1) & 1);
    if (!ok) {
      if (lane == 0) atomicExch(p.status, ST_TIMEOUT_EPILOGUE);
    } else {
      tc_fence_after();
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      const bool row_ok = row < seqlen;
      const long long tok = static_cast<long long>(seq_start) + row;
#pragma unroll 1
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t o[32];
        tmem_ld_32x32(tmem_base + TM_O + c * 32 + lane_off, o);
        tmem_ld_wait();
        if (row_ok) {
          __nv_bfloat16* dst = p.out + tok * p.ldo + static_cast<long long>(head) * HD + c * 32;
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 v;
            v.x = pack_bf16x2(__uint_as_float(o[i]) * inv, __uint_as_float(o[i + 1]) * inv);
            v.y = pack_bf16x2(__uint_as_float(o[i + 2]) * inv, __uint_as_float(o[i + 3]) * inv);
            v.z = pack_bf16x2(__uint_as_float(o[i + 4]) * inv, __uint_as_float(o[i + 5]) * inv);
            v.w = pack_bf16x2(__uint_as_float(o[i + 6]) * inv, __uint_as_float(o[i + 7]) * inv);
            *reinterpret_cast<uint4*>(dst + i) = v;
          }
        }
      }
      if (row_ok && p.lse != nullptr)
        p.lse[static_cast<long long>(head) * p.total_tokens + tok] = (m_run + log2f(l_run)) * 0.6931471805599453f;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 256);
  }
}

__device__ int g_attn_status[4];

template <int HD>
static cudaError_t launch_attn_fwd(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                                   const AttnFwdParams& p, int max_tiles, cudaStream_t stream) {
  auto kern = attn_fwd_kernel<HD>;
  constexpr int smem = AttnSmem<HD>::TOTAL;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    configured = true;
  }
  dim3 grid(max_tiles, p.nh);
  kern<<<grid, ATT_THREADS, smem, stream>>>(tq, tk, tv, p);
  return cudaGetLastError();
}

}  // namespace vb

using namespace vb;

// q: [T, nh, hd] view (row stride ldq elements), k/v: [T, nkv, hd] views. max_seqlen bounds nothing here; the tile
// count upper bound T/128 + num_seqs is used for the grid so no host copy of cu_seqlens is needed.
extern "C" int vb_attn_fwd(const void* q, const void* k, const void* v, long long ldq, long long ldk, long long ldv,
                           const int* cu_seqlens, int num_seqs, int total_tokens, int nh, int nkv, int hd, float scale,
                           void* out, long long ldo, float* lse, cudaStream_t stream) {
  if (total_tokens <= 0 || num_seqs <= 0) return 0;
  if (hd != 64 && hd != 128) return -2;
  if ((ldq % 8) || (ldk % 8) || (ldv % 8) || (ldo % 8) || (nh % nkv)) return -1;
  CUtensorMap tq, tk, tv;
  const auto bf = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  if (!make_tmap_2d(&tq, q, bf, 2, total_tokens, (uint64_t)nh * hd, ldq, 64, ATT_BQ, CU_TENSOR_MAP_SWIZZLE_128B)) return -3;
  if (!make_tmap_2d(&tk, k, bf, 2, total_tokens, (uint64_t)nkv * hd, ldk, 64, ATT_BKV, CU_TENSOR_MAP_SWIZZLE_128B)) return -3;
  if (!make_tmap_2d(&tv, v, bf, 2, total_tokens, (uint64_t)nkv * hd, ldv, 64, ATT_BKV, CU_TENSOR_MAP_SWIZZLE_128B)) return -3;
  static int* status = nullptr;
  if (status == nullptr) cudaGetSymbolAddress(reinterpret_cast<void**>(&status), g_attn_status);
  AttnFwdParams p{};
  p.cu_seqlens = cu_seqlens; p.num_seqs = num_seqs; p.nh = nh; p.nkv = nkv;
  p.out = reinterpret_cast<__nv_bfloat16*>(out); p.ldo = ldo; p.lse = lse; p.total_tokens = total_tokens;
  p.scale_log2 = scale * 1.4426950408889634f; p.status = status;
  const int max_tiles = (total_tokens + ATT_BQ - 1) / ATT_BQ + num_seqs;
  cudaError_t e = (hd == 128) ? launch_attn_fwd<128>(tq, tk, tv, p, max_tiles, stream)
                              : launch_attn_fwd<64>(tq, tk, tv, p, max_tiles, stream);
  return static_cast<int>(e);
}

extern "C" int vb_attn_status() {
  int h[4] = {0, 0, 0, 0};
  if (cudaMemcpyFromSymbol(h, g_attn_status, sizeof(h)) != cudaSuccess) return -1;
  if (h[0] != 0) {
    int z[4] = {0, 0, 0, 0};
    cudaMemcpyToSymbol(g_attn_status, z, sizeof(z));
  }
  return h[0];
}
