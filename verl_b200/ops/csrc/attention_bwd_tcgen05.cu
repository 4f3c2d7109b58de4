// Causal GQA attention backward over packed (varlen) sequences on tcgen05 tensor cores (head_dim 128).
//
// One CTA = one (sequence, block of 128 keys, KV head). K and V of the block stay in shared memory and dK, dV stay in
// TMEM for the whole CTA, which walks over every query head of the GQA group and every block of 64 queries at or
// below the diagonal. Everything is computed in the transposed frame so that the 128 keys are the M (TMEM lane)
// dimension and softmax threads own one key row each:
//
//   S^T  = K  Q^T            [128 keys, 64 q]   A = K  (K-major)     B = Q  (K-major)
//   dP^T = V  dO^T           [128 keys, 64 q]   A = V  (K-major)     B = dO (K-major)
//   P^T  = exp2(S^T * c - lse2[q]) (causal),   dS^T = P^T o (dP^T - D[q]) * scale          -> bf16, shared memory
//   dV  += P^T  dO           [128 keys, hd]     A = P^T  (K-major)   B = dO (MN-major)       TMEM-resident
//   dK  += dS^T Q            [128 keys, hd]     A = dS^T (K-major)   B = Q  (MN-major)       TMEM-resident
//   dQ^T = K^T dS^T          [hd, 64 q]         A = K  (MN-major)    B = dS^T (MN-major)     -> fp32 atomics into dQ
//
//   warp 0      TMA: K, V once; Q and dO tiles through a 2-stage ring
//   warp 1      MMA issue (one elected thread)
//   warps 2..5  thread == key row: tcgen05.ld S^T / dP^T -> P^T, dS^T -> swizzled shared memory; drain dQ^T with
//               coalesced red.add (lanes = 32 consecutive head-dim elements of one query); final dK / dV store
// D[q] = sum_d dO[q,d] O[q,d] comes from a small pre-pass; dQ is accumulated in fp32 and converted afterwards.
#include "tcgen05_common.cuh"

#include <math.h>

namespace vb {

constexpr int AB_BK = 128;  // keys per CTA
constexpr int AB_BQ = 64;   // queries per step
constexpr int AB_THREADS = 192;

struct AttnBwdParams {
  const int* cu_seqlens;
  int num_seqs, nh, nkv, total_tokens;
  const float* lse;    // [nh, T] natural log
  const float* delta;  // [nh, T]
  float* dq32;         // [T, nh*hd] fp32, zero on entry
  __nv_bfloat16* dk;   // [T, nkv*hd] (row stride lddk)
  __nv_bfloat16* dv;
  long long lddk, lddv;
  float scale, scale_log2;
  int* status;
};

template <int HD>
struct AttnBwdSmem {
  static constexpr int KV_BYTES = AB_BK * HD * 2;   // 32 KB each
  static constexpr int QO_BYTES = AB_BQ * HD * 2;   // 16 KB each, per stage
  static constexpr int PS_BYTES = AB_BK * AB_BQ * 2;  // 16 KB each
  static constexpr int OFF_K = 0;
  static constexpr int OFF_V = OFF_K + KV_BYTES;
  static constexpr int OFF_Q = OFF_V + KV_BYTES;          // 2 stages
  static constexpr int OFF_DO = OFF_Q + 2 * QO_BYTES;     // 2 stages
  static constexpr int OFF_P = OFF_DO + 2 * QO_BYTES;
  static constexpr int OFF_DS = OFF_P + PS_BYTES;
  static constexpr int OFF_VEC = OFF_DS + PS_BYTES;       // per softmax warp: [2 steps][lse2 | delta][64] fp32
  static constexpr int OFF_BAR = OFF_VEC + 4 * 2 * 2 * AB_BQ * 4;
  static constexpr int TOTAL = OFF_BAR + 128 + 1024;
};

template <int HD>
__global__ void __launch_bounds__(AB_THREADS, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
                const AttnBwdParams p) {
  using L = AttnBwdSmem<HD>;
  constexpr int PANELS = HD / 64;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem + L::OFF_K;
  uint8_t* sV = smem + L::OFF_V;
  uint8_t* sQ = smem + L::OFF_Q;
  uint8_t* sDO = smem + L::OFF_DO;
  uint8_t* sP = smem + L::OFF_P;
  uint8_t* sDS = smem + L::OFF_DS;
  float* sVec = reinterpret_cast<float*>(smem + L::OFF_VEC);  // [4 warps][2 steps][lse2 | delta][64]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::OFF_BAR);
  uint64_t* kv_full = bars;        // 1
  uint64_t* qdo_full = bars + 1;   // 2
  uint64_t* qdo_empty = bars + 3;  // 2
  uint64_t* bar_sdp = bars + 5;    // S^T, dP^T ready
  uint64_t* bar_pds = bars + 6;    // P^T, dS^T written (4 warps)
  uint64_t* bar_dq = bars + 7;     // dV, dK, dQ^T MMAs of a step done
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 8);
  __shared__ int s_tile[4];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kvh = blockIdx.y;
  const int G = p.nh / p.nkv;

  if (threadIdx.x == 0) {
    int t = blockIdx.x, found = 0, start = 0, k0 = 0, len = 0;
    for (int s = 0; s < p.num_seqs; ++s) {
      const int a = p.cu_seqlens[s], b = p.cu_seqlens[s + 1];
      const int nt = (b - a + AB_BK - 1) / AB_BK;
      if (t < nt) {
        start = a; len = b - a; k0 = t * AB_BK; found = 1;  // early key blocks (most query blocks) come first
        break;
      }
      t -= nt;
    }
    s_tile[0] = start; s_tile[1] = k0; s_tile[2] = len; s_tile[3] = found;
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
    tma_prefetch_desc(&tm_do);
    mbar_init(kv_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&qdo_full[i], 1);
      mbar_init(&qdo_empty[i], 1);
    }
    mbar_init(bar_sdp, 1);
    mbar_init(bar_pds, 4);
    mbar_init(bar_dq, 1);
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_holder, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  const int seq_start = s_tile[0], k0 = s_tile[1], seqlen = s_tile[2];
  const bool valid_tile = s_tile[3] != 0;
  const int i0 = k0 / AB_BQ;                                    // first query block at or below the diagonal
  const int nqb = valid_tile ? (seqlen + AB_BQ - 1) / AB_BQ : 0;
  const int per_head = valid_tile ? nqb - i0 : 0;
  const int n_it = per_head * G;
  constexpr uint32_t TM_DV = 0, TM_DK = HD, TM_S = 2 * HD, TM_DP = 2 * HD + AB_BQ, TM_DQ = 2 * HD + 2 * AB_BQ;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0 && n_it > 0) {
      mbar_expect_tx(kv_full, 2 * L::KV_BYTES);
#pragma unroll
      for (int c = 0; c < PANELS; ++c) {
        tma_load_2d(sK + c * (AB_BK * 128), &tm_k, kv_full, kvh * HD + 64 * c, seq_start + k0);
        tma_load_2d(sV + c * (AB_BK * 128), &tm_v, kv_full, kvh * HD + 64 * c, seq_start + k0);
      }
      for (int it = 0; it < n_it; ++it) {
        const int st = it & 1;
        if (!mbar_wait(&qdo_empty[st], ((it >> 1) & 1) ^ 1)) {
          atomicExch(p.status, ST_TIMEOUT_PRODUCER);
          break;
        }
        const int head = kvh * G + it / per_head;
        const int q0 = (i0 + it % per_head) * AB_BQ;
        mbar_expect_tx(&qdo_full[st], 2 * L::QO_BYTES);
#pragma unroll
        for (int c = 0; c < PANELS; ++c) {
          tma_load_2d(sQ + st * L::QO_BYTES + c * (AB_BQ * 128), &tm_q, &qdo_full[st], head * HD + 64 * c, seq_start + q0);
          tma_load_2d(sDO + st * L::QO_BYTES + c * (AB_BQ * 128), &tm_do, &qdo_full[st], head * HD + 64 * c, seq_start + q0);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && n_it > 0) {
      constexpr uint32_t idesc_s = make_idesc_f16(AB_BK, AB_BQ, false, false);   // S^T, dP^T
      constexpr uint32_t idesc_kv = make_idesc_f16(AB_BK, HD, false, true);      // dV, dK
      constexpr uint32_t idesc_dq = make_idesc_f16(HD, AB_BQ, true, true);       // dQ^T (M = hd = 128)
      const uint32_t aK = smem_u32(sK), aV = smem_u32(sV), aP = smem_u32(sP), aDS = smem_u32(sDS);
      auto issue_sdp = [&](int it) {
        const int st = it & 1;
        if (!mbar_wait(&qdo_full[st], (it >> 1) & 1)) return false;
        tc_fence_after();
        const uint32_t bQ = smem_u32(sQ + st * L::QO_BYTES), bDO = smem_u32(sDO + st * L::QO_BYTES);
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint64_t da = make_smem_desc_sw128(aK + (k >> 2) * (AB_BK * 128) + (k & 3) * 32, 16, 1024);
          const uint64_t db = make_smem_desc_sw128(bQ + (k >> 2) * (AB_BQ * 128) + (k & 3) * 32, 16, 1024);
          tc_mma_f16_ss(tmem_base + TM_S, da, db, idesc_s, k > 0 ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint64_t da = make_smem_desc_sw128(aV + (k >> 2) * (AB_BK * 128) + (k & 3) * 32, 16, 1024);
          const uint64_t db = make_smem_desc_sw128(bDO + (k >> 2) * (AB_BQ * 128) + (k & 3) * 32, 16, 1024);
          tc_mma_f16_ss(tmem_base + TM_DP, da, db, idesc_s, k > 0 ? 1u : 0u);
        }
        tc_commit(bar_sdp);
        return true;
      };
      bool ok = mbar_wait(kv_full, 0);
      if (ok) ok = issue_sdp(0);
      for (int it = 0; it < n_it && ok; ++it) {
        if (!mbar_wait(bar_pds, it & 1)) { ok = false; break; }
        tc_fence_after();
        if (it + 1 < n_it) ok = issue_sdp(it + 1);  // S^T/dP^T columns are free: the softmax of `it` has read them
        if (!ok) break;
        const int st = it & 1;
        const uint32_t bQ = smem_u32(sQ + st * L::QO_BYTES), bDO = smem_u32(sDO + st * L::QO_BYTES);
#pragma unroll
        for (int k = 0; k < AB_BQ / 16; ++k) {  // contraction over the 64 queries of the step
          const uint64_t dp = make_smem_desc_sw128(aP + k * 32, 16, 1024);
          const uint64_t dds = make_smem_desc_sw128(aDS + k * 32, 16, 1024);
          const uint64_t bdo = make_smem_desc_sw128(bDO + k * 2048, AB_BQ * 128, 1024);
          const uint64_t bq = make_smem_desc_sw128(bQ + k * 2048, AB_BQ * 128, 1024);
          tc_mma_f16_ss(tmem_base + TM_DV, dp, bdo, idesc_kv, (it > 0 || k > 0) ? 1u : 0u);
          tc_mma_f16_ss(tmem_base + TM_DK, dds, bq, idesc_kv, (it > 0 || k > 0) ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < AB_BK / 16; ++k) {  // contraction over the 128 keys
          const uint64_t da = make_smem_desc_sw128(aK + k * 2048, AB_BK * 128, 1024);
          const uint64_t db = make_smem_desc_sw128(aDS + k * 2048, AB_BK * 128, 1024);
          tc_mma_f16_ss(tmem_base + TM_DQ, da, db, idesc_dq, k > 0 ? 1u : 0u);
        }
        tc_commit(&qdo_empty[st]);
        tc_commit(bar_dq);
      }
      if (!ok) atomicExch(p.status, ST_TIMEOUT_MMA);
    }
  } else if (n_it > 0) {
    // ------------------------------------------------------------------ softmax backward / drains (thread == key row)
    const int q = warp & 3;
    const int r = q * 32 + lane;
    const int key = k0 + r;  // key index inside the sequence; also the head-dim index when draining dQ^T
    const uint32_t lane_off = static_cast<uint32_t>(q * 32) << 16;
    bool ok = true;
    constexpr float LOG2E = 1.4426950408889634f;

    auto drain_dq = [&](int it) {
      const int head = kvh * G + it / per_head;
      const int q0 = (i0 + it % per_head) * AB_BQ;
      float* base = p.dq32 + static_cast<long long>(seq_start + q0) * (static_cast<long long>(p.nh) * HD) +
                    static_cast<long long>(head) * HD + r;
#pragma unroll 1
      for (int c = 0; c < AB_BQ / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(tmem_base + TM_DQ + c * 32 + lane_off, v);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          if (q0 + c * 32 + j < seqlen)
            atomicAdd(base + static_cast<long long>(c * 32 + j) * (static_cast<long long>(p.nh) * HD), __uint_as_float(v[j]));
        }
      }
    };

    for (int it = 0; it < n_it && ok; ++it) {
      const int head = kvh * G + it / per_head;
      const int q0 = (i0 + it % per_head) * AB_BQ;
      // stage lse (log2 domain) and delta of the 64 queries of this step: every warp keeps its own copy, so no
      // barrier across warps is needed (a warp that gave up on a wait cannot leave the others stuck)
      float* vL = sVec + ((q * 2 + (it & 1)) * 2) * AB_BQ;
      float* vD = vL + AB_BQ;
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int c = lane + 32 * u;
        float l2 = 0.f, de = 0.f;
        if (q0 + c < seqlen) {
          const long long o = static_cast<long long>(head) * p.total_tokens + seq_start + q0 + c;
          l2 = p.lse[o] * LOG2E;
          de = p.delta[o];
        }
        vL[c] = l2;
        vD[c] = de;
      }
      __syncwarp();
      if (!mbar_wait(bar_sdp, it & 1)) { ok = false; break; }
      tc_fence_after();
      uint32_t pk[32], dk[32];  // packed bf16 pairs of P^T and dS^T for this key row (64 queries)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        uint32_t s[32], dp[32];
        tmem_ld_32x32(tmem_base + TM_S + h * 32 + lane_off, s);
        tmem_ld_32x32(tmem_base + TM_DP + h * 32 + lane_off, dp);
        tmem_ld_wait();
#pragma unroll
        for (int c = 0; c < 32; c += 2) {
          float pv[2], dsv[2];
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            const int col = h * 32 + c + u;
            const int qi = q0 + col;
            const bool live = (key <= qi) && (qi < seqlen);
            const float pe = live ? exp2f(__uint_as_float(s[c + u]) * p.scale_log2 - vL[col]) : 0.f;
            pv[u] = pe;
            dsv[u] = pe * (__uint_as_float(dp[c + u]) - vD[col]) * p.scale;
          }
          pk[h * 16 + (c >> 1)] = pack_bf16x2(pv[0], pv[1]);
          dk[h * 16 + (c >> 1)] = pack_bf16x2(dsv[0], dsv[1]);
        }
      }
      tc_fence_before();
      if (it > 0) {
        // P^T / dS^T buffers and the dQ^T columns are still in use by the MMAs of the previous step
        if (!mbar_wait(bar_dq, (it - 1) & 1)) { ok = false; break; }
        tc_fence_after();
        drain_dq(it - 1);
      }
      uint8_t* prow = sP + r * 128;
      uint8_t* drow = sDS + r * 128;
#pragma unroll
      for (int ch = 0; ch < 8; ++ch) {
        const int sw = (ch ^ (r & 7)) << 4;
        *reinterpret_cast<uint4*>(prow + sw) = make_uint4(pk[ch * 4], pk[ch * 4 + 1], pk[ch * 4 + 2], pk[ch * 4 + 3]);
        *reinterpret_cast<uint4*>(drow + sw) = make_uint4(dk[ch * 4], dk[ch * 4 + 1], dk[ch * 4 + 2], dk[ch * 4 + 3]);
      }
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_pds);
    }
    if (ok) ok = mbar_wait(bar_dq, (n_it - 1) & 1);
    if (!ok) {
      if (lane == 0) atomicExch(p.status, ST_TIMEOUT_EPILOGUE);
    } else {
      tc_fence_after();
      drain_dq(n_it - 1);
      // dK, dV of this key block: exclusive to this CTA, plain stores (the TMEM loads are warp-wide, the stores are
      // predicated on the key being inside the sequence)
      const bool key_ok = key < seqlen;
      const long long tok = static_cast<long long>(seq_start) + key;
#pragma unroll 1
      for (int which = 0; which < 2; ++which) {
        __nv_bfloat16* dst = (which == 0 ? p.dv + tok * p.lddv : p.dk + tok * p.lddk) + static_cast<long long>(kvh) * HD;
#pragma unroll 1
        for (int c = 0; c < HD / 32; ++c) {
          uint32_t o[32];
          tmem_ld_32x32(tmem_base + (which == 0 ? TM_DV : TM_DK) + c * 32 + lane_off, o);
          tmem_ld_wait();
          if (key_ok) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              uint4 v;
              v.x = pack_bf16x2(__uint_as_float(o[i]), __uint_as_float(o[i + 1]));
              v.y = pack_bf16x2(__uint_as_float(o[i + 2]), __uint_as_float(o[i + 3]));
              v.z = pack_bf16x2(__uint_as_float(o[i + 4]), __uint_as_float(o[i + 5]));
              v.w = pack_bf16x2(__uint_as_float(o[i + 6]), __uint_as_float(o[i + 7]));
              *reinterpret_cast<uint4*>(dst + c * 32 + i) = v;
            }
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// delta[h, t] = sum_d dO[t, h, d] * O[t, h, d]; one warp per (token, head)
__global__ void attn_bwd_delta_kernel(const __nv_bfloat16* __restrict__ dout, long long lddo,
                                      const __nv_bfloat16* __restrict__ out, long long ldo, float* __restrict__ delta,
                                      int T, int nh, int hd) {
  const long long w = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= static_cast<long long>(T) * nh) return;
  const int t = static_cast<int>(w / nh), h = static_cast<int>(w % nh);
  const __nv_bfloat16* a = dout + static_cast<long long>(t) * lddo + static_cast<long long>(h) * hd;
  const __nv_bfloat16* b = out + static_cast<long long>(t) * ldo + static_cast<long long>(h) * hd;
  float s = 0.f;
  for (int d = lane * 2; d < hd; d += 64) {
    const float2 x = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(a + d));
    const float2 y = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(b + d));
    s += x.x * y.x + x.y * y.y;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (lane == 0) delta[static_cast<long long>(h) * T + t] = s;
}

// dq (bf16, row stride lddq) = dq32 (fp32 [T, nh*hd])
__global__ void attn_bwd_dq_cast_kernel(const float* __restrict__ dq32, __nv_bfloat16* __restrict__ dq, long long lddq,
                                        int T, int width) {
  const long long i4 = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  const long long per_row = width / 4;
  if (i4 >= static_cast<long long>(T) * per_row) return;
  const long long t = i4 / per_row, c = (i4 % per_row) * 4;
  const float4 v = *reinterpret_cast<const float4*>(dq32 + t * width + c);
  uint2 o;
  o.x = pack_bf16x2(v.x, v.y);
  o.y = pack_bf16x2(v.z, v.w);
  *reinterpret_cast<uint2*>(dq + t * lddq + c) = o;
}

__device__ int g_attn_bwd_status[4];

}  // namespace vb

using namespace vb;

// Workspace (caller-provided, any content): delta [nh*T] fp32 and dq32 [T*nh*hd] fp32 (zeroed here).
// q/dout/out: [T, nh, hd] views, k/v: [T, nkv, hd] views; dq/dk/dv are written with their own row strides.
extern "C" int vb_attn_bwd(const void* q, const void* k, const void* v, const void* out, const void* dout, long long ldq,
                           long long ldk, long long ldv, long long ldo, long long lddo, const float* lse,
                           const int* cu_seqlens, int num_seqs, int total_tokens, int nh, int nkv, int hd, float scale,
                           void* dq, void* dk, void* dv, long long lddq, long long lddk, long long lddv, float* delta_ws,
                           float* dq32_ws, cudaStream_t stream) {
  if (total_tokens <= 0 || num_seqs <= 0) return 0;
  if (hd != 128) return -2;
  if ((ldq % 8) || (ldk % 8) || (ldv % 8) || (ldo % 8) || (lddo % 8) || (lddq % 8) || (lddk % 8) || (lddv % 8) || (nh % nkv)) return -1;
  CUtensorMap tq, tk, tv, tdo;
  const auto bf = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  if (!make_tmap_2d(&tq, q, bf, 2, total_tokens, (uint64_t)nh * hd, ldq, 64, AB_BQ, CU_TENSOR_MAP_SWIZZLE_128B)) return -3;
  if (!make_tmap_2d(&tdo, dout, bf, 2, total_tokens, (uint64_t)nh * hd, lddo, 64, AB_BQ, CU_TENSOR_MAP_SWIZZLE_128B)) return -3;
  if (!make_tmap_2d(&tk, k, bf, 2, total_tokens, (uint64_t)nkv * hd, ldk, 64, AB_BK, CU_TENSOR_MAP_SWIZZLE_128B)) return -3;
  if (!make_tmap_2d(&tv, v, bf, 2, total_tokens, (uint64_t)nkv * hd, ldv, 64, AB_BK, CU_TENSOR_MAP_SWIZZLE_128B)) return -3;
  static int* status = nullptr;
  if (status == nullptr) cudaGetSymbolAddress(reinterpret_cast<void**>(&status), g_attn_bwd_status);
  const long long warps = static_cast<long long>(total_tokens) * nh;
  attn_bwd_delta_kernel<<<static_cast<int>((warps * 32 + 255) / 256), 256, 0, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(dout), lddo, reinterpret_cast<const __nv_bfloat16*>(out), ldo, delta_ws,
      total_tokens, nh, hd);
  cudaError_t e = cudaMemsetAsync(dq32_ws, 0, sizeof(float) * static_cast<size_t>(total_tokens) * nh * hd, stream);
  if (e != cudaSuccess) return static_cast<int>(e);
  AttnBwdParams p{};
  p.cu_seqlens = cu_seqlens; p.num_seqs = num_seqs; p.nh = nh; p.nkv = nkv; p.total_tokens = total_tokens;
  p.lse = lse; p.delta = delta_ws; p.dq32 = dq32_ws;
  p.dk = reinterpret_cast<__nv_bfloat16*>(dk); p.dv = reinterpret_cast<__nv_bfloat16*>(dv);
  p.lddk = lddk; p.lddv = lddv; p.scale = scale; p.scale_log2 = scale * 1.4426950408889634f; p.status = status;
  auto kern = attn_bwd_kernel<128>;
  constexpr int smem = AttnBwdSmem<128>::TOTAL;
  static bool configured = false;
  if (!configured) {
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  dim3 grid((total_tokens + AB_BK - 1) / AB_BK + num_seqs, nkv);
  kern<<<grid, AB_THREADS, smem, stream>>>(tq, tk, tv, tdo, p);
  e = cudaGetLastError();
  if (e != cudaSuccess) return static_cast<int>(e);
  const long long n4 = static_cast<long long>(total_tokens) * nh * hd / 4;
  attn_bwd_dq_cast_kernel<<<static_cast<int>((n4 + 255) / 256), 256, 0, stream>>>(
      dq32_ws, reinterpret_cast<__nv_bfloat16*>(dq), lddq, total_tokens, nh * hd);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int vb_attn_bwd_status() {
  int h[4] = {0, 0, 0, 0};
  if (cudaMemcpyFromSymbol(h, g_attn_bwd_status, sizeof(h)) != cudaSuccess) return -1;
  if (h[0] != 0) {
    int z[4] = {0, 0, 0, 0};
    cudaMemcpyToSymbol(g_attn_bwd_status, z, sizeof(z));
  }
  return h[0];
}
