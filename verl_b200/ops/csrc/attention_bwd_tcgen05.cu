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
// dQ^T has two TMEM buffers: the atomics of step i run after the softmax warps have handed P^T / dS^T of step i + 1 to
// the MMA warp, i.e. under the tensor-core work of step i + 1 instead of in front of it.
// Grid = (KV head, sequence, key block counted from the END of the sequence, longest first): blocks are handed out in
// order of decreasing work (the first key block meets every query block, the last one only its own), which keeps the
// tail of the launch short.
//
//   warp 0      TMA: K, V once; Q and dO tiles through a 2-stage ring
//   warp 1      MMA issue (one elected thread)
//   warps 2..9  two threads per key row (32 of the step's 64 queries each): tcgen05.ld S^T / dP^T -> P^T, dS^T ->
//               swizzled shared memory; drain dQ^T with coalesced red.add (lanes = 32 consecutive head-dim elements of
//               one query); final dV (warps 2..5) / dK (warps 6..9) store
// D[q] = sum_d dO[q,d] O[q,d] comes from a small pre-pass; dQ is accumulated in fp32 and converted afterwards.
#include "tcgen05_common.cuh"

#include <math.h>

namespace vb {

constexpr int AB_BK = 128;  // keys per CTA
constexpr int AB_BQ = 64;   // queries per step
constexpr int AB_THREADS = 320;  // TMA warp, MMA warp, eight softmax warps

struct AttnBwdParams {
  const int* cu_seqlens;
  int num_seqs, nh, nkv, total_tokens, max_tiles;  // max_tiles: key blocks of the longest sequence
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
  static constexpr int OFF_VEC = OFF_DS + PS_BYTES;       // per softmax warp (8): [2 steps][lse2 | delta][32] fp32
  static constexpr int OFF_BAR = OFF_VEC + 8 * 2 * 2 * 32 * 4;
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
  float* sVec = reinterpret_cast<float*>(smem + L::OFF_VEC);  // [8 warps][2 steps][lse2 | delta][32]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::OFF_BAR);
  uint64_t* kv_full = bars;        // 1
  uint64_t* qdo_full = bars + 1;   // 2
  uint64_t* qdo_empty = bars + 3;  // 2
  uint64_t* bar_sdp = bars + 5;    // S^T, dP^T ready
  uint64_t* bar_pds = bars + 6;    // P^T, dS^T written (4 warps)
  uint64_t* bar_dq = bars + 7;     // dV, dK, dQ^T MMAs of a step done
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kvh = blockIdx.x;
  const int G = p.nh / p.nkv;
  const int seq_start = p.cu_seqlens[blockIdx.y];
  const int seqlen = p.cu_seqlens[blockIdx.y + 1] - seq_start;
  const int from_end = p.max_tiles - 1 - static_cast<int>(blockIdx.z);
  const int ntiles = (seqlen + AB_BK - 1) / AB_BK;
  if (from_end >= ntiles) return;  // shorter sequence: uniform over the CTA, nothing allocated yet
  if (ntiles > p.max_tiles && blockIdx.z == 0 && threadIdx.x == 0) atomicExch(p.status, ST_BAD_ARGS);  // max_seqlen too small
  const int k0 = (ntiles - 1 - from_end) * AB_BK;

  if (threadIdx.x == 0) {
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
    mbar_init(bar_pds, 8);
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
  const int i0 = k0 / AB_BQ;                                    // first query block at or below the diagonal
  const int nqb = (seqlen + AB_BQ - 1) / AB_BQ;
  const int per_head = nqb - i0;
  const int n_it = per_head * G;
  constexpr uint32_t TM_DV = 0, TM_DK = HD, TM_S = 2 * HD, TM_DP = 2 * HD + AB_BQ, TM_DQ = 2 * HD + 2 * AB_BQ;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
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
          tc_mma_f16_ss(tmem_base + TM_DQ + (it & 1) * AB_BQ, da, db, idesc_dq, k > 0 ? 1u : 0u);
        }
        tc_commit(&qdo_empty[st]);
        tc_commit(bar_dq);
      }
      if (!ok) atomicExch(p.status, ST_TIMEOUT_MMA);
    }
  } else if (n_it > 0) {
    // ------------------------------------------------------------------ softmax backward / drains
    // Eight warps: warp w serves TMEM lane quarter w % 4 (thread == key row) and the query columns of half (w - 2) / 4,
    // so every key row is shared by two threads that never need each other's values.
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;   // 0: query columns 0..31 of the step, 1: columns 32..63
    const int r = q * 32 + lane;
    const int key = k0 + r;  // key index inside the sequence; also the head-dim index when draining dQ^T
    const uint32_t lane_off = static_cast<uint32_t>(q * 32) << 16;
    const int cbase = half * 32;
    bool ok = true;
    constexpr float LOG2E = 1.4426950408889634f;

    auto drain_dq = [&](int it) {
      const int head = kvh * G + it / per_head;
      const int q0 = (i0 + it % per_head) * AB_BQ + cbase;
      const long long row_stride = static_cast<long long>(p.nh) * HD;
      float* base = p.dq32 + static_cast<long long>(seq_start + q0) * row_stride + static_cast<long long>(head) * HD + r;
      uint32_t v[32];
      tmem_ld_32x32(tmem_base + TM_DQ + (it & 1) * AB_BQ + cbase + lane_off, v);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        if (q0 + j < seqlen) atomicAdd(base + j * row_stride, __uint_as_float(v[j]));
      }
    };

    // lse (log2 domain) and delta of this warp's 32 queries of a step, one query per lane; fetched one step ahead
    float nl2 = 0.f, nde = 0.f;
    auto fetch_vec = [&](int it) {
      const int qi = (i0 + it % per_head) * AB_BQ + cbase + lane;
      nl2 = 0.f;
      nde = 0.f;
      if (it < n_it && qi < seqlen) {
        const long long o = static_cast<long long>(kvh * G + it / per_head) * p.total_tokens + seq_start + qi;
        nl2 = p.lse[o] * LOG2E;
        nde = p.delta[o] * p.scale;
      }
    };
    fetch_vec(0);
    for (int it = 0; it < n_it && ok; ++it) {
      const int q0 = (i0 + it % per_head) * AB_BQ;
      // a private copy per warp, so no barrier across warps is needed (a warp that gave up on a wait cannot leave the
      // others stuck)
      float* vL = sVec + (((warp - 2) * 2 + (it & 1)) * 2) * 32;
      float* vD = vL + 32;
      vL[lane] = nl2;
      vD[lane] = nde;
      __syncwarp();
      fetch_vec(it + 1);
      if (!mbar_wait(bar_sdp, it & 1)) { ok = false; break; }
      tc_fence_after();
      uint32_t pk[16], dk[16];  // packed bf16 pairs of P^T and dS^T: this key row, this warp's 32 queries
      {
        uint32_t s[32], dp[32];
        tmem_ld_32x32(tmem_base + TM_S + cbase + lane_off, s);
        tmem_ld_32x32(tmem_base + TM_DP + cbase + lane_off, dp);
        tmem_ld_wait();
        // only the blocks on the diagonal and the last (partial) query block of the sequence need the mask
        const bool masked = (q0 < k0 + AB_BK) || (q0 + AB_BQ > seqlen);
        const float4* vL4 = reinterpret_cast<const float4*>(vL);
        const float4* vD4 = reinterpret_cast<const float4*>(vD);
#pragma unroll
        for (int c = 0; c < 32; c += 4) {
          const float4 l4 = vL4[c >> 2], d4 = vD4[c >> 2];
          const float lv[4] = {l4.x, l4.y, l4.z, l4.w}, dv_[4] = {d4.x, d4.y, d4.z, d4.w};
          float pv[4], dsv[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            float pe = exp2f(fmaf(__uint_as_float(s[c + u]), p.scale_log2, -lv[u]));
            if (masked) {
              const int qi = q0 + cbase + c + u;
              if (!((key <= qi) && (qi < seqlen))) pe = 0.f;
            }
            pv[u] = pe;
            dsv[u] = pe * fmaf(__uint_as_float(dp[c + u]), p.scale, -dv_[u]);  // delta is stored pre-multiplied by scale
          }
          pk[c >> 1] = pack_bf16x2(pv[0], pv[1]);
          pk[(c >> 1) + 1] = pack_bf16x2(pv[2], pv[3]);
          dk[c >> 1] = pack_bf16x2(dsv[0], dsv[1]);
          dk[(c >> 1) + 1] = pack_bf16x2(dsv[2], dsv[3]);
        }
      }
      tc_fence_before();
      if (it > 0) {
        // the P^T / dS^T buffers are still read by the MMAs of the previous step
        if (!mbar_wait(bar_dq, (it - 1) & 1)) { ok = false; break; }
        tc_fence_after();
      }
      uint8_t* prow = sP + r * 128;
      uint8_t* drow = sDS + r * 128;
#pragma unroll
      for (int c4 = 0; c4 < 4; ++c4) {  // this warp's four 16-byte chunks of the 128-byte row
        const int sw = ((half * 4 + c4) ^ (r & 7)) << 4;
        *reinterpret_cast<uint4*>(prow + sw) = make_uint4(pk[c4 * 4], pk[c4 * 4 + 1], pk[c4 * 4 + 2], pk[c4 * 4 + 3]);
        *reinterpret_cast<uint4*>(drow + sw) = make_uint4(dk[c4 * 4], dk[c4 * 4 + 1], dk[c4 * 4 + 2], dk[c4 * 4 + 3]);
      }
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_pds);
      if (it > 0) {
        // dQ^T of the previous step sits in the other TMEM buffer; its next writer is the MMA of step it + 1, which
        // waits for this warp's next arrival
        drain_dq(it - 1);
        tc_fence_before();
      }
    }
    if (ok) ok = mbar_wait(bar_dq, (n_it - 1) & 1);
    if (!ok) {
      if (lane == 0) atomicExch(p.status, ST_TIMEOUT_EPILOGUE);
    } else {
      tc_fence_after();
      drain_dq(n_it - 1);
      // dV (first four warps) and dK (last four) of this key block: exclusive to this CTA, plain stores; the TMEM loads
      // are warp-wide, the stores are predicated on the key being inside the sequence
      const bool key_ok = key < seqlen;
      const long long tok = static_cast<long long>(seq_start) + key;
      __nv_bfloat16* dst = (half == 0 ? p.dv + tok * p.lddv : p.dk + tok * p.lddk) + static_cast<long long>(kvh) * HD;
#pragma unroll 1
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t o[32];
        tmem_ld_32x32(tmem_base + (half == 0 ? TM_DV : TM_DK) + c * 32 + lane_off, o);
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
                           float* dq32_ws, int max_seqlen, cudaStream_t stream) {
  if (total_tokens <= 0 || num_seqs <= 0) return 0;
  if (max_seqlen <= 0 || num_seqs > 65535) return -4;
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
  p.max_tiles = (max_seqlen + AB_BK - 1) / AB_BK;
  if (p.max_tiles > 65535) return -4;
  dim3 grid(nkv, num_seqs, p.max_tiles);
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
