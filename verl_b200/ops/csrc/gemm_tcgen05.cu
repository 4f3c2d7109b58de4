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

#include <math.h>
#include <stdio.h>
#include <stdlib.h>

namespace vb {

// --------------------------------------------------------------------------- kernel
constexpr int BM = 128;
constexpr int BK = 64;  // 64 bf16 = 128 bytes = one swizzle row
constexpr int GEMM_THREADS = 192;

// Epilogue kinds.
//  EPI_STORE    D = acc (+bias) as bf16 or fp32 (optionally +=)
//  EPI_LSE      LM head forward: per (row, 256-column tile) online-softmax partials (max, sum exp,
//               sum x*exp) of x = acc * inv_temp, plus the label logit; the [T, V] logits never exist.
//  EPI_DLOGITS  LM head backward: D = d loss / d acc for the recomputed tile, written as bf16:
//               inv_temp * ( g_lp * (onehot - p) - g_ent * p * (x - E[x]) ),  p = exp(x - lse).
//  EPI_ALLREDUCE  row-parallel (K-sharded) linear of a tensor-parallel group: every rank computes a partial tile,
//               publishes it as bf16 in its own peer-visible buffer, raises a per-(tile, warp) flag, then sums
//               the partials of all ranks in rank order (bitwise identical on every rank) and stores D.
//  EPI_SWIGLU   gated MLP up-projection: B is the stacked [gate; up] weight [2I, K], loaded through a 3-D tensor map that
//               interleaves the two halves row by row (accumulator column 2j = gate_j, 2j+1 = up_j), so that a thread
//               holds both members of a pair: D[M, I] = silu(gate) * up as bf16; optionally the pre-activation is
//               also written in the stacked layout ([M, 2I], what the backward pass of a kept layer reads).
enum { EPI_STORE = 0, EPI_LSE = 1, EPI_DLOGITS = 2, EPI_ALLREDUCE = 3, EPI_SWIGLU = 4 };

constexpr int AR_MAX_RANKS = 8;

struct GemmParams {
  int M, N, K;
  void* D;
  long long ldd;
  const __nv_bfloat16* bias;
  int out_f32;
  int accumulate;
  int* status;
  int k_splits;        // > 1: tile t also selects a K range; partials go to `D` as fp32 [k_splits][M][N]
  // LM-head epilogues
  const long long* labels;  // [M]; label column in the full vocabulary
  int label_offset;         // first vocabulary column covered by this launch
  float inv_temp;
  float* partial;           // EPI_LSE: [3][num_n_tiles][M]
  float* label_logit;       // EPI_LSE: [M]
  const float* lse;         // EPI_DLOGITS: [M]
  const float* ex;          // EPI_DLOGITS: [M]  E[x] = lse - entropy (may be null when g_ent is null)
  const float* g_lp;        // EPI_DLOGITS: [M]
  const float* g_ent;       // EPI_DLOGITS: [M] or null
  // EPI_ALLREDUCE
  int ar_world, ar_rank;
  unsigned long long ar_part[AR_MAX_RANKS];  // per rank: bf16 [2][ar_buf_elems] (two halves, selected by epoch parity)
  unsigned long long ar_flag[AR_MAX_RANKS];  // per rank: uint32 [num_tiles * 4]
  long long ar_buf_elems;
  unsigned int* ar_epoch;   // this rank's [2]: {calls completed, CTAs finished in the running call}
  unsigned long long ar_limit_ns;  // how long a slab waits for its peers before giving up
  int ar_rs_rows;  // > 0: reduce-scatter over rows: this rank sums (and stores, at row - rank * ar_rs_rows) only rows
                   // [rank * ar_rs_rows, (rank + 1) * ar_rs_rows); the other slabs are published and left to their owners
  // grouped (mixture-of-experts) modes; all row segments are padded to multiples of 128 rows
  //  1: rows grouped by expert  D[rows, N] = A[rows, K] * B_e^T, expert of each 128-row tile from grp_tile_expert
  //  2: contraction grouped     D_e[M, N] (+)= A[seg_e, M]^T * B[seg_e, N] for every expert e (weight gradients)
  int grp_mode;
  const int* grp_tile_expert;
  const int* grp_num_mtiles;
  const int* grp_seg_start;  // [E + 1]
  int grp_b_rows;            // rows one expert occupies in the stacked 2-D view of B
  int grp_E;
  // staged all-gather (FETCH variants). A byte range of `fetch_total` bytes is stored in equal slices of `fetch_slice`
  // bytes on the ranks of a group (rank r holds bytes [r * slice, (r + 1) * slice) at fetch_src[r], peer-mapped). The
  // copy warps of every CTA move 16 KB chunks [fetch_c0, fetch_c1) of it into local memory at fetch_dst while the
  // tensor pipe works. When B itself lies inside that range (at byte offset fetch_b_off, N * K * 2 bytes, rows
  // contiguous), fetch_panel counts the chunks that have landed per BN-row panel of B and the TMA producer holds a
  // tile back until its panel is complete; tiles then sweep all rows of the output per panel, so panels are needed
  // at an even rate over the whole GEMM.
  unsigned long long fetch_src[AR_MAX_RANKS];
  unsigned long long fetch_dst;
  long long fetch_total, fetch_slice, fetch_b_off;
  int fetch_c0, fetch_c1;
  unsigned int* fetch_panel;   // [ceil(N / BN)] zero at launch; null: B is local already, nothing waits
  unsigned long long fetch_limit_ns;
  // K-split with the fold inside the kernel: every split writes its fp32 partial slab to the workspace (D above) and
  // counts itself on the slab's counter; the split that arrives last sums all partials of the slab, adds the bias and
  // writes the real output. Counters return to zero, so they never need clearing between launches.
  unsigned int* fix_counter;   // [num output tiles * 4] or null (partials stay in the workspace for a later kernel)
  void* fix_out;
  long long fix_ldd;
  const __nv_bfloat16* fix_bias;
  int fix_out_f32, fix_accumulate;
  // EPI_SWIGLU: N counts accumulator columns (2 * I); D is the activation [M, I]
  __nv_bfloat16* gu_out;  // pre-activation [M, 2I] (gate columns first), or null
  long long gu_ld;
};

constexpr int FIX_COUNTERS = 16384;
__device__ unsigned int g_fix_counters[FIX_COUNTERS];

constexpr int FETCH_CHUNK = 16384;  // bytes per copy job of a fetch warp
constexpr int FETCH_WARPS = 4;      // copy warps per CTA (warps 6..9): peer loads are latency-bound, bytes in flight = rate
constexpr int ST_TIMEOUT_FETCH = 14;

__device__ __forceinline__ void st_release_sys_u32(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys_u32(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned int ld_acquire_gpu_u32(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long ar_now_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ int g_gemm_status[4];

template <int BN, int STAGES>
struct GemmSmem {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int RING = STAGES * (A_BYTES + B_BYTES);
  static constexpr int TOTAL = RING + 256 + 1024;  // barriers + alignment slack
};

// Pass B of the all-reduce epilogue for one warp's slab (32 rows x BN columns): sum the bf16 partials of all ranks in rank
// order (+ bias) and store the rows that lie in [rs_lo, rs_hi). Lanes sweep the columns of one (BN = 256) or two
// (BN = 128) rows at a time: the 16-byte pieces of a row are contiguous across lanes, so every peer read is a full 512-byte
// (256-byte) burst over NVLink. A peer read costs microseconds of latency, so the loads of UNR row groups from ALL W ranks
// are issued before the first is consumed: a slab costs 32 / (rows per group x UNR) dependent round trips, not that times
// the number of ranks.
template <int BN, int W, int UNR>
__device__ __forceinline__ void ar_sum_slab(const GemmParams& p, long long half, int row0, int n0, int lane, int rs_lo, int rs_hi) {
  static_assert(W <= AR_MAX_RANKS, "more ranks than pointer slots");
  constexpr int LPR = BN / 8;    // lanes per row
  constexpr int RPI = 32 / LPR;  // rows per row group
  static_assert(32 % (RPI * UNR) == 0, "a slab is a whole number of batches");
  const int col = n0 + (lane % LPR) * 8;
  const bool col_ok = col < p.N;
  float bias8[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (p.bias != nullptr && col_ok) {
#pragma unroll
    for (int j = 0; j < 8; ++j) bias8[j] = __bfloat162float(p.bias[col + j]);
  }
#pragma unroll 1
  for (int rr = 0; rr < 32; rr += RPI * UNR) {
    uint4 v[W][UNR];
#pragma unroll
    for (int r = 0; r < W; ++r) {
      if (r < p.ar_world) {
        const __nv_bfloat16* src = reinterpret_cast<const __nv_bfloat16*>(p.ar_part[r]);
#pragma unroll
        for (int u = 0; u < UNR; ++u) {
          const int orow = row0 + rr + u * RPI + lane / LPR;
          const bool ok = col_ok && orow < p.M && orow >= rs_lo && orow < rs_hi;
          v[r][u] = ok ? __ldcg(reinterpret_cast<const uint4*>(src + half + static_cast<long long>(orow) * p.N + col))
                       : make_uint4(0, 0, 0, 0);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < UNR; ++u) {
      const int orow = row0 + rr + u * RPI + lane / LPR;
      const bool ok = col_ok && orow < p.M && orow >= rs_lo && orow < rs_hi;
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int r = 0; r < W; ++r) {
        if (r < p.ar_world) {
          const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v[r][u]);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 f2 = __bfloat1622float2(h[j]);
            acc[2 * j] += f2.x;
            acc[2 * j + 1] += f2.y;
          }
        }
      }
      if (!ok) continue;
      uint4 o;
      o.x = pack_bf16x2(acc[0] + bias8[0], acc[1] + bias8[1]);
      o.y = pack_bf16x2(acc[2] + bias8[2], acc[3] + bias8[3]);
      o.z = pack_bf16x2(acc[4] + bias8[4], acc[5] + bias8[5]);
      o.w = pack_bf16x2(acc[6] + bias8[6], acc[7] + bias8[7]);
      *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.D) + static_cast<long long>(orow - rs_lo) * p.ldd + col) = o;
    }
  }
}

// Kernel body. FETCH adds copy warps that stage peer memory into local memory (see GemmParams::fetch_*).
template <int BN, bool A_MN, bool B_MN, int STAGES, int EPI, bool FETCH>
__device__ __forceinline__ void gemm_body(const CUtensorMap& tma_a, const CUtensorMap& tma_b, const GemmParams& p) {
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

  const int num_n = (p.N + BN - 1) / BN;
  const int num_m = (p.grp_mode == 1) ? *p.grp_num_mtiles : (p.M + BM - 1) / BM;
  const int splits = p.k_splits > 1 ? p.k_splits : 1;
  const int num_mn = num_m * num_n;
  const int num_tiles = (p.grp_mode == 2) ? num_mn * p.grp_E : num_mn * splits;
  const int num_kb_total = (p.K + BK - 1) / BK;
  const int kb_per = (num_kb_total + splits - 1) / splits;
  // rasterisation: groups of GROUP_M row tiles share their B panels through L2; a launch that waits for B panels to
  // arrive sweeps every row tile of a panel before it moves to the next panel
  const int GROUP_M = (FETCH && p.fetch_panel != nullptr) ? num_m : 8;

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
  unsigned int ar_epoch_now = 0;
  if constexpr (EPI == EPI_ALLREDUCE) ar_epoch_now = *reinterpret_cast<volatile unsigned int*>(p.ar_epoch) + 1u;

  // tile t -> output tile origin (m0, n0), k-block range, row offset of the B tile in its stacked view, row offset of
  // the output; returns false for a tile without work (an expert that received no rows)
  auto decode_tile = [&](int t, int& m0, int& n0, int& kb0, int& kb1, int& b_off, long long& d_off) -> bool {
    b_off = 0;
    d_off = 0;
    if (p.grp_mode == 1) {
      const int m_idx = t / num_n;
      m0 = m_idx * BM;
      n0 = (t - m_idx * num_n) * BN;
      kb0 = 0;
      kb1 = num_kb_total;
      b_off = p.grp_tile_expert[m_idx] * p.grp_b_rows;
      return true;
    }
    int tt = t;
    if (p.grp_mode == 2) {
      const int e = t / num_mn;
      tt = t - e * num_mn;
      kb0 = p.grp_seg_start[e] / BK;
      kb1 = p.grp_seg_start[e + 1] / BK;
      d_off = static_cast<long long>(e) * p.M;
    } else {
      const int sp = t / num_mn;
      tt = t - sp * num_mn;
      kb0 = sp * kb_per;
      kb1 = min(num_kb_total, kb0 + kb_per);
      d_off = static_cast<long long>(sp) * p.M;  // split-K partials are stacked [splits][M][N]
    }
    const int per_group = GROUP_M * num_n;
    const int g = tt / per_group;
    const int first_m = g * GROUP_M;
    const int gsize = min(num_m - first_m, GROUP_M);
    const int r = tt - g * per_group;
    m0 = (first_m + (r % gsize)) * BM;
    n0 = (r / gsize) * BN;
    return kb1 > kb0;
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int panel_ready = -1;  // FETCH: last panel of B known to be complete in local memory
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int m0, n0, kb0, kb1, b_off;
        long long d_off;
        if (!decode_tile(t, m0, n0, kb0, kb1, b_off, d_off)) continue;
        if constexpr (FETCH) {
          const int panel = n0 / BN;
          if (p.fetch_panel != nullptr && panel != panel_ready) {
            // chunks of this launch that intersect the panel's bytes
            const long long lo = p.fetch_b_off + static_cast<long long>(n0) * p.K * 2;
            const long long hi = p.fetch_b_off + static_cast<long long>(min(n0 + BN, p.N)) * p.K * 2;
            const long long e_lo = max(lo / FETCH_CHUNK, static_cast<long long>(p.fetch_c0));
            const long long e_hi = min((hi - 1) / FETCH_CHUNK, static_cast<long long>(p.fetch_c1) - 1);
            const unsigned int expect = e_hi >= e_lo ? static_cast<unsigned int>(e_hi - e_lo + 1) : 0u;
            const unsigned long long t0 = ar_now_ns();
            unsigned int spins = 0;
            while (ld_acquire_gpu_u32(p.fetch_panel + panel) < expect) {
              if ((++spins & 0x3f) == 0 && ar_now_ns() - t0 > p.fetch_limit_ns) {
                atomicExch(p.status, ST_TIMEOUT_FETCH);
                ok = false;
                break;
              }
            }
            if (!ok) break;
            // the chunks were written with ordinary stores; the tile loads below read them through the async proxy
            asm volatile("fence.proxy.async.global;" ::: "memory");
            panel_ready = panel;
          }
        }
        for (int kb = kb0; kb < kb1; ++kb) {
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
          if constexpr (EPI == EPI_SWIGLU) {
            // (k, half, row) box of 64 x 2 x BN/2: shared-memory row 2j holds gate row n0/2 + j, row 2j + 1 its up row
            tma_load_3d(sb, &tma_b, &full_bar[stage], k0, 0, n0 >> 1);
          } else if constexpr (!B_MN) {
            tma_load_2d(sb, &tma_b, &full_bar[stage], k0, b_off + n0);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_2d(sb + j * (BK * 128), &tma_b, &full_bar[stage], n0 + 64 * j, (p.grp_mode == 1 ? b_off : 0) + k0);
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
        int m0_, n0_, kb0, kb1, b_off_;
        long long d_off_;
        if (!decode_tile(t, m0_, n0_, kb0, kb1, b_off_, d_off_)) continue;
        if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1)) {
          atomicExch(p.status, ST_TIMEOUT_MMA);
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = kb0; kb < kb1; ++kb) {
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
            tc_mma_f16_ss(d_tmem, da, db, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
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
  } else if (FETCH && warp >= 6) {
    // ------------------------------------------------------------------ fetch warps: peer memory -> local memory
    // Chunks are dealt round-robin over all fetch warps of the grid in address order, so every CTA works on the panels
    // that are needed first. 16 independent 16-byte loads per lane are in flight before the first store (8 KB per warp).
    if constexpr (FETCH) {
      const long long panel_bytes = static_cast<long long>(BN) * p.K * 2;
      const long long b_end = p.fetch_b_off + static_cast<long long>(p.N) * p.K * 2;
      const int fw = static_cast<int>(blockIdx.x) * FETCH_WARPS + (warp - 6);
      const int fw_stride = static_cast<int>(gridDim.x) * FETCH_WARPS;
      for (int c = p.fetch_c0 + fw; c < p.fetch_c1; c += fw_stride) {
        const long long off = static_cast<long long>(c) * FETCH_CHUNK;
        const long long len = min(static_cast<long long>(FETCH_CHUNK), p.fetch_total - off);
        const int owner = static_cast<int>(off / p.fetch_slice);
        const uint4* src = reinterpret_cast<const uint4*>(p.fetch_src[owner] + (off - owner * p.fetch_slice));
        uint4* dst = reinterpret_cast<uint4*>(p.fetch_dst + off);
        const int n16 = static_cast<int>(len >> 4);
        for (int base = 0; base < n16; base += 32 * 16) {
          uint4 v[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int i = base + j * 32 + lane;
            if (i < n16) v[j] = src[i];
          }
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int i = base + j * 32 + lane;
            if (i < n16) dst[i] = v[j];
          }
        }
        if (p.fetch_panel != nullptr && off < b_end && off + len > p.fetch_b_off) {
          asm volatile("fence.proxy.async.global;" ::: "memory");
          __threadfence();
          __syncwarp();
          if (lane == 0) {
            const long long lo = max(off, p.fetch_b_off) - p.fetch_b_off;
            const long long hi = min(off + len, b_end) - p.fetch_b_off;
            for (long long pp = lo / panel_bytes; pp <= (hi - 1) / panel_bytes; ++pp) atomicAdd(p.fetch_panel + pp, 1u);
          }
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
      int m0, n0, kb0_, kb1_, b_off_;
      long long d_off;
      if (!decode_tile(t, m0, n0, kb0_, kb1_, b_off_, d_off)) continue;
      const int n_idx = n0 / BN;
      if (!mbar_wait(&acc_full[acc], acc_phase)) {
        if (lane == 0) atomicExch(p.status, ST_TIMEOUT_EPILOGUE);
        ok = false;
        break;
      }
      tc_fence_after();
      const int row = m0 + q * 32 + lane;
      const bool row_ok = (p.grp_mode == 1) ? true : row < p.M;  // grouped rows are padded to whole tiles
      // per-row state of the LM-head epilogues (thread == row)
      float run_m = -INFINITY, run_l = 0.f, run_s = 0.f;
      long long label = -1;
      float r_lse = 0.f, r_ex = 0.f, r_glp = 0.f, r_gent = 0.f;
      if constexpr (EPI != EPI_STORE) {
        if (row_ok) {
          label = p.labels[row] - p.label_offset;
          if constexpr (EPI == EPI_DLOGITS) {
            r_lse = p.lse[row];
            r_glp = p.g_lp[row];
            if (p.g_ent != nullptr) {
              r_gent = p.g_ent[row];
              r_ex = p.ex[row];
            }
          }
        }
      }
      constexpr float LOG2E = 1.4426950408889634f;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        const int col0 = n0 + c * 32;
        if (col0 >= p.N) break;  // uniform across the warp
        uint32_t r[32];
        tmem_ld_32x32(tmem_base + acc * BN + c * 32 + (static_cast<uint32_t>(q * 32) << 16), r);
        tmem_ld_wait();
        const int ncols = min(32, p.N - col0);  // multiple of 8
        if constexpr (EPI == EPI_LSE) {
          float x[32];
          float cmax = -INFINITY;
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            x[j] = (j < ncols) ? __uint_as_float(r[j]) * p.inv_temp : -INFINITY;
            cmax = fmaxf(cmax, x[j]);
          }
          const float new_m = fmaxf(run_m, cmax);
          const float resc = exp2f((run_m - new_m) * LOG2E);  // 0 on the first chunk (run_m = -inf)
          float cl = 0.f, cs = 0.f;
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float e = exp2f((x[j] - new_m) * LOG2E);
            cl += e;
            cs += (j < ncols) ? e * x[j] : 0.f;
          }
          run_l = run_l * resc + cl;
          run_s = run_s * resc + cs;
          run_m = new_m;
          const long long rel = label - col0;
          if (rel >= 0 && rel < ncols && row_ok) {
            float lab = 0.f;
#pragma unroll
            for (int j = 0; j < 32; ++j) lab = (j == rel) ? x[j] : lab;
            p.label_logit[row] = lab;
          }
        } else if constexpr (EPI == EPI_DLOGITS) {
          if (row_ok) {
            const long long rel = label - col0;
            __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.D) + static_cast<long long>(row) * p.ldd + col0;
            float d[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const float x = __uint_as_float(r[j]) * p.inv_temp;
              const float pj = exp2f((x - r_lse) * LOG2E);
              float g = r_glp * (((j == rel) ? 1.f : 0.f) - pj);
              g -= r_gent * pj * (x - r_ex);
              d[j] = g * p.inv_temp;
            }
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              if (j < ncols) {
                uint4 v;
                v.x = pack_bf16x2(d[j], d[j + 1]);
                v.y = pack_bf16x2(d[j + 2], d[j + 3]);
                v.z = pack_bf16x2(d[j + 4], d[j + 5]);
                v.w = pack_bf16x2(d[j + 6], d[j + 7]);
                *reinterpret_cast<uint4*>(out + j) = v;
              }
            }
          }
        } else if constexpr (EPI == EPI_SWIGLU) {
          if (row_ok) {
            const int ac0 = col0 >> 1;        // first activation column of this chunk
            const int npairs = ncols >> 1;    // multiple of 4
            const int inter = p.N >> 1;
            float act[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const float g = __uint_as_float(r[2 * j]), u = __uint_as_float(r[2 * j + 1]);
              act[j] = g / (1.f + __expf(-g)) * u;
            }
            __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.D) + static_cast<long long>(row) * p.ldd + ac0;
#pragma unroll
            for (int j = 0; j < 16; j += 4) {
              if (j < npairs) {
                uint2 v;
                v.x = pack_bf16x2(act[j], act[j + 1]);
                v.y = pack_bf16x2(act[j + 2], act[j + 3]);
                *reinterpret_cast<uint2*>(out + j) = v;
              }
            }
            if (p.gu_out != nullptr) {
              __nv_bfloat16* go = p.gu_out + static_cast<long long>(row) * p.gu_ld + ac0;
#pragma unroll
              for (int j = 0; j < 16; j += 4) {
                if (j < npairs) {
                  uint2 g4, u4;
                  g4.x = pack_bf16x2(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 2]));
                  g4.y = pack_bf16x2(__uint_as_float(r[2 * j + 4]), __uint_as_float(r[2 * j + 6]));
                  u4.x = pack_bf16x2(__uint_as_float(r[2 * j + 1]), __uint_as_float(r[2 * j + 3]));
                  u4.y = pack_bf16x2(__uint_as_float(r[2 * j + 5]), __uint_as_float(r[2 * j + 7]));
                  *reinterpret_cast<uint2*>(go + j) = g4;
                  *reinterpret_cast<uint2*>(go + inter + j) = u4;
                }
              }
            }
          }
        } else if constexpr (EPI == EPI_ALLREDUCE) {
          // pass A: this rank's partial, rounded to bf16, into its own peer-visible buffer
          if (row_ok) {
            __nv_bfloat16* mine = reinterpret_cast<__nv_bfloat16*>(p.ar_part[p.ar_rank]) +
                                  static_cast<long long>(ar_epoch_now & 1u) * p.ar_buf_elems +
                                  static_cast<long long>(row) * p.N + col0;
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              if (j < ncols) {
                uint4 v;
                v.x = pack_bf16x2(__uint_as_float(r[j]), __uint_as_float(r[j + 1]));
                v.y = pack_bf16x2(__uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
                v.z = pack_bf16x2(__uint_as_float(r[j + 4]), __uint_as_float(r[j + 5]));
                v.w = pack_bf16x2(__uint_as_float(r[j + 6]), __uint_as_float(r[j + 7]));
                *reinterpret_cast<uint4*>(mine + j) = v;
              }
            }
          }
        } else if (row_ok) {
          if (p.bias != nullptr) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              if (j < ncols) r[j] = __float_as_uint(__uint_as_float(r[j]) + __bfloat162float(p.bias[col0 + j]));
            }
          }
          if (p.out_f32) {
            float* out = reinterpret_cast<float*>(p.D) + (d_off + row) * p.ldd + col0;
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
            __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.D) + (d_off + row) * p.ldd + col0;
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
      if constexpr (EPI == EPI_LSE) {
        if (row_ok) {
          const long long plane = static_cast<long long>(num_n) * p.M;
          const long long o = static_cast<long long>(n_idx) * p.M + row;
          p.partial[o] = run_m;
          p.partial[plane + o] = run_l;
          p.partial[2 * plane + o] = run_s;
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[acc]);  // the accumulator is free: the next tile's MMAs may start
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1;
      }
      if constexpr (EPI == EPI_STORE) {
        if (p.fix_counter != nullptr && splits > 1) {
          __threadfence();  // this warp's slab of its split is in the workspace before it counts itself
          __syncwarp();
          const int slab = (t % num_mn) * 4 + q;
          unsigned int before = 0;
          if (lane == 0) before = atomicAdd(p.fix_counter + slab, 1u);
          before = __shfl_sync(0xffffffffu, before, 0);
          if (before == static_cast<unsigned int>(splits - 1)) {
            if (lane == 0) p.fix_counter[slab] = 0;
            __threadfence();
            // lanes across the columns (coalesced 1 KB row reads), eight rows per round: the sixteen loads of a split are
            // all issued before the first is consumed (one warp folds a slab alone, so its latency is on the critical
            // path of the launch)
            const int colw = n0 + lane * 8;
            if (lane * 8 < BN && colw < p.N) {
              float b8[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
              if (p.fix_bias != nullptr) {
#pragma unroll
                for (int j = 0; j < 8; ++j) b8[j] = __bfloat162float(p.fix_bias[colw + j]);
              }
              const float* __restrict__ wsb = reinterpret_cast<const float*>(p.D) + colw;
              const long long split_stride = static_cast<long long>(p.M) * p.ldd;
              constexpr int RB = 8;
#pragma unroll 1
              for (int rr = 0; rr < 32; rr += RB) {
                const int rbase = m0 + q * 32 + rr;
                if (rbase >= p.M) break;
                float a8[RB][8];
#pragma unroll
                for (int u = 0; u < RB; ++u)
#pragma unroll
                  for (int j = 0; j < 8; ++j) a8[u][j] = b8[j];
                for (int sp = 0; sp < splits; ++sp) {
                  float4 v[RB][2];
#pragma unroll
                  for (int u = 0; u < RB; ++u) {
                    const int rw = min(rbase + u, p.M - 1);  // rows past the end re-read the last row; they are not stored
                    const float* src = wsb + sp * split_stride + static_cast<long long>(rw) * p.ldd;
                    v[u][0] = __ldcg(reinterpret_cast<const float4*>(src));
                    v[u][1] = __ldcg(reinterpret_cast<const float4*>(src + 4));
                  }
#pragma unroll
                  for (int u = 0; u < RB; ++u) {
                    a8[u][0] += v[u][0].x; a8[u][1] += v[u][0].y; a8[u][2] += v[u][0].z; a8[u][3] += v[u][0].w;
                    a8[u][4] += v[u][1].x; a8[u][5] += v[u][1].y; a8[u][6] += v[u][1].z; a8[u][7] += v[u][1].w;
                  }
                }
#pragma unroll
                for (int u = 0; u < RB; ++u) {
                  const int rw = rbase + u;
                  if (rw >= p.M) break;
                  if (p.fix_out_f32) {
                    float* o = reinterpret_cast<float*>(p.fix_out) + static_cast<long long>(rw) * p.fix_ldd + colw;
                    if (p.fix_accumulate) {
#pragma unroll
                      for (int j = 0; j < 8; ++j) a8[u][j] += o[j];
                    }
                    *reinterpret_cast<float4*>(o) = make_float4(a8[u][0], a8[u][1], a8[u][2], a8[u][3]);
                    *reinterpret_cast<float4*>(o + 4) = make_float4(a8[u][4], a8[u][5], a8[u][6], a8[u][7]);
                  } else {
                    uint4 v4;
                    v4.x = pack_bf16x2(a8[u][0], a8[u][1]); v4.y = pack_bf16x2(a8[u][2], a8[u][3]);
                    v4.z = pack_bf16x2(a8[u][4], a8[u][5]); v4.w = pack_bf16x2(a8[u][6], a8[u][7]);
                    *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.fix_out) + static_cast<long long>(rw) * p.fix_ldd + colw) = v4;
                  }
                }
              }
            }
          }
        }
      }
      if constexpr (EPI == EPI_ALLREDUCE) {
        // publish: all 32 rows of this warp's slab are written -> raise flag (tile, q) with release semantics
        __threadfence_system();
        __syncwarp();
        const int slot = (t % num_mn) * 4 + q;
        if (lane == 0) st_release_sys_u32(reinterpret_cast<unsigned int*>(p.ar_flag[p.ar_rank]) + slot, ar_epoch_now);
        // pass B: wait (bounded) for the same slab of every peer, then sum all partials in rank order
        int rs_lo = 0, rs_hi = 0x7fffffff;
        bool mine = true;
        if (p.ar_rs_rows > 0) {
          rs_lo = p.ar_rank * p.ar_rs_rows;
          rs_hi = rs_lo + p.ar_rs_rows;
          const int s0 = m0 + q * 32;
          mine = s0 < rs_hi && s0 + 32 > rs_lo;  // uniform over the warp
        }
        bool peers_ok = true;
        const unsigned long long t_start = ar_now_ns();
        for (int r = 0; mine && r < p.ar_world; ++r) {
          if (r == p.ar_rank) continue;
          const unsigned int* f = reinterpret_cast<const unsigned int*>(p.ar_flag[r]) + slot;
          while (static_cast<int>(ld_acquire_sys_u32(f) - ar_epoch_now) < 0) {
            if (ar_now_ns() - t_start > p.ar_limit_ns) {  // the peer never arrived
              peers_ok = false;
              break;
            }
            __nanosleep(64);
          }
          if (!peers_ok) break;
        }
        peers_ok = __all_sync(0xffffffffu, peers_ok);
        if (!peers_ok) {
          if (lane == 0) atomicExch(p.status, ST_TIMEOUT_EPILOGUE + 10);
        } else if (mine) {
          const long long half = static_cast<long long>(ar_epoch_now & 1u) * p.ar_buf_elems;
          // 16 sixteen-byte loads per lane are in flight per round trip whatever the group size (more would spill): more
          // rows per round trip on few ranks, every rank's piece of fewer rows on many
          if (p.ar_world <= 2) ar_sum_slab<BN, 2, 8>(p, half, m0 + q * 32, n0, lane, rs_lo, rs_hi);
          else if (p.ar_world <= 4) ar_sum_slab<BN, 4, 4>(p, half, m0 + q * 32, n0, lane, rs_lo, rs_hi);
          else ar_sum_slab<BN, AR_MAX_RANKS, 2>(p, half, m0 + q * 32, n0, lane, rs_lo, rs_hi);
        }
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
  if constexpr (EPI == EPI_ALLREDUCE) {
    // the last CTA to finish closes the call: every CTA of this launch has read the epoch by now
    if (threadIdx.x == 0) {
      __threadfence();
      const unsigned int done = atomicAdd(p.ar_epoch + 1, 1u);
      if (done == gridDim.x - 1) {
        p.ar_epoch[1] = 0;
        __threadfence();
        atomicAdd(p.ar_epoch, 1u);
      }
    }
  }
}

template <int BN, bool A_MN, bool B_MN, int STAGES, int EPI>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                 const GemmParams p) {
  gemm_body<BN, A_MN, B_MN, STAGES, EPI, false>(tma_a, tma_b, p);
}

constexpr int GEMM_FETCH_THREADS = GEMM_THREADS + 32 * FETCH_WARPS;

// The same GEMM with fetch warps: the all-gather of a sharded byte range (the GEMM's own B operand, or whatever a later
// kernel needs) runs inside the GEMM, over peer loads, behind the tensor pipe.
template <int BN, bool A_MN, bool B_MN, int STAGES>
__global__ void __launch_bounds__(GEMM_FETCH_THREADS, 1)
gemm_bf16_fetch_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                       const GemmParams p) {
  gemm_body<BN, A_MN, B_MN, STAGES, EPI_STORE, true>(tma_a, tma_b, p);
}

// Device address of the status word, resolved once (outside any stream capture).
static int* status_ptr() {
  static int* p = nullptr;
  if (p == nullptr) cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_gemm_status);
  return p;
}

// --------------------------------------------------------------------------- launcher
template <int BN, bool A_MN, bool B_MN, int STAGES, int EPI = EPI_STORE>
static cudaError_t launch_variant(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int sms,
                                  cudaStream_t stream) {
  auto kern = gemm_bf16_kernel<BN, A_MN, B_MN, STAGES, EPI>;
  constexpr int smem = GemmSmem<BN, STAGES>::TOTAL;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    configured = true;
  }
  const int tiles = ((p.M + BM - 1) / BM) * ((p.N + BN - 1) / BN) * (p.k_splits > 1 ? p.k_splits : 1);
  const int grid = tiles < sms ? tiles : sms;
  kern<<<grid, GEMM_THREADS, smem, stream>>>(ta, tb, p);
  return cudaGetLastError();
}

}  // namespace vb

using namespace vb;

// Returns 0 on success, a negative code for bad arguments, a positive cudaError_t otherwise.
//  a_mn / b_mn: operand is stored [K, M|N] (MN contiguous) instead of [M|N, K].
//  lda / ldb / ldd: row stride in elements of the stored matrix.
namespace vb {
__global__ void splitk_reduce_kernel(const float* __restrict__ ws, const __nv_bfloat16* __restrict__ bias, void* D,
                                     long long ldd, int M, int N, int splits, int out_f32, int accumulate) {
  const long long i4 = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  const long long total4 = static_cast<long long>(M) * N / 4;
  if (i4 >= total4) return;
  const long long e = i4 * 4;
  const int row = static_cast<int>(e / N), col = static_cast<int>(e % N);
  float4 a = reinterpret_cast<const float4*>(ws)[i4];
  for (int s = 1; s < splits; ++s) {
    const float4 b = reinterpret_cast<const float4*>(ws + static_cast<long long>(s) * M * N)[i4];
    a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
  }
  if (bias != nullptr) {
    a.x += __bfloat162float(bias[col]); a.y += __bfloat162float(bias[col + 1]);
    a.z += __bfloat162float(bias[col + 2]); a.w += __bfloat162float(bias[col + 3]);
  }
  if (out_f32) {
    float4* o = reinterpret_cast<float4*>(reinterpret_cast<float*>(D) + static_cast<long long>(row) * ldd + col);
    if (accumulate) { const float4 c = *o; a.x += c.x; a.y += c.y; a.z += c.z; a.w += c.w; }
    *o = a;
  } else {
    uint2 v;
    v.x = pack_bf16x2(a.x, a.y);
    v.y = pack_bf16x2(a.z, a.w);
    *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(D) + static_cast<long long>(row) * ldd + col) = v;
  }
}

// Split-K reduction fused with the tensor-parallel all-reduce (decode-sized row-parallel linears: few output tiles, deep
// K). Every CTA owns 2048 consecutive output elements: it folds this rank's K-split partial sums, publishes the bf16
// result in the rank's peer-visible buffer, raises the chunk's flag, waits (bounded) for the same chunk of every peer and
// sums all ranks' chunks in rank order, so every rank obtains identical bits.
struct SplitKAllReduceParams {
  const float* ws;   // [splits][M*N] fp32 partial sums of this rank
  int splits;
  long long total;   // M * N
  int N;
  const __nv_bfloat16* bias;
  __nv_bfloat16* D;
  long long ldd;
  unsigned long long part[AR_MAX_RANKS];
  unsigned long long flag[AR_MAX_RANKS];
  long long buf_elems;
  unsigned int* epoch;
  unsigned long long limit_ns;
  int world, rank;
  int* status;
};

constexpr int SKAR_THREADS = 256;

__global__ void __launch_bounds__(SKAR_THREADS)
splitk_reduce_allreduce_kernel(const SplitKAllReduceParams p) {
  __shared__ int s_ok;
  const unsigned int epoch_now = *reinterpret_cast<volatile unsigned int*>(p.epoch) + 1u;
  const long long half = static_cast<long long>(epoch_now & 1u) * p.buf_elems;
  const long long e = (blockIdx.x * static_cast<long long>(SKAR_THREADS) + threadIdx.x) * 8;
  const bool live = e < p.total;
  if (live) {
    float a[8];
    const float4* w0 = reinterpret_cast<const float4*>(p.ws + e);
    float4 x = w0[0], y = w0[1];
    a[0] = x.x; a[1] = x.y; a[2] = x.z; a[3] = x.w; a[4] = y.x; a[5] = y.y; a[6] = y.z; a[7] = y.w;
    for (int s = 1; s < p.splits; ++s) {
      const float4* w = reinterpret_cast<const float4*>(p.ws + static_cast<long long>(s) * p.total + e);
      x = w[0]; y = w[1];
      a[0] += x.x; a[1] += x.y; a[2] += x.z; a[3] += x.w; a[4] += y.x; a[5] += y.y; a[6] += y.z; a[7] += y.w;
    }
    uint4 v;
    v.x = pack_bf16x2(a[0], a[1]); v.y = pack_bf16x2(a[2], a[3]); v.z = pack_bf16x2(a[4], a[5]); v.w = pack_bf16x2(a[6], a[7]);
    *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.part[p.rank]) + half + e) = v;
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    st_release_sys_u32(reinterpret_cast<unsigned int*>(p.flag[p.rank]) + blockIdx.x, epoch_now);
    int ok = 1;
    const unsigned long long t0 = ar_now_ns();
    for (int r = 0; r < p.world && ok; ++r) {
      if (r == p.rank) continue;
      const unsigned int* f = reinterpret_cast<const unsigned int*>(p.flag[r]) + blockIdx.x;
      while (static_cast<int>(ld_acquire_sys_u32(f) - epoch_now) < 0) {
        if (ar_now_ns() - t0 > p.limit_ns) {  // the peer never arrived
          ok = 0;
          break;
        }
        __nanosleep(64);
      }
    }
    if (!ok) atomicExch(p.status, ST_TIMEOUT_EPILOGUE + 10);
    s_ok = ok;
  }
  __syncthreads();
  if (s_ok && live) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    uint4 v[AR_MAX_RANKS];
#pragma unroll
    for (int r = 0; r < AR_MAX_RANKS; ++r) {  // all peers' loads in flight before the first is consumed
      if (r < p.world) v[r] = __ldcg(reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(p.part[r]) + half + e));
    }
#pragma unroll
    for (int r = 0; r < AR_MAX_RANKS; ++r) {
      if (r < p.world) {
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v[r]);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f2 = __bfloat1622float2(h[j]);
          acc[2 * j] += f2.x;
          acc[2 * j + 1] += f2.y;
        }
      }
    }
    const long long row = e / p.N;
    const int col = static_cast<int>(e % p.N);
    if (p.bias != nullptr) {
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += __bfloat162float(p.bias[col + j]);
    }
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]); o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
    *reinterpret_cast<uint4*>(p.D + row * p.ldd + col) = o;
  }
  // the last CTA to finish closes the call: every CTA of this launch has read the epoch by now
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned int done = atomicAdd(p.epoch + 1, 1u);
    if (done == gridDim.x - 1) {
      p.epoch[1] = 0;
      __threadfence();
      atomicAdd(p.epoch, 1u);
    }
  }
}
}  // namespace vb

// Suggested number of K splits for a skinny GEMM (few output tiles, deep K); 1 = no split.
extern "C" int vb_gemm_suggest_splits(int M, int N, int K) {
  const int BN = N > 128 ? 256 : 128;
  const int tiles = ((M + 127) / 128) * ((N + BN - 1) / BN);
  const int sms = num_sms();
  if (tiles * 2 > sms || K < 2048) return 1;
  int s = sms / tiles;
  const int by_k = K / 1024;
  if (s > by_k) s = by_k;
  if (s > 8) s = 8;
  return s < 2 ? 1 : s;
}

extern "C" int vb_gemm_bf16_ex(const void* A, const void* B, void* D, const void* bias, int M, int N, int K,
                               long long lda, long long ldb, long long ldd, int a_mn, int b_mn, int out_f32,
                               int accumulate, int max_ctas, int k_splits, float* splitk_ws, cudaStream_t stream);

extern "C" int vb_gemm_bf16(const void* A, const void* B, void* D, const void* bias, int M, int N, int K,
                            long long lda, long long ldb, long long ldd, int a_mn, int b_mn, int out_f32,
                            int accumulate, int max_ctas, cudaStream_t stream) {
  return vb_gemm_bf16_ex(A, B, D, bias, M, N, K, lda, ldb, ldd, a_mn, b_mn, out_f32, accumulate, max_ctas, 1, nullptr,
                         stream);
}

// VERL_B200_SPLITK_FOLD=1 folds the partial sums of a K-split GEMM inside the GEMM kernel instead of a second launch
// (read once per process). Off by default: inside the decode graph the fold by the last-arriving warp measured 0.3 ms
// per step slower than the reduce kernel, which spreads the same reads over every SM.
extern "C" int vb_gemm_fold_in_kernel() {
  static const bool on = [] { const char* v = getenv("VERL_B200_SPLITK_FOLD"); return v != nullptr && v[0] == '1'; }();
  return on ? 1 : 0;
}

// k_splits > 1 needs splitk_ws of k_splits * M * N floats.
static bool g_partials_only = false;  // set by the all-reduce launcher: leave the K-split partial sums in the workspace

extern "C" int vb_gemm_bf16_ex(const void* A, const void* B, void* D, const void* bias, int M, int N, int K,
                               long long lda, long long ldb, long long ldd, int a_mn, int b_mn, int out_f32,
                               int accumulate, int max_ctas, int k_splits, float* splitk_ws, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  // TMA needs 16-byte aligned bases and row strides; the epilogue stores 8-column vectors.
  if ((N % 8) || (lda % 8) || (ldb % 8) || (ldd % (out_f32 ? 4 : 8))) return -1;
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
  int* status = status_ptr();
  GemmParams p{};
  p.M = M; p.N = N; p.K = K; p.D = D; p.ldd = ldd;
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.out_f32 = out_f32; p.accumulate = accumulate; p.status = status;
  p.k_splits = 1;
  bool fold_in_kernel = false;
  if (splitk_ws != nullptr && k_splits > 1) {
    // partial sums as fp32 [k_splits][M][N] in the workspace; the split that finishes a slab last folds them (+bias)
    // into D inside the GEMM kernel. (When the partials are wanted as they are, or the output has more slabs than the
    // counter table, the separate reduce kernel below does it.)
    const long long slabs = 4LL * ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
    fold_in_kernel = vb_gemm_fold_in_kernel() && !g_partials_only && slabs <= FIX_COUNTERS;
    if (fold_in_kernel) {
      static unsigned int* counters = nullptr;
      if (counters == nullptr) cudaGetSymbolAddress(reinterpret_cast<void**>(&counters), g_fix_counters);
      p.fix_counter = counters; p.fix_out = D; p.fix_ldd = ldd; p.fix_bias = reinterpret_cast<const __nv_bfloat16*>(bias);
      p.fix_out_f32 = out_f32; p.fix_accumulate = accumulate;
    }
    p.k_splits = k_splits; p.D = splitk_ws; p.ldd = N; p.bias = nullptr; p.out_f32 = 1; p.accumulate = 0;
  }
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
  if (e == cudaSuccess && p.k_splits > 1 && !g_partials_only && !fold_in_kernel) {
    const long long total4 = static_cast<long long>(M) * N / 4;
    splitk_reduce_kernel<<<static_cast<int>((total4 + 255) / 256), 256, 0, stream>>>(
        splitk_ws, reinterpret_cast<const __nv_bfloat16*>(bias), D, ldd, M, N, p.k_splits, out_f32, accumulate);
    e = cudaGetLastError();
  }
  return static_cast<int>(e);
}

// Gated MLP up-projection with the activation in the epilogue: act[M, I] = silu(A W_gate^T) * (A W_up^T) for the stacked
// weight W = [W_gate; W_up] ([2I, K], K-major, row stride ldw). gu_out (or null): the pre-activation [M, 2I] in the
// stacked layout, row stride gu_ld, for a backward pass that keeps it. I must be a multiple of 4.
extern "C" int vb_gemm_bf16_swiglu(const void* A, const void* W, void* act, void* gu_out, int M, int I, int K,
                                   long long lda, long long ldw, long long ldd, long long gu_ld, cudaStream_t stream) {
  if (M <= 0 || I <= 0 || K <= 0) return 0;
  if ((I % 4) || (lda % 8) || (ldw % 8) || (ldd % 4) || (gu_out != nullptr && (gu_ld % 4))) return -1;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(W)) & 15) return -2;
  if ((reinterpret_cast<uintptr_t>(act) | reinterpret_cast<uintptr_t>(gu_out)) & 7) return -2;
  CUtensorMap ta, tb;
  if (!make_tmap_2d(&ta, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, K, lda, BK, BM, CU_TENSOR_MAP_SWIZZLE_128B)) return -3;
  // (k, half, row): half 0 = gate rows [0, I), half 1 = up rows [I, 2I)
  if (!make_tmap_3d(&tb, W, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, 2, I, static_cast<uint64_t>(I) * ldw, ldw, BK, 2, 128,
                    CU_TENSOR_MAP_SWIZZLE_128B))
    return -3;
  GemmParams p{};
  p.M = M; p.N = 2 * I; p.K = K; p.D = act; p.ldd = ldd; p.status = status_ptr(); p.k_splits = 1;
  p.gu_out = reinterpret_cast<__nv_bfloat16*>(gu_out); p.gu_ld = gu_ld;
  return static_cast<int>(launch_variant<256, false, false, 4, EPI_SWIGLU>(ta, tb, p, num_sms(), stream));
}

// Row-parallel linear of a tensor-parallel group with the all-reduce done inside the GEMM epilogue over peer memory:
// D[M,N] = sum_r A_r[M,K_r] B_r[N,K_r]^T (+bias), identical bits on every rank. A and B are K-major.
//  part_ptrs[r]  rank r's partial buffer (bf16, 2 * buf_elems elements, peer-mapped); buf_elems >= M*N
//  flag_ptrs[r]  rank r's flags (uint32, >= 4 * ceil(M/128) * ceil(N/BN) entries, zero before the first call)
//  epoch         this rank's two-word call counter (zero before the first call); all ranks must issue the same
//                sequence of calls on these buffers. Waits on peers give up after limit_s seconds and report through
//                vb_gemm_status() (code 13); the output is then undefined but the kernel returns.
extern "C" int vb_gemm_bf16_allreduce_ex(const void* A, const void* B, void* D, const void* bias, int M, int N, int K,
                                         long long lda, long long ldb, long long ldd, int b_mn, int rs_rows,
                                         const unsigned long long* part_ptrs, const unsigned long long* flag_ptrs,
                                         unsigned int* epoch, long long buf_elems, int world, int rank, double limit_s,
                                         cudaStream_t stream);

extern "C" int vb_gemm_bf16_allreduce(const void* A, const void* B, void* D, const void* bias, int M, int N, int K,
                                      long long lda, long long ldb, long long ldd, const unsigned long long* part_ptrs,
                                      const unsigned long long* flag_ptrs, unsigned int* epoch, long long buf_elems,
                                      int world, int rank, double limit_s, cudaStream_t stream) {
  return vb_gemm_bf16_allreduce_ex(A, B, D, bias, M, N, K, lda, ldb, ldd, 0, 0, part_ptrs, flag_ptrs, epoch, buf_elems,
                                   world, rank, limit_s, stream);
}

// b_mn != 0: B is stored [K, N] (the input gradient of a column-parallel layer: D = dY_r W_r summed over the ranks).
// rs_rows > 0: reduce-scatter over rows instead of all-reduce: D is this rank's [rs_rows, N] slice (rows
// [rank * rs_rows, (rank + 1) * rs_rows) of the sum; rows at or beyond M are not written). Every rank must own at least one
// row below M (the wait on its own slabs is what keeps a rank from running two calls ahead of a peer).
extern "C" int vb_gemm_bf16_allreduce_ex(const void* A, const void* B, void* D, const void* bias, int M, int N, int K,
                                         long long lda, long long ldb, long long ldd, int b_mn, int rs_rows,
                                         const unsigned long long* part_ptrs, const unsigned long long* flag_ptrs,
                                         unsigned int* epoch, long long buf_elems, int world, int rank, double limit_s,
                                         cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((N % 8) || (lda % 8) || (ldb % 8) || (ldd % 8)) return -1;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(D)) & 15) return -2;
  if (world < 1 || world > AR_MAX_RANKS || rank < 0 || rank >= world) return -4;
  if (static_cast<long long>(M) * N > buf_elems) return -5;
  const int sms = num_sms();
  // small M (decode): narrow tiles give more CTAs to hide the peer latency; large M (prefill): wide tiles
  const bool wide = N > 128 && M > 1024;
  const int BN = wide ? 256 : 128;
  CUtensorMap ta, tb;
  if (!make_tmap_2d(&ta, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, K, lda, BK, BM, CU_TENSOR_MAP_SWIZZLE_128B)) return -3;
  if (!b_mn) {
    if (!make_tmap_2d(&tb, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, K, ldb, BK, BN, CU_TENSOR_MAP_SWIZZLE_128B)) return -3;
  } else {
    if (!make_tmap_2d(&tb, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, N, ldb, 64, BK, CU_TENSOR_MAP_SWIZZLE_128B)) return -3;
  }
  GemmParams p{};
  p.M = M; p.N = N; p.K = K; p.D = D; p.ldd = ldd;
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.status = status_ptr();
  p.k_splits = 1;
  p.ar_world = world; p.ar_rank = rank; p.ar_buf_elems = buf_elems; p.ar_epoch = epoch;
  p.ar_limit_ns = static_cast<unsigned long long>((limit_s > 0.0 ? limit_s : 2.0) * 1e9);
  if (rs_rows > 0 && static_cast<long long>(rs_rows) * (world - 1) >= M) return -6;  // a rank without rows
  p.ar_rs_rows = rs_rows > 0 ? rs_rows : 0;
  for (int r = 0; r < world; ++r) {
    p.ar_part[r] = part_ptrs[r];
    p.ar_flag[r] = flag_ptrs[r];
  }
  cudaError_t e;
  if (wide) e = b_mn ? launch_variant<256, false, true, 4, EPI_ALLREDUCE>(ta, tb, p, sms, stream)
                     : launch_variant<256, false, false, 4, EPI_ALLREDUCE>(ta, tb, p, sms, stream);
  else e = b_mn ? launch_variant<128, false, true, 6, EPI_ALLREDUCE>(ta, tb, p, sms, stream)
                : launch_variant<128, false, false, 6, EPI_ALLREDUCE>(ta, tb, p, sms, stream);
  return static_cast<int>(e);
}

// GEMM with a staged all-gather running inside it (see GemmParams::fetch_*): D = op(A) * op(B) as vb_gemm_bf16, while
// the copy warps of every CTA move chunks [chunk_begin, chunk_end) (16 KB each) of a byte range that is stored in
// equal slices on the ranks of a group (src_ptrs[r]: rank r's slice, peer-mapped; slice_bytes a multiple of 16 KB) to
// local memory at dst. With b_off_bytes >= 0 the B operand is the K-major matrix at dst + b_off_bytes (rows contiguous,
// ldb == K) and is being gathered by this very launch: `panel_counters` (ceil(N / tile width) words, cleared here) then
// hold every tile back until the rows it reads have landed. With b_off_bytes < 0 the copy is unrelated to this GEMM's
// operands (it prefetches what a later kernel needs) and nothing waits for it inside the kernel. Peers' slices must not
// change while the kernel runs. A wait that runs out after limit_s reports code 14 through vb_gemm_status().
extern "C" int vb_gemm_bf16_fetch(const void* A, const void* B, void* D, const void* bias, int M, int N, int K,
                                  long long lda, long long ldb, long long ldd, int a_mn, int b_mn, int out_f32,
                                  int accumulate, const unsigned long long* src_ptrs, int world, unsigned long long dst,
                                  long long total_bytes, long long slice_bytes, int chunk_begin, int chunk_end,
                                  long long b_off_bytes, unsigned int* panel_counters, double limit_s,
                                  cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda % 8) || (ldb % 8) || (ldd % (out_f32 ? 4 : 8))) return -1;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(D)) & 15) return -2;
  if (world < 1 || world > AR_MAX_RANKS) return -4;
  if (total_bytes < 0 || (total_bytes & 15) || (dst & 15) || slice_bytes <= 0 || total_bytes > slice_bytes * world) return -7;
  if (world > 1 && (slice_bytes % FETCH_CHUNK)) return -7;
  const long long num_chunks = (total_bytes + FETCH_CHUNK - 1) / FETCH_CHUNK;
  if (chunk_begin < 0 || chunk_end < chunk_begin || chunk_end > num_chunks) return -8;
  const bool panel_mode = b_off_bytes >= 0;
  const bool wide = N > 128;
  const int BN = wide ? 256 : 128;
  if (panel_mode) {
    if (a_mn || b_mn || ldb != K || panel_counters == nullptr) return -9;
    if (reinterpret_cast<unsigned long long>(B) != dst + static_cast<unsigned long long>(b_off_bytes)) return -9;
    if (b_off_bytes + static_cast<long long>(N) * K * 2 > total_bytes) return -9;
    // every chunk of B must be copied by this launch, or its panel would never complete
    if (chunk_begin > b_off_bytes / FETCH_CHUNK || chunk_end <= (b_off_bytes + static_cast<long long>(N) * K * 2 - 1) / FETCH_CHUNK)
      return -9;
    cudaError_t em = cudaMemsetAsync(panel_counters, 0, sizeof(unsigned int) * ((N + BN - 1) / BN), stream);
    if (em != cudaSuccess) return static_cast<int>(em);
  }
  CUtensorMap ta, tb;
  bool ok;
  if (!a_mn) ok = make_tmap_2d(&ta, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, K, lda, BK, BM, CU_TENSOR_MAP_SWIZZLE_128B);
  else       ok = make_tmap_2d(&ta, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, M, lda, 64, BK, CU_TENSOR_MAP_SWIZZLE_128B);
  if (!ok) return -3;
  if (!b_mn) ok = make_tmap_2d(&tb, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, K, ldb, BK, BN, CU_TENSOR_MAP_SWIZZLE_128B);
  else       ok = make_tmap_2d(&tb, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, N, ldb, 64, BK, CU_TENSOR_MAP_SWIZZLE_128B);
  if (!ok) return -3;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K; p.D = D; p.ldd = ldd;
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.out_f32 = out_f32; p.accumulate = accumulate;
  p.status = status_ptr();
  p.k_splits = 1;
  for (int r = 0; r < world; ++r) {
    if (src_ptrs[r] & 15) return -2;
    p.fetch_src[r] = src_ptrs[r];
  }
  p.fetch_dst = dst; p.fetch_total = total_bytes; p.fetch_slice = slice_bytes;
  p.fetch_b_off = panel_mode ? b_off_bytes : 0;
  p.fetch_c0 = chunk_begin; p.fetch_c1 = chunk_end;
  p.fetch_panel = panel_mode ? panel_counters : nullptr;
  p.fetch_limit_ns = static_cast<unsigned long long>((limit_s > 0.0 ? limit_s : 2.0) * 1e9);
  const int sms = num_sms();
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  // the copy needs its warps even when the GEMM has few tiles: one CTA per SM, idle tensor pipes cost nothing
  const int grid = (chunk_end > chunk_begin) ? sms : (tiles < sms ? tiles : sms);
  cudaError_t e = cudaSuccess;
#define VB_FETCH(BN_, AM, BMJ, ST)                                                                              \
  do {                                                                                                          \
    auto kern = gemm_bf16_fetch_kernel<BN_, AM, BMJ, ST>;                                                       \
    constexpr int smem = GemmSmem<BN_, ST>::TOTAL;                                                              \
    static bool configured = false;                                                                             \
    if (!configured) {                                                                                          \
      e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);                        \
      if (e != cudaSuccess) return static_cast<int>(e);                                                         \
      configured = true;                                                                                        \
    }                                                                                                           \
    kern<<<grid, GEMM_FETCH_THREADS, smem, stream>>>(ta, tb, p);                                                \
  } while (0)
  if (wide) {
    if (!a_mn && !b_mn) VB_FETCH(256, false, false, 4);
    else if (!a_mn && b_mn) VB_FETCH(256, false, true, 4);
    else if (a_mn && b_mn) VB_FETCH(256, true, true, 4);
    else VB_FETCH(256, true, false, 4);
  } else {
    if (!a_mn && !b_mn) VB_FETCH(128, false, false, 6);
    else if (!a_mn && b_mn) VB_FETCH(128, false, true, 6);
    else if (a_mn && b_mn) VB_FETCH(128, true, true, 6);
    else VB_FETCH(128, true, false, 6);
  }
#undef VB_FETCH
  return static_cast<int>(cudaGetLastError());
}

// Decode-sized variant of the row-parallel linear: the GEMM runs K-split over all SMs into ``splitk_ws``
// (k_splits * M * N floats), then one kernel folds the splits and performs the all-reduce over peer memory.
// flag_ptrs need ceil(M * N / 2048) entries; part_ptrs / epoch / limit_s as for vb_gemm_bf16_allreduce.
extern "C" int vb_gemm_skinny(const void* X, const void* W, void* D, const void* bias, int M, int N, int K, long long ldx,
                              long long ldw, long long ldd, int splits, float* ws, int ws_rows, int partials_only,
                              cudaStream_t stream);
extern "C" int vb_gemm_bf16_splitk_allreduce(const void* A, const void* B, void* D, const void* bias, int M, int N, int K,
                                             long long lda, long long ldb, long long ldd, const unsigned long long* part_ptrs,
                                             const unsigned long long* flag_ptrs, unsigned int* epoch, long long buf_elems,
                                             int world, int rank, double limit_s, int k_splits, float* splitk_ws,
                                             int skinny, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((N % 8) || (ldd % 8) || k_splits < 2 || splitk_ws == nullptr) return -1;
  if (world < 1 || world > AR_MAX_RANKS || rank < 0 || rank >= world) return -4;
  if (static_cast<long long>(M) * N > buf_elems) return -5;
  int rc;
  if (skinny > 0) {
    // the transposed kernel for few tokens: k_splits comes from vb_gemm_skinny_splits
    rc = vb_gemm_skinny(A, B, nullptr, nullptr, M, N, K, lda, ldb, N, k_splits, splitk_ws, M, 1, stream);
  } else {
    g_partials_only = true;
    rc = vb_gemm_bf16_ex(A, B, splitk_ws, nullptr, M, N, K, lda, ldb, N, 0, 0, 1, 0, 0, k_splits, splitk_ws, stream);
    g_partials_only = false;
  }
  if (rc != 0) return rc;
  SplitKAllReduceParams p{};
  p.ws = splitk_ws; p.splits = k_splits; p.total = static_cast<long long>(M) * N; p.N = N;
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias); p.D = reinterpret_cast<__nv_bfloat16*>(D); p.ldd = ldd;
  p.buf_elems = buf_elems; p.epoch = epoch; p.world = world; p.rank = rank; p.status = status_ptr();
  p.limit_ns = static_cast<unsigned long long>((limit_s > 0.0 ? limit_s : 2.0) * 1e9);
  for (int r = 0; r < world; ++r) {
    p.part[r] = part_ptrs[r];
    p.flag[r] = flag_ptrs[r];
  }
  const long long chunks = (p.total / 8 + SKAR_THREADS - 1) / SKAR_THREADS;
  splitk_reduce_allreduce_kernel<<<static_cast<unsigned int>(chunks), SKAR_THREADS, 0, stream>>>(p);
  return static_cast<int>(cudaGetLastError());
}

// Grouped GEMMs of a mixture-of-experts layer; every expert's rows start at a multiple of 128 (zero-padded).
//  mode 1 (forward / dgrad):  D[rows, N] = A[rows, K] * B_e^T for the expert e of each 128-row tile.
//      b_mn = 0: B stacked [E*N, K]; b_mn = 1: B stacked [E*K, N] (K % 64 == 0). tile_expert[i] = expert of tile i,
//      num_mtiles (device scalar) = number of 128-row tiles in use; rows_cap bounds the rows of A and D.
//  mode 2 (wgrad):  D_e[M, N] (+)= A[seg_e, M]^T * B[seg_e, N], D stacked fp32 [E*M, N], seg_start [E+1] (device).
extern "C" int vb_gemm_grouped(int mode, const void* A, const void* B, void* D, int rows_cap, int M, int N, int K, long long lda,
                               long long ldb, long long ldd, int b_mn, int accumulate, int E, const int* tile_expert,
                               const int* num_mtiles, const int* seg_start, cudaStream_t stream) {
  if (rows_cap <= 0 || N <= 0 || E <= 0) return 0;
  if ((N % 8) || (lda % 8) || (ldb % 8) || (rows_cap % 128)) return -1;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(D)) & 15) return -2;
  const int sms = num_sms();
  const bool wide = N > 128;
  const int BN = wide ? 256 : 128;
  CUtensorMap ta, tb;
  GemmParams p{};
  p.status = status_ptr();
  p.k_splits = 1;
  p.grp_mode = mode; p.grp_E = E; p.grp_tile_expert = tile_expert; p.grp_num_mtiles = num_mtiles; p.grp_seg_start = seg_start;
  p.D = D; p.ldd = ldd; p.N = N;
  cudaError_t e;
  int max_tiles;
  const auto bf = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  if (mode == 1) {
    if ((ldd % 8) || (b_mn && (K % 64))) return -1;
    p.M = rows_cap; p.K = K; p.out_f32 = 0; p.accumulate = 0;
    p.grp_b_rows = b_mn ? K : N;
    if (!make_tmap_2d(&ta, A, bf, 2, rows_cap, K, lda, BK, BM, CU_TENSOR_MAP_SWIZZLE_128B)) return -3;
    const bool ok = b_mn ? make_tmap_2d(&tb, B, bf, 2, (uint64_t)E * K, N, ldb, 64, BK, CU_TENSOR_MAP_SWIZZLE_128B)
                         : make_tmap_2d(&tb, B, bf, 2, (uint64_t)E * N, K, ldb, BK, BN, CU_TENSOR_MAP_SWIZZLE_128B);
    if (!ok) return -3;
    max_tiles = (rows_cap / 128) * ((N + BN - 1) / BN);
    const int grid = max_tiles < sms ? max_tiles : sms;
    auto launch = [&](auto kern, int smem) {
      cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
      kern<<<grid, GEMM_THREADS, smem, stream>>>(ta, tb, p);
    };
    if (wide) {
      if (b_mn) launch(gemm_bf16_kernel<256, false, true, 4, EPI_STORE>, GemmSmem<256, 4>::TOTAL);
      else launch(gemm_bf16_kernel<256, false, false, 4, EPI_STORE>, GemmSmem<256, 4>::TOTAL);
    } else {
      if (b_mn) launch(gemm_bf16_kernel<128, false, true, 6, EPI_STORE>, GemmSmem<128, 6>::TOTAL);
      else launch(gemm_bf16_kernel<128, false, false, 6, EPI_STORE>, GemmSmem<128, 6>::TOTAL);
    }
    e = cudaGetLastError();
  } else if (mode == 2) {
    if ((ldd % 4) || (M % 8)) return -1;
    p.M = M; p.K = rows_cap; p.out_f32 = 1; p.accumulate = accumulate;
    if (!make_tmap_2d(&ta, A, bf, 2, rows_cap, M, lda, 64, BK, CU_TENSOR_MAP_SWIZZLE_128B)) return -3;
    if (!make_tmap_2d(&tb, B, bf, 2, rows_cap, N, ldb, 64, BK, CU_TENSOR_MAP_SWIZZLE_128B)) return -3;
    max_tiles = E * ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
    const int grid = max_tiles < sms ? max_tiles : sms;
    if (wide) {
      auto kern = gemm_bf16_kernel<256, true, true, 4, EPI_STORE>;
      cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmSmem<256, 4>::TOTAL);
      kern<<<grid, GEMM_THREADS, GemmSmem<256, 4>::TOTAL, stream>>>(ta, tb, p);
    } else {
      auto kern = gemm_bf16_kernel<128, true, true, 6, EPI_STORE>;
      cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmSmem<128, 6>::TOTAL);
      kern<<<grid, GEMM_THREADS, GemmSmem<128, 6>::TOTAL, stream>>>(ta, tb, p);
    }
    e = cudaGetLastError();
  } else {
    return -4;
  }
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

namespace vb {

// logprob / entropy from the per-tile partials written by EPI_LSE.
__global__ void lmhead_merge_kernel(const float* __restrict__ partial, const float* __restrict__ label_logit,
                                    float* __restrict__ logprob, float* __restrict__ entropy,
                                    float* __restrict__ lse_out, int T, int num_n) {
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= T) return;
  const long long plane = static_cast<long long>(num_n) * T;
  float M = -INFINITY;
  for (int n = 0; n < num_n; ++n) M = fmaxf(M, partial[static_cast<long long>(n) * T + row]);
  float L = 0.f, S = 0.f;
  for (int n = 0; n < num_n; ++n) {
    const long long o = static_cast<long long>(n) * T + row;
    const float w = __expf(partial[o] - M);
    L += partial[plane + o] * w;
    S += partial[2 * plane + o] * w;
  }
  const float lse = M + __logf(L);
  if (logprob) logprob[row] = label_logit[row] - lse;
  if (entropy) entropy[row] = lse - S / L;
  if (lse_out) lse_out[row] = lse;
}

}  // namespace vb

// Number of 256-column tiles (rows of the partial buffer) for a vocabulary of V columns.
extern "C" int vb_lmhead_num_tiles(int V) { return (V + 255) / 256; }

// Forward: hidden [T,H] bf16, weight [V,H] bf16, labels [T] int64 -> logprob/entropy/lse [T] fp32.
// partial: scratch of 3 * num_tiles(V) * T floats; label_logit: scratch of T floats.
extern "C" int vb_lmhead_fwd(const void* hidden, const void* weight, const long long* labels, float inv_temp,
                             float* partial, float* label_logit, float* logprob, float* entropy, float* lse, int T,
                             int V, int H, long long ldh, long long ldw, cudaStream_t stream) {
  if (T <= 0) return 0;
  if ((V % 8) || (H % 8) || (ldh % 8) || (ldw % 8)) return -1;
  CUtensorMap ta, tb;
  if (!make_tmap_2d(&ta, hidden, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, T, H, ldh, BK, BM, CU_TENSOR_MAP_SWIZZLE_128B)) return -3;
  if (!make_tmap_2d(&tb, weight, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, V, H, ldw, BK, 256, CU_TENSOR_MAP_SWIZZLE_128B)) return -3;
  int* status = status_ptr();
  GemmParams p{};
  p.M = T; p.N = V; p.K = H; p.status = status;
  p.labels = labels; p.label_offset = 0; p.inv_temp = inv_temp; p.partial = partial; p.label_logit = label_logit;
  cudaError_t e = launch_variant<256, false, false, 4, EPI_LSE>(ta, tb, p, num_sms(), stream);
  if (e != cudaSuccess) return static_cast<int>(e);
  lmhead_merge_kernel<<<(T + 127) / 128, 128, 0, stream>>>(partial, label_logit, logprob, entropy, lse, T,
                                                         vb_lmhead_num_tiles(V));
  return static_cast<int>(cudaGetLastError());
}

// Backward, one vocabulary chunk [v0, v0+Vc): writes dlogits [T, Vc] bf16 (row stride ldd).
extern "C" int vb_lmhead_dlogits(const void* hidden, const void* weight_chunk, const long long* labels, int v0,
                                 float inv_temp, const float* lse, const float* ex, const float* g_lp,
                                 const float* g_ent, void* dlogits, int T, int Vc, int H, long long ldh, long long ldw,
                                 long long ldd, cudaStream_t stream) {
  if (T <= 0 || Vc <= 0) return 0;
  if ((Vc % 8) || (H % 8) || (ldh % 8) || (ldw % 8) || (ldd % 8)) return -1;
  CUtensorMap ta, tb;
  if (!make_tmap_2d(&ta, hidden, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, T, H, ldh, BK, BM, CU_TENSOR_MAP_SWIZZLE_128B)) return -3;
  if (!make_tmap_2d(&tb, weight_chunk, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, Vc, H, ldw, BK, 256, CU_TENSOR_MAP_SWIZZLE_128B)) return -3;
  int* status = status_ptr();
  GemmParams p{};
  p.M = T; p.N = Vc; p.K = H; p.D = dlogits; p.ldd = ldd; p.status = status;
  p.labels = labels; p.label_offset = v0; p.inv_temp = inv_temp;
  p.lse = lse; p.ex = ex; p.g_lp = g_lp; p.g_ent = g_ent;
  cudaError_t e = launch_variant<256, false, false, 4, EPI_DLOGITS>(ta, tb, p, num_sms(), stream);
  return static_cast<int>(e);
}
