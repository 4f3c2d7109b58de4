// Paged decode attention, bandwidth-oriented version: one CTA per (sequence, KV head [, KV split]).
//
// The KV cache of a sequence is streamed once, block by block (64 tokens = one cache page), by TMA into a
// 3-stage shared-memory ring (128B swizzle); the whole GQA group (<= 16 query heads sharing the KV head)
// is processed together on the tensor cores with the query heads as the M dimension of m16n8k16 MMAs:
//   S[16 heads, 16 tokens] = Q[16, hd] K^T       (B fragments by ldmatrix from the swizzled K tile)
//   O[16 heads, hd]       += P[16, 16] V          (P reuses the S accumulator registers; V by ldmatrix.trans)
// Each of the 4 warps owns 16 of the 64 tokens of a page and keeps its own online-softmax state; the warps
// (and optional KV splits) are merged at the end.  The work per cache byte is ~8x lower than a CUDA-core
// formulation, so the kernel is limited by HBM bandwidth rather than by instruction issue.
// (The MMA shape here is a 16-row sliver: tcgen05's 128-row tiles would idle 7/8 of the tensor core and need
// the same traffic, so the warp-level MMA is the right tool for this memory-bound op.)
#include "tcgen05_common.cuh"

#include <math.h>

namespace vb {

constexpr int PD_PAGE = 64;
constexpr int PD_STAGES = 3;
constexpr int PD_THREADS = 128;

struct PagedDecodeParams {
  const __nv_bfloat16* q;  // [B, nh, hd], row stride ldq
  long long ldq;
  const int* block_table;  // [B, max_blocks]
  int max_blocks;
  const int* ctx_len;  // [B]
  __nv_bfloat16* out;  // [B, nh, hd], row stride ldo
  long long ldo;
  float* part_o;   // [B, nh, nsplit, hd]   (nsplit > 1)
  float* part_ml;  // [B, nh, nsplit, 2]
  int nh, nkv, nsplit;
  float scale_log2;
  int* status;
  // grouped-prefix mode: the leading skip[b] pages of sequence b are covered by the group kernel below; this kernel then
  // starts behind them and writes its partial results into slots [slot0, slot0 + nsplit) of nslots per (sequence, head)
  const int* skip;  // [B] or null
  int slot0, nslots;
};

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <int HD>
struct PDSmem {
  static constexpr int TILE = PD_PAGE * HD * 2;           // one of K or V
  static constexpr int STAGE = 2 * TILE;
  static constexpr int OFF_Q = PD_STAGES * STAGE;          // 16 x HD bf16
  static constexpr int OFF_MERGE = 0;                      // 4 warps x 16 heads x (HD + 2) floats, aliases the ring
  static constexpr int OFF_BAR = OFF_Q + 16 * HD * 2;
  static_assert(4 * 16 * (HD + 2) * 4 <= PD_STAGES * STAGE, "merge buffer must fit in the ring");
  static constexpr int TOTAL = OFF_BAR + 64 + 1024;
};

template <int HD>
__global__ void __launch_bounds__(PD_THREADS, 2)
paged_decode_tma_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                        const PagedDecodeParams p) {
  using L = PDSmem<HD>;
  constexpr int PANELS = HD / 64;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(smem + L::OFF_Q);
  float* sM = reinterpret_cast<float*>(smem + L::OFF_MERGE);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + L::OFF_BAR);
  uint64_t* empty = full + PD_STAGES;

  const int b = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = p.nh / p.nkv;
  const int len = p.ctx_len[b];
  const int npages = (len + PD_PAGE - 1) / PD_PAGE;
  const int first = p.skip != nullptr ? min(p.skip[b], npages) : 0;
  const int per = (npages - first + p.nsplit - 1) / p.nsplit;
  const int pg0 = first + split * per, pg1 = min(npages, pg0 + per);
  const int n = max(0, pg1 - pg0);
  const int* bt = p.block_table + static_cast<long long>(b) * p.max_blocks;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
    for (int s = 0; s < PD_STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 4);
    }
    mbar_fence_init();
  }
  // Q (zero padded to 16 heads) -> smem, row-major [16][HD]
  for (int i = threadIdx.x; i < 16 * HD / 8; i += PD_THREADS) {
    const int g = i / (HD / 8), c = i % (HD / 8);
    uint4 v = make_uint4(0, 0, 0, 0);
    if (g < G) v = *reinterpret_cast<const uint4*>(p.q + b * p.ldq + static_cast<long long>(kvh * G + g) * HD + c * 8);
    *reinterpret_cast<uint4*>(sQ + g * HD + c * 8) = v;
  }
  __syncthreads();

  auto issue = [&](int i) {  // page i of this CTA's range into stage i % STAGES (thread 0 only)
    const int s = i % PD_STAGES;
    const int row = bt[pg0 + i] * PD_PAGE;
    uint8_t* dst = smem + s * L::STAGE;
    mbar_expect_tx(&full[s], L::STAGE);
#pragma unroll
    for (int c = 0; c < PANELS; ++c) {
      tma_load_2d(dst + c * (PD_PAGE * 128), &tm_k, &full[s], kvh * HD + 64 * c, row);
      tma_load_2d(dst + L::TILE + c * (PD_PAGE * 128), &tm_v, &full[s], kvh * HD + 64 * c, row);
    }
  };
  if (threadIdx.x == 0) {
    for (int i = 0; i < min(n, PD_STAGES); ++i) issue(i);
  }

  // Q fragments (A operand), all k-steps, kept in registers
  uint32_t qa[HD / 16][4];
  {
    const int mi = lane >> 3, r = lane & 7;
#pragma unroll
    for (int k = 0; k < HD / 16; ++k) {
      const int row = (mi & 1) * 8 + r, col = k * 16 + (mi >> 1) * 8;
      ldsm_x4(qa[k], smem_u32(sQ + row * HD + col));
    }
  }
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  float o[HD / 8][4];
#pragma unroll
  for (int j = 0; j < HD / 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;

  bool ok = true;
  const int t0w = warp * 16;  // this warp's tokens inside a page
  for (int i = 0; i < n; ++i) {
    const int s = i % PD_STAGES;
    if (!__all_sync(0xffffffffu, mbar_wait(&full[s], (i / PD_STAGES) & 1))) { ok = false; break; }
    const uint32_t kbase = smem_u32(smem + s * L::STAGE), vbase = kbase + L::TILE;
    // ---- S = Q K^T for tokens [t0w, t0w+16): two 8-token column blocks
    float sacc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
    {
      const int mi = lane >> 3, r = lane & 7;
#pragma unroll
      for (int nb = 0; nb < 2; ++nb) {
        const int tok = t0w + nb * 8 + r;
#pragma unroll
        for (int k2 = 0; k2 < HD / 32; ++k2) {  // two k-steps per ldmatrix.x4
          const int dc = k2 * 4 + mi;           // 16-byte chunk index along d
          uint32_t kb[4];
          ldsm_x4(kb, kbase + (dc >> 3) * (PD_PAGE * 128) + tok * 128 + (((dc & 7) ^ (tok & 7)) << 4));
          mma_bf16_16816(sacc[nb], qa[2 * k2], kb[0], kb[1]);
          mma_bf16_16816(sacc[nb], qa[2 * k2 + 1], kb[2], kb[3]);
        }
      }
    }
    // ---- online softmax (rows: heads lane/4 and lane/4 + 8; columns: this warp's 16 tokens)
    const int tok_base = (pg0 + i) * PD_PAGE + t0w + (lane & 3) * 2;
    float alpha[2];
    uint32_t pa[4];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      float v[4];
#pragma unroll
      for (int nb = 0; nb < 2; ++nb)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int t = tok_base + nb * 8 + e;
          v[nb * 2 + e] = (t < len) ? sacc[nb][h * 2 + e] * p.scale_log2 : -INFINITY;
        }
      float mx = fmaxf(fmaxf(v[0], v[1]), fmaxf(v[2], v[3]));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float mn = fmaxf(m_run[h], mx);
      const float mu = (mn == -INFINITY) ? 0.f : mn;
      alpha[h] = (mn == -INFINITY) ? 1.f : exp2f(m_run[h] - mn);
      float e0 = exp2f(v[0] - mu), e1 = exp2f(v[1] - mu), e2 = exp2f(v[2] - mu), e3 = exp2f(v[3] - mu);
      float sum = (e0 + e1) + (e2 + e3);
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      l_run[h] = l_run[h] * alpha[h] + sum;
      m_run[h] = mn;
      pa[h] = pack_bf16x2(e0, e1);       // a0 (h=0) / a1 (h=1): tokens 0..7 of the warp's 16
      pa[2 + h] = pack_bf16x2(e2, e3);   // a2 / a3: tokens 8..15
    }
    // ---- O = O * alpha + P V
    {
      const int mi = lane >> 3, r = lane & 7;
      const int tok = t0w + (mi & 1) * 8 + r;
#pragma unroll
      for (int j2 = 0; j2 < HD / 16; ++j2) {  // two 8-wide d blocks per ldmatrix.x4.trans
        const int dc = j2 * 2 + (mi >> 1);
        uint32_t vb[4];
        ldsm_x4_t(vb, vbase + (dc >> 3) * (PD_PAGE * 128) + tok * 128 + (((dc & 7) ^ (tok & 7)) << 4));
#pragma unroll
        for (int q2 = 0; q2 < 2; ++q2) {
          float* oo = o[2 * j2 + q2];
          oo[0] *= alpha[0]; oo[1] *= alpha[0]; oo[2] *= alpha[1]; oo[3] *= alpha[1];
          mma_bf16_16816(o[2 * j2 + q2], pa, vb[2 * q2], vb[2 * q2 + 1]);
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty[s]);
    if (threadIdx.x == 0 && i + PD_STAGES < n) {
      if (mbar_wait(&empty[s], (i / PD_STAGES) & 1)) issue(i + PD_STAGES);
      else atomicExch(p.status, ST_TIMEOUT_PRODUCER);  // the consumers' next wait on this stage then runs out too
    }
    __syncwarp();
  }
  if (!ok && lane == 0) atomicExch(p.status, ST_TIMEOUT_EPILOGUE);

  // ---- merge the 4 warps: sM[warp][head][HD + 2] = {o..., m, l}  (the ring is idle now)
  __syncthreads();
  {
    const int h0 = lane >> 2, cpair = (lane & 3) * 2;
#pragma unroll
    for (int j = 0; j < HD / 8; ++j) {
      float* r0 = sM + (warp * 16 + h0) * (HD + 2) + j * 8 + cpair;
      float* r1 = sM + (warp * 16 + h0 + 8) * (HD + 2) + j * 8 + cpair;
      r0[0] = o[j][0]; r0[1] = o[j][1]; r1[0] = o[j][2]; r1[1] = o[j][3];
    }
    if ((lane & 3) == 0) {
      sM[(warp * 16 + h0) * (HD + 2) + HD] = m_run[0];
      sM[(warp * 16 + h0) * (HD + 2) + HD + 1] = l_run[0];
      sM[(warp * 16 + h0 + 8) * (HD + 2) + HD] = m_run[1];
      sM[(warp * 16 + h0 + 8) * (HD + 2) + HD + 1] = l_run[1];
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * HD; idx += PD_THREADS) {
    const int g = idx / HD, d = idx % HD;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) M = fmaxf(M, sM[(w * 16 + g) * (HD + 2) + HD]);
    float Lsum = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float mw = sM[(w * 16 + g) * (HD + 2) + HD];
      const float f = (mw == -INFINITY) ? 0.f : exp2f(mw - M);
      Lsum += sM[(w * 16 + g) * (HD + 2) + HD + 1] * f;
      acc += sM[(w * 16 + g) * (HD + 2) + d] * f;
    }
    const int head = kvh * G + g;
    if (p.nslots <= 1) {
      p.out[b * p.ldo + static_cast<long long>(head) * HD + d] = __float2bfloat16(Lsum > 0.f ? acc / Lsum : 0.f);
    } else {
      const long long base = (static_cast<long long>(b) * p.nh + head) * p.nslots + p.slot0 + split;
      p.part_o[base * HD + d] = acc;
      if (d == 0) {
        p.part_ml[base * 2] = M;
        p.part_ml[base * 2 + 1] = Lsum;
        if (p.skip != nullptr && split == 0 && first == 0) {
          // a sequence outside every group: its prefix slots hold the neutral element of the merge
          for (int sl = 0; sl < p.slot0; ++sl) {
            p.part_ml[(base - p.slot0 - split + sl) * 2] = -INFINITY;
            p.part_ml[(base - p.slot0 - split + sl) * 2 + 1] = 0.f;
          }
        }
      }
    }
  }
}

// ---- grouped prefix: the sequences of a group (the samples of one prompt) share their leading pages. One CTA per
// (group, KV head, split of the shared pages) streams those pages ONCE; warp w holds the query heads of member w and
// runs all 64 tokens of every page against them (four 16-token sub-blocks, one online softmax per member). The result
// of each member goes to partial slot `split` of that sequence; the per-sequence kernel above covers the pages behind
// the shared ones and paged_decode_merge_kernel joins the slots by their log-sum-exp.
constexpr int PG_MEMBERS = 8;

struct PagedDecodeGroupParams {
  const __nv_bfloat16* q;
  long long ldq;
  const int* block_table;
  int max_blocks;
  const int* members;    // [NG, PG_MEMBERS] sequence index or -1; member 0 of a live group is valid
  const int* grp_pages;  // [NG] shared pages (0: empty group)
  float* part_o;
  float* part_ml;
  int nh, nkv, psplit, nslots;
  float scale_log2;
  int* status;
};

template <int HD>
struct PGSmem {
  static constexpr int TILE = PD_PAGE * HD * 2;
  static constexpr int STAGE = 2 * TILE;
  static constexpr int OFF_Q = PD_STAGES * STAGE;            // PG_MEMBERS x 16 x HD bf16
  static constexpr int OFF_BAR = OFF_Q + PG_MEMBERS * 16 * HD * 2;
  static constexpr int TOTAL = OFF_BAR + 64 + 1024;
};

template <int HD>
__global__ void __launch_bounds__(PG_MEMBERS * 32, 1)
paged_decode_group_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                          const PagedDecodeGroupParams p) {
  using L = PGSmem<HD>;
  constexpr int PANELS = HD / 64;
  const int g = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
  const int npages = p.grp_pages[g];
  if (npages <= 0) return;  // uniform over the CTA
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(smem + L::OFF_Q);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + L::OFF_BAR);
  uint64_t* empty = full + PD_STAGES;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = p.nh / p.nkv;
  const int b = p.members[g * PG_MEMBERS + warp];
  const int per = (npages + p.psplit - 1) / p.psplit;
  const int pg0 = split * per, pg1 = min(npages, pg0 + per);
  const int n = max(0, pg1 - pg0);
  const int* bt = p.block_table + static_cast<long long>(p.members[g * PG_MEMBERS]) * p.max_blocks;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
    for (int s = 0; s < PD_STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], PG_MEMBERS);
    }
    mbar_fence_init();
  }
  // this warp's member: query heads of the KV head, zero padded to 16 rows
  for (int i = lane; i < 16 * HD / 8; i += 32) {
    const int gh = i / (HD / 8), c = i % (HD / 8);
    uint4 v = make_uint4(0, 0, 0, 0);
    if (b >= 0 && gh < G) v = *reinterpret_cast<const uint4*>(p.q + b * p.ldq + static_cast<long long>(kvh * G + gh) * HD + c * 8);
    *reinterpret_cast<uint4*>(sQ + (warp * 16 + gh) * HD + c * 8) = v;
  }
  __syncthreads();

  auto issue = [&](int i) {
    const int s = i % PD_STAGES;
    const int row = bt[pg0 + i] * PD_PAGE;
    uint8_t* dst = smem + s * L::STAGE;
    mbar_expect_tx(&full[s], L::STAGE);
#pragma unroll
    for (int c = 0; c < PANELS; ++c) {
      tma_load_2d(dst + c * (PD_PAGE * 128), &tm_k, &full[s], kvh * HD + 64 * c, row);
      tma_load_2d(dst + L::TILE + c * (PD_PAGE * 128), &tm_v, &full[s], kvh * HD + 64 * c, row);
    }
  };
  if (threadIdx.x == 0) {
    for (int i = 0; i < min(n, PD_STAGES); ++i) issue(i);
  }
  uint32_t qa[HD / 16][4];
  {
    const int mi = lane >> 3, r = lane & 7;
#pragma unroll
    for (int k = 0; k < HD / 16; ++k) {
      const int row = (mi & 1) * 8 + r, col = k * 16 + (mi >> 1) * 8;
      ldsm_x4(qa[k], smem_u32(sQ + (warp * 16 + row) * HD + col));
    }
  }
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  float o[HD / 8][4];
#pragma unroll
  for (int j = 0; j < HD / 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;

  bool ok = true;
  for (int i = 0; i < n; ++i) {
    const int s = i % PD_STAGES;
    if (!__all_sync(0xffffffffu, mbar_wait(&full[s], (i / PD_STAGES) & 1))) { ok = false; break; }
    const uint32_t kbase = smem_u32(smem + s * L::STAGE), vbase = kbase + L::TILE;
    if (b >= 0) {
#pragma unroll 1
      for (int tb = 0; tb < PD_PAGE / 16; ++tb) {
        const int t0w = tb * 16;
        float sacc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
        {
          const int mi = lane >> 3, r = lane & 7;
#pragma unroll
          for (int nb = 0; nb < 2; ++nb) {
            const int tok = t0w + nb * 8 + r;
#pragma unroll
            for (int k2 = 0; k2 < HD / 32; ++k2) {
              const int dc = k2 * 4 + mi;
              uint32_t kb[4];
              ldsm_x4(kb, kbase + (dc >> 3) * (PD_PAGE * 128) + tok * 128 + (((dc & 7) ^ (tok & 7)) << 4));
              mma_bf16_16816(sacc[nb], qa[2 * k2], kb[0], kb[1]);
              mma_bf16_16816(sacc[nb], qa[2 * k2 + 1], kb[2], kb[3]);
            }
          }
        }
        float alpha[2];
        uint32_t pa[4];
#pragma unroll
        for (int h = 0; h < 2; ++h) {  // every token of a shared page lies inside every member's context
          const float v0 = sacc[0][h * 2] * p.scale_log2, v1 = sacc[0][h * 2 + 1] * p.scale_log2;
          const float v2 = sacc[1][h * 2] * p.scale_log2, v3 = sacc[1][h * 2 + 1] * p.scale_log2;
          float mx = fmaxf(fmaxf(v0, v1), fmaxf(v2, v3));
          mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
          mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
          const float mn = fmaxf(m_run[h], mx);
          alpha[h] = exp2f(m_run[h] - mn);
          const float e0 = exp2f(v0 - mn), e1 = exp2f(v1 - mn), e2 = exp2f(v2 - mn), e3 = exp2f(v3 - mn);
          float sum = (e0 + e1) + (e2 + e3);
          sum += __shfl_xor_sync(0xffffffffu, sum, 1);
          sum += __shfl_xor_sync(0xffffffffu, sum, 2);
          l_run[h] = l_run[h] * alpha[h] + sum;
          m_run[h] = mn;
          pa[h] = pack_bf16x2(e0, e1);
          pa[2 + h] = pack_bf16x2(e2, e3);
        }
        {
          const int mi = lane >> 3, r = lane & 7;
          const int tok = t0w + (mi & 1) * 8 + r;
#pragma unroll
          for (int j2 = 0; j2 < HD / 16; ++j2) {
            const int dc = j2 * 2 + (mi >> 1);
            uint32_t vb[4];
            ldsm_x4_t(vb, vbase + (dc >> 3) * (PD_PAGE * 128) + tok * 128 + (((dc & 7) ^ (tok & 7)) << 4));
#pragma unroll
            for (int q2 = 0; q2 < 2; ++q2) {
              float* oo = o[2 * j2 + q2];
              oo[0] *= alpha[0]; oo[1] *= alpha[0]; oo[2] *= alpha[1]; oo[3] *= alpha[1];
              mma_bf16_16816(o[2 * j2 + q2], pa, vb[2 * q2], vb[2 * q2 + 1]);
            }
          }
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty[s]);
    if (threadIdx.x == 0 && i + PD_STAGES < n) {
      if (mbar_wait(&empty[s], (i / PD_STAGES) & 1)) issue(i + PD_STAGES);
      else atomicExch(p.status, ST_TIMEOUT_PRODUCER);
    }
    __syncwarp();
  }
  if (!ok && lane == 0) atomicExch(p.status, ST_TIMEOUT_EPILOGUE);
  if (b < 0) return;
  // this member's partial result for slot `split` (a split without pages writes the neutral element)
  const int h0 = lane >> 2, cpair = (lane & 3) * 2;
#pragma unroll
  for (int hh = 0; hh < 2; ++hh) {
    const int gh = h0 + hh * 8;
    if (gh >= G) continue;
    const long long base = (static_cast<long long>(b) * p.nh + kvh * G + gh) * p.nslots + split;
#pragma unroll
    for (int j = 0; j < HD / 8; ++j)
      *reinterpret_cast<float2*>(p.part_o + base * HD + j * 8 + cpair) = make_float2(o[j][hh * 2], o[j][hh * 2 + 1]);
    if ((lane & 3) == 0) {
      p.part_ml[base * 2] = m_run[hh];
      p.part_ml[base * 2 + 1] = l_run[hh];
    }
  }
}

// merge KV splits: one thread per (b, head, d)
__global__ void paged_decode_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                          __nv_bfloat16* __restrict__ out, long long ldo, int B, int nh, int hd,
                                          int nsplit) {
  const long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (idx >= static_cast<long long>(B) * nh * hd) return;
  const int d = idx % hd;
  const long long bh = idx / hd;
  float M = -INFINITY;
  for (int s = 0; s < nsplit; ++s) M = fmaxf(M, part_ml[(bh * nsplit + s) * 2]);
  float L = 0.f, acc = 0.f;
  for (int s = 0; s < nsplit; ++s) {
    const float ms = part_ml[(bh * nsplit + s) * 2];
    if (ms == -INFINITY) continue;  // an empty slot: its values were never written
    const float f = exp2f(ms - M);
    L += part_ml[(bh * nsplit + s) * 2 + 1] * f;
    acc += part_o[(bh * nsplit + s) * hd + d] * f;
  }
  const long long b = bh / nh, h = bh % nh;
  out[b * ldo + h * hd + d] = __float2bfloat16(L > 0.f ? acc / L : 0.f);
}

__device__ int g_pd_status[4];

template <int HD>
static cudaError_t launch_pd(const CUtensorMap& tk, const CUtensorMap& tv, const PagedDecodeParams& p, int B,
                             cudaStream_t stream) {
  auto kern = paged_decode_tma_kernel<HD>;
  constexpr int smem = PDSmem<HD>::TOTAL;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    configured = true;
  }
  dim3 grid(B, p.nkv, p.nsplit);
  kern<<<grid, PD_THREADS, smem, stream>>>(tk, tv, p);
  return cudaGetLastError();
}

}  // namespace vb

using namespace vb;

// Scratch needed for nsplit > 1: part_o of B*nh*nsplit*hd floats and part_ml of B*nh*nsplit*2 floats.
extern "C" int vb_paged_decode_v2(const void* q, long long ldq, const void* kc, const void* vc, long long num_slots,
                                  const int* block_table, int max_blocks, const int* ctx_len, void* out, long long ldo,
                                  int B, int nh, int nkv, int hd, int block_size, float scale, int nsplit, float* part_o,
                                  float* part_ml, cudaStream_t stream) {
  if (B == 0) return 0;
  if (block_size != PD_PAGE || (hd != 64 && hd != 128) || nh % nkv || nh / nkv > 16) return -2;
  if (nsplit < 1) nsplit = 1;
  CUtensorMap tk, tv;
  const auto bf = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const uint64_t cols = static_cast<uint64_t>(nkv) * hd;
  if (!make_tmap_2d(&tk, kc, bf, 2, num_slots, cols, cols, 64, PD_PAGE, CU_TENSOR_MAP_SWIZZLE_128B)) return -3;
  if (!make_tmap_2d(&tv, vc, bf, 2, num_slots, cols, cols, 64, PD_PAGE, CU_TENSOR_MAP_SWIZZLE_128B)) return -3;
  static int* status = nullptr;
  if (status == nullptr) cudaGetSymbolAddress(reinterpret_cast<void**>(&status), g_pd_status);
  PagedDecodeParams p{};
  p.q = reinterpret_cast<const __nv_bfloat16*>(q); p.ldq = ldq; p.block_table = block_table; p.max_blocks = max_blocks;
  p.ctx_len = ctx_len; p.out = reinterpret_cast<__nv_bfloat16*>(out); p.ldo = ldo; p.part_o = part_o; p.part_ml = part_ml;
  p.nh = nh; p.nkv = nkv; p.nsplit = nsplit; p.scale_log2 = scale * 1.4426950408889634f; p.status = status;
  p.skip = nullptr; p.slot0 = 0; p.nslots = nsplit;
  cudaError_t e = (hd == 128) ? launch_pd<128>(tk, tv, p, B, stream) : launch_pd<64>(tk, tv, p, B, stream);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (nsplit > 1) {
    const long long total = static_cast<long long>(B) * nh * hd;
    paged_decode_merge_kernel<<<static_cast<int>((total + 255) / 256), 256, 0, stream>>>(
        part_o, part_ml, reinterpret_cast<__nv_bfloat16*>(out), ldo, B, nh, hd, nsplit);
    e = cudaGetLastError();
  }
  return static_cast<int>(e);
}

template <int HD>
static cudaError_t launch_pg(const CUtensorMap& tk, const CUtensorMap& tv, const PagedDecodeGroupParams& p, int NG,
                             cudaStream_t stream) {
  auto kern = paged_decode_group_kernel<HD>;
  constexpr int smem = PGSmem<HD>::TOTAL;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    configured = true;
  }
  dim3 grid(NG, p.nkv, p.psplit);
  kern<<<grid, PG_MEMBERS * 32, smem, stream>>>(tk, tv, p);
  return cudaGetLastError();
}

// Decode attention for sequences that share their leading pages in groups (the samples of one prompt).
//  members [NG, 8]   sequence index of every member of a group (-1: none; entry 0 valid when grp_pages > 0)
//  grp_pages [NG]    pages shared by the members of the group (0: no such group)
//  skip [B]          for every sequence the number of leading pages its group covers (0: in no group)
// The group kernel reads the shared pages once per group into `psplit` partial slots, the per-sequence kernel covers the
// rest of every context in `nsplit` slots, and the merge kernel joins the psplit + nsplit slots.
// Scratch: part_o of B*nh*(psplit+nsplit)*hd floats, part_ml of B*nh*(psplit+nsplit)*2 floats.
extern "C" int vb_paged_decode_grouped(const void* q, long long ldq, const void* kc, const void* vc, long long num_slots,
                                       const int* block_table, int max_blocks, const int* ctx_len, const int* members,
                                       const int* grp_pages, const int* skip, int NG, void* out, long long ldo, int B, int nh,
                                       int nkv, int hd, int block_size, float scale, int psplit, int nsplit, float* part_o,
                                       float* part_ml, cudaStream_t stream) {
  if (B == 0) return 0;
  if (block_size != PD_PAGE || (hd != 64 && hd != 128) || nh % nkv || nh / nkv > 16) return -2;
  if (psplit < 1 || nsplit < 1 || NG < 1 || part_o == nullptr || part_ml == nullptr) return -4;
  CUtensorMap tk, tv;
  const auto bf = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const uint64_t cols = static_cast<uint64_t>(nkv) * hd;
  if (!make_tmap_2d(&tk, kc, bf, 2, num_slots, cols, cols, 64, PD_PAGE, CU_TENSOR_MAP_SWIZZLE_128B)) return -3;
  if (!make_tmap_2d(&tv, vc, bf, 2, num_slots, cols, cols, 64, PD_PAGE, CU_TENSOR_MAP_SWIZZLE_128B)) return -3;
  static int* status = nullptr;
  if (status == nullptr) cudaGetSymbolAddress(reinterpret_cast<void**>(&status), g_pd_status);
  const int nslots = psplit + nsplit;
  PagedDecodeGroupParams g{};
  g.q = reinterpret_cast<const __nv_bfloat16*>(q); g.ldq = ldq; g.block_table = block_table; g.max_blocks = max_blocks;
  g.members = members; g.grp_pages = grp_pages; g.part_o = part_o; g.part_ml = part_ml; g.nh = nh; g.nkv = nkv;
  g.psplit = psplit; g.nslots = nslots; g.scale_log2 = scale * 1.4426950408889634f; g.status = status;
  cudaError_t e = (hd == 128) ? launch_pg<128>(tk, tv, g, NG, stream) : launch_pg<64>(tk, tv, g, NG, stream);
  if (e != cudaSuccess) return static_cast<int>(e);
  PagedDecodeParams p{};
  p.q = g.q; p.ldq = ldq; p.block_table = block_table; p.max_blocks = max_blocks; p.ctx_len = ctx_len;
  p.out = reinterpret_cast<__nv_bfloat16*>(out); p.ldo = ldo; p.part_o = part_o; p.part_ml = part_ml;
  p.nh = nh; p.nkv = nkv; p.nsplit = nsplit; p.scale_log2 = g.scale_log2; p.status = status;
  p.skip = skip; p.slot0 = psplit; p.nslots = nslots;
  e = (hd == 128) ? launch_pd<128>(tk, tv, p, B, stream) : launch_pd<64>(tk, tv, p, B, stream);
  if (e != cudaSuccess) return static_cast<int>(e);
  const long long total = static_cast<long long>(B) * nh * hd;
  paged_decode_merge_kernel<<<static_cast<int>((total + 255) / 256), 256, 0, stream>>>(
      part_o, part_ml, reinterpret_cast<__nv_bfloat16*>(out), ldo, B, nh, hd, nslots);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int vb_pd_status() {
  int h[4] = {0, 0, 0, 0};
  if (cudaMemcpyFromSymbol(h, g_pd_status, sizeof(h)) != cudaSuccess) return -1;
  if (h[0] != 0) {
    int z[4] = {0, 0, 0, 0};
    cudaMemcpyToSymbol(g_pd_status, z, sizeof(z));
  }
  return h[0];
}
