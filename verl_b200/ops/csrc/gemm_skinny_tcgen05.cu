// Skinny bf16 GEMM for decode-sized activations: D[M, N] = X[M, K] * W[rows, K]^T (+bias) with M <= 1024 tokens.
//
// The product is computed transposed. A CTA owns 128 rows of W (the UMMA M dimension: no padding of the token count up
// to a multiple of 128) and a block of up to 512 tokens (the UMMA N dimension, one or two instructions of up to 256
// columns), so a weight tile is read from L2 once per K range and token block instead of once per 128-token row tile,
// and the token count only has to be a multiple of 16. The rows of W may be up to four separate row ranges of one
// matrix ("segments": the q | k | v rows, or the gate | up rows, of one tensor-parallel rank inside the replicated
// fused weight); their outputs are written side by side. With few work tiles the K range is split over CTAs until the
// machine is full; the partial sums go to a workspace as fp32 and every split CTA of a tile, once all of them have
// arrived, folds its own share of the token rows (+bias) into the bf16 output: the reduction is spread over all SMs and
// needs no second launch. A launch whose CTAs wait for one another is issued as a cooperative launch (co-residency is
// guaranteed by the driver) and every wait is bounded.
//
// Warp roles (192 threads): warp 0 = TMA producer, warp 1 = MMA issuer (tcgen05.mma, accumulator in TMEM),
// warps 2..5 = epilogue (tcgen05.ld: thread == weight row, registers == tokens) and fold.

#include "tcgen05_common.cuh"

#include <cuda_bf16.h>
#include <stdlib.h>

namespace vb {

constexpr int SK_BM = 128;  // weight rows per tile
constexpr int SK_BK = 64;   // 64 bf16 = 128 bytes = one swizzle row
constexpr int SK_THREADS = 192;
constexpr int SK_BLOCK_TOKENS = 512;  // tokens one CTA covers (TMEM has 512 fp32 columns)
constexpr int SK_MAX_TOKENS = 1024;
constexpr int SK_MAX_SEGS = 4;
constexpr int SK_MAX_STAGES = 8;
constexpr int SK_COUNTERS = 4096;
constexpr int SK_SLOT = 512;  // counters per launch: launches take the eight slots of the table in turn
constexpr int SK_W_BYTES = SK_BM * SK_BK * 2;
constexpr int SK_SMEM_LIMIT = 232448;  // 227 KB of dynamic shared memory per CTA

enum SkinnyStatus : int { SK_OK = 0, SK_TIMEOUT_PRODUCER = 21, SK_TIMEOUT_MMA = 22, SK_TIMEOUT_EPILOGUE = 23, SK_TIMEOUT_FOLD = 24 };

struct SkinnyParams {
  int M, N, K;    // tokens, output columns (sum of the segments' rows), depth
  int mb;         // tokens per block (multiple of 16, <= 512)
  int tblocks;    // token blocks (1 or 2)
  int mh;         // tokens per MMA instruction (multiple of 16, <= 256)
  int halves;     // 1 or 2 instructions cover a block
  int stages;     // depth of the shared-memory ring
  int tmem_cols;  // power of two >= halves * mh
  int splits;     // K splits (1 = none)
  int num_tiles;  // weight tiles over all segments
  int nseg;
  int seg_w0[SK_MAX_SEGS];    // first weight row of the segment
  int seg_rows[SK_MAX_SEGS];  // rows (= output columns) of the segment, a multiple of 8
  int seg_c0[SK_MAX_SEGS];    // first output column of the segment
  int seg_t0[SK_MAX_SEGS + 1];  // first tile of the segment
  int partials_only;  // leave the fp32 partial sums [splits][M][N] in the workspace (the caller folds them)
  __nv_bfloat16* D;
  long long ldd;
  const __nv_bfloat16* bias;  // indexed by weight row
  float* ws;
  long long ws_split_stride;  // floats between the partial sums of consecutive splits
  unsigned int* arrive;  // per (token block, weight tile): split CTAs that have written their partial sums
  unsigned int* done;    // per (token block, weight tile): split CTAs that have finished folding
  int* status;
  unsigned long long wait_ns;
};

__device__ int g_skinny_status[1];
__device__ unsigned int g_sk_arrive[SK_COUNTERS];
__device__ unsigned int g_sk_done[SK_COUNTERS];

__device__ __forceinline__ unsigned int sk_ld_acquire(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void sk_epi_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// Work item -> (K split, token block, weight tile) and the tile's place: first weight row, first output column, valid rows.
struct SkItem {
  int sp, tb, tile, w_row0, out_col0, rows_valid;
};
__device__ __forceinline__ SkItem sk_item(const SkinnyParams& p, int it) {
  SkItem r;
  const int per_split = p.num_tiles * p.tblocks;
  r.sp = it / per_split;
  const int rem = it - r.sp * per_split;
  r.tb = rem / p.num_tiles;
  r.tile = rem - r.tb * p.num_tiles;
  int s = 0;
  while (s + 1 < p.nseg && r.tile >= p.seg_t0[s + 1]) ++s;
  const int off = (r.tile - p.seg_t0[s]) * SK_BM;
  r.w_row0 = p.seg_w0[s] + off;
  r.out_col0 = p.seg_c0[s] + off;
  r.rows_valid = min(SK_BM, p.seg_rows[s] - off);
  return r;
}

__global__ void __launch_bounds__(SK_THREADS, 1)
gemm_skinny_kernel(const __grid_constant__ CUtensorMap tma_w, const __grid_constant__ CUtensorMap tma_x,
                   const SkinnyParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int x_bytes = p.halves * p.mh * (SK_BK * 2);
  const int stage_bytes = SK_W_BYTES + x_bytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + p.stages * stage_bytes);
  uint64_t* full_bar = bars;                       // [stages]
  uint64_t* empty_bar = bars + SK_MAX_STAGES;      // [stages]
  uint64_t* acc_full = bars + 2 * SK_MAX_STAGES;   // accumulator complete
  uint64_t* acc_empty = acc_full + 1;              // accumulator drained by the four epilogue warps
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(acc_empty + 1);
  volatile int* fold_ok = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_items = p.num_tiles * p.tblocks * p.splits;
  const int kb_total = (p.K + SK_BK - 1) / SK_BK;
  const int kb_per = (kb_total + p.splits - 1) / p.splits;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tma_w);
    tma_prefetch_desc(&tma_x);
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(acc_full, 1);
    mbar_init(acc_empty, 4);
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_holder, static_cast<uint32_t>(p.tmem_cols));
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int it = blockIdx.x; it < num_items && ok; it += gridDim.x) {
        const SkItem w = sk_item(p, it);
        const int kb0 = w.sp * kb_per;
        const int kb1 = min(kb_total, kb0 + kb_per);
        const int tok0 = w.tb * p.mb;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1)) {
            atomicExch(p.status, SK_TIMEOUT_PRODUCER);
            ok = false;
            break;
          }
          mbar_expect_tx(&full_bar[stage], static_cast<uint32_t>(stage_bytes));
          uint8_t* sw = smem + stage * stage_bytes;
          uint8_t* sx = sw + SK_W_BYTES;
          const int k0 = kb * SK_BK;
          tma_load_2d(sw, &tma_w, &full_bar[stage], k0, w.w_row0);
          tma_load_2d(sx, &tma_x, &full_bar[stage], k0, tok0);
          if (p.halves == 2) tma_load_2d(sx + p.mh * (SK_BK * 2), &tma_x, &full_bar[stage], k0, tok0 + p.mh);
          if (++stage == p.stages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = make_idesc_f16(SK_BM, p.mh, false, false);
      int stage = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      for (int it = blockIdx.x; it < num_items && ok; it += gridDim.x) {
        const int sp = it / (p.num_tiles * p.tblocks);
        const int kb0 = sp * kb_per;
        const int kb1 = min(kb_total, kb0 + kb_per);
        if (!mbar_wait(acc_empty, acc_phase ^ 1)) {
          atomicExch(p.status, SK_TIMEOUT_MMA);
          break;
        }
        tc_fence_after();
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase)) {
            atomicExch(p.status, SK_TIMEOUT_MMA);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sw = smem_u32(smem + stage * stage_bytes);
          const uint32_t sx = sw + SK_W_BYTES;
#pragma unroll
          for (int k = 0; k < SK_BK / 16; ++k) {
            const uint64_t da = make_smem_desc_sw128(sw + k * 32, 16, 1024);
            const uint32_t accum = (kb > kb0 || k > 0) ? 1u : 0u;
            tc_mma_f16_ss(tmem_base, da, make_smem_desc_sw128(sx + k * 32, 16, 1024), idesc, accum);
            if (p.halves == 2)
              tc_mma_f16_ss(tmem_base + p.mh, da, make_smem_desc_sw128(sx + p.mh * (SK_BK * 2) + k * 32, 16, 1024), idesc, accum);
          }
          tc_commit(&empty_bar[stage]);
          if (++stage == p.stages) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        tc_commit(acc_full);
        acc_phase ^= 1;
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue + fold (warps 2..5)
    const int q = warp & 3;  // TMEM lane quarter this warp may access
    const int et = threadIdx.x - 64;
    uint32_t acc_phase = 0;
    for (int it = blockIdx.x; it < num_items; it += gridDim.x) {
      const SkItem w = sk_item(p, it);
      const int nl = q * 32 + lane;          // weight row within the tile
      const bool n_ok = nl < w.rows_valid;
      const int tok0 = w.tb * p.mb;
      const int mvalid = min(p.mb, p.M - tok0);   // tokens of this block
      const int chunks = (mvalid + 31) / 32;
      if (!mbar_wait(acc_full, acc_phase)) {
        if (lane == 0) atomicExch(p.status, SK_TIMEOUT_EPILOGUE);
        break;
      }
      tc_fence_after();
      acc_phase ^= 1;
      const bool direct = p.splits == 1;
      const float bv = (direct && p.bias != nullptr && n_ok) ? __bfloat162float(p.bias[w.w_row0 + nl]) : 0.f;
      float* wsp = p.ws + static_cast<long long>(w.sp) * p.ws_split_stride + static_cast<long long>(tok0) * p.N + w.out_col0 + nl;
      __nv_bfloat16* dp = p.D + static_cast<long long>(tok0) * p.ldd + w.out_col0 + nl;
#pragma unroll 1
      for (int c = 0; c < chunks; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(tmem_base + c * 32 + (static_cast<uint32_t>(q * 32) << 16), r);
        tmem_ld_wait();
        if (n_ok) {
          const int mrem = mvalid - c * 32;
          if (direct) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (j < mrem) dp[static_cast<long long>(c * 32 + j) * p.ldd] = __float2bfloat16(__uint_as_float(r[j]) + bv);
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (j < mrem) wsp[static_cast<long long>(c * 32 + j) * p.N] = __uint_as_float(r[j]);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty);
      if (direct || p.partials_only) continue;

      // ---- fold: wait until every split of this tile has written its partial sums, then reduce this CTA's rows
      const int slot = w.tb * p.num_tiles + w.tile;
      __threadfence();
      sk_epi_sync();
      if (et == 0) {
        atomicAdd(p.arrive + slot, 1u);
        const uint64_t t0 = global_timer_ns();
        uint32_t spins = 0;
        int ok = 1;
        while (sk_ld_acquire(p.arrive + slot) < static_cast<unsigned int>(p.splits)) {
          if ((++spins & 0x3f) == 0 && global_timer_ns() - t0 > p.wait_ns) {
            atomicExch(p.status, SK_TIMEOUT_FOLD);
            ok = 0;
            break;
          }
        }
        *fold_ok = ok;
      }
      sk_epi_sync();
      if (*fold_ok) {
        const int rows_per = (mvalid + p.splits - 1) / p.splits;
        const int r0 = tok0 + w.sp * rows_per;
        const int r1 = min(tok0 + mvalid, r0 + rows_per);
        const int cl = (et & 31) * 4;  // column within the tile; rows_valid is a multiple of 4
        if (cl < w.rows_valid && r0 < r1) {
          const int col = w.out_col0 + cl;
          float4 b4 = make_float4(0.f, 0.f, 0.f, 0.f);
          if (p.bias != nullptr) {
            const __nv_bfloat16* bp = p.bias + w.w_row0 + cl;
            b4.x = __bfloat162float(bp[0]); b4.y = __bfloat162float(bp[1]);
            b4.z = __bfloat162float(bp[2]); b4.w = __bfloat162float(bp[3]);
          }
          const float* __restrict__ src = p.ws + col;
          const long long split_stride = p.ws_split_stride;
          constexpr int RB = 4;  // rows in flight per thread
#pragma unroll 1
          for (int m = r0 + (et >> 5); m < r1; m += 4 * RB) {
            float4 a[RB];
#pragma unroll
            for (int u = 0; u < RB; ++u) a[u] = b4;
            for (int s = 0; s < p.splits; ++s) {
              float4 v[RB];
#pragma unroll
              for (int u = 0; u < RB; ++u) {
                const int mm = min(m + 4 * u, r1 - 1);  // rows past the end re-read a valid row; they are not stored
                v[u] = __ldcg(reinterpret_cast<const float4*>(src + s * split_stride + static_cast<long long>(mm) * p.N));
              }
#pragma unroll
              for (int u = 0; u < RB; ++u) {
                a[u].x += v[u].x; a[u].y += v[u].y; a[u].z += v[u].z; a[u].w += v[u].w;
              }
            }
#pragma unroll
            for (int u = 0; u < RB; ++u) {
              const int mm = m + 4 * u;
              if (mm < r1) {
                uint2 o;
                o.x = pack_bf16x2(a[u].x, a[u].y);
                o.y = pack_bf16x2(a[u].z, a[u].w);
                *reinterpret_cast<uint2*>(p.D + static_cast<long long>(mm) * p.ldd + col) = o;
              }
            }
          }
        }
      }
      sk_epi_sync();
      if (et == 0) {
        // the split that finishes last returns the tile's counters to zero for the next launch
        __threadfence();
        if (atomicAdd(p.done + slot, 1u) == static_cast<unsigned int>(p.splits - 1)) {
          p.arrive[slot] = 0;
          p.done[slot] = 0;
          __threadfence();
        }
      }
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, static_cast<uint32_t>(p.tmem_cols));
  }
}

// Fills the shape-dependent fields of `p` (token blocks, MMA halves, ring depth, tiles, K splits). force_splits > 0: use that
// many K splits (the caller sized its workspace for them); else choose. Returns false for shapes the kernel does not serve.
static bool sk_plan(int M, int K, int nseg, const int* seg_w0, const int* seg_rows, int force_splits, SkinnyParams& p) {
  if (M <= 0 || M > SK_MAX_TOKENS || K <= 0 || (K % 8) || nseg < 1 || nseg > SK_MAX_SEGS) return false;
  p.M = M; p.K = K; p.nseg = nseg;
  int tiles = 0, cols = 0;
  for (int s = 0; s < nseg; ++s) {
    if (seg_rows[s] <= 0 || (seg_rows[s] % 8) || seg_w0[s] < 0) return false;
    p.seg_w0[s] = seg_w0[s]; p.seg_rows[s] = seg_rows[s]; p.seg_c0[s] = cols; p.seg_t0[s] = tiles;
    tiles += (seg_rows[s] + SK_BM - 1) / SK_BM;
    cols += seg_rows[s];
  }
  p.seg_t0[nseg] = tiles;
  p.num_tiles = tiles;
  p.N = cols;
  p.tblocks = (M + SK_BLOCK_TOKENS - 1) / SK_BLOCK_TOKENS;
  p.mb = ((M + p.tblocks - 1) / p.tblocks + 15) / 16 * 16;
  if (p.mb <= 256) { p.halves = 1; p.mh = p.mb; }
  else { p.halves = 2; p.mh = (p.mb / 2 + 15) / 16 * 16; }
  int tc = 32;
  while (tc < p.halves * p.mh) tc *= 2;
  p.tmem_cols = tc;
  const int stage_bytes = SK_W_BYTES + p.halves * p.mh * (SK_BK * 2);
  int stages = (SK_SMEM_LIMIT - 2048) / stage_bytes;
  if (stages > SK_MAX_STAGES) stages = SK_MAX_STAGES;
  if (stages < 2) return false;
  p.stages = stages;
  const int kb_total = (K + SK_BK - 1) / SK_BK;
  const int sms = num_sms();
  const int work = tiles * p.tblocks;
  int s = 1;
  if (force_splits > 0) s = force_splits;
  else if (work * 2 <= sms && work <= SK_SLOT) {
    s = sms / work;
    if (s > kb_total / 4) s = kb_total / 4;  // at least four k-blocks per split
    if (s > 8) s = 8;
    if (s < 1) s = 1;
  }
  if (s > kb_total) s = kb_total;
  const int kb_per = (kb_total + s - 1) / s;
  p.splits = (kb_total + kb_per - 1) / kb_per;  // every split owns at least one k-block
  return true;
}

}  // namespace vb

using namespace vb;

// Number of K splits the launcher will use for these row ranges (1 = none; the workspace needs splits * M * N floats, N the
// sum of the ranges' rows), or 0 when the shape is not served by the skinny kernel.
extern "C" int vb_gemm_skinny_seg_splits(int M, int K, int nseg, const int* seg_w0, const int* seg_rows) {
  SkinnyParams p{};
  return sk_plan(M, K, nseg, seg_w0, seg_rows, 0, p) ? p.splits : 0;
}
extern "C" int vb_gemm_skinny_splits(int M, int N, int K) {
  const int w0 = 0;
  return vb_gemm_skinny_seg_splits(M, K, 1, &w0, &N);
}

// Status of the launches so far (0 = fine, else the SkinnyStatus of the first wait that ran out); reading a non-zero
// status clears it.
extern "C" int vb_gemm_skinny_status() {
  int h = 0;
  if (cudaMemcpyFromSymbol(&h, g_skinny_status, sizeof(int)) != cudaSuccess) return -1;
  if (h != 0) {
    const int z = 0;
    cudaMemcpyToSymbol(g_skinny_status, &z, sizeof(int));
  }
  return h;
}

// D[M, N] (bf16, row stride ldd) = X[M, K] W_sel^T (+bias_sel), where W_sel stacks the row ranges
// [seg_w0[s], seg_w0[s] + seg_rows[s]) of W (w_rows x K, row stride ldw) and N is the sum of their rows; bias (or null) is
// indexed by the row of W. splits: the value vb_gemm_skinny_seg_splits returned; ws: fp32 workspace of splits * ws_rows * N
// floats when splits > 1 (ws_rows = 0 means M).
// partials_only != 0: leave the partial sums in ws as [splits][ws_rows][N] and do not touch D (bias is ignored).
// Returns 0 on success, a negative code for arguments the kernel does not serve, a positive cudaError_t otherwise.
extern "C" int vb_gemm_skinny_seg(const void* X, const void* W, void* D, const void* bias, int M, int K, int w_rows,
                                  long long ldx, long long ldw, long long ldd, int nseg, const int* seg_w0,
                                  const int* seg_rows, int splits, float* ws, int ws_rows, int partials_only,
                                  cudaStream_t stream) {
  SkinnyParams p{};
  if (!sk_plan(M, K, nseg, seg_w0, seg_rows, splits, p)) return -1;
  if (splits > 0 && p.splits != splits) return -4;  // the caller sized ws for another split count
  for (int s = 0; s < nseg; ++s)
    if (seg_w0[s] + seg_rows[s] > w_rows) return -1;
  if ((ldx % 8) || (ldw % 8)) return -1;
  if ((reinterpret_cast<uintptr_t>(X) | reinterpret_cast<uintptr_t>(W)) & 15) return -2;
  if (p.splits > 1 && ws == nullptr) return -5;
  if (!partials_only && ((ldd % 4) || (reinterpret_cast<uintptr_t>(D) & 7))) return -2;
  const int sms = num_sms();
  const int work = p.num_tiles * p.tblocks;
  if (p.splits > 1 && !partials_only && (work * p.splits > sms || work > SK_SLOT)) return -6;
  CUtensorMap tw, tx;
  if (!make_tmap_2d(&tw, W, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, w_rows, K, ldw, SK_BK, SK_BM, CU_TENSOR_MAP_SWIZZLE_128B)) return -3;
  if (!make_tmap_2d(&tx, X, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, K, ldx, SK_BK, p.mh, CU_TENSOR_MAP_SWIZZLE_128B)) return -3;
  static int* status = nullptr;
  static unsigned int* arrive = nullptr;
  static unsigned int* done = nullptr;
  if (status == nullptr) {
    cudaGetSymbolAddress(reinterpret_cast<void**>(&status), g_skinny_status);
    cudaGetSymbolAddress(reinterpret_cast<void**>(&arrive), g_sk_arrive);
    cudaGetSymbolAddress(reinterpret_cast<void**>(&done), g_sk_done);
  }
  p.partials_only = partials_only ? 1 : 0;
  p.D = reinterpret_cast<__nv_bfloat16*>(D);
  p.ldd = ldd;
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.ws = ws;
  p.ws_split_stride = static_cast<long long>(ws_rows > 0 ? ws_rows : M) * p.N;
  // launches in flight at the same time (several streams) must not share counters
  static unsigned int launch_seq = 0;
  const unsigned int slot = (launch_seq++ % (SK_COUNTERS / SK_SLOT)) * SK_SLOT;
  p.arrive = arrive + slot; p.done = done + slot; p.status = status;
  p.wait_ns = VB_WAIT_LIMIT_NS;
  const int stage_bytes = SK_W_BYTES + p.halves * p.mh * (SK_BK * 2);
  const int smem = p.stages * stage_bytes + 1024 + 256;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_skinny_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SK_SMEM_LIMIT);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  const int items = work * p.splits;
  const bool waits = p.splits > 1 && !partials_only;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(static_cast<unsigned>(items < sms ? items : sms));
  cfg.blockDim = dim3(SK_THREADS);
  cfg.dynamicSmemBytes = static_cast<size_t>(smem);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  // CTAs of a K-split launch wait for one another: a cooperative launch makes the driver guarantee that they are all
  // resident. VERL_B200_SKINNY_COOP=0 launches plainly (the grid never exceeds the SM count and the waits are bounded).
  static const bool coop = [] { const char* v = getenv("VERL_B200_SKINNY_COOP"); return v == nullptr || v[0] != '0'; }();
  if (waits && coop) {
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
  }
  cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_skinny_kernel, tw, tx, p);
  return static_cast<int>(e);
}

// All rows of W[N, K]: one segment.
extern "C" int vb_gemm_skinny(const void* X, const void* W, void* D, const void* bias, int M, int N, int K,
                              long long ldx, long long ldw, long long ldd, int splits, float* ws, int ws_rows,
                              int partials_only, cudaStream_t stream) {
  const int w0 = 0;
  return vb_gemm_skinny_seg(X, W, D, bias, M, K, N, ldx, ldw, ldd, 1, &w0, &N, splits, ws, ws_rows, partials_only, stream);
}
