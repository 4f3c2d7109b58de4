// Mixture-of-experts bookkeeping kernels: softmax + top-k router, row gather into the expert-grouped (128-row padded)
// layout, weighted combine back to token order, and the routing-weight gradient.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

namespace vb {

// One warp per token. logits [T, E] (bf16), E <= 1024. Writes the k largest softmax probabilities
// (optionally renormalised to sum 1), their expert ids, and bumps the per-expert histogram.
template <int MAX_PER_LANE>
__global__ void moe_route_topk_kernel(const __nv_bfloat16* __restrict__ logits, long long ld, int T, int E, int k, int renorm,
                                      float* __restrict__ weights, int* __restrict__ experts, int* __restrict__ counts) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= T) return;
  const __nv_bfloat16* row = logits + static_cast<long long>(warp) * ld;
  float v[MAX_PER_LANE];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < MAX_PER_LANE; ++i) {
    const int e = lane + 32 * i;
    v[i] = e < E ? __bfloat162float(row[e]) : -INFINITY;
    mx = fmaxf(mx, v[i]);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < MAX_PER_LANE; ++i) {
    v[i] = (lane + 32 * i < E) ? __expf(v[i] - mx) : -1.f;  // probabilities (unnormalised); -1 marks "taken / absent"
    sum += fmaxf(v[i], 0.f);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  const float inv = 1.f / sum;
  float top_sum = 0.f;
  float my_w = 0.f;
  int my_e = 0;
  for (int j = 0; j < k; ++j) {
    float best = -1.f;
    int bi = 0;
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i) {
      if (v[i] > best) { best = v[i]; bi = lane + 32 * i; }
    }
    // warp arg-max; ties go to the smaller expert id (as torch.topk on a sorted-stable backend does not guarantee an
    // order for exact ties, any fixed rule is acceptable)
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
    }
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i) {
      if (lane + 32 * i == bi) v[i] = -1.f;
    }
    top_sum += best;
    if (lane == j) { my_w = best; my_e = bi; }
  }
  if (lane < k) {
    const float w = renorm ? my_w / top_sum : my_w * inv;
    weights[static_cast<long long>(warp) * k + lane] = w;
    experts[static_cast<long long>(warp) * k + lane] = my_e;
    atomicAdd(counts + my_e, 1);
  }
}

// dst[r, :] = src[map[r], :] * (scale ? scale[r] : 1), or zeros where map[r] < 0.   H % 8 == 0, 16-byte vectors.
__global__ void moe_gather_rows_kernel(const __nv_bfloat16* __restrict__ src, long long lds, const int* __restrict__ map,
                                       const float* __restrict__ scale, __nv_bfloat16* __restrict__ dst, long long ldd,
                                       int rows, int H) {
  const int vec = H >> 3;
  const long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (i >= static_cast<long long>(rows) * vec) return;
  const int r = static_cast<int>(i / vec), c = static_cast<int>(i % vec) * 8;
  const int s = map[r];
  uint4 out = make_uint4(0u, 0u, 0u, 0u);
  if (s >= 0) {
    out = *reinterpret_cast<const uint4*>(src + static_cast<long long>(s) * lds + c);
    if (scale != nullptr) {
      const float f = scale[r];
      __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 t = __bfloat1622float2(h[j]);
        h[j] = __floats2bfloat162_rn(t.x * f, t.y * f);
      }
    }
  }
  *reinterpret_cast<uint4*>(dst + static_cast<long long>(r) * ldd + c) = out;
}

// out[t, :] = sum_j w[t, j] * y[slot[t, j], :]   (fp32 accumulation in a fixed order: deterministic)
__global__ void moe_combine_kernel(const __nv_bfloat16* __restrict__ y, long long ldy, const int* __restrict__ slot,
                                   const float* __restrict__ w, __nv_bfloat16* __restrict__ out, long long ldo, int T, int H,
                                   int k) {
  const int vec = H >> 3;
  const long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (i >= static_cast<long long>(T) * vec) return;
  const int t = static_cast<int>(i / vec), c = static_cast<int>(i % vec) * 8;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  for (int j = 0; j < k; ++j) {
    const int s = slot[static_cast<long long>(t) * k + j];
    const float f = w != nullptr ? w[static_cast<long long>(t) * k + j] : 1.f;
    const uint4 v = *reinterpret_cast<const uint4*>(y + static_cast<long long>(s) * ldy + c);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float2 p2 = __bfloat1622float2(h[q]);
      acc[2 * q] += f * p2.x;
      acc[2 * q + 1] += f * p2.y;
    }
  }
  uint4 o;
  __nv_bfloat162* ho = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
  for (int q = 0; q < 4; ++q) ho[q] = __floats2bfloat162_rn(acc[2 * q], acc[2 * q + 1]);
  *reinterpret_cast<uint4*>(out + static_cast<long long>(t) * ldo + c) = o;
}

// gw[t, j] = <g[t, :], y[slot[t, j], :]>   one warp per (t, j)
__global__ void moe_combine_bwd_w_kernel(const __nv_bfloat16* __restrict__ g, long long ldg, const __nv_bfloat16* __restrict__ y,
                                         long long ldy, const int* __restrict__ slot, float* __restrict__ gw, int T, int H,
                                         int k) {
  const long long warp = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= static_cast<long long>(T) * k) return;
  const int t = static_cast<int>(warp / k);
  const int s = slot[warp];
  const __nv_bfloat16* a = g + static_cast<long long>(t) * ldg;
  const __nv_bfloat16* b = y + static_cast<long long>(s) * ldy;
  float acc = 0.f;
  for (int c = lane * 8; c < H; c += 256) {
    const uint4 va = *reinterpret_cast<const uint4*>(a + c), vb_ = *reinterpret_cast<const uint4*>(b + c);
    const __nv_bfloat162* ha = reinterpret_cast<const __nv_bfloat162*>(&va);
    const __nv_bfloat162* hb = reinterpret_cast<const __nv_bfloat162*>(&vb_);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float2 x = __bfloat1622float2(ha[q]), z = __bfloat1622float2(hb[q]);
      acc += x.x * z.x + x.y * z.y;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) gw[warp] = acc;
}

// ---- expert parallelism over peer memory ------------------------------------------------------------------------
// Dispatch: the permutation into the expert-grouped layout writes each token copy straight into the buffer of the rank
// that owns the expert (peer stores over NVLink): permutation and all-to-all are one kernel, nothing is staged.
//   dst_ptrs[r] = base of rank r's grouped activation buffer [cap, H]; (dest_rank, dest_row) per (token, choice)
__global__ void moe_dispatch_peer_kernel(const __nv_bfloat16* __restrict__ src, long long lds, const unsigned long long* __restrict__ dst_ptrs,
                                         const int* __restrict__ dest_rank, const int* __restrict__ dest_row, int pairs, int k, int H) {
  const int vec = H >> 3;
  const long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (i >= static_cast<long long>(pairs) * vec) return;
  const int pr = static_cast<int>(i / vec), c = static_cast<int>(i % vec) * 8;
  const int row = dest_row[pr];
  if (row < 0) return;  // dropped by the capacity limit
  const uint4 v = *reinterpret_cast<const uint4*>(src + static_cast<long long>(pr / k) * lds + c);
  __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(dst_ptrs[dest_rank[pr]]);
  *reinterpret_cast<uint4*>(dst + static_cast<long long>(row) * H + c) = v;
}

// Combine: out[t] = sum_j w[t,j] * y_{rank(t,j)}[row(t,j)] with the expert outputs read from the owners' buffers (peer
// loads): un-permutation, all-to-all and the weighted sum are one kernel.
__global__ void moe_combine_peer_kernel(const unsigned long long* __restrict__ y_ptrs, const int* __restrict__ src_rank,
                                        const int* __restrict__ src_row, const float* __restrict__ w, __nv_bfloat16* __restrict__ out,
                                        long long ldo, int T, int H, int k) {
  const int vec = H >> 3;
  const long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (i >= static_cast<long long>(T) * vec) return;
  const int t = static_cast<int>(i / vec), c = static_cast<int>(i % vec) * 8;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  for (int j = 0; j < k; ++j) {
    const long long pr = static_cast<long long>(t) * k + j;
    const int row = src_row[pr];
    if (row < 0) continue;
    const float f = w != nullptr ? w[pr] : 1.f;
    const __nv_bfloat16* y = reinterpret_cast<const __nv_bfloat16*>(y_ptrs[src_rank[pr]]);
    const uint4 v = *reinterpret_cast<const uint4*>(y + static_cast<long long>(row) * H + c);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float2 p2 = __bfloat1622float2(h[q]);
      acc[2 * q] += f * p2.x;
      acc[2 * q + 1] += f * p2.y;
    }
  }
  uint4 o;
  __nv_bfloat162* ho = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
  for (int q = 0; q < 4; ++q) ho[q] = __floats2bfloat162_rn(acc[2 * q], acc[2 * q + 1]);
  *reinterpret_cast<uint4*>(out + static_cast<long long>(t) * ldo + c) = o;
}

// Every rank publishes its per-expert token counts into row `rank` of every peer's [W, E] table.
__global__ void moe_publish_counts_kernel(const int* __restrict__ counts, const unsigned long long* __restrict__ table_ptrs, int W,
                                          int rank, int E) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= W * E) return;
  const int r = i / E, e = i % E;
  reinterpret_cast<int*>(table_ptrs[r])[rank * E + e] = counts[e];
}

}  // namespace vb

using namespace vb;

extern "C" int vb_moe_dispatch_peer(const void* src, long long lds, const unsigned long long* dst_ptrs_dev, const int* dest_rank,
                                    const int* dest_row, int pairs, int k, int H, cudaStream_t s) {
  if (pairs <= 0) return 0;
  if (H % 8 || lds % 8) return -1;
  const long long n = static_cast<long long>(pairs) * (H / 8);
  moe_dispatch_peer_kernel<<<static_cast<int>((n + 255) / 256), 256, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(src), lds, dst_ptrs_dev,
                                                                             dest_rank, dest_row, pairs, k, H);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int vb_moe_combine_peer(const unsigned long long* y_ptrs_dev, const int* src_rank, const int* src_row, const float* w, void* out,
                                   long long ldo, int T, int H, int k, cudaStream_t s) {
  if (T <= 0) return 0;
  if (H % 8 || ldo % 8) return -1;
  const long long n = static_cast<long long>(T) * (H / 8);
  moe_combine_peer_kernel<<<static_cast<int>((n + 255) / 256), 256, 0, s>>>(y_ptrs_dev, src_rank, src_row, w,
                                                                            reinterpret_cast<__nv_bfloat16*>(out), ldo, T, H, k);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int vb_moe_publish_counts(const int* counts, const unsigned long long* table_ptrs_dev, int W, int rank, int E, cudaStream_t s) {
  moe_publish_counts_kernel<<<(W * E + 255) / 256, 256, 0, s>>>(counts, table_ptrs_dev, W, rank, E);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int vb_moe_route_topk(const void* logits, long long ld, int T, int E, int k, int renorm, float* weights, int* experts,
                                 int* counts, cudaStream_t s) {
  if (T <= 0) return 0;
  if (E > 1024 || k > 32 || k > E) return -1;
  const int blocks = (T * 32 + 255) / 256;
  const auto* lg = reinterpret_cast<const __nv_bfloat16*>(logits);
  if (E <= 128) moe_route_topk_kernel<4><<<blocks, 256, 0, s>>>(lg, ld, T, E, k, renorm, weights, experts, counts);
  else if (E <= 256) moe_route_topk_kernel<8><<<blocks, 256, 0, s>>>(lg, ld, T, E, k, renorm, weights, experts, counts);
  else moe_route_topk_kernel<32><<<blocks, 256, 0, s>>>(lg, ld, T, E, k, renorm, weights, experts, counts);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int vb_moe_gather_rows(const void* src, long long lds, const int* map, const float* scale, void* dst, long long ldd,
                                  int rows, int H, cudaStream_t s) {
  if (rows <= 0) return 0;
  if (H % 8 || lds % 8 || ldd % 8) return -1;
  const long long n = static_cast<long long>(rows) * (H / 8);
  moe_gather_rows_kernel<<<static_cast<int>((n + 255) / 256), 256, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(src), lds, map, scale,
                                                                           reinterpret_cast<__nv_bfloat16*>(dst), ldd, rows, H);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int vb_moe_combine(const void* y, long long ldy, const int* slot, const float* w, void* out, long long ldo, int T, int H,
                              int k, cudaStream_t s) {
  if (T <= 0) return 0;
  if (H % 8 || ldy % 8 || ldo % 8) return -1;
  const long long n = static_cast<long long>(T) * (H / 8);
  moe_combine_kernel<<<static_cast<int>((n + 255) / 256), 256, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(y), ldy, slot, w,
                                                                       reinterpret_cast<__nv_bfloat16*>(out), ldo, T, H, k);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int vb_moe_combine_bwd_w(const void* g, long long ldg, const void* y, long long ldy, const int* slot, float* gw, int T,
                                    int H, int k, cudaStream_t s) {
  if (T <= 0) return 0;
  if (H % 8 || ldg % 8 || ldy % 8) return -1;
  const long long threads = static_cast<long long>(T) * k * 32;
  moe_combine_bwd_w_kernel<<<static_cast<int>((threads + 255) / 256), 256, 0, s>>>(
      reinterpret_cast<const __nv_bfloat16*>(g), ldg, reinterpret_cast<const __nv_bfloat16*>(y), ldy, slot, gw, T, H, k);
  return static_cast<int>(cudaGetLastError());
}
