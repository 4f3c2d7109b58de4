// Rollout-engine kernels: paged KV-cache append, paged decode attention (GQA-aware, one pass over the
// cache per KV head), and the token sampler (temperature + Gumbel-max with the sampled token's log-prob).
// All are bandwidth-bound: the design goal is one coalesced read of every cache byte per decode step.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

namespace vb {

__device__ __forceinline__ float wsum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float wmax(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// ------------------------------------------------------------------------------------------ KV append
// k/v: [T, nkv, hd] with row stride ld (elements); slot[t] = physical cache row (block * block_size + off),
// negative slots are skipped.  Cache layout: [num_slots, nkv, hd].
__global__ void kv_append_kernel(const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v,
                                 long long ldk, long long ldv, const long long* __restrict__ slot,
                                 __nv_bfloat16* __restrict__ kc, __nv_bfloat16* __restrict__ vc, int row_elems) {
  const long long t = blockIdx.x;
  const long long s = slot[t];
  if (s < 0) return;
  const uint4* ks = reinterpret_cast<const uint4*>(k + t * ldk);
  const uint4* vs = reinterpret_cast<const uint4*>(v + t * ldv);
  uint4* kd = reinterpret_cast<uint4*>(kc + s * row_elems);
  uint4* vd = reinterpret_cast<uint4*>(vc + s * row_elems);
  for (int i = threadIdx.x; i < (row_elems >> 3); i += blockDim.x) {
    kd[i] = ks[i];
    vd[i] = vs[i];
  }
}

// Decode step, one launch per layer instead of three: rotary embedding of q (in place), rotary embedding of k, and the
// append of the rotated k and of v to the paged cache. qkv is the projection output [T, (nh + 2 nkv) * hd] (row stride ld):
// q heads first, then k heads, then v heads. One block per token; threads cover the rotary pairs of all q and k heads and
// the 16-byte pieces of v. A token whose slot is negative (an inactive sequence) only gets its q rotated.
__global__ void rope_kv_append_kernel(__nv_bfloat16* __restrict__ qkv, long long ld, const int* __restrict__ pos,
                                      const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                      const long long* __restrict__ slot, __nv_bfloat16* __restrict__ kc,
                                      __nv_bfloat16* __restrict__ vc, int nh, int nkv, int hd) {
  const long long t = blockIdx.x;
  const int half = hd >> 1, pairs = half >> 1;  // two rotary pairs per thread
  const int p = pos[t];
  const long long s = slot[t];
  __nv_bfloat16* row = qkv + t * ld;
  const int rot_heads = nh + nkv;
  for (int idx = threadIdx.x; idx < rot_heads * pairs; idx += blockDim.x) {
    const int h = idx / pairs, i = (idx - h * pairs) * 2;
    __nv_bfloat16* base = row + static_cast<long long>(h) * hd;
    const float2 c = *reinterpret_cast<const float2*>(cos_t + static_cast<long long>(p) * half + i);
    const float2 sn = *reinterpret_cast<const float2*>(sin_t + static_cast<long long>(p) * half + i);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(base + i));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(base + half + i));
    const __nv_bfloat162 lo = __floats2bfloat162_rn(a.x * c.x - b.x * sn.x, a.y * c.y - b.y * sn.y);
    const __nv_bfloat162 hi = __floats2bfloat162_rn(b.x * c.x + a.x * sn.x, b.y * c.y + a.y * sn.y);
    *reinterpret_cast<__nv_bfloat162*>(base + i) = lo;
    *reinterpret_cast<__nv_bfloat162*>(base + half + i) = hi;
    if (h >= nh && s >= 0) {  // a key head: the rotated values also go to the cache
      __nv_bfloat16* kd = kc + s * static_cast<long long>(nkv) * hd + static_cast<long long>(h - nh) * hd;
      *reinterpret_cast<__nv_bfloat162*>(kd + i) = lo;
      *reinterpret_cast<__nv_bfloat162*>(kd + half + i) = hi;
    }
  }
  if (s >= 0) {
    const uint4* vs = reinterpret_cast<const uint4*>(row + static_cast<long long>(nh + nkv) * hd);
    uint4* vd = reinterpret_cast<uint4*>(vc + s * static_cast<long long>(nkv) * hd);
    for (int i = threadIdx.x; i < (nkv * hd) >> 3; i += blockDim.x) vd[i] = vs[i];
  }
}

// ------------------------------------------------------------------------------------------ decode attention
// q: [B, nh, hd] (row stride ldq); cache: [num_slots, nkv, hd]; block_table: [B, max_blocks]; ctx_len: [B].
// grid = (B, nkv); 4 warps; each warp walks 32-token tiles: the score phase is lane-per-token (no shuffles
// in the dot products), the value phase lane-per-dimension (coalesced 256-byte rows).
constexpr int DEC_WARPS = 4;
constexpr int MAXG = 8;

template <int HD>
__global__ void __launch_bounds__(DEC_WARPS * 32)
paged_decode_kernel(const __nv_bfloat16* __restrict__ q, long long ldq, const __nv_bfloat16* __restrict__ kc,
                    const __nv_bfloat16* __restrict__ vc, const int* __restrict__ block_table, int max_blocks,
                    const int* __restrict__ ctx_len, __nv_bfloat16* __restrict__ out, long long ldo, int nh, int nkv,
                    int block_size, float scale_log2) {
  constexpr int DPL = HD / 32;  // dims per lane in the value phase
  const int b = blockIdx.x, kvh = blockIdx.y;
  const int G = nh / nkv;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int len = ctx_len[b];

  __shared__ float q_s[MAXG][HD];
  __shared__ float p_s[DEC_WARPS][MAXG][32];
  __shared__ float o_s[DEC_WARPS][MAXG][HD];
  __shared__ float ml_s[DEC_WARPS][MAXG][2];

  for (int i = threadIdx.x; i < G * HD; i += blockDim.x) {
    const int g = i / HD, d = i % HD;
    q_s[g][d] = __bfloat162float(q[b * ldq + static_cast<long long>(kvh * G + g) * HD + d]) * scale_log2;
  }
  __syncthreads();

  float m[MAXG], l[MAXG], o[MAXG][DPL];
#pragma unroll
  for (int g = 0; g < MAXG; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int d = 0; d < DPL; ++d) o[g][d] = 0.f;
  }
  const int* bt = block_table + static_cast<long long>(b) * max_blocks;
  const long long row_stride = static_cast<long long>(nkv) * HD;

  for (int t0 = warp * 32; t0 < len; t0 += DEC_WARPS * 32) {
    const int t = t0 + lane;
    const bool valid = t < len;
    long long row = 0;
    if (valid) row = (static_cast<long long>(bt[t / block_size]) * block_size + (t % block_size)) * row_stride +
                     static_cast<long long>(kvh) * HD;
    float s[MAXG];
#pragma unroll
    for (int g = 0; g < MAXG; ++g) s[g] = 0.f;
    if (valid) {
      const uint4* kr = reinterpret_cast<const uint4*>(kc + row);
#pragma unroll 4
      for (int c = 0; c < HD / 8; ++c) {
        const uint4 kv = kr[c];
        const __nv_bfloat162* k2 = reinterpret_cast<const __nv_bfloat162*>(&kv);
        float kf[8];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(k2[j]);
          kf[2 * j] = f.x;
          kf[2 * j + 1] = f.y;
        }
#pragma unroll
        for (int g = 0; g < MAXG; ++g) {
          if (g < G) {
            const float4 qa = *reinterpret_cast<const float4*>(&q_s[g][c * 8]);
            const float4 qb = *reinterpret_cast<const float4*>(&q_s[g][c * 8 + 4]);
            s[g] += qa.x * kf[0] + qa.y * kf[1] + qa.z * kf[2] + qa.w * kf[3] + qb.x * kf[4] + qb.y * kf[5] +
                    qb.z * kf[6] + qb.w * kf[7];
          }
        }
      }
    }
    float alpha[MAXG];
#pragma unroll
    for (int g = 0; g < MAXG; ++g) {
      if (g < G) {
        const float sv = valid ? s[g] : -INFINITY;
        const float mn = fmaxf(m[g], wmax(sv));
        const float p = exp2f(sv - mn);
        alpha[g] = exp2f(m[g] - mn);
        l[g] = l[g] * alpha[g] + wsum(p);
        m[g] = mn;
        p_s[warp][g][lane] = p;
      }
    }
    __syncwarp();
#pragma unroll
    for (int g = 0; g < MAXG; ++g) {
      if (g < G) {
#pragma unroll
        for (int d = 0; d < DPL; ++d) o[g][d] *= alpha[g];
      }
    }
    const int nt = min(32, len - t0);
    for (int tt = 0; tt < nt; ++tt) {
      const long long r = __shfl_sync(0xffffffffu, row, tt);
      float vf[DPL];
      if constexpr (DPL == 4) {
        const uint2 raw = *reinterpret_cast<const uint2*>(vc + r + lane * 4);
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
        const float2 c = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
        vf[0] = a.x; vf[1] = a.y; vf[2] = c.x; vf[3] = c.y;
      } else {
        const uint32_t raw = *reinterpret_cast<const uint32_t*>(vc + r + lane * 2);
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw));
        vf[0] = a.x; vf[1] = a.y;
      }
#pragma unroll
      for (int g = 0; g < MAXG; ++g) {
        if (g < G) {
          const float p = p_s[warp][g][tt];
#pragma unroll
          for (int d = 0; d < DPL; ++d) o[g][d] += p * vf[d];
        }
      }
    }
    __syncwarp();
  }

  // merge the four warps
#pragma unroll
  for (int g = 0; g < MAXG; ++g) {
    if (g < G) {
      if (lane == 0) {
        ml_s[warp][g][0] = m[g];
        ml_s[warp][g][1] = l[g];
      }
#pragma unroll
      for (int d = 0; d < DPL; ++d) o_s[warp][g][lane * DPL + d] = o[g][d];
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < G * HD; i += blockDim.x) {
    const int g = i / HD, d = i % HD;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) M = fmaxf(M, ml_s[w][g][0]);
    float L = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) {
      const float f = (ml_s[w][g][0] == -INFINITY) ? 0.f : exp2f(ml_s[w][g][0] - M);
      L += ml_s[w][g][1] * f;
      acc += o_s[w][g][d] * f;
    }
    out[b * ldo + static_cast<long long>(kvh * G + g) * HD + d] = __float2bfloat16(L > 0.f ? acc / L : 0.f);
  }
}

// ------------------------------------------------------------------------------------------ sampler
__device__ __forceinline__ uint64_t mix64(uint64_t z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

// One block per row. logits [B, V] bf16 (row stride ld). Columns >= valid_vocab are masked out.
// Greedy when inv_temp <= 0 (the log-prob is then reported at temperature 1).
__global__ void sample_kernel(const __nv_bfloat16* __restrict__ logits, long long ld, int V, int valid_vocab,
                              float inv_temp, const long long* __restrict__ seeds, long long step,
                              long long* __restrict__ tokens, float* __restrict__ logprobs) {
  const int row = blockIdx.x;
  const bool greedy = inv_temp <= 0.f;
  const float it = greedy ? 1.f : inv_temp;
  const __nv_bfloat16* lr = logits + row * ld;
  const uint64_t key = mix64(static_cast<uint64_t>(seeds[row]) ^ (static_cast<uint64_t>(step) * 0xD1342543DE82EF95ull));
  float m = -INFINITY, l = 0.f, best = -INFINITY, best_x = 0.f;
  int best_i = 0;
  for (int i = threadIdx.x; i < valid_vocab; i += blockDim.x) {
    const float x = __bfloat162float(lr[i]) * it;
    const float mn = fmaxf(m, x);
    l = l * __expf(m - mn) + __expf(x - mn);
    m = mn;
    float score = x;
    if (!greedy) {
      const uint64_t h = mix64(key + static_cast<uint64_t>(i));
      const float u = (static_cast<float>(h >> 40) + 0.5f) * (1.0f / 16777216.0f);  // (0,1)
      score = x - __logf(-__logf(u));
    }
    if (score > best) {
      best = score;
      best_i = i;
      best_x = x;
    }
  }
  __shared__ float sm[32], sl[32], sb[32], sx[32];
  __shared__ int si[32];
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float m2 = __shfl_xor_sync(0xffffffffu, m, o), l2 = __shfl_xor_sync(0xffffffffu, l, o);
    const float b2 = __shfl_xor_sync(0xffffffffu, best, o), x2 = __shfl_xor_sync(0xffffffffu, best_x, o);
    const int i2 = __shfl_xor_sync(0xffffffffu, best_i, o);
    const float mn = fmaxf(m, m2);
    l = (mn == -INFINITY) ? 0.f : l * __expf(m - mn) + l2 * __expf(m2 - mn);
    m = mn;
    if (b2 > best || (b2 == best && i2 < best_i)) {
      best = b2;
      best_i = i2;
      best_x = x2;
    }
  }
  if (lane == 0) {
    sm[w] = m; sl[w] = l; sb[w] = best; sx[w] = best_x; si[w] = best_i;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const int nw = blockDim.x >> 5;
    for (int k = 1; k < nw; ++k) {
      const float mn = fmaxf(m, sm[k]);
      l = (mn == -INFINITY) ? 0.f : l * __expf(m - mn) + sl[k] * __expf(sm[k] - mn);
      m = mn;
      if (sb[k] > best || (sb[k] == best && si[k] < best_i)) {
        best = sb[k];
        best_i = si[k];
        best_x = sx[k];
      }
    }
    tokens[row] = best_i;
    if (logprobs) logprobs[row] = best_x - (m + __logf(l));
  }
}

// ---- top-k / top-p (nucleus) sampling without a sort.
// bf16 logits have at most 65536 distinct values, so the k-th largest value and the nucleus boundary are found exactly by
// two rounds of 256-bin histograms over an order-preserving 16-bit key (high byte, then low byte inside the boundary
// bin): counts for top-k, probability mass for top-p (evaluated on the distribution that top-k left, as the reference
// samplers do). Every element whose key is >= the boundary key is kept: elements that tie with the boundary value stay
// in. The token is then drawn by Gumbel-max among the kept ones and its log-prob is that of the renormalised
// distribution. One block per row; the row (V * 2 bytes) is re-read from L2 by each pass.
__device__ __forceinline__ unsigned int bf16_key(__nv_bfloat16 v) {
  const unsigned int u = __bfloat16_as_ushort(v);
  return (u & 0x8000u) ? (~u & 0xffffu) : (u | 0x8000u);
}

__global__ void sample_topkp_kernel(const __nv_bfloat16* __restrict__ logits, long long ld, int valid_vocab, float inv_temp,
                                    int top_k, float top_p, const long long* __restrict__ seeds, long long step,
                                    long long* __restrict__ tokens, float* __restrict__ logprobs) {
  const int row = blockIdx.x;
  const __nv_bfloat16* lr = logits + row * ld;
  __shared__ int cnt[256];
  __shared__ float mass[256];
  __shared__ float red[32];
  __shared__ int sh_i[4];
  __shared__ float sh_f[4];
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
  auto block_max = [&](float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    if (lane == 0) red[w] = v;
    __syncthreads();
    if (threadIdx.x == 0) {
      float t = red[0];
      for (int k = 1; k < nw; ++k) t = fmaxf(t, red[k]);
      sh_f[0] = t;
    }
    __syncthreads();
    const float r = sh_f[0];
    __syncthreads();
    return r;
  };
  auto block_sum = [&](float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (lane == 0) red[w] = v;
    __syncthreads();
    if (threadIdx.x == 0) {
      float t = 0.f;
      for (int k = 0; k < nw; ++k) t += red[k];   // fixed order
      sh_f[0] = t;
    }
    __syncthreads();
    const float r = sh_f[0];
    __syncthreads();
    return r;
  };
  // pass A: row maximum (of the temperature-scaled logits)
  float m = -INFINITY;
  for (int i = threadIdx.x; i < valid_vocab; i += blockDim.x) m = fmaxf(m, __bfloat162float(lr[i]) * inv_temp);
  m = block_max(m);
  unsigned int thr = 0;  // keep key >= thr
  if (top_k > 0 && top_k < valid_vocab) {
    // passes B, C: the key of the k-th largest element
    for (int b = threadIdx.x; b < 256; b += blockDim.x) cnt[b] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < valid_vocab; i += blockDim.x) atomicAdd(&cnt[bf16_key(lr[i]) >> 8], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
      int c = 0, b = 255;
      for (; b > 0; --b) {
        if (c + cnt[b] >= top_k) break;
        c += cnt[b];
      }
      sh_i[0] = b;
      sh_i[1] = c;  // elements strictly above bin b
    }
    __syncthreads();
    const int hb = sh_i[0], above = sh_i[1];
    __syncthreads();
    for (int b = threadIdx.x; b < 256; b += blockDim.x) cnt[b] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < valid_vocab; i += blockDim.x) {
      const unsigned int k = bf16_key(lr[i]);
      if (static_cast<int>(k >> 8) == hb) atomicAdd(&cnt[k & 255u], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int c = above, b = 255;
      for (; b > 0; --b) {
        if (c + cnt[b] >= top_k) break;
        c += cnt[b];
      }
      sh_i[2] = (hb << 8) | b;
    }
    __syncthreads();
    thr = static_cast<unsigned int>(sh_i[2]);
    __syncthreads();
  }
  if (top_p < 1.f) {
    // passes D, E: the smallest set of the largest elements whose mass reaches top_p of what top-k kept
    for (int b = threadIdx.x; b < 256; b += blockDim.x) mass[b] = 0.f;
    __syncthreads();
    float z = 0.f;
    for (int i = threadIdx.x; i < valid_vocab; i += blockDim.x) {
      const unsigned int k = bf16_key(lr[i]);
      if (k >= thr) {
        const float e = __expf(__bfloat162float(lr[i]) * inv_temp - m);
        z += e;
        atomicAdd(&mass[k >> 8], e);
      }
    }
    z = block_sum(z);
    if (threadIdx.x == 0) {
      float c = 0.f;
      int b = 255;
      for (; b > 0; --b) {
        if (c + mass[b] >= top_p * z) break;
        c += mass[b];
      }
      sh_i[0] = b;
      sh_f[1] = c;
    }
    __syncthreads();
    const int hb = sh_i[0];
    const float above = sh_f[1];
    __syncthreads();
    for (int b = threadIdx.x; b < 256; b += blockDim.x) mass[b] = 0.f;
    __syncthreads();
    for (int i = threadIdx.x; i < valid_vocab; i += blockDim.x) {
      const unsigned int k = bf16_key(lr[i]);
      if (k >= thr && static_cast<int>(k >> 8) == hb) atomicAdd(&mass[k & 255u], __expf(__bfloat162float(lr[i]) * inv_temp - m));
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      float c = above;
      int b = 255;
      for (; b > 0; --b) {
        if (c + mass[b] >= top_p * z) break;
        c += mass[b];
      }
      const unsigned int tp = (static_cast<unsigned int>(hb) << 8) | static_cast<unsigned int>(b);
      sh_i[2] = static_cast<int>(tp > thr ? tp : thr);
    }
    __syncthreads();
    thr = static_cast<unsigned int>(sh_i[2]);
    __syncthreads();
  }
  // pass F: Gumbel-max among the kept elements, normaliser of the kept set
  const uint64_t key = mix64(static_cast<uint64_t>(seeds[row]) ^ (static_cast<uint64_t>(step) * 0xD1342543DE82EF95ull));
  float l = 0.f, best = -INFINITY, best_x = 0.f;
  int best_i = 0;
  for (int i = threadIdx.x; i < valid_vocab; i += blockDim.x) {
    if (bf16_key(lr[i]) < thr) continue;
    const float x = __bfloat162float(lr[i]) * inv_temp;
    l += __expf(x - m);
    const uint64_t h = mix64(key + static_cast<uint64_t>(i));
    const float u = (static_cast<float>(h >> 40) + 0.5f) * (1.0f / 16777216.0f);
    const float score = x - __logf(-__logf(u));
    if (score > best) {
      best = score;
      best_i = i;
      best_x = x;
    }
  }
  l = block_sum(l);
  __shared__ float sb[32], sx[32];
  __shared__ int si[32];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float b2 = __shfl_xor_sync(0xffffffffu, best, o), x2 = __shfl_xor_sync(0xffffffffu, best_x, o);
    const int i2 = __shfl_xor_sync(0xffffffffu, best_i, o);
    if (b2 > best || (b2 == best && i2 < best_i)) {
      best = b2;
      best_i = i2;
      best_x = x2;
    }
  }
  if (lane == 0) {
    sb[w] = best; sx[w] = best_x; si[w] = best_i;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int k = 1; k < nw; ++k) {
      if (sb[k] > best || (sb[k] == best && si[k] < best_i)) {
        best = sb[k];
        best_i = si[k];
        best_x = sx[k];
      }
    }
    tokens[row] = best_i;
    if (logprobs) logprobs[row] = best_x - (m + __logf(l));
  }
}

}  // namespace vb

using namespace vb;

extern "C" {

int vb_kv_append(const void* k, const void* v, long long ldk, long long ldv, const long long* slot, void* kc, void* vc,
                 int T, int nkv, int hd, cudaStream_t s) {
  if (T == 0) return 0;
  if ((nkv * hd) % 8) return -1;
  kv_append_kernel<<<T, 128, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(k), reinterpret_cast<const __nv_bfloat16*>(v),
                                     ldk, ldv, slot, reinterpret_cast<__nv_bfloat16*>(kc),
                                     reinterpret_cast<__nv_bfloat16*>(vc), nkv * hd);
  return static_cast<int>(cudaGetLastError());
}

int vb_rope_kv_append(void* qkv, long long ld, const int* pos, const float* cos_t, const float* sin_t, const long long* slot,
                      void* kc, void* vc, int T, int nh, int nkv, int hd, cudaStream_t s) {
  if (T == 0) return 0;
  if ((hd % 8) || (ld % 8) || ((nkv * hd) % 8)) return -1;
  if ((reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(vc)) & 15) return -2;
  rope_kv_append_kernel<<<T, 256, 0, s>>>(reinterpret_cast<__nv_bfloat16*>(qkv), ld, pos, cos_t, sin_t, slot,
                                          reinterpret_cast<__nv_bfloat16*>(kc), reinterpret_cast<__nv_bfloat16*>(vc), nh, nkv, hd);
  return static_cast<int>(cudaGetLastError());
}

int vb_paged_decode(const void* q, long long ldq, const void* kc, const void* vc, const int* block_table,
                    int max_blocks, const int* ctx_len, void* out, long long ldo, int B, int nh, int nkv, int hd,
                    int block_size, float scale, cudaStream_t s) {
  if (B == 0) return 0;
  if (nh % nkv || nh / nkv > MAXG) return -1;
  const float sl2 = scale * 1.4426950408889634f;
  dim3 grid(B, nkv);
  if (hd == 128)
    paged_decode_kernel<128><<<grid, DEC_WARPS * 32, 0, s>>>(
        reinterpret_cast<const __nv_bfloat16*>(q), ldq, reinterpret_cast<const __nv_bfloat16*>(kc),
        reinterpret_cast<const __nv_bfloat16*>(vc), block_table, max_blocks, ctx_len,
        reinterpret_cast<__nv_bfloat16*>(out), ldo, nh, nkv, block_size, sl2);
  else if (hd == 64)
    paged_decode_kernel<64><<<grid, DEC_WARPS * 32, 0, s>>>(
        reinterpret_cast<const __nv_bfloat16*>(q), ldq, reinterpret_cast<const __nv_bfloat16*>(kc),
        reinterpret_cast<const __nv_bfloat16*>(vc), block_table, max_blocks, ctx_len,
        reinterpret_cast<__nv_bfloat16*>(out), ldo, nh, nkv, block_size, sl2);
  else
    return -2;
  return static_cast<int>(cudaGetLastError());
}

int vb_sample_topkp(const void* logits, long long ld, int B, int V, int valid_vocab, float inv_temp, int top_k, float top_p,
                    const long long* seeds, long long step, long long* tokens, float* logprobs, cudaStream_t s) {
  if (B == 0) return 0;
  if (valid_vocab <= 0 || valid_vocab > V) valid_vocab = V;
  if (inv_temp <= 0.f || top_p <= 0.f) return -1;  // greedy decoding goes through vb_sample
  sample_topkp_kernel<<<B, 1024, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(logits), ld, valid_vocab, inv_temp, top_k, top_p,
                                         seeds, step, tokens, logprobs);
  return static_cast<int>(cudaGetLastError());
}

int vb_sample(const void* logits, long long ld, int B, int V, int valid_vocab, float inv_temp, const long long* seeds,
              long long step, long long* tokens, float* logprobs, cudaStream_t s) {
  if (B == 0) return 0;
  if (valid_vocab <= 0 || valid_vocab > V) valid_vocab = V;
  sample_kernel<<<B, 1024, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(logits), ld, V, valid_vocab, inv_temp, seeds,
                                   step, tokens, logprobs);
  return static_cast<int>(cudaGetLastError());
}

}  // extern "C"
