// Advantage estimators on the device: GRPO group-normalised outcome advantage and GAE (reverse scan with
// mask carry-through) plus masked whitening.  Semantics follow verl/trainer/ppo/core_algos.py:216-331.
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

namespace vb {

// scores[b] = sum_t rewards[b,t]; group statistics accumulated with atomics: stats[g] = {sum, sumsq, count}.
__global__ void grpo_scores_kernel(const float* __restrict__ rewards, const int* __restrict__ group, int B, int L,
                                   float* __restrict__ scores, float* __restrict__ stats) {
  const int b = blockIdx.x;
  __shared__ float red[32];
  float s = 0.f;
  for (int t = threadIdx.x; t < L; t += blockDim.x) s += rewards[static_cast<long long>(b) * L + t];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float tot = 0.f;
    for (int w = 0; w < (blockDim.x + 31) / 32; ++w) tot += red[w];
    scores[b] = tot;
    const int g = group[b];
    atomicAdd(&stats[3 * g], tot);
    atomicAdd(&stats[3 * g + 1], tot * tot);
    atomicAdd(&stats[3 * g + 2], 1.f);
  }
}

// adv[b,t] = (score - mean_g) / (std_g + eps) * mask[b,t]   (unbiased std; singleton group: mean 0, std 1)
__global__ void grpo_adv_kernel(const float* __restrict__ scores, const int* __restrict__ group,
                                const float* __restrict__ stats, const float* __restrict__ mask, int B, int L,
                                float eps, int norm_by_std, float* __restrict__ adv) {
  const int b = blockIdx.x;
  const int g = group[b];
  const float n = stats[3 * g + 2];
  float mean = 0.f, sd = 1.f;
  if (n > 1.5f) {
    mean = stats[3 * g] / n;
    const float var = fmaxf((stats[3 * g + 1] - n * mean * mean) / (n - 1.f), 0.f);
    sd = sqrtf(var);
  }
  const float a = norm_by_std ? (scores[b] - mean) / (sd + eps) : (scores[b] - mean);
  for (int t = threadIdx.x; t < L; t += blockDim.x) {
    const long long i = static_cast<long long>(b) * L + t;
    adv[i] = a * mask[i];
  }
}

// GAE: one thread per sequence, reverse scan. On masked tokens next-value and last-gae carry through.
__global__ void gae_kernel(const float* __restrict__ rewards, const float* __restrict__ values,
                           const float* __restrict__ mask, int B, int L, float gamma, float lam,
                           float* __restrict__ adv, float* __restrict__ ret) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  float nextv = 0.f, last = 0.f;
  for (int t = L - 1; t >= 0; --t) {
    const long long i = static_cast<long long>(b) * L + t;
    const float v = values[i], mk = mask[i];
    const float delta = rewards[i] + gamma * nextv - v;
    const float cand = delta + gamma * lam * last;
    nextv = v * mk + (1.f - mk) * nextv;
    last = cand * mk + (1.f - mk) * last;
    adv[i] = last;
    ret[i] = last + v;
  }
}

// acc = {sum(x*m), sum(x*x*m), sum(m)}
__global__ void masked_moments_kernel(const float* __restrict__ x, const float* __restrict__ mask, long long n,
                                      float* __restrict__ acc) {
  float s = 0.f, ss = 0.f, c = 0.f;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float m = mask[i], v = x[i];
    s += v * m;
    ss += v * v * m;
    c += m;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    s += __shfl_xor_sync(0xffffffffu, s, o);
    ss += __shfl_xor_sync(0xffffffffu, ss, o);
    c += __shfl_xor_sync(0xffffffffu, c, o);
  }
  if ((threadIdx.x & 31) == 0) {
    atomicAdd(&acc[0], s);
    atomicAdd(&acc[1], ss);
    atomicAdd(&acc[2], c);
  }
}
// x <- (x - mean) * rsqrt(var + 1e-8) * (apply_mask ? mask : 1), unbiased variance
__global__ void whiten_kernel(float* __restrict__ x, const float* __restrict__ mask, long long n,
                              const float* __restrict__ acc, int apply_mask) {
  const long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (i >= n) return;
  const float c = acc[2];
  const float mean = acc[0] / (c + 1e-8f);
  float var = acc[1] / (c + 1e-8f) - mean * mean;
  var = fmaxf(var, 0.f) * (c / fmaxf(c - 1.f, 1.f));
  const float w = (x[i] - mean) * rsqrtf(var + 1e-8f);
  x[i] = apply_mask ? w * mask[i] : w;
}

}  // namespace vb

using namespace vb;

extern "C" {

// stats: scratch of 3 * num_groups floats, zeroed by this call.
int vb_grpo_advantage(const float* rewards, const float* mask, const int* group, int B, int L, int num_groups,
                      float eps, int norm_by_std, float* scores, float* stats, float* adv, cudaStream_t s) {
  if (B == 0) return 0;
  cudaMemsetAsync(stats, 0, sizeof(float) * 3 * num_groups, s);
  grpo_scores_kernel<<<B, 128, 0, s>>>(rewards, group, B, L, scores, stats);
  grpo_adv_kernel<<<B, 128, 0, s>>>(scores, group, stats, mask, B, L, eps, norm_by_std, adv);
  return static_cast<int>(cudaGetLastError());
}

// acc: scratch of 4 floats, zeroed by this call. Whitening of the advantages over the whole batch (statistics
// over unmasked tokens, result not re-masked) is applied when `whiten` is non-zero.
int vb_gae(const float* rewards, const float* values, const float* mask, int B, int L, float gamma, float lam,
           int whiten, float* adv, float* ret, float* acc, cudaStream_t s) {
  if (B == 0) return 0;
  gae_kernel<<<(B + 63) / 64, 64, 0, s>>>(rewards, values, mask, B, L, gamma, lam, adv, ret);
  if (whiten) {
    const long long n = static_cast<long long>(B) * L;
    cudaMemsetAsync(acc, 0, sizeof(float) * 4, s);
    masked_moments_kernel<<<148 * 2, 256, 0, s>>>(adv, mask, n, acc);
    whiten_kernel<<<static_cast<int>((n + 255) / 256), 256, 0, s>>>(adv, mask, n, acc, 0);
  }
  return static_cast<int>(cudaGetLastError());
}

}  // extern "C"
