// Collectives fused with their compute, over NVLink peer memory (symmetric buffers mapped into every rank).
//
//   peer_barrier        flag exchange through per-rank signal pads (st.release.sys / ld.acquire.sys), bounded wait
//   rs_sumsq            gradient reduce-scatter fused with the mean, the fp32 shard write and the squared-norm
//                       partial: every rank pulls ITS shard of every peer's fp32 gradient buffer with 16-byte
//                       peer loads (or one multimem.ld_reduce through the NVSwitch when a multicast mapping exists)
//   adamw_allgather     clipped AdamW on the shard fused with the all-gather of the new bf16 weights: the update
//                       is computed once and stored straight into every peer's working-weight buffer (or with a
//                       single multimem.st), i.e. the train -> rollout weight hand-over needs no further copy
//   allreduce_peer      one-shot all-reduce of a small bf16 tensor (tensor-parallel activations)
// No kernel here waits on another launch of the same GPU; cross-GPU waits are bounded by %globaltimer and report
// through a status word.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

namespace vb {

constexpr int MAX_PEERS = 16;
struct PeerPtrs {
  void* p[MAX_PEERS];
};

__device__ __forceinline__ uint64_t gtimer() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void st_release_sys(uint32_t* addr, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* addr) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}

__device__ int g_comm_status[4];

// Each rank owns a pad of uint32 slots. Rank r writes `epoch` into slot [r] of every peer's pad, then waits until
// all W slots of its own pad hold a value >= epoch. Epochs only grow, so pads never need clearing.
// When the wait runs out the kernel records ST_TIMEOUT_PEER in the status word and, if `poison` is given, stores
// +inf there: a caller that points it at the squared-gradient-norm accumulator makes the step that follows see a
// non-finite norm on every rank (after the norm is summed over ranks) and skip its update on the device, before any
// host has read the status.
__global__ void peer_barrier_kernel(PeerPtrs pads, int rank, int W, uint32_t epoch, unsigned long long limit_ns,
                                    int* status, float* poison) {
  const int t = threadIdx.x;
  if (t < W) {
    __threadfence_system();
    st_release_sys(reinterpret_cast<uint32_t*>(pads.p[t]) + rank, epoch);
    const uint32_t* mine = reinterpret_cast<const uint32_t*>(pads.p[rank]) + t;
    const uint64_t t0 = gtimer();
    uint32_t spins = 0;
    while (static_cast<int32_t>(ld_acquire_sys(mine) - epoch) < 0) {
      if ((++spins & 0xff) == 0 && gtimer() - t0 > limit_ns) {
        atomicExch(status, 4);  // ST_TIMEOUT_PEER
        if (poison != nullptr) *poison = __int_as_float(0x7f800000);
        break;
      }
    }
  }
}

__device__ __forceinline__ float block_sum_f(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = (threadIdx.x < (blockDim.x >> 5)) ? red[threadIdx.x] : 0.f;
  if (threadIdx.x < 32) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  }
  return t;
}

// out[i] = scale * sum_r grads[r][lo + i];  ctrl[0] += sum out^2.   n % 4 == 0.
__global__ void rs_sumsq_kernel(PeerPtrs grads, float* __restrict__ out, long long lo, long long n, int W, int rank,
                                float scale, float* ctrl) {
  __shared__ float red[32];
  float acc = 0.f;
  const long long n4 = n >> 2;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n4;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int k = 0; k < W; ++k) {
      const int r = (rank + k) % W;  // start with the local copy, then spread the peers
      const float4 v = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(grads.p[r]) + lo)[i];
      s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
    }
    s.x *= scale; s.y *= scale; s.z *= scale; s.w *= scale;
    reinterpret_cast<float4*>(out)[i] = s;
    acc += s.x * s.x + s.y * s.y + s.z * s.z + s.w * s.w;
  }
  acc = block_sum_f(acc, red);
  if (threadIdx.x == 0) atomicAdd(ctrl, acc);
}

// Same through an NVSwitch multicast mapping: one multimem.ld_reduce returns the sum over all ranks.
__global__ void rs_sumsq_mc_kernel(const float* mc_grads, float* __restrict__ out, long long lo, long long n,
                                   float scale, float* ctrl) {
  __shared__ float red[32];
  float acc = 0.f;
  const long long n4 = n >> 2;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n4;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float4 s;
    const float* src = mc_grads + lo + i * 4;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=f"(s.x), "=f"(s.y), "=f"(s.z), "=f"(s.w) : "l"(src) : "memory");
    s.x *= scale; s.y *= scale; s.z *= scale; s.w *= scale;
    reinterpret_cast<float4*>(out)[i] = s;
    acc += s.x * s.x + s.y * s.y + s.z * s.z + s.w * s.w;
  }
  acc = block_sum_f(acc, red);
  if (threadIdx.x == 0) atomicAdd(ctrl, acc);
}

struct AdamHyper {
  float lr, beta1, beta2, eps, wd, bc1, bc2_sqrt;
};

// AdamW on the shard; the new bf16 values go to params[r][lo + i] for every rank r (n % 8 == 0).
template <bool MULTICAST>
__global__ void adamw_allgather_kernel(float* __restrict__ master, const float* __restrict__ grad, float* __restrict__ m,
                                       float* __restrict__ v, PeerPtrs params, __nv_bfloat16* mc_params, long long lo,
                                       long long n, int W, int rank, const float* __restrict__ ctrl, AdamHyper h) {
  const long long i8 = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (i8 * 8 >= n) return;
  const bool skip = ctrl[2] != 0.f;
  const float coef = ctrl[1];
  uint32_t packed[4];
  float p8[8];
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const long long i = i8 * 8 + half * 4;
    float4 pm = *reinterpret_cast<const float4*>(master + i);
    if (!skip) {
      const float4 g4 = *reinterpret_cast<const float4*>(grad + i);
      float4 m4 = *reinterpret_cast<const float4*>(m + i);
      float4 v4 = *reinterpret_cast<const float4*>(v + i);
      float* pp = reinterpret_cast<float*>(&pm);
      const float* gp = reinterpret_cast<const float*>(&g4);
      float* mp = reinterpret_cast<float*>(&m4);
      float* vp = reinterpret_cast<float*>(&v4);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float g = gp[j] * coef;
        mp[j] = h.beta1 * mp[j] + (1.f - h.beta1) * g;
        vp[j] = h.beta2 * vp[j] + (1.f - h.beta2) * g * g;
        float p = pp[j] * (1.f - h.lr * h.wd);
        p -= (h.lr / h.bc1) * (mp[j] / (sqrtf(vp[j]) / h.bc2_sqrt + h.eps));
        pp[j] = p;
      }
      *reinterpret_cast<float4*>(master + i) = pm;
      *reinterpret_cast<float4*>(m + i) = m4;
      *reinterpret_cast<float4*>(v + i) = v4;
    }
    p8[half * 4 + 0] = pm.x; p8[half * 4 + 1] = pm.y; p8[half * 4 + 2] = pm.z; p8[half * 4 + 3] = pm.w;
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    __nv_bfloat162 t = __floats2bfloat162_rn(p8[2 * j], p8[2 * j + 1]);
    packed[j] = *reinterpret_cast<uint32_t*>(&t);
  }
  const long long off = lo + i8 * 8;
  if constexpr (MULTICAST) {
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc_params + off),
                 "f"(__uint_as_float(packed[0])), "f"(__uint_as_float(packed[1])), "f"(__uint_as_float(packed[2])),
                 "f"(__uint_as_float(packed[3]))
                 : "memory");
  } else {
    const uint4 val = make_uint4(packed[0], packed[1], packed[2], packed[3]);
    for (int k = 0; k < W; ++k) {
      const int r = (rank + k) % W;
      *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(params.p[r]) + off) = val;
    }
  }
}

// out[i] = sum_r bufs[r][i] (bf16 in, fp32 accumulate, bf16 out); n % 8 == 0. Every rank computes the full result.
__global__ void allreduce_peer_kernel(PeerPtrs bufs, __nv_bfloat16* __restrict__ out, long long n, int W, int rank) {
  const long long i8 = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (i8 * 8 >= n) return;
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  for (int k = 0; k < W; ++k) {
    const int r = (rank + k) % W;
    const uint4 raw = reinterpret_cast<const uint4*>(bufs.p[r])[i8];
    const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __bfloat1622float2(b2[j]);
      acc[2 * j] += f.x;
      acc[2 * j + 1] += f.y;
    }
  }
  uint4 o;
  uint32_t* op = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    __nv_bfloat162 t = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
    op[j] = *reinterpret_cast<uint32_t*>(&t);
  }
  reinterpret_cast<uint4*>(out)[i8] = o;
}

// ---- train -> rollout reshard: a table of 2-D copy jobs, any of whose destinations may be peer memory.
// Job j copies rows[j] rows of row_bytes[j] bytes (a multiple of 16) from src (row stride src_stride) to dst (row stride
// dst_stride); addresses 16-byte aligned. Blocks [block_start[j], block_start[j + 1]) belong to job j, 16 KB each.
struct CopyJob {
  unsigned long long dst, src;
  long long rows, row_bytes, dst_stride, src_stride;
};

__global__ void scatter_copy_kernel(const CopyJob* __restrict__ jobs, const int* __restrict__ block_start, int njobs) {
  // the job of this block: last j with block_start[j] <= blockIdx.x
  int lo = 0, hi = njobs - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (block_start[mid] <= static_cast<int>(blockIdx.x)) lo = mid; else hi = mid - 1;
  }
  const CopyJob jb = jobs[lo];
  const long long per_row = jb.row_bytes >> 4;                 // 16-byte units per row
  const long long total = jb.rows * per_row;
  const long long u0 = static_cast<long long>(blockIdx.x - block_start[lo]) * 1024;   // 1024 units = 16 KB per block
  for (long long u = u0 + threadIdx.x; u < min(total, u0 + 1024); u += blockDim.x) {
    const long long r = u / per_row, c = u - r * per_row;
    const uint4 v = *reinterpret_cast<const uint4*>(jb.src + r * jb.src_stride + (c << 4));
    *reinterpret_cast<uint4*>(jb.dst + r * jb.dst_stride + (c << 4)) = v;
  }
}

// Small all-gather over peer memory whose call counter lives on the device, so that it can sit inside a captured graph:
// every rank stores its n words into slot [parity of the call][its rank] of every rank's buffer, raises its flag on every
// rank to the call number, waits (bounded) until all flags of its own pad have reached it and copies the W slots out.
// Two halves alternate by call parity: a rank can be at most one call ahead of a peer (its next call waits for that
// peer's flag), so a slot is never overwritten while its owner still reads it.
//  bufs.p[r]: 2 * W * cap words; flags.p[r]: W words, zero before the first call; epoch: this rank's call counter.
__global__ void peer_share_kernel(PeerPtrs bufs, PeerPtrs flags, uint32_t* epoch, const uint32_t* __restrict__ src,
                                  uint32_t* __restrict__ out, int n, int cap, int rank, int W, unsigned long long limit_ns,
                                  int* status) {
  __shared__ uint32_t s_e;
  if (threadIdx.x == 0) s_e = *epoch + 1u;
  __syncthreads();
  const uint32_t e = s_e;
  const long long slot = (static_cast<long long>(e & 1u) * W + rank) * cap;
  for (int r = 0; r < W; ++r) {
    uint32_t* dst = reinterpret_cast<uint32_t*>(bufs.p[(rank + r) % W]) + slot;
    for (int i = threadIdx.x; i < n; i += blockDim.x) dst[i] = src[i];
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < W) {
    st_release_sys(reinterpret_cast<uint32_t*>(flags.p[threadIdx.x]) + rank, e);
    const uint32_t* mine = reinterpret_cast<const uint32_t*>(flags.p[rank]) + threadIdx.x;
    const uint64_t t0 = gtimer();
    uint32_t spins = 0;
    while (static_cast<int32_t>(ld_acquire_sys(mine) - e) < 0) {
      if ((++spins & 0xff) == 0 && gtimer() - t0 > limit_ns) {
        atomicExch(status, 4);  // ST_TIMEOUT_PEER
        break;
      }
    }
  }
  __syncthreads();
  const volatile uint32_t* mybuf = reinterpret_cast<const volatile uint32_t*>(bufs.p[rank]) + static_cast<long long>(e & 1u) * W * cap;
  for (int r = 0; r < W; ++r)
    for (int i = threadIdx.x; i < n; i += blockDim.x) out[static_cast<long long>(r) * n + i] = mybuf[static_cast<long long>(r) * cap + i];
  if (threadIdx.x == 0) *epoch = e;
}

static int* comm_status_ptr() {
  static int* p = nullptr;
  if (p == nullptr) cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_comm_status);
  return p;
}
static PeerPtrs make_peers(const unsigned long long* ptrs, int W) {
  PeerPtrs pp{};
  for (int i = 0; i < W && i < MAX_PEERS; ++i) pp.p[i] = reinterpret_cast<void*>(ptrs[i]);
  return pp;
}

}  // namespace vb

using namespace vb;

extern "C" {

int vb_peer_barrier(const unsigned long long* pad_ptrs, int rank, int W, unsigned int epoch, double limit_s,
                    float* poison_on_timeout, cudaStream_t s) {
  if (W > MAX_PEERS) return -1;
  peer_barrier_kernel<<<1, 32, 0, s>>>(make_peers(pad_ptrs, W), rank, W, epoch,
                                       static_cast<unsigned long long>(limit_s * 1e9), comm_status_ptr(), poison_on_timeout);
  return static_cast<int>(cudaGetLastError());
}

int vb_rs_sumsq(const unsigned long long* grad_ptrs, unsigned long long mc_ptr, float* out, long long lo, long long n,
                int W, int rank, float scale, float* ctrl, cudaStream_t s) {
  if (W > MAX_PEERS || (n % 4) || (lo % 4)) return -1;
  if (n == 0) return 0;
  long long blocks = (n / 4 + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (mc_ptr != 0)
    rs_sumsq_mc_kernel<<<static_cast<int>(blocks), 256, 0, s>>>(reinterpret_cast<const float*>(mc_ptr), out, lo, n, scale, ctrl);
  else
    rs_sumsq_kernel<<<static_cast<int>(blocks), 256, 0, s>>>(make_peers(grad_ptrs, W), out, lo, n, W, rank, scale, ctrl);
  return static_cast<int>(cudaGetLastError());
}

int vb_adamw_allgather(float* master, const float* grad, float* m, float* v, const unsigned long long* param_ptrs,
                       unsigned long long mc_ptr, long long lo, long long n, int W, int rank, const float* ctrl, float lr,
                       float beta1, float beta2, float eps, float wd, int step, cudaStream_t s) {
  if (W > MAX_PEERS || (n % 8) || (lo % 8)) return -1;
  if (n == 0) return 0;
  AdamHyper h{lr, beta1, beta2, eps, wd, 1.f - powf(beta1, static_cast<float>(step)),
              sqrtf(1.f - powf(beta2, static_cast<float>(step)))};
  const int blocks = static_cast<int>((n / 8 + 255) / 256);
  if (mc_ptr != 0)
    adamw_allgather_kernel<true><<<blocks, 256, 0, s>>>(master, grad, m, v, PeerPtrs{},
                                                        reinterpret_cast<__nv_bfloat16*>(mc_ptr), lo, n, W, rank, ctrl, h);
  else
    adamw_allgather_kernel<false><<<blocks, 256, 0, s>>>(master, grad, m, v, make_peers(param_ptrs, W), nullptr, lo, n, W,
                                                         rank, ctrl, h);
  return static_cast<int>(cudaGetLastError());
}

int vb_allreduce_peer(const unsigned long long* buf_ptrs, void* out, long long n, int W, int rank, cudaStream_t s) {
  if (W > MAX_PEERS || (n % 8)) return -1;
  if (n == 0) return 0;
  allreduce_peer_kernel<<<static_cast<int>((n / 8 + 255) / 256), 256, 0, s>>>(make_peers(buf_ptrs, W),
                                                                              reinterpret_cast<__nv_bfloat16*>(out), n, W, rank);
  return static_cast<int>(cudaGetLastError());
}

int vb_scatter_copy(const void* jobs, const int* block_start, int njobs, int total_blocks, cudaStream_t s) {
  if (njobs <= 0 || total_blocks <= 0) return 0;
  scatter_copy_kernel<<<total_blocks, 256, 0, s>>>(reinterpret_cast<const CopyJob*>(jobs), block_start, njobs);
  return static_cast<int>(cudaGetLastError());
}

int vb_peer_share(const unsigned long long* buf_ptrs, const unsigned long long* flag_ptrs, unsigned int* epoch, const void* src,
                  void* out, int n, int cap, int rank, int W, double limit_s, cudaStream_t s) {
  if (W > MAX_PEERS || n < 0 || n > cap) return -1;
  peer_share_kernel<<<1, 256, 0, s>>>(make_peers(buf_ptrs, W), make_peers(flag_ptrs, W), epoch, reinterpret_cast<const uint32_t*>(src),
                                      reinterpret_cast<uint32_t*>(out), n, cap, rank, W,
                                      static_cast<unsigned long long>((limit_s > 0 ? limit_s : 2.0) * 1e9), comm_status_ptr());
  return static_cast<int>(cudaGetLastError());
}

int vb_comm_status() {
  int h[4] = {0, 0, 0, 0};
  if (cudaMemcpyFromSymbol(h, g_comm_status, sizeof(h)) != cudaSuccess) return -1;
  if (h[0] != 0) {
    int z[4] = {0, 0, 0, 0};
    cudaMemcpyToSymbol(g_comm_status, z, sizeof(z));
  }
  return h[0];
}

}  // extern "C"
