// Small kernels around the fused tensor-parallel GEMMs (gemm_tp.cu):
//
//   lb_peer_barrier   all ranks of a tensor-parallel group meet; every store a rank made before
//                     the barrier (to its own or to a peer's memory) is visible to every rank's
//                     kernels launched after it. One counter per (destination, source) pair in
//                     peer-visible memory, bumped with a system-scope release and polled with a
//                     system-scope acquire. The wait is bounded: after LB_WAIT_LIMIT_NS the kernel
//                     records ST_TIMEOUT_FLAG in the status word and returns.
//   lb_reduce_norm    h = residual + sum over slots (the partial products that gemm_tp mode 2
//                     scattered to this rank), y = RMSNorm(h) * w, for this rank's rows. It is the
//                     "reduce" half of the reduce-scatter fused with the residual add and the norm
//                     that follows every attention / feed-forward output projection
//                     (lingua/transformer.py:520-527).
#include "common.cuh"
#include "lingua_b200.h"

namespace lb {

struct BarrierParams {
  uint32_t* pads[LB_MAX_PEERS];
  int world, rank;
  uint32_t epoch;
  uint32_t* status;
  unsigned long long limit_ns;
};

__global__ void peer_barrier_kernel(const BarrierParams p) {
  const int r = threadIdx.x;
  if (r >= p.world) return;
  __threadfence_system();
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p.pads[r] + p.rank), "r"(1u) : "memory");
  const uint32_t* mine = p.pads[p.rank] + r;
  uint64_t t0 = 0;
  for (uint32_t it = 0;; ++it) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
    if (static_cast<int32_t>(v - p.epoch) >= 0) break;
    __nanosleep(100);
    if ((it & 0xFFu) == 0xFFu) {
      const uint64_t now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      if (now - t0 > p.limit_ns) {
        if (p.status) atomicOr(p.status, ST_TIMEOUT_FLAG | 7u);
        break;
      }
    }
  }
  __threadfence_system();
}

constexpr int RN_THREADS = 256;
constexpr int RN_MAXV = 4;  // 8-element vectors per thread kept in registers: D <= 8192

__global__ void __launch_bounds__(RN_THREADS)
reduce_norm_kernel(const __nv_bfloat16* __restrict__ slots, int n_slots, long long slot_stride,
                   const __nv_bfloat16* resid, const __nv_bfloat16* __restrict__ w, float eps,
                   __nv_bfloat16* h_out, __nv_bfloat16* __restrict__ y_out,
                   float* __restrict__ rstd_out, int D) {
  const long long row = blockIdx.x;
  const int nvec = D / 8;
  float h[RN_MAXV][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < RN_MAXV; ++i) {
    const int v = threadIdx.x + i * RN_THREADS;
    if (v < nvec) {
      float acc[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
      for (int s = 0; s < n_slots; ++s) {
        const uint4 q = *reinterpret_cast<const uint4*>(slots + s * slot_stride + row * D + v * 8);
        const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(b[j]);
          acc[2 * j] += f.x;
          acc[2 * j + 1] += f.y;
        }
      }
      if (resid) {
        const uint4 q = *reinterpret_cast<const uint4*>(resid + row * D + v * 8);
        const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(b[j]);
          acc[2 * j] += f.x;
          acc[2 * j + 1] += f.y;
        }
      }
      // the residual stream is stored in bf16; the norm sees the stored value
      uint4 o;
      uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        ow[j] = pack_bf16(acc[2 * j], acc[2 * j + 1]);
        const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&ow[j]));
        h[i][2 * j] = f.x;
        h[i][2 * j + 1] = f.y;
        ss += f.x * f.x + f.y * f.y;
      }
      if (h_out) *reinterpret_cast<uint4*>(h_out + row * D + v * 8) = o;
    }
  }
  if (!y_out) return;
  __shared__ float red[RN_THREADS / 32];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < RN_THREADS / 32; ++i) tot += red[i];
  const float rstd = rsqrtf(tot / D + eps);
  if (rstd_out && threadIdx.x == 0) rstd_out[row] = rstd;
#pragma unroll
  for (int i = 0; i < RN_MAXV; ++i) {
    const int v = threadIdx.x + i * RN_THREADS;
    if (v < nvec) {
      const uint4 q = *reinterpret_cast<const uint4*>(w + v * 8);
      const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&q);
      uint4 o;
      uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 g = __bfloat1622float2(b[j]);
        ow[j] = pack_bf16(h[i][2 * j] * rstd * g.x, h[i][2 * j + 1] * rstd * g.y);
      }
      *reinterpret_cast<uint4*>(y_out + row * D + v * 8) = o;
    }
  }
}

}  // namespace lb

extern "C" int lb_peer_barrier_limit(void* const* pads, int world, int rank, uint32_t epoch, uint32_t* status,
                                     unsigned long long limit_ns, void* stream);

extern "C" int lb_peer_barrier(void* const* pads, int world, int rank, uint32_t epoch, uint32_t* status,
                               void* stream) {
  return lb_peer_barrier_limit(pads, world, rank, epoch, status, LB_WAIT_LIMIT_NS, stream);
}

// Same with an explicit wait limit: ranks of a training job may drift apart by more than the default limit
// (a slow data loader, a checkpoint write) without anything being wrong.
extern "C" int lb_peer_barrier_limit(void* const* pads, int world, int rank, uint32_t epoch, uint32_t* status,
                                     unsigned long long limit_ns, void* stream) {
  if (!pads || world < 1 || world > LB_MAX_PEERS || rank < 0 || rank >= world) return 1;
  lb::BarrierParams p;
  p.limit_ns = limit_ns;
  for (int r = 0; r < LB_MAX_PEERS; ++r) p.pads[r] = reinterpret_cast<uint32_t*>(pads[r < world ? r : 0]);
  p.world = world; p.rank = rank; p.epoch = epoch; p.status = status;
  lb::peer_barrier_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(p);
  lb::g_launches.fetch_add(1, std::memory_order_relaxed);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}

extern "C" int lb_reduce_norm(const void* slots, int n_slots, long long slot_stride, const void* resid,
                              const void* w, float eps, void* h_out, void* y_out, float* rstd_out,
                              long long rows, int D, void* stream) {
  if (!slots || n_slots < 1 || rows <= 0) return 1;
  if (D % 8 != 0 || D > 8 * lb::RN_THREADS * lb::RN_MAXV || slot_stride % 8 != 0) return 2;
  if (y_out && !w) return 3;
  using bf = __nv_bfloat16;
  lb::reduce_norm_kernel<<<(unsigned)rows, lb::RN_THREADS, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const bf*>(slots), n_slots, slot_stride, reinterpret_cast<const bf*>(resid),
      reinterpret_cast<const bf*>(w), eps, reinterpret_cast<bf*>(h_out), reinterpret_cast<bf*>(y_out), rstd_out, D);
  lb::g_launches.fetch_add(1, std::memory_order_relaxed);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}

// out[i] = scale * (own[i] + sum_s slots[s * slot_stride + i]); *sumsq += sum_i out[i]^2.
// The reduce half of a reduce-scatter whose transfer half was done by the copy engines (every peer pushed its
// fp32 gradient slice for this rank into one slot), fused with the squared-norm pass the optimiser needs.
namespace lb {
__global__ void __launch_bounds__(256)
reduce_slots_kernel(const float* __restrict__ own, const float* __restrict__ slots, int n_slots, long long slot_stride,
                    float* __restrict__ out, long long n, float scale, float* __restrict__ sumsq) {
  float acc = 0.f;
  const long long n4 = n / 4;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    // streaming accesses (evict first): the kernel runs next to the backward GEMMs, whose operand tiles
    // should stay in L2
    float4 v = __ldcs(reinterpret_cast<const float4*>(own) + i);
    for (int s = 0; s < n_slots; ++s) {
      const float4 w = __ldcs(reinterpret_cast<const float4*>(slots + s * slot_stride) + i);
      v.x += w.x; v.y += w.y; v.z += w.z; v.w += w.w;
    }
    v.x *= scale; v.y *= scale; v.z *= scale; v.w *= scale;
    __stcs(reinterpret_cast<float4*>(out) + i, v);
    acc += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  if (blockIdx.x == 0) {
    for (long long i = n4 * 4 + threadIdx.x; i < n; i += blockDim.x) {
      float v = own[i];
      for (int s = 0; s < n_slots; ++s) v += slots[s * slot_stride + i];
      v *= scale;
      out[i] = v;
      acc += v * v;
    }
  }
  __shared__ float red[8];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0 && sumsq) {
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) t += red[i];
    atomicAdd(sumsq, t);
  }
}
// Reduce-scatter by pulling: out[i] = scale * sum_r src[r][i], where src[r] points at this rank's slice inside
// rank r's gradient buffer (peer-visible memory, plain loads over NVLink; src[0] is the local one), fused with
// the squared-norm pass. No staging copy: each gradient byte is read once where it lives and crosses NVLink
// once. All loads of an element are issued before the first add, so a thread keeps n_src requests in flight.
struct PeerSrcs {
  const float* p[LB_MAX_PEERS];
};
template <int NS>
__global__ void __launch_bounds__(256)
reduce_peers_kernel(PeerSrcs srcs, float* __restrict__ out, long long n, float scale, float* __restrict__ sumsq) {
  float acc = 0.f;
  const long long n4 = n / 4;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    float4 v[NS];
#pragma unroll
    for (int s = 0; s < NS; ++s) v[s] = __ldcs(reinterpret_cast<const float4*>(srcs.p[s]) + i);
#pragma unroll
    for (int s = 1; s < NS; ++s) {
      v[0].x += v[s].x; v[0].y += v[s].y; v[0].z += v[s].z; v[0].w += v[s].w;
    }
    v[0].x *= scale; v[0].y *= scale; v[0].z *= scale; v[0].w *= scale;
    __stcs(reinterpret_cast<float4*>(out) + i, v[0]);
    acc += v[0].x * v[0].x + v[0].y * v[0].y + v[0].z * v[0].z + v[0].w * v[0].w;
  }
  if (blockIdx.x == 0) {
    for (long long i = n4 * 4 + threadIdx.x; i < n; i += blockDim.x) {
      float v = 0.f;
      for (int s = 0; s < NS; ++s) v += srcs.p[s][i];
      v *= scale;
      out[i] = v;
      acc += v * v;
    }
  }
  __shared__ float red[8];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0 && sumsq) {
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) t += red[i];
    atomicAdd(sumsq, t);
  }
}
}  // namespace lb

extern "C" int lb_reduce_peers(const void* const* srcs, int n_src, float* out, long long n, float scale, float* sumsq,
                               void* stream) {
  if (!srcs || !out || n <= 0 || n_src < 1 || n_src > LB_MAX_PEERS) return 1;
  lb::PeerSrcs ps{};
  for (int s = 0; s < n_src; ++s) {
    if (!srcs[s] || reinterpret_cast<uintptr_t>(srcs[s]) % 16) return 2;
    ps.p[s] = static_cast<const float*>(srcs[s]);
  }
  if (reinterpret_cast<uintptr_t>(out) % 16) return 2;
  long long blocks = (n / 4 + 255) / 256;
  const long long cap = (long long)lb::num_sms() * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  switch (n_src) {
#define LB_RP(NS) case NS: lb::reduce_peers_kernel<NS><<<(unsigned)blocks, 256, 0, st>>>(ps, out, n, scale, sumsq); break;
    LB_RP(1) LB_RP(2) LB_RP(3) LB_RP(4) LB_RP(5) LB_RP(6) LB_RP(7) LB_RP(8)
#undef LB_RP
  }
  lb::g_launches.fetch_add(1, std::memory_order_relaxed);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}

// dst[i] += src[i] with fp32 reductions that are atomic at the destination (dst may be a peer's memory: several
// ranks add into the same shard at the same time).
namespace lb {
__global__ void __launch_bounds__(256) red_add_kernel(float* __restrict__ dst, const float* __restrict__ src, long long n) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    asm volatile("red.global.add.f32 [%0], %1;" ::"l"(dst + i), "f"(src[i]) : "memory");
}
}  // namespace lb
extern "C" int lb_red_add(float* dst, const float* src, long long n, void* stream) {
  if (!dst || !src || n <= 0) return 1;
  long long blocks = (n + 255) / 256;
  if (blocks > (long long)lb::num_sms() * 4) blocks = (long long)lb::num_sms() * 4;
  lb::red_add_kernel<<<(unsigned)blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(dst, src, n);
  lb::g_launches.fetch_add(1, std::memory_order_relaxed);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}

// max_blocks > 0 caps the grid: a reduction that runs beside the backward GEMMs has a whole layer's time to finish and
// should trickle (few blocks, little pressure on the SMs and on L2) rather than burst; 0 = LB_REDUCE_BLOCKS or 8 per SM.
extern "C" int lb_reduce_slots_grid(const float* own, const float* slots, int n_slots, long long slot_stride, float* out,
                                    long long n, float scale, float* sumsq, int max_blocks, void* stream) {
  if (!own || !out || n <= 0 || n_slots < 0 || (n_slots > 0 && !slots)) return 1;
  if (reinterpret_cast<uintptr_t>(own) % 16 || reinterpret_cast<uintptr_t>(out) % 16 ||
      reinterpret_cast<uintptr_t>(slots) % 16 || slot_stride % 4)
    return 2;
  long long blocks = (n / 4 + 255) / 256;
  static const long long env_cap = [] {
    const char* s = getenv("LB_REDUCE_BLOCKS");
    return s ? atoll(s) : 0LL;
  }();
  const long long cap = max_blocks > 0 ? max_blocks : env_cap > 0 ? env_cap : (long long)lb::num_sms() * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  lb::reduce_slots_kernel<<<(unsigned)blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      own, slots, n_slots, slot_stride, out, n, scale, sumsq);
  lb::g_launches.fetch_add(1, std::memory_order_relaxed);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}

extern "C" int lb_reduce_slots(const float* own, const float* slots, int n_slots, long long slot_stride, float* out,
                               long long n, float scale, float* sumsq, void* stream) {
  return lb_reduce_slots_grid(own, slots, n_slots, slot_stride, out, n, scale, sumsq, 0, stream);
}
