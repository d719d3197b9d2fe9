// Single-step (decoding) kernels of the recurrent / state-space models and the fused gate
// arithmetic of the RG-LRU. All memory-bound: one pass over their operands, fp32 math.
//
//   conv1d_update      one decoding step of the causal depthwise convolution: shift the window of
//                      every (sequence, channel), insert the new input, weight, SiLU
//                      (causal_conv1d_update as used by apps/mamba/core_mamba.py:197 and
//                      apps/fastRNN/component/rnn_common.py:62-70)
//   conv_states        last W inputs of every document of a packed sequence, i.e. the window a
//                      decoder continues from (causal_conv1d_varlen_states, core_mamba.py:181-186)
//   ssm_state_update   one step of the selective state space recurrence with its read-out
//                      (selective_state_update, core_mamba.py:283)
//   rnn_step           h = a * h + b on a cached fp32 state (sequential_step,
//                      apps/fastRNN/component/rnn_common.py:83-86)
//   rglru_gates_fwd/bwd  a = exp(-8 sigmoid(ga) softplus(lambda)), b = sqrt(1 - a^2) sigmoid(gx) x
//                      and its gradient with the bounded derivative of the square root
//                      (apps/fastRNN/hawk/core_hawk.py:110-131)
#include "common.cuh"
#include "lingua_b200.h"

namespace lb {

using bf16 = __nv_bfloat16;

__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + __expf(-x)); }

// ---------------------------------------------------------------- conv1d update
template <int W>
__global__ void __launch_bounds__(256)
conv1d_update_kernel(const bf16* __restrict__ x, long long ldx, bf16* __restrict__ state,
                     const bf16* __restrict__ w, bf16* __restrict__ out, long long ldo, int N, int C, int act) {
  const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (i >= (long long)N * C) return;
  const int n = (int)(i / C), c = (int)(i - (long long)n * C);
  bf16* s = state + i * W;
  float win[W];
#pragma unroll
  for (int j = 0; j < W - 1; ++j) win[j] = __bfloat162float(s[j + 1]);
  const bf16 xn = x[n * ldx + c];
  win[W - 1] = __bfloat162float(xn);
  float acc = 0.f;
#pragma unroll
  for (int j = 0; j < W; ++j) acc += win[j] * __bfloat162float(w[c * W + j]);
#pragma unroll
  for (int j = 0; j < W - 1; ++j) s[j] = __float2bfloat16(win[j]);
  s[W - 1] = xn;
  if (act) acc = acc * sigmoidf_(acc);
  out[n * ldo + c] = __float2bfloat16(acc);
}

// ---------------------------------------------------------------- conv states of packed documents
__global__ void __launch_bounds__(256)
conv_states_kernel(const bf16* __restrict__ x, long long ldx, const long long* __restrict__ starts,
                   const long long* __restrict__ ends, bf16* __restrict__ out, int n_docs, int C, int W) {
  const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (i >= (long long)n_docs * C) return;
  const int d = (int)(i / C), c = (int)(i - (long long)d * C);
  const long long s0 = starts[d], e = ends[d];
  for (int j = 0; j < W; ++j) {
    const long long t = e - W + j;
    out[i * W + j] = t >= s0 ? x[t * ldx + c] : __float2bfloat16(0.f);
  }
}

// ---------------------------------------------------------------- selective state update
// one warp per (sequence, head, row p): state[n, h, p, :] (N floats) is decayed, fed and read out
__global__ void __launch_bounds__(256)
ssm_state_update_kernel(float* __restrict__ state, const bf16* __restrict__ x, long long ldx,
                        const float* __restrict__ dt, const float* __restrict__ A, const bf16* __restrict__ B,
                        long long ldb, const bf16* __restrict__ Cm, long long ldc, const float* __restrict__ D,
                        int d_has_p, bf16* __restrict__ y, int nseq, int H, int P, int N, int G) {
  const long long row = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= (long long)nseq * H * P) return;
  const int p = (int)(row % P);
  const int h = (int)((row / P) % H);
  const int n = (int)(row / ((long long)P * H));
  const int g = h / (H / G);
  const float dtv = dt[n * H + h];
  const float decay = __expf(dtv * A[h]);
  const float xv = __bfloat162float(x[n * ldx + h * P + p]);
  const float dx = dtv * xv;
  float* s = state + row * N;
  const bf16* b = B + n * ldb + g * N;
  const bf16* c = Cm + n * ldc + g * N;
  float acc = 0.f;
  for (int k = lane * 4; k < N; k += 128) {
    float4 v = *reinterpret_cast<float4*>(s + k);
    const uint2 bb = *reinterpret_cast<const uint2*>(b + k);
    const uint2 cc = *reinterpret_cast<const uint2*>(c + k);
    const float2 b01 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&bb.x));
    const float2 b23 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&bb.y));
    const float2 c01 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&cc.x));
    const float2 c23 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&cc.y));
    v.x = v.x * decay + dx * b01.x;
    v.y = v.y * decay + dx * b01.y;
    v.z = v.z * decay + dx * b23.x;
    v.w = v.w * decay + dx * b23.y;
    *reinterpret_cast<float4*>(s + k) = v;
    acc += v.x * c01.x + v.y * c01.y + v.z * c23.x + v.w * c23.y;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) {
    if (D) acc += D[d_has_p ? h * P + p : h] * xv;
    y[row] = __float2bfloat16(acc);
  }
}

// ---------------------------------------------------------------- one step of h = a h + b
__global__ void __launch_bounds__(256)
rnn_step_kernel(const bf16* __restrict__ a, const bf16* __restrict__ b, float* __restrict__ state,
                bf16* __restrict__ out, long long n) {
  const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float h = __bfloat162float(a[i]) * state[i] + __bfloat162float(b[i]);
  state[i] = h;
  out[i] = __float2bfloat16(h);
}

// ---------------------------------------------------------------- RG-LRU gates
constexpr float RGLRU_C = 8.0f;
constexpr float RGLRU_SQRT_MIN = 1e-6f;  // 1 / (max sqrt gradient 1000)^2

// 8 channels per thread (16-byte vectors); rows = tokens
__global__ void __launch_bounds__(256)
rglru_gates_fwd_kernel(const bf16* __restrict__ gx, const bf16* __restrict__ ga, const bf16* __restrict__ x,
                       const float* __restrict__ sp, bf16* __restrict__ a_out, bf16* __restrict__ b_out,
                       long long rows, int C) {
  const int cv = C / 8;
  const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (i >= rows * cv) return;
  const int c0 = (int)(i % cv) * 8;
  const uint4 vgx = reinterpret_cast<const uint4*>(gx)[i];
  const uint4 vga = reinterpret_cast<const uint4*>(ga)[i];
  const uint4 vx = reinterpret_cast<const uint4*>(x)[i];
  const bf16* pgx = reinterpret_cast<const bf16*>(&vgx);
  const bf16* pga = reinterpret_cast<const bf16*>(&vga);
  const bf16* px = reinterpret_cast<const bf16*>(&vx);
  uint4 va, vb;
  bf16* pa = reinterpret_cast<bf16*>(&va);
  bf16* pb = reinterpret_cast<bf16*>(&vb);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float gate_x = sigmoidf_(__bfloat162float(pgx[j]));
    const float gate_a = sigmoidf_(__bfloat162float(pga[j]));
    const float log_a = -RGLRU_C * gate_a * sp[c0 + j];
    const float a = __expf(log_a);
    const float mult = sqrtf(fmaxf(1.f - __expf(2.f * log_a), 0.f));
    pa[j] = __float2bfloat16(a);
    pb[j] = __float2bfloat16(mult * gate_x * __bfloat162float(px[j]));
  }
  reinterpret_cast<uint4*>(a_out)[i] = va;
  reinterpret_cast<uint4*>(b_out)[i] = vb;
}

// Each block walks a strip of rows for 8 * blockDim.x... channels: thread t owns 8 channels of one column group and
// loops over the block's rows, so the per-channel sum for d softplus(lambda) stays in registers until the end.
__global__ void __launch_bounds__(128)
rglru_gates_bwd_kernel(const bf16* __restrict__ gx, const bf16* __restrict__ ga, const bf16* __restrict__ x,
                       const float* __restrict__ sp, const bf16* __restrict__ da, const bf16* __restrict__ db,
                       bf16* __restrict__ dgx, bf16* __restrict__ dga, bf16* __restrict__ dx,
                       float* __restrict__ dsp, long long rows, int C, int rows_per_block) {
  const int cv = C / 8;
  const int col = blockIdx.x * blockDim.x + threadIdx.x;
  if (col >= cv) return;
  const int c0 = col * 8;
  const long long r0 = (long long)blockIdx.y * rows_per_block;
  const long long r1 = r0 + rows_per_block < rows ? r0 + rows_per_block : rows;
  float spv[8], acc[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    spv[j] = sp[c0 + j];
    acc[j] = 0.f;
  }
  for (long long r = r0; r < r1; ++r) {
    const long long i = r * cv + col;
    const uint4 vgx = reinterpret_cast<const uint4*>(gx)[i];
    const uint4 vga = reinterpret_cast<const uint4*>(ga)[i];
    const uint4 vx = reinterpret_cast<const uint4*>(x)[i];
    const uint4 vda = reinterpret_cast<const uint4*>(da)[i];
    const uint4 vdb = reinterpret_cast<const uint4*>(db)[i];
    const bf16* pgx = reinterpret_cast<const bf16*>(&vgx);
    const bf16* pga = reinterpret_cast<const bf16*>(&vga);
    const bf16* px = reinterpret_cast<const bf16*>(&vx);
    const bf16* pda = reinterpret_cast<const bf16*>(&vda);
    const bf16* pdb = reinterpret_cast<const bf16*>(&vdb);
    uint4 ogx, oga, ox;
    bf16* qgx = reinterpret_cast<bf16*>(&ogx);
    bf16* qga = reinterpret_cast<bf16*>(&oga);
    bf16* qx = reinterpret_cast<bf16*>(&ox);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float gate_x = sigmoidf_(__bfloat162float(pgx[j]));
      const float gate_a = sigmoidf_(__bfloat162float(pga[j]));
      const float xv = __bfloat162float(px[j]);
      const float log_a = -RGLRU_C * gate_a * spv[j];
      const float a = __expf(log_a);
      const float a2 = __expf(2.f * log_a);
      const float u = 1.f - a2;
      const float mult = sqrtf(fmaxf(u, 0.f));
      const float g_a = __bfloat162float(pda[j]);
      const float g_b = __bfloat162float(pdb[j]);
      qx[j] = __float2bfloat16(g_b * mult * gate_x);
      qgx[j] = __float2bfloat16(g_b * mult * xv * gate_x * (1.f - gate_x));
      const float d_mult = g_b * gate_x * xv;
      const float d_u = d_mult * rsqrtf(fmaxf(4.f * u, RGLRU_SQRT_MIN));
      const float d_log_a = g_a * a - 2.f * a2 * d_u;
      qga[j] = __float2bfloat16(d_log_a * (-RGLRU_C * spv[j]) * gate_a * (1.f - gate_a));
      acc[j] += d_log_a * (-RGLRU_C * gate_a);
    }
    reinterpret_cast<uint4*>(dgx)[i] = ogx;
    reinterpret_cast<uint4*>(dga)[i] = oga;
    reinterpret_cast<uint4*>(dx)[i] = ox;
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) atomicAdd(dsp + c0 + j, acc[j]);
}

static inline unsigned blocks_for(long long n, int threads) { return (unsigned)((n + threads - 1) / threads); }

}  // namespace lb

using lb::bf16;

extern "C" int lb_conv1d_update(const void* x, long long ldx, void* state, const void* w, void* out, long long ldo,
                                int N, int C, int W, int act, void* stream) {
  if (!x || !state || !w || !out || N <= 0 || C <= 0) return 1;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const unsigned grid = lb::blocks_for((long long)N * C, 256);
#define LB_CU(WW)                                                                                              \
  case WW:                                                                                                     \
    lb::conv1d_update_kernel<WW><<<grid, 256, 0, st>>>((const bf16*)x, ldx, (bf16*)state, (const bf16*)w, (bf16*)out, \
                                                       ldo, N, C, act);                                        \
    break;
  switch (W) {
    LB_CU(2) LB_CU(3) LB_CU(4)
    default: return 2;
  }
#undef LB_CU
  lb::g_launches.fetch_add(1, std::memory_order_relaxed);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}

extern "C" int lb_conv_states(const void* x, long long ldx, const long long* starts, const long long* ends, void* out,
                              int n_docs, int C, int W, void* stream) {
  if (!x || !starts || !ends || !out || n_docs <= 0 || C <= 0 || W <= 0) return 1;
  lb::conv_states_kernel<<<lb::blocks_for((long long)n_docs * C, 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      (const bf16*)x, ldx, starts, ends, (bf16*)out, n_docs, C, W);
  lb::g_launches.fetch_add(1, std::memory_order_relaxed);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}

extern "C" int lb_ssm_state_update(float* state, const void* x, long long ldx, const float* dt, const float* A,
                                   const void* B, long long ldb, const void* Cm, long long ldc, const float* D,
                                   int d_has_p, void* y, int nseq, int H, int P, int N, int G, void* stream) {
  if (!state || !x || !dt || !A || !B || !Cm || !y || nseq <= 0) return 1;
  if (N % 4 || G <= 0 || H % G || ldb % 4 || ldc % 4) return 2;
  if (reinterpret_cast<uintptr_t>(B) % 8 || reinterpret_cast<uintptr_t>(Cm) % 8) return 3;
  const long long rows = (long long)nseq * H * P;
  lb::ssm_state_update_kernel<<<lb::blocks_for(rows * 32, 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      state, (const bf16*)x, ldx, dt, A, (const bf16*)B, ldb, (const bf16*)Cm, ldc, D, d_has_p, (bf16*)y, nseq, H, P, N,
      G);
  lb::g_launches.fetch_add(1, std::memory_order_relaxed);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}

extern "C" int lb_rnn_step(const void* a, const void* b, float* state, void* out, long long n, void* stream) {
  if (!a || !b || !state || !out || n <= 0) return 1;
  lb::rnn_step_kernel<<<lb::blocks_for(n, 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      (const bf16*)a, (const bf16*)b, state, (bf16*)out, n);
  lb::g_launches.fetch_add(1, std::memory_order_relaxed);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}

extern "C" int lb_rglru_gates_fwd(const void* gx, const void* ga, const void* x, const float* sp, void* a_out,
                                  void* b_out, long long rows, int C, void* stream) {
  if (!gx || !ga || !x || !sp || !a_out || !b_out || rows <= 0 || C <= 0 || C % 8) return 1;
  lb::rglru_gates_fwd_kernel<<<lb::blocks_for(rows * (C / 8), 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      (const bf16*)gx, (const bf16*)ga, (const bf16*)x, sp, (bf16*)a_out, (bf16*)b_out, rows, C);
  lb::g_launches.fetch_add(1, std::memory_order_relaxed);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}

// dsp (fp32 [C]) is accumulated into: clear it before the first call of a step.
extern "C" int lb_rglru_gates_bwd(const void* gx, const void* ga, const void* x, const float* sp, const void* da,
                                  const void* db, void* dgx, void* dga, void* dx, float* dsp, long long rows, int C,
                                  void* stream) {
  if (!gx || !ga || !x || !sp || !da || !db || !dgx || !dga || !dx || !dsp || rows <= 0 || C <= 0 || C % 8) return 1;
  const int cv = C / 8;
  const unsigned gx_blocks = (unsigned)((cv + 127) / 128);
  // enough row strips to fill the GPU a few times over, each long enough to amortise the atomics
  long long strips = (long long)lb::num_sms() * 8 / gx_blocks;
  if (strips < 1) strips = 1;
  long long rpb = (rows + strips - 1) / strips;
  if (rpb < 16) rpb = 16;
  const unsigned gy = (unsigned)((rows + rpb - 1) / rpb);
  lb::rglru_gates_bwd_kernel<<<dim3(gx_blocks, gy), 128, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      (const bf16*)gx, (const bf16*)ga, (const bf16*)x, sp, (const bf16*)da, (const bf16*)db, (bf16*)dgx, (bf16*)dga,
      (bf16*)dx, dsp, rows, C, (int)rpb);
  lb::g_launches.fetch_add(1, std::memory_order_relaxed);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}
