// Sequence kernels of the recurrent / state-space models, all on channel-last [B, S, C] tensors
// (one row per token, as the GEMMs produce them), so no transposes surround them:
//
//   * causal depthwise conv1d (+ SiLU) forward / backward with document resets, replacing the
//     causal_conv1d extension used through apps/mamba/component/causal_conv1d_compilable.py;
//   * first-order linear recurrence h_t = a_t h_{t-1} + b_t forward / backward for any sequence
//     length, with document resets, replacing accelerated_scan
//     (apps/fastRNN/component/compilable_scan.py), whose warp kernel needs power-of-two lengths.
//
// The scan is chunked: pass 1 reduces every chunk of SCAN_CHUNK steps to its transfer pair
// (prod a, local h_end); pass 2 lets every chunk fold the pairs of the chunks before it (a few
// dozen steps over a tiny array) and then replays its own steps with the right carry. Work is
// (batch x chunks x channels) threads, reads are coalesced across channels.
#include "common.cuh"
#include "conv1d_vec.cuh"
#include "lingua_b200.h"

namespace lb {

constexpr int SCAN_CHUNK = 64;

__device__ __forceinline__ float bf2f(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float silu_f(float x) { return x / (1.f + __expf(-x)); }
__device__ __forceinline__ float dsilu_f(float x) {
  const float s = 1.f / (1.f + __expf(-x));
  return s * (1.f + x * (1.f - s));
}

// ------------------------------------------------------------------ conv1d
// y[b,s,c] = act(sum_j w[c,j] * x[b, s-(W-1)+j, c]); taps before doc_start[b,s] (or before 0) are 0.
template <int W>
__global__ void conv1d_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                  const int* __restrict__ doc_start, __nv_bfloat16* __restrict__ y, int B, int S,
                                  int C, long long ldx, long long ldy, int act) {
  const long long total = (long long)B * S * C;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int c = i % C;
    const long long bs = i / C;
    const int s = bs % S;
    const int b = bs / S;
    const int lo = doc_start ? doc_start[bs] : 0;
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < W; ++j) {
      const int t = s - (W - 1) + j;
      if (t >= lo) acc += bf2f(w[c * W + j]) * bf2f(x[((long long)b * S + t) * ldx + c]);
    }
    y[bs * ldy + c] = __float2bfloat16(act ? silu_f(acc) : acc);
  }
}
// dx[b,t,c] = sum_j w[c,j] * g[b, t+(W-1)-j, c] where g = dy * act'(pre) and the tap is valid for
// the receiving token (t >= its doc_start); dw[c,j] accumulated with atomics from per-thread sums.
template <int W>
__global__ void conv1d_bwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                  const int* __restrict__ doc_start, const __nv_bfloat16* __restrict__ dy,
                                  __nv_bfloat16* __restrict__ dx, float* __restrict__ dw, int B, int S, int C,
                                  long long ldx, long long ldy, long long lddx, int act, int rows_per_thread) {
  // thread = (channel c, block of rows); rows are consecutive tokens of one sequence
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const long long n_rows = (long long)B * S;
  const long long r0 = (long long)blockIdx.y * rows_per_thread;
  float wv[W], dwacc[W];
#pragma unroll
  for (int j = 0; j < W; ++j) {
    wv[j] = bf2f(w[c * W + j]);
    dwacc[j] = 0.f;
  }
  for (long long r = r0; r < r0 + rows_per_thread && r < n_rows; ++r) {
    const int s = r % S;
    const long long b = r / S;
    // dx for token (b, s): contributions of outputs s .. s+W-1 of the same sequence
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < W; ++j) {
      const int so = s + (W - 1) - j;  // output position that used x[s] with tap j
      if (so < S) {
        const long long ro = b * S + so;
        const int lo = doc_start ? doc_start[ro] : 0;
        if (s >= lo) {
          float g = bf2f(dy[ro * ldy + c]);
          if (act) {
            float pre = 0.f;
#pragma unroll
            for (int jj = 0; jj < W; ++jj) {
              const int t = so - (W - 1) + jj;
              if (t >= lo) pre += wv[jj] * bf2f(x[(b * S + t) * ldx + c]);
            }
            g *= dsilu_f(pre);
          }
          acc += wv[j] * g;
          dwacc[j] += g * bf2f(x[r * ldx + c]);
        }
      }
    }
    dx[r * lddx + c] = __float2bfloat16(acc);
  }
#pragma unroll
  for (int j = 0; j < W; ++j) atomicAdd(dw + c * W + j, dwacc[j]);
}

// ------------------------------------------------------------------ linear recurrence
// Every thread owns V adjacent channels (V = 2: one 4-byte load per tensor and step, a warp covers 128 bytes
// per row; V = 1 for odd channel counts).
template <int V>
__device__ __forceinline__ void ldv(const __nv_bfloat16* p, float (&f)[V]) {
  if (V == 2) {
    const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
    f[0] = v.x;
    f[V - 1] = v.y;
  } else {
    f[0] = __bfloat162float(*p);
  }
}
template <int V>
__device__ __forceinline__ void stv(__nv_bfloat16* p, const float (&f)[V]) {
  if (V == 2)
    *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(f[0], f[V - 1]);
  else
    *p = __float2bfloat16(f[0]);
}

// Forward pass 1: per (b, chunk, c): A = prod a, H = local end state (zero carry). A document
// start inside the chunk cuts the product (a is taken as 0 at the first token of a document).
template <int V>
__global__ void scan_reduce_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ bb,
                                   const int* __restrict__ doc_start, float* __restrict__ agg_a,
                                   float* __restrict__ agg_h, int B, int S, int C, int n_chunks, int reverse,
                                   const __nv_bfloat16* __restrict__ shifted_a) {
  const int CV = C / V;
  const long long total = (long long)B * n_chunks * CV;
  const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int c = (i % CV) * V;
  const long long bk = i / CV;
  const int k = bk % n_chunks;
  const int b = bk / n_chunks;
  const int s0 = k * SCAN_CHUNK, s1 = min(S, s0 + SCAN_CHUNK);
  float A[V], H[V];
#pragma unroll
  for (int v = 0; v < V; ++v) { A[v] = 1.f; H[v] = 0.f; }
  if (!reverse) {
    for (int s = s0; s < s1; ++s) {
      const long long idx = ((long long)b * S + s) * C + c;
      float av[V], bv[V];
      ldv<V>(a + idx, av);
      ldv<V>(bb + idx, bv);
      const bool cut = doc_start && doc_start[(long long)b * S + s] == s;
#pragma unroll
      for (int v = 0; v < V; ++v) {
        const float x = cut ? 0.f : av[v];
        H[v] = x * H[v] + bv[v];
        A[v] *= x;
      }
    }
  } else {
    // reverse recurrence g_s = dh_s + a_{s+1} g_{s+1}: coefficient of step s is a_{s+1} (0 past the
    // end or when s+1 starts a new document)
    for (int s = s1 - 1; s >= s0; --s) {
      const long long idx = ((long long)b * S + s) * C + c;
      float av[V], bv[V];
#pragma unroll
      for (int v = 0; v < V; ++v) av[v] = 0.f;
      if (s + 1 < S && !(doc_start && doc_start[(long long)b * S + s + 1] == s + 1)) ldv<V>(shifted_a + idx + C, av);
      ldv<V>(bb + idx, bv);
#pragma unroll
      for (int v = 0; v < V; ++v) {
        H[v] = av[v] * H[v] + bv[v];
        A[v] *= av[v];
      }
    }
  }
  const long long o = bk * C + c;
#pragma unroll
  for (int v = 0; v < V; ++v) {
    agg_a[o + v] = A[v];
    agg_h[o + v] = H[v];
  }
}

// Forward pass 2: fold the aggregates of the earlier chunks into a carry, then replay.
// mode 0: h (bf16) out. Optionally h0 [B, C] initial state and h_last [B, C] final state.
template <int V>
__global__ void scan_apply_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ bb,
                                  const int* __restrict__ doc_start, const float* __restrict__ agg_a,
                                  const float* __restrict__ agg_h, const float* __restrict__ h0,
                                  __nv_bfloat16* __restrict__ h, float* __restrict__ h_last, int B, int S, int C,
                                  int n_chunks) {
  const int CV = C / V;
  const long long total = (long long)B * n_chunks * CV;
  const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int c = (i % CV) * V;
  const long long bk = i / CV;
  const int k = bk % n_chunks;
  const int b = bk / n_chunks;
  float H[V];
#pragma unroll
  for (int v = 0; v < V; ++v) H[v] = h0 ? h0[(long long)b * C + c + v] : 0.f;
  for (int kk = 0; kk < k; ++kk) {
    const long long j = ((long long)b * n_chunks + kk) * C + c;
#pragma unroll
    for (int v = 0; v < V; ++v) H[v] = agg_a[j + v] * H[v] + agg_h[j + v];
  }
  const int s0 = k * SCAN_CHUNK, s1 = min(S, s0 + SCAN_CHUNK);
  for (int s = s0; s < s1; ++s) {
    const long long idx = ((long long)b * S + s) * C + c;
    float av[V], bv[V];
    ldv<V>(a + idx, av);
    ldv<V>(bb + idx, bv);
    const bool cut = doc_start && doc_start[(long long)b * S + s] == s;
#pragma unroll
    for (int v = 0; v < V; ++v) H[v] = (cut ? 0.f : av[v]) * H[v] + bv[v];
    stv<V>(h + idx, H);
  }
  if (h_last && k == n_chunks - 1) {
#pragma unroll
    for (int v = 0; v < V; ++v) h_last[(long long)b * C + c + v] = H[v];
  }
}

// Backward pass 2: g_s = dh_s + a_{s+1} g_{s+1} (reverse); db_s = g_s; da_s = g_s * h_{s-1}
// (h_{-1} = h0 or 0; 0 at a document start).
template <int V>
__global__ void scan_bwd_apply_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ h,
                                      const __nv_bfloat16* __restrict__ dh, const int* __restrict__ doc_start,
                                      const float* __restrict__ agg_a, const float* __restrict__ agg_h,
                                      const float* __restrict__ h0, __nv_bfloat16* __restrict__ da,
                                      __nv_bfloat16* __restrict__ db, int B, int S, int C, int n_chunks) {
  const int CV = C / V;
  const long long total = (long long)B * n_chunks * CV;
  const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int c = (i % CV) * V;
  const long long bk = i / CV;
  const int k = bk % n_chunks;
  const int b = bk / n_chunks;
  float G[V];
#pragma unroll
  for (int v = 0; v < V; ++v) G[v] = 0.f;
  for (int kk = n_chunks - 1; kk > k; --kk) {
    const long long j = ((long long)b * n_chunks + kk) * C + c;
#pragma unroll
    for (int v = 0; v < V; ++v) G[v] = agg_a[j + v] * G[v] + agg_h[j + v];
  }
  const int s0 = k * SCAN_CHUNK, s1 = min(S, s0 + SCAN_CHUNK);
  for (int s = s1 - 1; s >= s0; --s) {
    const long long idx = ((long long)b * S + s) * C + c;
    float av[V], dv[V], hp[V], o[V];
#pragma unroll
    for (int v = 0; v < V; ++v) { av[v] = 0.f; hp[v] = 0.f; }
    if (s + 1 < S && !(doc_start && doc_start[(long long)b * S + s + 1] == s + 1)) ldv<V>(a + idx + C, av);
    ldv<V>(dh + idx, dv);
#pragma unroll
    for (int v = 0; v < V; ++v) G[v] = av[v] * G[v] + dv[v];
    stv<V>(db + idx, G);
    // forward took a_s = 0 at the first token of a document: no gradient flows into it
    const bool cut = doc_start && doc_start[(long long)b * S + s] == s;
    if (!cut) {
      if (s > 0) {
        ldv<V>(h + idx - C, hp);
      } else if (h0) {
#pragma unroll
        for (int v = 0; v < V; ++v) hp[v] = h0[(long long)b * C + c + v];
      }
    }
#pragma unroll
    for (int v = 0; v < V; ++v) o[v] = G[v] * hp[v];
    stv<V>(da + idx, o);
  }
}

static inline int blocks_for(long long n, int t) { return (int)((n + t - 1) / t); }

}  // namespace lb

using namespace lb;
typedef __nv_bfloat16 bf16;

extern "C" int lb_conv1d_fwd(const void* x, const void* w, const int* doc_start, void* y, int B, int S, int C,
                             int W, long long ldx, long long ldy, int act, void* stream) {
  const long long total = (long long)B * S * C;
  if (total == 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  if (C % 8 == 0 && ldx % 8 == 0 && ldy % 8 == 0 && reinterpret_cast<uintptr_t>(x) % 16 == 0 &&
      reinterpret_cast<uintptr_t>(y) % 16 == 0 && W >= 2 && W <= 4) {
    const long long n_rows = (long long)B * S;
    dim3 vgrid((C / CONV_NV + 127) / 128, (unsigned)((n_rows + CONV_ROWS - 1) / CONV_ROWS));
    switch (W) {
      case 2: conv1d_fwd_vec_kernel<2><<<vgrid, 128, 0, st>>>((const bf16*)x, (const bf16*)w, doc_start, (bf16*)y, n_rows, S, C, ldx, ldy, act); break;
      case 3: conv1d_fwd_vec_kernel<3><<<vgrid, 128, 0, st>>>((const bf16*)x, (const bf16*)w, doc_start, (bf16*)y, n_rows, S, C, ldx, ldy, act); break;
      default: conv1d_fwd_vec_kernel<4><<<vgrid, 128, 0, st>>>((const bf16*)x, (const bf16*)w, doc_start, (bf16*)y, n_rows, S, C, ldx, ldy, act); break;
    }
    g_launches.fetch_add(1, std::memory_order_relaxed);
    cudaError_t ev = cudaGetLastError();
    return ev == cudaSuccess ? 0 : 400 + (int)ev;
  }
  long long nb = (total + 255) / 256;
  const long long cap = (long long)num_sms() * 16;
  int grid = (int)(nb < cap ? nb : cap);
  switch (W) {
    case 2: conv1d_fwd_kernel<2><<<grid, 256, 0, st>>>((const bf16*)x, (const bf16*)w, doc_start, (bf16*)y, B, S, C, ldx, ldy, act); break;
    case 3: conv1d_fwd_kernel<3><<<grid, 256, 0, st>>>((const bf16*)x, (const bf16*)w, doc_start, (bf16*)y, B, S, C, ldx, ldy, act); break;
    case 4: conv1d_fwd_kernel<4><<<grid, 256, 0, st>>>((const bf16*)x, (const bf16*)w, doc_start, (bf16*)y, B, S, C, ldx, ldy, act); break;
    default: return 1;
  }
  g_launches.fetch_add(1, std::memory_order_relaxed);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}

// dw: fp32 [C, W], accumulated into (zero it first for a fresh gradient)
extern "C" int lb_conv1d_bwd(const void* x, const void* w, const int* doc_start, const void* dy, void* dx, float* dw,
                             int B, int S, int C, int W, long long ldx, long long ldy, long long lddx, int act,
                             void* stream) {
  if ((long long)B * S * C == 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  if (C % 8 == 0 && ldx % 8 == 0 && ldy % 8 == 0 && lddx % 8 == 0 && reinterpret_cast<uintptr_t>(x) % 16 == 0 &&
      reinterpret_cast<uintptr_t>(dy) % 16 == 0 && reinterpret_cast<uintptr_t>(dx) % 16 == 0 && W >= 2 && W <= 4) {
    const long long n_rows = (long long)B * S;
    dim3 vgrid((C / CONV_NV + 127) / 128, (unsigned)((n_rows + CONV_ROWS - 1) / CONV_ROWS));
    switch (W) {
      case 2: conv1d_bwd_vec_kernel<2><<<vgrid, 128, 0, st>>>((const bf16*)x, (const bf16*)w, doc_start, (const bf16*)dy, (bf16*)dx, dw, n_rows, S, C, ldx, ldy, lddx, act); break;
      case 3: conv1d_bwd_vec_kernel<3><<<vgrid, 128, 0, st>>>((const bf16*)x, (const bf16*)w, doc_start, (const bf16*)dy, (bf16*)dx, dw, n_rows, S, C, ldx, ldy, lddx, act); break;
      default: conv1d_bwd_vec_kernel<4><<<vgrid, 128, 0, st>>>((const bf16*)x, (const bf16*)w, doc_start, (const bf16*)dy, (bf16*)dx, dw, n_rows, S, C, ldx, ldy, lddx, act); break;
    }
    g_launches.fetch_add(1, std::memory_order_relaxed);
    cudaError_t ev = cudaGetLastError();
    return ev == cudaSuccess ? 0 : 400 + (int)ev;
  }
  const int rows_per_thread = 64;
  dim3 grid((C + 127) / 128, (unsigned)(((long long)B * S + rows_per_thread - 1) / rows_per_thread));
  switch (W) {
    case 2: conv1d_bwd_kernel<2><<<grid, 128, 0, st>>>((const bf16*)x, (const bf16*)w, doc_start, (const bf16*)dy, (bf16*)dx, dw, B, S, C, ldx, ldy, lddx, act, rows_per_thread); break;
    case 3: conv1d_bwd_kernel<3><<<grid, 128, 0, st>>>((const bf16*)x, (const bf16*)w, doc_start, (const bf16*)dy, (bf16*)dx, dw, B, S, C, ldx, ldy, lddx, act, rows_per_thread); break;
    case 4: conv1d_bwd_kernel<4><<<grid, 128, 0, st>>>((const bf16*)x, (const bf16*)w, doc_start, (const bf16*)dy, (bf16*)dx, dw, B, S, C, ldx, ldy, lddx, act, rows_per_thread); break;
    default: return 1;
  }
  g_launches.fetch_add(1, std::memory_order_relaxed);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}

// a, b, h: contiguous [B, S, C] bf16. scratch: 2 * B * ceil(S/64) * C floats. h0 / h_last: [B, C]
// fp32 or NULL.
extern "C" int lb_scan_fwd(const void* a, const void* b, const int* doc_start, const float* h0, void* h,
                           float* h_last, float* scratch, int B, int S, int C, void* stream) {
  if ((long long)B * S * C == 0) return 0;
  const int n_chunks = (S + SCAN_CHUNK - 1) / SCAN_CHUNK;
  const long long n = (long long)B * n_chunks * C;
  float* agg_a = scratch;
  float* agg_h = scratch + n;
  cudaStream_t st = (cudaStream_t)stream;
  if (C % 2 == 0) {
    scan_reduce_kernel<2><<<blocks_for(n / 2, 256), 256, 0, st>>>((const bf16*)a, (const bf16*)b, doc_start, agg_a,
                                                                  agg_h, B, S, C, n_chunks, 0, nullptr);
    scan_apply_kernel<2><<<blocks_for(n / 2, 256), 256, 0, st>>>((const bf16*)a, (const bf16*)b, doc_start, agg_a,
                                                                 agg_h, h0, (bf16*)h, h_last, B, S, C, n_chunks);
  } else {
    scan_reduce_kernel<1><<<blocks_for(n, 256), 256, 0, st>>>((const bf16*)a, (const bf16*)b, doc_start, agg_a,
                                                              agg_h, B, S, C, n_chunks, 0, nullptr);
    scan_apply_kernel<1><<<blocks_for(n, 256), 256, 0, st>>>((const bf16*)a, (const bf16*)b, doc_start, agg_a, agg_h,
                                                             h0, (bf16*)h, h_last, B, S, C, n_chunks);
  }
  g_launches.fetch_add(2, std::memory_order_relaxed);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}

extern "C" int lb_scan_bwd(const void* a, const void* h, const void* dh, const int* doc_start, const float* h0,
                           void* da, void* db, float* scratch, int B, int S, int C, void* stream) {
  if ((long long)B * S * C == 0) return 0;
  const int n_chunks = (S + SCAN_CHUNK - 1) / SCAN_CHUNK;
  const long long n = (long long)B * n_chunks * C;
  float* agg_a = scratch;
  float* agg_h = scratch + n;
  cudaStream_t st = (cudaStream_t)stream;
  if (C % 2 == 0) {
    scan_reduce_kernel<2><<<blocks_for(n / 2, 256), 256, 0, st>>>(nullptr, (const bf16*)dh, doc_start, agg_a, agg_h,
                                                                  B, S, C, n_chunks, 1, (const bf16*)a);
    scan_bwd_apply_kernel<2><<<blocks_for(n / 2, 256), 256, 0, st>>>((const bf16*)a, (const bf16*)h, (const bf16*)dh,
                                                                     doc_start, agg_a, agg_h, h0, (bf16*)da,
                                                                     (bf16*)db, B, S, C, n_chunks);
  } else {
    scan_reduce_kernel<1><<<blocks_for(n, 256), 256, 0, st>>>(nullptr, (const bf16*)dh, doc_start, agg_a, agg_h, B, S,
                                                              C, n_chunks, 1, (const bf16*)a);
    scan_bwd_apply_kernel<1><<<blocks_for(n, 256), 256, 0, st>>>((const bf16*)a, (const bf16*)h, (const bf16*)dh,
                                                                 doc_start, agg_a, agg_h, h0, (bf16*)da, (bf16*)db, B,
                                                                 S, C, n_chunks);
  }
  g_launches.fetch_add(2, std::memory_order_relaxed);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}
