// Vectorised causal depthwise conv1d (forward / backward) for channel counts and row pitches that
// are multiples of 8: one thread owns 4 adjacent channels (one 8-byte vector per token) and walks
// a run of consecutive tokens with the last W-1 inputs kept in registers, so every token costs one
// vector load and one vector store and a warp reads 256 contiguous bytes per token.
// Included by scan.cu; same arithmetic and masking rules as the scalar kernels there.
#pragma once
#include "common.cuh"

namespace lb {

constexpr int CONV_ROWS = 32;  // tokens per thread

constexpr int CONV_NV = 4;  // channels per thread: 8-byte vectors keep the register count low enough for
                            // full occupancy, and a warp still covers 256 contiguous bytes per token
__device__ __forceinline__ void ld8(const __nv_bfloat16* p, float (&f)[CONV_NV]) {
  const uint2 q = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
  for (int j = 0; j < CONV_NV / 2; ++j) {
    const float2 v = __bfloat1622float2(b[j]);
    f[2 * j] = v.x;
    f[2 * j + 1] = v.y;
  }
}
__device__ __forceinline__ void st8(__nv_bfloat16* p, const float (&f)[CONV_NV]) {
  uint2 q;
  q.x = pack_bf16(f[0], f[1]);
  q.y = pack_bf16(f[2], f[3]);
  *reinterpret_cast<uint2*>(p) = q;
}
__device__ __forceinline__ float conv_silu(float x) { return x / (1.f + __expf(-x)); }
__device__ __forceinline__ float conv_dsilu(float x) {
  const float s = 1.f / (1.f + __expf(-x));
  return s * (1.f + x * (1.f - s));
}

// grid: (ceil(C/CONV_NV / blockDim.x), ceil(B*S / CONV_ROWS))
template <int W>
__global__ void __launch_bounds__(128)
conv1d_fwd_vec_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                      const int* __restrict__ doc_start, __nv_bfloat16* __restrict__ y, long long n_rows, int S,
                      int C, long long ldx, long long ldy, int act) {
  const int c0 = (blockIdx.x * blockDim.x + threadIdx.x) * CONV_NV;
  if (c0 >= C) return;
  float wv[W][CONV_NV];  // wv[j][k]: tap j of channel c0 + k
#pragma unroll
  for (int k = 0; k < CONV_NV; ++k)
#pragma unroll
    for (int j = 0; j < W; ++j) wv[j][k] = __bfloat162float(w[(c0 + k) * W + j]);
  const long long r0 = (long long)blockIdx.y * CONV_ROWS;
  const long long r1 = min(n_rows, r0 + CONV_ROWS);
  float win[W][CONV_NV];  // win[j]: input of token s - (W-1) + j
  for (long long r = r0; r < r1; ++r) {
    const int s = r % S;
    if (r == r0 || s == 0) {  // (re)fill the history at the start of the run or of a sequence
#pragma unroll
      for (int j = 0; j < W - 1; ++j) {
        const int t = s - (W - 1) + j;
        if (t >= 0) {
          ld8(x + (r - (W - 1) + j) * ldx + c0, win[j]);
        } else {
#pragma unroll
          for (int k = 0; k < CONV_NV; ++k) win[j][k] = 0.f;
        }
      }
    }
    ld8(x + r * ldx + c0, win[W - 1]);
    const int lo = doc_start ? doc_start[r] : 0;
    float acc[CONV_NV];
#pragma unroll
    for (int k = 0; k < CONV_NV; ++k) acc[k] = 0.f;
#pragma unroll
    for (int j = 0; j < W; ++j) {
      if (s - (W - 1) + j >= lo) {
#pragma unroll
        for (int k = 0; k < CONV_NV; ++k) acc[k] += wv[j][k] * win[j][k];
      }
    }
    if (act) {
#pragma unroll
      for (int k = 0; k < CONV_NV; ++k) acc[k] = conv_silu(acc[k]);
    }
    st8(y + r * ldy + c0, acc);
#pragma unroll
    for (int j = 0; j < W - 1; ++j)
#pragma unroll
      for (int k = 0; k < CONV_NV; ++k) win[j][k] = win[j + 1][k];
  }
}

// Backward. For the run of tokens [r0, r1) this thread
//   * recomputes g(so) = dy(so) * act'(pre(so)) for so in [r0, r1 + W - 1) (same sequence only),
//   * emits dx(t) = sum_j w[j] g(t + W-1-j) [t >= lo(t + W-1-j)] for t in [r0, r1),
//   * adds g(so) x(so - (W-1) + j) [valid tap] to dw[., j] for so in [r0, r1) only, so that every
//     output position is counted once over the grid.
template <int W>
__global__ void __launch_bounds__(128)
conv1d_bwd_vec_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                      const int* __restrict__ doc_start, const __nv_bfloat16* __restrict__ dy,
                      __nv_bfloat16* __restrict__ dx, float* __restrict__ dw, long long n_rows, int S, int C,
                      long long ldx, long long ldy, long long lddx, int act) {
  const int c0 = (blockIdx.x * blockDim.x + threadIdx.x) * CONV_NV;
  if (c0 >= C) return;
  float wv[W][CONV_NV], dwacc[W][CONV_NV];
#pragma unroll
  for (int k = 0; k < CONV_NV; ++k)
#pragma unroll
    for (int j = 0; j < W; ++j) {
      wv[j][k] = __bfloat162float(w[(c0 + k) * W + j]);
      dwacc[j][k] = 0.f;
    }
  const long long r0 = (long long)blockIdx.y * CONV_ROWS;
  const long long r1 = min(n_rows, r0 + CONV_ROWS);
  float xin[W][CONV_NV];  // inputs of tokens so - (W-1) .. so
  float gw[W][CONV_NV];   // gw[j] = g(so - (W-1) + j), 0 where that output does not exist
  int low[W];       // lo of the same outputs (INT_MAX marks "no such output")
#pragma unroll
  for (int j = 0; j < W; ++j) {
    low[j] = 0x7FFFFFFF;
#pragma unroll
    for (int k = 0; k < CONV_NV; ++k) gw[j][k] = 0.f;
  }
  // so runs over the outputs that read any token of [r0, r1): same-sequence rows up to r1 + W - 2
  for (long long so = r0; so < r1 + W - 1; ++so) {
    // outputs past the end of the sequence of the token they would feed do not exist
    const long long t_emit = so - (W - 1);  // token whose dx is complete after this step
    bool exists = so < n_rows;
    const int s_o = exists ? (int)(so % S) : 0;
    // slide the windows
#pragma unroll
    for (int j = 0; j < W - 1; ++j) {
      low[j] = low[j + 1];
#pragma unroll
      for (int k = 0; k < CONV_NV; ++k) gw[j][k] = gw[j + 1][k];
    }
    if (exists) {
      if (so == r0 || s_o == 0) {
#pragma unroll
        for (int j = 0; j < W - 1; ++j) {
          const int t = s_o - (W - 1) + j;
          if (t >= 0) {
            ld8(x + (so - (W - 1) + j) * ldx + c0, xin[j]);
          } else {
#pragma unroll
            for (int k = 0; k < CONV_NV; ++k) xin[j][k] = 0.f;
          }
        }
      }
      ld8(x + so * ldx + c0, xin[W - 1]);
      const int lo = doc_start ? doc_start[so] : 0;
      float g[CONV_NV];
      ld8(dy + so * ldy + c0, g);
      if (act) {
        float pre[CONV_NV];
#pragma unroll
        for (int k = 0; k < CONV_NV; ++k) pre[k] = 0.f;
#pragma unroll
        for (int j = 0; j < W; ++j)
          if (s_o - (W - 1) + j >= lo) {
#pragma unroll
            for (int k = 0; k < CONV_NV; ++k) pre[k] += wv[j][k] * xin[j][k];
          }
#pragma unroll
        for (int k = 0; k < CONV_NV; ++k) g[k] *= conv_dsilu(pre[k]);
      }
      if (so < r1) {  // this run owns output so: its share of dw
#pragma unroll
        for (int j = 0; j < W; ++j)
          if (s_o - (W - 1) + j >= lo) {
#pragma unroll
            for (int k = 0; k < CONV_NV; ++k) dwacc[j][k] += g[k] * xin[j][k];
          }
      }
      low[W - 1] = lo;
#pragma unroll
      for (int k = 0; k < CONV_NV; ++k) gw[W - 1][k] = g[k];
#pragma unroll
      for (int j = 0; j < W - 1; ++j)
#pragma unroll
        for (int k = 0; k < CONV_NV; ++k) xin[j][k] = xin[j + 1][k];
    } else {
      low[W - 1] = 0x7FFFFFFF;
#pragma unroll
      for (int k = 0; k < CONV_NV; ++k) gw[W - 1][k] = 0.f;
    }
    // dx of token t_emit: outputs t_emit .. t_emit + W - 1 = window entries 0 .. W-1, tap W-1-j
    if (t_emit >= r0 && t_emit < r1) {
      const int s_t = (int)(t_emit % S);
      float acc[CONV_NV];
#pragma unroll
      for (int k = 0; k < CONV_NV; ++k) acc[k] = 0.f;
#pragma unroll
      for (int j = 0; j < W; ++j) {
        // window entry j is output t_emit + j; it exists, lies in the same sequence (s_t + j < S) and
        // used token t_emit (tap W-1-j) iff s_t >= its lo
        if (low[j] != 0x7FFFFFFF && s_t + j < S && s_t >= low[j]) {
#pragma unroll
          for (int k = 0; k < CONV_NV; ++k) acc[k] += wv[W - 1 - j][k] * gw[j][k];
        }
      }
      st8(dx + t_emit * lddx + c0, acc);
    }
  }
#pragma unroll
  for (int j = 0; j < W; ++j)
#pragma unroll
    for (int k = 0; k < CONV_NV; ++k) atomicAdd(dw + (c0 + k) * W + j, dwacc[j][k]);
}

}  // namespace lb
