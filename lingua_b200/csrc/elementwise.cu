// Memory-bound kernels of the transformer path: RMSNorm (+ residual add), RoPE, SwiGLU /
// squared-ReLU, embedding gather / scatter-add, softmax cross-entropy over a logits chunk,
// AdamW on flat shards, gradient sum of squares. All take bf16 activations, do their math
// in fp32 (as lingua/transformer.py:51-56,126-139,283-289 do) and move 16 bytes per access.
#include "common.cuh"
#include "lingua_b200.h"

namespace lb {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
  return v;
}
// Block-wide sum; `red` holds >= 33 floats. Every thread gets the result.
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  if (w == 0) {
    float t = lane < nw ? red[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}
__device__ __forceinline__ float block_max(float v, float* red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  if (w == 0) {
    float t = lane < nw ? red[lane] : -INFINITY;
    t = warp_max(t);
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}

struct bf16x8 {
  uint4 raw;
  __device__ __forceinline__ void unpack(float (&f)[8]) const {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 t = __bfloat1622float2(h[i]);
      f[2 * i] = t.x;
      f[2 * i + 1] = t.y;
    }
  }
  __device__ __forceinline__ void pack(const float (&f)[8]) {
    raw.x = pack_bf16(f[0], f[1]);
    raw.y = pack_bf16(f[2], f[3]);
    raw.z = pack_bf16(f[4], f[5]);
    raw.w = pack_bf16(f[6], f[7]);
  }
};
__device__ __forceinline__ bf16x8 ld8(const __nv_bfloat16* p) {
  bf16x8 v;
  v.raw = *reinterpret_cast<const uint4*>(p);
  return v;
}
__device__ __forceinline__ void st8(__nv_bfloat16* p, const bf16x8& v) {
  *reinterpret_cast<uint4*>(p) = v.raw;
}

// ------------------------------------------------------------------ RMSNorm
// h = x (+ res); y = h * rsqrt(mean(h^2) + eps) * w.
// If res != null the sum h is also written to h_out (the new residual stream).
constexpr int NORM_MAX_VEC = 4;  // widest row: D <= 256 * 8 * 4

// One warp per row (eight rows per block): every lane keeps its part of the row packed in registers, all loads
// of a row are in flight together and the only exchange is a shuffle reduction -- no block barrier. VPL is the
// number of 16-byte vectors per lane (D <= 256 * VPL).
__device__ __forceinline__ void unpack8(const uint4& raw, float (&f)[8]) {
  bf16x8 v;
  v.raw = raw;
  v.unpack(f);
}
// WPR warps share a row (its halves); their partial sums meet in shared memory.
// Keeps the packed form live across a phase boundary: without it the compiler carries the unpacked fp32 values of
// the first pass over the row into the second one, which costs four times the registers.
__device__ __forceinline__ void keep_packed(uint4& v) {
  asm volatile("" : "+r"(v.x), "+r"(v.y), "+r"(v.z), "+r"(v.w));
}
template <int WPR>
__device__ __forceinline__ float row_sum(float v, float* part) {
  v = warp_sum(v);
  if (WPR == 1) return v;
  const int w = threadIdx.x >> 5;
  if ((threadIdx.x & 31) == 0) part[w] = v;
  __syncthreads();
  return part[w] + part[w ^ 1];
}
template <int VPL, int WPR>
__global__ void __launch_bounds__(256, 2) rmsnorm_fwd_warp_kernel(
    const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
    const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
    __nv_bfloat16* __restrict__ h_out, float* __restrict__ rstd_out, long long M, int D, float eps) {
  __shared__ float part[8];
  const int sub = (threadIdx.x >> 5) % WPR;  // which part of the row this warp holds
  const int lane = (threadIdx.x & 31) + 32 * sub;
  constexpr int LPR = 32 * WPR;  // lanes per row
  long long row = blockIdx.x * (long long)(8 / WPR) + (threadIdx.x >> 5) / WPR;
  // rows past the end are computed on the last row and not stored (no early exit: the block meets at a barrier)
  const int nvec = row < M ? D / 8 : 0;
  if (row >= M) row = M - 1;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * D);
  uint4 h[VPL];
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int v = lane + i * LPR;
    h[i] = v < nvec ? xr[v] : make_uint4(0u, 0u, 0u, 0u);
  }
  if (res) {
    const uint4* rr = reinterpret_cast<const uint4*>(res + row * D);
    uint4* ho = reinterpret_cast<uint4*>(h_out + row * D);
    constexpr int CH = VPL < 8 ? VPL : (VPL > 8 ? 4 : 8);
#pragma unroll
    for (int c = 0; c < VPL; c += CH) {
      uint4 r[CH];
#pragma unroll
      for (int i = 0; i < CH; ++i) {
        const int v = lane + (c + i) * LPR;
        r[i] = v < nvec ? rr[v] : make_uint4(0u, 0u, 0u, 0u);
      }
#pragma unroll
      for (int i = 0; i < CH; ++i) {
        const int v = lane + (c + i) * LPR;
        float a[8], b[8];
        unpack8(h[c + i], a);
        unpack8(r[i], b);
#pragma unroll
        for (int j = 0; j < 8; ++j) a[j] += b[j];
        bf16x8 o;
        o.pack(a);
        h[c + i] = o.raw;  // the normalised value uses the rounded residual, as a reload would
        if (v < nvec) ho[v] = o.raw;
      }
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    float a[8];
    unpack8(h[i], a);
#pragma unroll
    for (int j = 0; j < 8; ++j) ss += a[j] * a[j];
  }
  ss = row_sum<WPR>(ss, part);
#pragma unroll
  for (int i = 0; i < VPL; ++i) keep_packed(h[i]);
  const float rstd = rsqrtf(ss / D + eps);
  if (lane == 0 && nvec && rstd_out) rstd_out[row] = rstd;
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  uint4* yr = reinterpret_cast<uint4*>(y + row * D);
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int v = lane + i * LPR;
    if (v < nvec) {
      float a[8], wv[8];
      unpack8(h[i], a);
      unpack8(__ldg(wr + v), wv);
#pragma unroll
      for (int j = 0; j < 8; ++j) a[j] = a[j] * rstd * wv[j];
      bf16x8 o;
      o.pack(a);
      yr[v] = o.raw;
    }
  }
}

template <int VPL, int WPR>
__global__ void __launch_bounds__(256, 2) rmsnorm_bwd_dx_warp_kernel(
    const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
    const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd,
    const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx, long long M, int D) {
  __shared__ float part[8];
  const int sub = (threadIdx.x >> 5) % WPR;
  const int lane = (threadIdx.x & 31) + 32 * sub;
  constexpr int LPR = 32 * WPR;
  long long row = blockIdx.x * (long long)(8 / WPR) + (threadIdx.x >> 5) / WPR;
  const int nvec = row < M ? D / 8 : 0;
  if (row >= M) row = M - 1;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * D);
  const uint4* dr = reinterpret_cast<const uint4*>(dy + row * D);
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  uint4 xv[VPL], dv[VPL];
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int v = lane + i * LPR;
    xv[i] = v < nvec ? xr[v] : make_uint4(0u, 0u, 0u, 0u);
    dv[i] = v < nvec ? dr[v] : make_uint4(0u, 0u, 0u, 0u);
  }
  const float rs = rstd[row];
  float dot = 0.f;
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int v = lane + i * LPR;
    if (v < nvec) {
      float a[8], g[8], wv[8];
      unpack8(xv[i], a);
      unpack8(dv[i], g);
      unpack8(__ldg(wr + v), wv);
#pragma unroll
      for (int j = 0; j < 8; ++j) dot += g[j] * wv[j] * (a[j] * rs);
    }
  }
  dot = row_sum<WPR>(dot, part) / D;
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    keep_packed(xv[i]);
    keep_packed(dv[i]);
  }
  uint4* ox = reinterpret_cast<uint4*>(dx + row * D);
  const uint4* rr = reinterpret_cast<const uint4*>(dres ? dres + row * D : dy);
  constexpr int CH = VPL < 8 ? VPL : 8;
#pragma unroll
  for (int c = 0; c < VPL; c += CH) {
    uint4 r[CH];
    if (dres) {
#pragma unroll
      for (int i = 0; i < CH; ++i) {
        const int v = lane + (c + i) * LPR;
        r[i] = v < nvec ? rr[v] : make_uint4(0u, 0u, 0u, 0u);
      }
    }
#pragma unroll
    for (int i = 0; i < CH; ++i) {
      const int v = lane + (c + i) * LPR;
      if (v < nvec) {
        float a[8], g[8], wv[8], o[8];
        unpack8(xv[c + i], a);
        unpack8(dv[c + i], g);
        unpack8(__ldg(wr + v), wv);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = rs * (g[j] * wv[j] - a[j] * rs * dot);
        if (dres) {
          float b[8];
          unpack8(r[i], b);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += b[j];
        }
        bf16x8 ov;
        ov.pack(o);
        ox[v] = ov.raw;
      }
    }
  }
}

// Backward in two kernels. (1) one block per row: dx = rstd * (dy*w - xhat * mean(dy*w*xhat)) (+ dres).
// (2) dw += sum_rows dy * xhat as a column reduction: a block owns 256 columns and a band of rows,
// 8 row lanes accumulate in registers, are combined in shared memory and added with one atomic
// per column. Splitting costs one extra read of dy and x but keeps both kernels small enough for
// full occupancy (the fused single-kernel form was latency bound at 24 % of copy bandwidth).
__global__ void __launch_bounds__(256) rmsnorm_bwd_dx_kernel(
    const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
    const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd,
    const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx, int D) {
  __shared__ float red[33];
  const long long row = blockIdx.x;
  const int nvec = D / 8;
  const float rs = rstd[row];
  float xh[NORM_MAX_VEC][8], g[NORM_MAX_VEC][8];
  float dot = 0.f;
#pragma unroll
  for (int i = 0; i < NORM_MAX_VEC; ++i) {
    const int v = threadIdx.x + i * blockDim.x;
    if (v < nvec) {
      float xv[8], dv[8], wv[8];
      ld8(x + row * D + v * 8).unpack(xv);
      ld8(dy + row * D + v * 8).unpack(dv);
      ld8(w + v * 8).unpack(wv);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        xh[i][j] = xv[j] * rs;
        g[i][j] = dv[j] * wv[j];
        dot += g[i][j] * xh[i][j];
      }
    }
  }
  dot = block_sum(dot, red) / D;
#pragma unroll
  for (int i = 0; i < NORM_MAX_VEC; ++i) {
    const int v = threadIdx.x + i * blockDim.x;
    if (v < nvec) {
      float o[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = rs * (g[i][j] - xh[i][j] * dot);
      if (dres) {
        float r[8];
        ld8(dres + row * D + v * 8).unpack(r);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] += r[j];
      }
      bf16x8 ov;
      ov.pack(o);
      st8(dx + row * D + v * 8, ov);
    }
  }
}

constexpr int DW_ROWS_PER_BLOCK = 128;
__global__ void __launch_bounds__(256) rmsnorm_bwd_dw_kernel(
    const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x, const float* __restrict__ rstd,
    float* __restrict__ dw, long long M, int D) {
  __shared__ float part[8][32][8];
  const int cv = blockIdx.x * 32 + threadIdx.x;  // 8-column vector index
  const int ry = threadIdx.y;
  const long long r0 = (long long)blockIdx.y * DW_ROWS_PER_BLOCK;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (cv * 8 < D) {
    for (long long r = r0 + ry; r < r0 + DW_ROWS_PER_BLOCK && r < M; r += 8) {
      float xv[8], dv[8];
      ld8(x + r * D + cv * 8).unpack(xv);
      ld8(dy + r * D + cv * 8).unpack(dv);
      const float rs = rstd[r];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += dv[j] * xv[j] * rs;
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) part[ry][threadIdx.x][j] = acc[j];
  __syncthreads();
  if (ry == 0 && cv * 8 < D) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float t = 0.f;
#pragma unroll
      for (int y = 0; y < 8; ++y) t += part[y][threadIdx.x][j];
      atomicAdd(dw + cv * 8 + j, t);
    }
  }
}

// ------------------------------------------------------------------ RoPE
// In-place rotation of interleaved pairs of the first n_rot_heads heads of every token row
// (row stride `ld` elements). cs[pos][i] = (cos, sin) of pos * theta^(-2i/Dh).
// sign = +1 forward, -1 backward (the transpose of a rotation is the opposite rotation).
// A thread owns one 16-byte vector position of the head (4 rotation pairs) for one token and walks over the heads:
// the cos / sin values are loaded once per token instead of once per head, and eight heads are in flight at a time.
__global__ void __launch_bounds__(256) rope_kernel(__nv_bfloat16* __restrict__ qk, const float2* __restrict__ cs,
                                                   const int* __restrict__ pos_idx, long long n_tok, int seq_len,
                                                   int ld, int n_rot_heads, int head_dim, float sign) {
  const int vec_per_head = head_dim / 8;
  const long long total = n_tok * vec_per_head;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int v = i % vec_per_head;
    const long long tok = i / vec_per_head;
    const int pos = pos_idx ? pos_idx[tok] : (int)(tok % seq_len);
    const float4* c4 = reinterpret_cast<const float4*>(cs + (long long)pos * (head_dim / 2) + v * 4);
    const float4 c01 = __ldg(c4), c23 = __ldg(c4 + 1);
    const float cc[4] = {c01.x, c01.z, c23.x, c23.z};
    const float sn[4] = {c01.y * sign, c01.w * sign, c23.y * sign, c23.w * sign};
    __nv_bfloat16* base = qk + tok * ld + v * 8;
    int h = 0;
    for (; h + 8 <= n_rot_heads; h += 8) {
      bf16x8 in[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) in[u] = ld8(base + (h + u) * head_dim);
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        float f[8], o[8];
        in[u].unpack(f);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          o[2 * j] = f[2 * j] * cc[j] - f[2 * j + 1] * sn[j];
          o[2 * j + 1] = f[2 * j] * sn[j] + f[2 * j + 1] * cc[j];
        }
        bf16x8 ov;
        ov.pack(o);
        st8(base + (h + u) * head_dim, ov);
      }
    }
    for (; h < n_rot_heads; ++h) {
      float f[8], o[8];
      ld8(base + h * head_dim).unpack(f);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        o[2 * j] = f[2 * j] * cc[j] - f[2 * j + 1] * sn[j];
        o[2 * j + 1] = f[2 * j] * sn[j] + f[2 * j + 1] * cc[j];
      }
      bf16x8 ov;
      ov.pack(o);
      st8(base + h * head_dim, ov);
    }
  }
}

// ------------------------------------------------------------------ gated activations
// gu: [M, 2H] with the gate in columns [0,H) and the linear branch in [H,2H).
// mode 0: silu(g) * u (SwiGLU).  mode 1: relu(g)^2 * u.
__device__ __forceinline__ float act_f(float g, int mode) {
  if (mode == 0) return g / (1.f + __expf(-g));
  const float r = fmaxf(g, 0.f);
  return r * r;
}
__device__ __forceinline__ float act_df(float g, int mode) {
  if (mode == 0) {
    const float s = 1.f / (1.f + __expf(-g));
    return s * (1.f + g * (1.f - s));
  }
  return 2.f * fmaxf(g, 0.f);
}
__global__ void glu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out,
                               long long M, int H, int mode) {
  const int hv = H / 8;
  const long long total = M * hv;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / hv;
    const int c = (i % hv) * 8;
    float g[8], u[8], o[8];
    ld8(gu + r * 2 * H + c).unpack(g);
    ld8(gu + r * 2 * H + H + c).unpack(u);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = act_f(g[j], mode) * u[j];
    bf16x8 ov;
    ov.pack(o);
    st8(out + r * H + c, ov);
  }
}
// dgu[:, :H] = dout * u * act'(g); dgu[:, H:] = dout * act(g). dgu may alias gu.
__global__ void glu_bwd_kernel(const __nv_bfloat16* gu, const __nv_bfloat16* __restrict__ dout,
                               __nv_bfloat16* dgu, long long M, int H, int mode) {
  const int hv = H / 8;
  const long long total = M * hv;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / hv;
    const int c = (i % hv) * 8;
    float g[8], u[8], d[8], dg[8], du[8];
    ld8(gu + r * 2 * H + c).unpack(g);
    ld8(gu + r * 2 * H + H + c).unpack(u);
    ld8(dout + r * H + c).unpack(d);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      dg[j] = d[j] * u[j] * act_df(g[j], mode);
      du[j] = d[j] * act_f(g[j], mode);
    }
    bf16x8 a, b;
    a.pack(dg);
    b.pack(du);
    st8(dgu + r * 2 * H + c, a);
    st8(dgu + r * 2 * H + H + c, b);
  }
}
// Ungated activation on [n]: mode 0 silu, 1 relu^2. bwd: dx = dy * act'(x).
__global__ void act_fwd_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y,
                               long long n8, int mode) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n8;
       i += (long long)gridDim.x * blockDim.x) {
    float f[8];
    ld8(x + i * 8).unpack(f);
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = act_f(f[j], mode);
    bf16x8 o;
    o.pack(f);
    st8(y + i * 8, o);
  }
}
__global__ void act_bwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dy,
                               __nv_bfloat16* __restrict__ dx, long long n8, int mode) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n8;
       i += (long long)gridDim.x * blockDim.x) {
    float f[8], d[8];
    ld8(x + i * 8).unpack(f);
    ld8(dy + i * 8).unpack(d);
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = d[j] * act_df(f[j], mode);
    bf16x8 o;
    o.pack(f);
    st8(dx + i * 8, o);
  }
}

// out = a + b (bf16, fp32 math)
__global__ void add_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b,
                           __nv_bfloat16* __restrict__ out, long long n8) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n8;
       i += (long long)gridDim.x * blockDim.x) {
    float x[8], y[8];
    ld8(a + i * 8).unpack(x);
    ld8(b + i * 8).unpack(y);
#pragma unroll
    for (int j = 0; j < 8; ++j) x[j] += y[j];
    bf16x8 o;
    o.pack(x);
    st8(out + i * 8, o);
  }
}

// ------------------------------------------------------------------ embedding
__global__ void embed_fwd_kernel(const long long* __restrict__ tok, const __nv_bfloat16* __restrict__ table,
                                 __nv_bfloat16* __restrict__ out, long long n_tok, int D, int V) {
  const int dv = D / 8;
  const long long total = n_tok * dv;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / dv;
    const int c = (i % dv) * 8;
    long long id = tok[t];
    id = id < 0 ? 0 : (id >= V ? V - 1 : id);
    st8(out + t * D + c, ld8(table + id * D + c));
  }
}
// dtable[tok] += dy  (fp32 accumulation buffer)
__global__ void embed_bwd_kernel(const long long* __restrict__ tok, const __nv_bfloat16* __restrict__ dy,
                                 float* __restrict__ dtable, long long n_tok, int D, int V) {
  const int dv = D / 8;
  const long long total = n_tok * dv;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / dv;
    const int c = (i % dv) * 8;
    long long id = tok[t];
    if (id < 0 || id >= V) continue;
    float f[8];
    ld8(dy + t * D + c).unpack(f);
    float* dst = dtable + id * D + c;
#pragma unroll
    for (int j = 0; j < 8; ++j) atomicAdd(dst + j, f[j]);
  }
}

// ------------------------------------------------------------------ cross-entropy
// One block per row of fp32 logits [rows, V]. Writes loss[row] = lse - logit[target] and
// lse[row]; rows whose target is ignore_index (< 0) get loss 0.
__global__ void __launch_bounds__(512) ce_fwd_kernel(const float* __restrict__ logits,
                                                     const long long* __restrict__ target,
                                                     float* __restrict__ loss, float* __restrict__ lse,
                                                     int V, long long ld) {
  __shared__ float red[33];
  const long long row = blockIdx.x;
  const float* lr = logits + row * ld;
  const int nv = V / 4;
  float mx = -INFINITY;
  for (int i = threadIdx.x; i < nv; i += blockDim.x) {
    const float4 v = reinterpret_cast<const float4*>(lr)[i];
    mx = fmaxf(mx, fmaxf(fmaxf(v.x, v.y), fmaxf(v.z, v.w)));
  }
  for (int i = nv * 4 + threadIdx.x; i < V; i += blockDim.x) mx = fmaxf(mx, lr[i]);
  mx = block_max(mx, red);
  float s = 0.f;
  for (int i = threadIdx.x; i < nv; i += blockDim.x) {
    const float4 v = reinterpret_cast<const float4*>(lr)[i];
    s += __expf(v.x - mx) + __expf(v.y - mx) + __expf(v.z - mx) + __expf(v.w - mx);
  }
  for (int i = nv * 4 + threadIdx.x; i < V; i += blockDim.x) s += __expf(lr[i] - mx);
  s = block_sum(s, red);
  if (threadIdx.x == 0) {
    const float l = mx + logf(s);
    lse[row] = l;
    const long long t = target[row];
    loss[row] = (t >= 0 && t < V) ? l - lr[t] : 0.f;
  }
}
// dlogits[row] = (softmax(logits[row]) - onehot(target)) * scale[0] * gscale, as bf16.
__global__ void __launch_bounds__(512) ce_bwd_kernel(const float* __restrict__ logits,
                                                     const long long* __restrict__ target,
                                                     const float* __restrict__ lse,
                                                     const float* __restrict__ gscale_ptr, float scale,
                                                     __nv_bfloat16* __restrict__ dlogits, int V,
                                                     long long ld, long long ldd) {
  const long long row = blockIdx.x;
  const float* lr = logits + row * ld;
  __nv_bfloat16* dr = dlogits + row * ldd;
  const long long t = target[row];
  const bool valid = t >= 0 && t < V;
  const float sc = valid ? scale * (gscale_ptr ? gscale_ptr[0] : 1.f) : 0.f;
  const float l = lse[row];
  const int nv = V / 8;
  for (int i = threadIdx.x; i < nv; i += blockDim.x) {
    const float4 a = reinterpret_cast<const float4*>(lr)[2 * i];
    const float4 b = reinterpret_cast<const float4*>(lr)[2 * i + 1];
    float f[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float p = __expf(f[j] - l);
      if (i * 8 + j == t) p -= 1.f;
      f[j] = p * sc;
    }
    bf16x8 o;
    o.pack(f);
    st8(dr + i * 8, o);
  }
  for (int i = nv * 8 + threadIdx.x; i < V; i += blockDim.x) {
    float p = __expf(lr[i] - l);
    if (i == t) p -= 1.f;
    dr[i] = __float2bfloat16(p * sc);
  }
}

// ------------------------------------------------------------------ optimiser
// sum of squares of a flat fp32 buffer, accumulated into out[0] (fp32 atomics of per-block
// partials that were reduced in double).
__global__ void __launch_bounds__(512) sumsq_kernel(const float* __restrict__ g, long long n,
                                                    float* __restrict__ out) {
  __shared__ float red[33];
  float s = 0.f;
  const long long n4 = n / 4;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4;
       i += (long long)gridDim.x * blockDim.x) {
    // streaming load (evict first): this pass runs next to the GEMMs of the backward pass and must not
    // push their operand tiles out of L2
    const float4 v = __ldcs(reinterpret_cast<const float4*>(g) + i);
    s += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  if (blockIdx.x == 0)
    for (long long i = n4 * 4 + threadIdx.x; i < n; i += blockDim.x) s += g[i] * g[i];
  s = block_sum(s, red);
  if (threadIdx.x == 0) atomicAdd(out, s);
}

// AdamW on a flat fp32 shard (torch.optim.AdamW semantics: decoupled weight decay, bias
// correction), with the clip coefficient min(1, max_norm / (sqrt(sumsq) + 1e-6)) taken from
// a device scalar so that no host synchronisation is needed, and the updated weights
// written back both as fp32 master and as bf16 compute copy.
__global__ void __launch_bounds__(256) adamw_kernel(float* __restrict__ p, float* __restrict__ m,
                                                    float* __restrict__ v, const float* __restrict__ g,
                                                    __nv_bfloat16* __restrict__ p16, long long n,
                                                    const float* __restrict__ sumsq, float max_norm,
                                                    float grad_mul, float lr, float beta1, float beta2,
                                                    float eps, float wd, float bc1, float bc2_sqrt) {
  float clip = grad_mul;
  if (sumsq && max_norm > 0.f) {
    const float nrm = sqrtf(sumsq[0]) * grad_mul;
    clip *= fminf(1.f, max_norm / (nrm + 1e-6f));
  }
  const long long n4 = n / 4;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4;
       i += (long long)gridDim.x * blockDim.x) {
    float4 pv = reinterpret_cast<float4*>(p)[i];
    float4 mv = reinterpret_cast<float4*>(m)[i];
    float4 vv = reinterpret_cast<float4*>(v)[i];
    const float4 gv = reinterpret_cast<const float4*>(g)[i];
    float pa[4] = {pv.x, pv.y, pv.z, pv.w}, ma[4] = {mv.x, mv.y, mv.z, mv.w};
    float va[4] = {vv.x, vv.y, vv.z, vv.w};
    const float ga[4] = {gv.x * clip, gv.y * clip, gv.z * clip, gv.w * clip};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      pa[j] *= (1.f - lr * wd);
      ma[j] = beta1 * ma[j] + (1.f - beta1) * ga[j];
      va[j] = beta2 * va[j] + (1.f - beta2) * ga[j] * ga[j];
      const float denom = sqrtf(va[j]) / bc2_sqrt + eps;
      pa[j] -= (lr / bc1) * ma[j] / denom;
    }
    reinterpret_cast<float4*>(p)[i] = make_float4(pa[0], pa[1], pa[2], pa[3]);
    reinterpret_cast<float4*>(m)[i] = make_float4(ma[0], ma[1], ma[2], ma[3]);
    reinterpret_cast<float4*>(v)[i] = make_float4(va[0], va[1], va[2], va[3]);
    if (p16) {
      uint2 o;
      o.x = pack_bf16(pa[0], pa[1]);
      o.y = pack_bf16(pa[2], pa[3]);
      reinterpret_cast<uint2*>(p16)[i] = o;
    }
  }
  if (blockIdx.x == 0) {
    for (long long i = n4 * 4 + threadIdx.x; i < n; i += blockDim.x) {
      float pa = p[i] * (1.f - lr * wd);
      const float ga = g[i] * clip;
      const float ma = beta1 * m[i] + (1.f - beta1) * ga;
      const float va = beta2 * v[i] + (1.f - beta2) * ga * ga;
      pa -= (lr / bc1) * ma / (sqrtf(va) / bc2_sqrt + eps);
      p[i] = pa; m[i] = ma; v[i] = va;
      if (p16) p16[i] = __float2bfloat16(pa);
    }
  }
}

__global__ void cast_f32_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst,
                                     long long n) {
  const long long n4 = n / 4;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4;
       i += (long long)gridDim.x * blockDim.x) {
    const float4 v = reinterpret_cast<const float4*>(src)[i];
    uint2 o;
    o.x = pack_bf16(v.x, v.y);
    o.y = pack_bf16(v.z, v.w);
    reinterpret_cast<uint2*>(dst)[i] = o;
  }
  if (blockIdx.x == 0)
    for (long long i = n4 * 4 + threadIdx.x; i < n; i += blockDim.x) dst[i] = __float2bfloat16(src[i]);
}

static inline int grid_for(long long work_items, int threads, int per_sm = 8) {
  long long b = (work_items + threads - 1) / threads;
  const long long cap = (long long)num_sms() * per_sm;
  if (b > cap) b = cap;
  if (b < 1) b = 1;
  return (int)b;
}
#define LB_LAUNCH_END()                                  \
  g_launches.fetch_add(1, std::memory_order_relaxed);    \
  {                                                      \
    cudaError_t e__ = cudaGetLastError();                \
    return e__ == cudaSuccess ? 0 : 400 + (int)e__;      \
  }

}  // namespace lb

using namespace lb;
typedef __nv_bfloat16 bf16;
#define S_(s) reinterpret_cast<cudaStream_t>(s)

extern "C" int lb_rmsnorm_fwd(const void* x, const void* res, const void* w, void* y, void* h_out,
                              float* rstd, long long M, int D, float eps, void* stream) {
  if (D % 8 || D > 256 * 8 * NORM_MAX_VEC) return 1;
  if (M == 0) return 0;
  if (res && !h_out) return 2;
#define LB_NORM_FWD(V, W)                                                                                  \
  rmsnorm_fwd_warp_kernel<V, W><<<(unsigned)((M + 8 / W - 1) / (8 / W)), 256, 0, S_(stream)>>>(              \
      (const bf16*)x, (const bf16*)res, (const bf16*)w, (bf16*)y, (bf16*)h_out, rstd, M, D, eps)
  if (D <= 256 * 4) LB_NORM_FWD(4, 1);
  else if (D <= 256 * 8) LB_NORM_FWD(8, 1);
  else if (D <= 256 * 16) LB_NORM_FWD(8, 2);
  else LB_NORM_FWD(16, 2);
#undef LB_NORM_FWD
  LB_LAUNCH_END();
}
extern "C" int lb_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd,
                              const void* dres, void* dx, float* dw, long long M, int D, void* stream) {
  if (D % 8 || D > 256 * 8 * NORM_MAX_VEC) return 1;
  if (M == 0) return 0;
#define LB_NORM_BWD(V, W)                                                                                  \
  rmsnorm_bwd_dx_warp_kernel<V, W><<<(unsigned)((M + 8 / W - 1) / (8 / W)), 256, 0, S_(stream)>>>(           \
      (const bf16*)dy, (const bf16*)x, (const bf16*)w, rstd, (const bf16*)dres, (bf16*)dx, M, D)
  if (D <= 256 * 4) LB_NORM_BWD(4, 1);
  else if (D <= 256 * 8) LB_NORM_BWD(8, 1);
  else if (D <= 256 * 16) LB_NORM_BWD(8, 2);
  else  // two packed operands of a wider row do not fit the lanes' registers: one block per row
    rmsnorm_bwd_dx_kernel<<<(unsigned)M, 256, 0, S_(stream)>>>((const bf16*)dy, (const bf16*)x, (const bf16*)w, rstd,
                                                              (const bf16*)dres, (bf16*)dx, D);
#undef LB_NORM_BWD
  if (dw) {
    dim3 grid((D / 8 + 31) / 32, (unsigned)((M + DW_ROWS_PER_BLOCK - 1) / DW_ROWS_PER_BLOCK));
    rmsnorm_bwd_dw_kernel<<<grid, dim3(32, 8), 0, S_(stream)>>>((const bf16*)dy, (const bf16*)x, rstd, dw, M, D);
    g_launches.fetch_add(1, std::memory_order_relaxed);
  }
  LB_LAUNCH_END();
}
extern "C" int lb_rope(void* qk, const void* cs, const int* pos_idx, long long n_tok, int seq_len, int ld,
                       int n_rot_heads, int head_dim, int backward, void* stream) {
  if (head_dim % 8 || ld % 8) return 1;
  const long long total = n_tok * (head_dim / 8);
  if (total == 0 || n_rot_heads == 0) return 0;
  rope_kernel<<<grid_for(total, 256), 256, 0, S_(stream)>>>((bf16*)qk, (const float2*)cs, pos_idx, n_tok, seq_len,
                                                            ld, n_rot_heads, head_dim, backward ? -1.f : 1.f);
  LB_LAUNCH_END();
}
extern "C" int lb_glu_fwd(const void* gu, void* out, long long M, int H, int mode, void* stream) {
  if (H % 8) return 1;
  glu_fwd_kernel<<<grid_for(M * (H / 8), 256), 256, 0, S_(stream)>>>((const bf16*)gu, (bf16*)out, M, H, mode);
  LB_LAUNCH_END();
}
extern "C" int lb_glu_bwd(const void* gu, const void* dout, void* dgu, long long M, int H, int mode, void* stream) {
  if (H % 8) return 1;
  glu_bwd_kernel<<<grid_for(M * (H / 8), 256), 256, 0, S_(stream)>>>((const bf16*)gu, (const bf16*)dout, (bf16*)dgu, M, H, mode);
  LB_LAUNCH_END();
}
extern "C" int lb_act_fwd(const void* x, void* y, long long n, int mode, void* stream) {
  if (n % 8) return 1;
  act_fwd_kernel<<<grid_for(n / 8, 256), 256, 0, S_(stream)>>>((const bf16*)x, (bf16*)y, n / 8, mode);
  LB_LAUNCH_END();
}
extern "C" int lb_act_bwd(const void* x, const void* dy, void* dx, long long n, int mode, void* stream) {
  if (n % 8) return 1;
  act_bwd_kernel<<<grid_for(n / 8, 256), 256, 0, S_(stream)>>>((const bf16*)x, (const bf16*)dy, (bf16*)dx, n / 8, mode);
  LB_LAUNCH_END();
}
extern "C" int lb_add(const void* a, const void* b, void* out, long long n, void* stream) {
  if (n % 8) return 1;
  add_kernel<<<grid_for(n / 8, 256), 256, 0, S_(stream)>>>((const bf16*)a, (const bf16*)b, (bf16*)out, n / 8);
  LB_LAUNCH_END();
}
extern "C" int lb_embed_fwd(const long long* tok, const void* table, void* out, long long n_tok, int D, int V,
                            void* stream) {
  if (D % 8) return 1;
  embed_fwd_kernel<<<grid_for(n_tok * (D / 8), 256), 256, 0, S_(stream)>>>(tok, (const bf16*)table, (bf16*)out, n_tok, D, V);
  LB_LAUNCH_END();
}
extern "C" int lb_embed_bwd(const long long* tok, const void* dy, float* dtable, long long n_tok, int D, int V,
                            void* stream) {
  if (D % 8) return 1;
  embed_bwd_kernel<<<grid_for(n_tok * (D / 8), 256), 256, 0, S_(stream)>>>(tok, (const bf16*)dy, dtable, n_tok, D, V);
  LB_LAUNCH_END();
}
extern "C" int lb_ce_fwd(const float* logits, const long long* target, float* loss, float* lse, long long rows,
                         int V, long long ld, void* stream) {
  if (ld % 4) return 1;
  if (rows == 0) return 0;
  ce_fwd_kernel<<<(unsigned)rows, 512, 0, S_(stream)>>>(logits, target, loss, lse, V, ld);
  LB_LAUNCH_END();
}
extern "C" int lb_ce_bwd(const float* logits, const long long* target, const float* lse, const float* gscale,
                         float scale, void* dlogits, long long rows, int V, long long ld, long long ldd,
                         void* stream) {
  if (ld % 4 || ldd % 8) return 1;
  if (rows == 0) return 0;
  ce_bwd_kernel<<<(unsigned)rows, 512, 0, S_(stream)>>>(logits, target, lse, gscale, scale, (bf16*)dlogits, V, ld, ldd);
  LB_LAUNCH_END();
}
extern "C" int lb_sumsq(const float* g, long long n, float* out, void* stream) {
  if (n == 0) return 0;
  if (reinterpret_cast<uintptr_t>(g) % 16) return 1;
  sumsq_kernel<<<grid_for(n / 4 + 1, 512, 4), 512, 0, S_(stream)>>>(g, n, out);
  LB_LAUNCH_END();
}
extern "C" int lb_adamw(float* p, float* m, float* v, const float* g, void* p16, long long n, const float* sumsq,
                        float max_norm, float grad_mul, float lr, float beta1, float beta2, float eps, float wd,
                        int step, void* stream) {
  if (n == 0) return 0;
  if ((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(m) | reinterpret_cast<uintptr_t>(v) |
       reinterpret_cast<uintptr_t>(g)) % 16 || reinterpret_cast<uintptr_t>(p16) % 8)
    return 1;
  const float bc1 = 1.f - powf(beta1, (float)step);
  const float bc2s = sqrtf(1.f - powf(beta2, (float)step));
  adamw_kernel<<<grid_for(n / 4 + 1, 256, 8), 256, 0, S_(stream)>>>(p, m, v, g, (bf16*)p16, n, sumsq, max_norm,
                                                                    grad_mul, lr, beta1, beta2, eps, wd, bc1, bc2s);
  LB_LAUNCH_END();
}
extern "C" int lb_cast_f32_bf16(const float* src, void* dst, long long n, void* stream) {
  if (n == 0) return 0;
  if (reinterpret_cast<uintptr_t>(src) % 16 || reinterpret_cast<uintptr_t>(dst) % 8) return 1;
  cast_f32_bf16_kernel<<<grid_for(n / 4 + 1, 256, 8), 256, 0, S_(stream)>>>(src, (bf16*)dst, n);
  LB_LAUNCH_END();
}
