// Mamba-2 chunked scan (SSD): everything around its four batched matrix products that is not the decay kernel
// of ssd.cu. Three steps, one kernel each way, replacing some forty elementwise / reduction / copy launches per
// layer and direction of a PyTorch formulation (the role of the _chunk_cumsum, _chunk_state, _state_passing and
// _chunk_scan pieces of mamba_ssm.ops.triton.ssd_combined, apps/mamba/component/ssm_compilable.py:17-90):
//
//   prep     cs = running sum of dt * A inside each chunk, xdt = x * dt, xw = xdt * exp(cs_last - cs)
//            (the operand of the chunk-state product; zero where the token's document ends before the chunk does)
//   carry    the state handed from chunk to chunk: prev[c] = S_c, S_{c+1} = a_c * S_c + T_c
//   combine  y = y_diag + y_off * exp(cs) (only for tokens that continue the carried document) + D * x
//
// Layouts (contiguous unless a pitch is given): x [b, s, h, p] bf16 with token pitch ldx; dt [b, s, h] fp32;
// cs [b, h, nc, L] fp32; xdt / xw / y / dy [b, s, h, p] bf16; doc [b, nc, L] int32 document id per token or NULL;
// chunk states T / prev [b, nc, h, p, n] bf16; a [b, h, nc] fp32; y_diag [b, nc, h, L, p] bf16;
// y_off [b, nc, g, L, (h / g) * p] bf16. p % 8 == 0, p <= 256, L <= 1024.
#include "common.cuh"
#include "lingua_b200.h"

namespace lb {

using bf16 = __nv_bfloat16;
constexpr int SG_THREADS = 256;
constexpr int SG_MAXL = 1024;

__device__ __forceinline__ void sg_ld8(const bf16* p, float (&f)[8]) {
  const uint4 q = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 v = __bfloat1622float2(b[j]);
    f[2 * j] = v.x;
    f[2 * j + 1] = v.y;
  }
}
__device__ __forceinline__ void sg_st8(bf16* p, const float (&f)[8]) {
  uint4 q;
  q.x = pack_bf16(f[0], f[1]);
  q.y = pack_bf16(f[2], f[3]);
  q.z = pack_bf16(f[4], f[5]);
  q.w = pack_bf16(f[6], f[7]);
  *reinterpret_cast<uint4*>(p) = q;
}
// sum over the `width` (power of two, <= 32) consecutive lanes that share one row
__device__ __forceinline__ float sg_row_sum(float v, int width) {
  for (int o = width >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float sg_block_sum(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = 0.f;
  for (int i = 0; i < SG_THREADS / 32; ++i) t += red[i];
  return t;
}

// ---------------------------------------------------------------- prep. grid (h, nc, b)
__global__ void __launch_bounds__(SG_THREADS)
ssd_prep_fwd_kernel(const bf16* __restrict__ x, long long ldx, const float* __restrict__ dt,
                    const float* __restrict__ A, const int* __restrict__ doc, float* __restrict__ cs,
                    bf16* __restrict__ xdt, bf16* __restrict__ xw, int S, int H, int P, int NC, int L) {
  __shared__ float s_cs[SG_MAXL], s_dt[SG_MAXL];
  const int h = blockIdx.x, c = blockIdx.y, b = blockIdx.z;
  const long long tok0 = (long long)b * S + (long long)c * L;
  const float a = A[h];
  for (int l = threadIdx.x; l < L; l += SG_THREADS) {
    const float d = dt[(tok0 + l) * H + h];
    s_dt[l] = d;
    s_cs[l] = d * a;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float run = 0.f;
    for (int l = 0; l < L; ++l) {
      run += s_cs[l];
      s_cs[l] = run;
    }
  }
  __syncthreads();
  float* csr = cs + (((long long)b * H + h) * NC + c) * L;
  for (int l = threadIdx.x; l < L; l += SG_THREADS) csr[l] = s_cs[l];
  const float cs_last = s_cs[L - 1];
  const int* dr = doc ? doc + ((long long)b * NC + c) * L : nullptr;
  const int d_last = dr ? dr[L - 1] : 0;
  const int vp = P / 8;
  for (int i = threadIdx.x; i < L * vp; i += SG_THREADS) {
    const int l = i / vp, v = i - l * vp;
    float f[8], o1[8], o2[8];
    sg_ld8(x + (tok0 + l) * ldx + h * P + v * 8, f);
    const float d = s_dt[l];
    const float e = (!dr || dr[l] == d_last) ? __expf(cs_last - s_cs[l]) : 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      o1[j] = f[j] * d;
      o2[j] = o1[j] * e;
    }
    const long long off = ((tok0 + l) * H + h) * P + v * 8;
    sg_st8(xdt + off, o1);
    sg_st8(xw + off, o2);
  }
}

// d_cs / d_xdt / d_xw may be NULL (no gradient from that output). dA must be zero on entry (atomics).
__global__ void __launch_bounds__(SG_THREADS)
ssd_prep_bwd_kernel(const bf16* __restrict__ x, long long ldx, const float* __restrict__ dt,
                    const float* __restrict__ A, const int* __restrict__ doc, const float* __restrict__ cs,
                    const float* __restrict__ d_cs, const bf16* __restrict__ d_xdt, const bf16* __restrict__ d_xw,
                    bf16* __restrict__ dx, float* __restrict__ ddt, float* __restrict__ dA, int S, int H, int P, int NC,
                    int L) {
  __shared__ float s_cs[SG_MAXL], s_dt[SG_MAXL], s_s1[SG_MAXL], s_s2[SG_MAXL];
  __shared__ float red[SG_THREADS / 32];
  const int h = blockIdx.x, c = blockIdx.y, b = blockIdx.z;
  const long long tok0 = (long long)b * S + (long long)c * L;
  const float a = A[h];
  const float* csr = cs + (((long long)b * H + h) * NC + c) * L;
  for (int l = threadIdx.x; l < L; l += SG_THREADS) {
    s_dt[l] = dt[(tok0 + l) * H + h];
    s_cs[l] = csr[l];
  }
  __syncthreads();
  const float cs_last = s_cs[L - 1];
  const int* dr = doc ? doc + ((long long)b * NC + c) * L : nullptr;
  const int d_last = dr ? dr[L - 1] : 0;
  const int vp = P / 8;
  // rows are walked by groups of vp lanes; all lanes of a warp stay in the loop together (L * vp % 32 == 0 is not
  // required: the row sums use shuffles only among the vp lanes of a row, and vp divides 32)
  const int n_items = L * vp;
  for (int i0 = 0; i0 < n_items; i0 += SG_THREADS) {
    const int i = i0 + threadIdx.x;
    const bool live = i < n_items;
    const int l = live ? i / vp : 0, v = live ? i - l * vp : 0;
    float s1 = 0.f, s2 = 0.f;
    if (live) {
      float f[8], g1[8], g2[8], o[8];
      const long long off = ((tok0 + l) * H + h) * P + v * 8;
      sg_ld8(x + (tok0 + l) * ldx + h * P + v * 8, f);
      if (d_xdt) sg_ld8(d_xdt + off, g1);
      if (d_xw) sg_ld8(d_xw + off, g2);
      const float d = s_dt[l];
      const float e = (!dr || dr[l] == d_last) ? __expf(cs_last - s_cs[l]) : 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float tot = (d_xdt ? g1[j] : 0.f) + (d_xw ? g2[j] * e : 0.f);
        o[j] = tot * d;
        s1 += tot * f[j];
        if (d_xw) s2 += g2[j] * f[j];
      }
      sg_st8(dx + off, o);
    }
    s1 = sg_row_sum(s1, vp);
    s2 = sg_row_sum(s2, vp);
    if (live && v == 0) {
      s_s1[l] = s1;
      s_s2[l] = s2;
    }
  }
  __syncthreads();
  // gradient of cs: from outside, and through E_l = exp(cs_last - cs_l)
  float to_last = 0.f;
  const float* dcs_in = d_cs ? d_cs + (((long long)b * H + h) * NC + c) * L : nullptr;
  for (int l = threadIdx.x; l < L; l += SG_THREADS) {
    const float e = (!dr || dr[l] == d_last) ? __expf(cs_last - s_cs[l]) : 0.f;
    const float dE = s_dt[l] * s_s2[l];
    s_s2[l] = (dcs_in ? dcs_in[l] : 0.f) - dE * e;
    to_last += dE * e;
  }
  to_last = sg_block_sum(to_last, red);
  __syncthreads();
  if (threadIdx.x == 0) {
    s_s2[L - 1] += to_last;
    float run = 0.f;  // reverse running sum: gradient of dt * A at l collects every later cs
    for (int l = L - 1; l >= 0; --l) {
      run += s_s2[l];
      s_s2[l] = run;
    }
  }
  __syncthreads();
  float da = 0.f;
  for (int l = threadIdx.x; l < L; l += SG_THREADS) {
    ddt[(tok0 + l) * H + h] = s_s1[l] + s_s2[l] * a;
    da += s_s2[l] * s_dt[l];
  }
  da = sg_block_sum(da, red);
  if (threadIdx.x == 0) atomicAdd(dA + h, da);
}

// ---------------------------------------------------------------- carry. one thread per 4 state elements
// grid (ceil(P * N / 4 / 256), h, b)
__global__ void __launch_bounds__(SG_THREADS)
ssd_carry_fwd_kernel(const bf16* __restrict__ T, const float* __restrict__ a, const float* __restrict__ init,
                     bf16* __restrict__ prev, float* __restrict__ fin, int H, int NC, long long PN) {
  const int h = blockIdx.y, b = blockIdx.z;
  const long long e = ((long long)blockIdx.x * SG_THREADS + threadIdx.x) * 4;
  if (e >= PN) return;
  const long long bh = ((long long)b * H + h);
  float4 st = init ? *reinterpret_cast<const float4*>(init + bh * PN + e) : make_float4(0.f, 0.f, 0.f, 0.f);
  for (int c = 0; c < NC; ++c) {
    const long long off = (((long long)b * NC + c) * H + h) * PN + e;
    uint2 o;
    o.x = pack_bf16(st.x, st.y);
    o.y = pack_bf16(st.z, st.w);
    *reinterpret_cast<uint2*>(prev + off) = o;
    const uint2 t = *reinterpret_cast<const uint2*>(T + off);
    const float2 t01 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&t.x));
    const float2 t23 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&t.y));
    const float ac = a[bh * NC + c];
    st.x = ac * st.x + t01.x;
    st.y = ac * st.y + t01.y;
    st.z = ac * st.z + t23.x;
    st.w = ac * st.w + t23.y;
  }
  *reinterpret_cast<float4*>(fin + bh * PN + e) = st;
}

// da must be zero on entry (atomics). d_prev / d_fin may be NULL.
__global__ void __launch_bounds__(SG_THREADS)
ssd_carry_bwd_kernel(const bf16* __restrict__ prev, const float* __restrict__ a, const bf16* __restrict__ d_prev,
                     const float* __restrict__ d_fin, bf16* __restrict__ dT, float* __restrict__ da,
                     float* __restrict__ d_init, int H, int NC, long long PN) {
  __shared__ float red[SG_THREADS / 32];
  const int h = blockIdx.y, b = blockIdx.z;
  const long long e = ((long long)blockIdx.x * SG_THREADS + threadIdx.x) * 4;
  const bool live = e < PN;
  const long long bh = ((long long)b * H + h);
  float4 g = (live && d_fin) ? *reinterpret_cast<const float4*>(d_fin + bh * PN + e) : make_float4(0.f, 0.f, 0.f, 0.f);
  for (int c = NC - 1; c >= 0; --c) {
    const long long off = (((long long)b * NC + c) * H + h) * PN + e;
    float dot = 0.f;
    if (live) {
      uint2 o;
      o.x = pack_bf16(g.x, g.y);
      o.y = pack_bf16(g.z, g.w);
      *reinterpret_cast<uint2*>(dT + off) = o;
      const uint2 s = *reinterpret_cast<const uint2*>(prev + off);
      const float2 s01 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&s.x));
      const float2 s23 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&s.y));
      dot = g.x * s01.x + g.y * s01.y + g.z * s23.x + g.w * s23.y;
      const float ac = a[bh * NC + c];
      float4 dp = make_float4(0.f, 0.f, 0.f, 0.f);
      if (d_prev) {
        const uint2 q = *reinterpret_cast<const uint2*>(d_prev + off);
        const float2 q01 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&q.x));
        const float2 q23 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&q.y));
        dp = make_float4(q01.x, q01.y, q23.x, q23.y);
      }
      g.x = dp.x + ac * g.x;
      g.y = dp.y + ac * g.y;
      g.z = dp.z + ac * g.z;
      g.w = dp.w + ac * g.w;
    }
    const float tot = sg_block_sum(dot, red);
    if (threadIdx.x == 0) atomicAdd(da + bh * NC + c, tot);
  }
  if (live && d_init) *reinterpret_cast<float4*>(d_init + bh * PN + e) = g;
}

// ---------------------------------------------------------------- combine. grid (h, nc, b)
__global__ void __launch_bounds__(SG_THREADS)
ssd_combine_fwd_kernel(const bf16* __restrict__ y_diag, const bf16* __restrict__ y_off, const float* __restrict__ cs,
                       const int* __restrict__ doc, const bf16* __restrict__ x, long long ldx,
                       const float* __restrict__ D, int d_has_p, bf16* __restrict__ y, int S, int H, int G, int P,
                       int NC, int L) {
  const int h = blockIdx.x, c = blockIdx.y, b = blockIdx.z;
  const int rep = H / G, g = h / rep, r = h - g * rep;
  const long long tok0 = (long long)b * S + (long long)c * L;
  const float* csr = cs + (((long long)b * H + h) * NC + c) * L;
  const int* dr = doc ? doc + ((long long)b * NC + c) * L : nullptr;
  const int prev_last = (dr && c > 0) ? dr[-1] : -1;  // document of the last token of the previous chunk
  const bf16* yd = y_diag + (((long long)b * NC + c) * H + h) * (long long)L * P;
  const bf16* yo = y_off + (((long long)b * NC + c) * G + g) * (long long)L * rep * P + (long long)r * P;
  const int vp = P / 8;
  for (int i = threadIdx.x; i < L * vp; i += SG_THREADS) {
    const int l = i / vp, v = i - l * vp;
    float a[8], o[8], f[8], out[8];
    sg_ld8(yd + (long long)l * P + v * 8, a);
    sg_ld8(yo + (long long)l * rep * P + v * 8, o);
    const bool carried = !dr || (c > 0 && dr[l] == prev_last);
    const float e = (dr ? carried : true) ? __expf(csr[l]) : 0.f;
    if (D) sg_ld8(x + (tok0 + l) * ldx + h * P + v * 8, f);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      out[j] = a[j] + o[j] * e;
      if (D) out[j] += (d_has_p ? D[h * P + v * 8 + j] : D[h]) * f[j];
    }
    sg_st8(y + ((tok0 + l) * H + h) * P + v * 8, out);
  }
}

// dD must be zero on entry (atomics). dx_d (the D * x path's share of dx) is written only when D is given.
__global__ void __launch_bounds__(SG_THREADS)
ssd_combine_bwd_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ y_off, const float* __restrict__ cs,
                       const int* __restrict__ doc, const bf16* __restrict__ x, long long ldx,
                       const float* __restrict__ D, int d_has_p, bf16* __restrict__ d_ydiag,
                       bf16* __restrict__ d_yoff, float* __restrict__ dcs, bf16* __restrict__ dx_d,
                       float* __restrict__ dD, int S, int H, int G, int P, int NC, int L) {
  __shared__ float s_dD[256];
  __shared__ float red[SG_THREADS / 32];
  const int h = blockIdx.x, c = blockIdx.y, b = blockIdx.z;
  const int rep = H / G, g = h / rep, r = h - g * rep;
  const long long tok0 = (long long)b * S + (long long)c * L;
  const float* csr = cs + (((long long)b * H + h) * NC + c) * L;
  float* dcsr = dcs + (((long long)b * H + h) * NC + c) * L;
  const int* dr = doc ? doc + ((long long)b * NC + c) * L : nullptr;
  const int prev_last = (dr && c > 0) ? dr[-1] : -1;
  bf16* gd = d_ydiag + (((long long)b * NC + c) * H + h) * (long long)L * P;
  const long long yo_base = (((long long)b * NC + c) * G + g) * (long long)L * rep * P + (long long)r * P;
  const int vp = P / 8;
  for (int i = threadIdx.x; i < P; i += SG_THREADS) s_dD[i] = 0.f;
  __syncthreads();
  float dd_h = 0.f;
  const int n_items = L * vp;
  for (int i0 = 0; i0 < n_items; i0 += SG_THREADS) {
    const int i = i0 + threadIdx.x;
    const bool live = i < n_items;
    const int l = live ? i / vp : 0, v = live ? i - l * vp : 0;
    float rowdot = 0.f;
    if (live) {
      float gy[8], o[8], f[8], t[8];
      sg_ld8(dy + ((tok0 + l) * H + h) * P + v * 8, gy);
      sg_ld8(y_off + yo_base + (long long)l * rep * P + v * 8, o);
      const bool carried = !dr || (c > 0 && dr[l] == prev_last);
      const float e = (dr ? carried : true) ? __expf(csr[l]) : 0.f;
      sg_st8(gd + (long long)l * P + v * 8, gy);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        t[j] = gy[j] * e;
        rowdot += gy[j] * o[j] * e;
      }
      sg_st8(d_yoff + yo_base + (long long)l * rep * P + v * 8, t);
      if (D) {
        sg_ld8(x + (tok0 + l) * ldx + h * P + v * 8, f);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          t[j] = gy[j] * (d_has_p ? D[h * P + v * 8 + j] : D[h]);
          if (d_has_p)
            atomicAdd(&s_dD[v * 8 + j], gy[j] * f[j]);
          else
            dd_h += gy[j] * f[j];
        }
        sg_st8(dx_d + ((tok0 + l) * H + h) * P + v * 8, t);
      }
    }
    rowdot = sg_row_sum(rowdot, vp);
    if (live && v == 0) dcsr[l] = rowdot;
  }
  if (D) {
    if (d_has_p) {
      __syncthreads();
      for (int i = threadIdx.x; i < P; i += SG_THREADS) atomicAdd(dD + h * P + i, s_dD[i]);
    } else {
      dd_h = sg_block_sum(dd_h, red);
      if (threadIdx.x == 0) atomicAdd(dD + h, dd_h);
    }
  }
}

static inline bool sg_shape_ok(int P, int L) {
  const int vp = P / 8;
  return P % 8 == 0 && P <= 256 && vp > 0 && (32 % vp) == 0 && L > 0 && L <= SG_MAXL;
}

}  // namespace lb

using lb::bf16;

extern "C" int lb_ssd_prep_fwd(const void* x, long long ldx, const float* dt, const float* A, const int* doc, float* cs,
                               void* xdt, void* xw, int B, int S, int H, int P, int NC, int L, void* stream) {
  if (B <= 0 || NC <= 0 || H <= 0) return 0;
  if (!lb::sg_shape_ok(P, L) || NC * L != S || ldx % 8) return 1;
  lb::ssd_prep_fwd_kernel<<<dim3(H, NC, B), lb::SG_THREADS, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      (const bf16*)x, ldx, dt, A, doc, cs, (bf16*)xdt, (bf16*)xw, S, H, P, NC, L);
  lb::g_launches.fetch_add(1, std::memory_order_relaxed);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}

extern "C" int lb_ssd_prep_bwd(const void* x, long long ldx, const float* dt, const float* A, const int* doc,
                               const float* cs, const float* d_cs, const void* d_xdt, const void* d_xw, void* dx,
                               float* ddt, float* dA, int B, int S, int H, int P, int NC, int L, void* stream) {
  if (B <= 0 || NC <= 0 || H <= 0) return 0;
  if (!lb::sg_shape_ok(P, L) || NC * L != S || ldx % 8) return 1;
  lb::ssd_prep_bwd_kernel<<<dim3(H, NC, B), lb::SG_THREADS, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      (const bf16*)x, ldx, dt, A, doc, cs, d_cs, (const bf16*)d_xdt, (const bf16*)d_xw, (bf16*)dx, ddt, dA, S, H, P, NC,
      L);
  lb::g_launches.fetch_add(1, std::memory_order_relaxed);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}

extern "C" int lb_ssd_carry_fwd(const void* T, const float* a, const float* init, void* prev, float* fin, int B, int H,
                                int NC, long long PN, void* stream) {
  if (B <= 0 || NC <= 0 || H <= 0) return 0;
  if (PN % 4) return 1;
  const unsigned gx = (unsigned)((PN / 4 + lb::SG_THREADS - 1) / lb::SG_THREADS);
  lb::ssd_carry_fwd_kernel<<<dim3(gx, H, B), lb::SG_THREADS, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      (const bf16*)T, a, init, (bf16*)prev, fin, H, NC, PN);
  lb::g_launches.fetch_add(1, std::memory_order_relaxed);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}

extern "C" int lb_ssd_carry_bwd(const void* prev, const float* a, const void* d_prev, const float* d_fin, void* dT,
                                float* da, float* d_init, int B, int H, int NC, long long PN, void* stream) {
  if (B <= 0 || NC <= 0 || H <= 0) return 0;
  if (PN % 4) return 1;
  const unsigned gx = (unsigned)((PN / 4 + lb::SG_THREADS - 1) / lb::SG_THREADS);
  lb::ssd_carry_bwd_kernel<<<dim3(gx, H, B), lb::SG_THREADS, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      (const bf16*)prev, a, (const bf16*)d_prev, d_fin, (bf16*)dT, da, d_init, H, NC, PN);
  lb::g_launches.fetch_add(1, std::memory_order_relaxed);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}

extern "C" int lb_ssd_combine_fwd(const void* y_diag, const void* y_off, const float* cs, const int* doc, const void* x,
                                  long long ldx, const float* D, int d_has_p, void* y, int B, int S, int H, int G, int P,
                                  int NC, int L, void* stream) {
  if (B <= 0 || NC <= 0 || H <= 0) return 0;
  if (!lb::sg_shape_ok(P, L) || NC * L != S || G <= 0 || H % G || ldx % 8) return 1;
  lb::ssd_combine_fwd_kernel<<<dim3(H, NC, B), lb::SG_THREADS, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      (const bf16*)y_diag, (const bf16*)y_off, cs, doc, (const bf16*)x, ldx, D, d_has_p, (bf16*)y, S, H, G, P, NC, L);
  lb::g_launches.fetch_add(1, std::memory_order_relaxed);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}

extern "C" int lb_ssd_combine_bwd(const void* dy, const void* y_off, const float* cs, const int* doc, const void* x,
                                  long long ldx, const float* D, int d_has_p, void* d_ydiag, void* d_yoff, float* dcs,
                                  void* dx_d, float* dD, int B, int S, int H, int G, int P, int NC, int L,
                                  void* stream) {
  if (B <= 0 || NC <= 0 || H <= 0) return 0;
  if (!lb::sg_shape_ok(P, L) || NC * L != S || G <= 0 || H % G || ldx % 8) return 1;
  lb::ssd_combine_bwd_kernel<<<dim3(H, NC, B), lb::SG_THREADS, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      (const bf16*)dy, (const bf16*)y_off, cs, doc, (const bf16*)x, ldx, D, d_has_p, (bf16*)d_ydiag, (bf16*)d_yoff,
      dcs, (bf16*)dx_d, dD, S, H, G, P, NC, L);
  lb::g_launches.fetch_add(1, std::memory_order_relaxed);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}
