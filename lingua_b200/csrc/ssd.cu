// Mamba-2 chunked scan (SSD): the decay / mask step between the two intra-chunk matrix products.
//
// Inside a chunk of L tokens the output is (C B^T  o  K) (dt x) with the lower-triangular decay kernel
//     K[l, s] = exp(cs[l] - cs[s])   for s <= l and tokens l, s in the same document, else 0
// where cs is the running sum of dt * A inside the chunk. The matrix products run on the tcgen05 GEMM;
// this file builds W = (C B^T) o K directly in bf16 (forward) and turns dW into the gradients of C B^T and of
// cs (backward), without materialising K, the broadcast of C B^T over the heads of a group, or any other
// [batch, heads, chunks, L, L] fp32 temporary. It is the role of the chunk-scan kernels of
// mamba_ssm.ops.triton.ssd_combined used through apps/mamba/component/ssm_compilable.py:17-90.
//
// Layouts: scores [b, nc, g, L, L] bf16, cs [b, h, nc, L] fp32, doc [b, nc, L] int32 (document id of each
// token, or NULL), w / dw [b, nc, h, L, L] bf16. One block per (head, chunk, batch); a warp walks rows, a lane
// owns 8 consecutive columns, so every access is a 16-byte vector and a warp reads 512 contiguous bytes.
#include "common.cuh"
#include "lingua_b200.h"

namespace lb {

constexpr int SSD_THREADS = 256;

__device__ __forceinline__ void ssd_ld8(const __nv_bfloat16* p, float (&f)[8]) {
  const uint4 q = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 v = __bfloat1622float2(b[j]);
    f[2 * j] = v.x;
    f[2 * j + 1] = v.y;
  }
}

// grid (h, nc, b). L % 8 == 0.
__global__ void __launch_bounds__(SSD_THREADS)
ssd_decay_fwd_kernel(const __nv_bfloat16* __restrict__ scores, const float* __restrict__ cs,
                     const int* __restrict__ doc, __nv_bfloat16* __restrict__ w, int H, int G, int NC, int L) {
  const int h = blockIdx.x, c = blockIdx.y, b = blockIdx.z;
  const int g = h / (H / G);
  const __nv_bfloat16* sc = scores + (((long long)b * NC + c) * G + g) * L * L;
  const float* csr = cs + (((long long)b * H + h) * NC + c) * L;
  const int* dr = doc ? doc + ((long long)b * NC + c) * L : nullptr;
  __nv_bfloat16* wr = w + (((long long)b * NC + c) * H + h) * (long long)L * L;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nvec = L / 8;
  for (int l = warp; l < L; l += SSD_THREADS / 32) {
    const float cl = csr[l];
    const int dl = dr ? dr[l] : 0;
    for (int v = lane; v < nvec; v += 32) {
      const int s0 = v * 8;
      uint4 out = make_uint4(0u, 0u, 0u, 0u);
      if (s0 <= l) {
        float sv[8], o[8];
        ssd_ld8(sc + (long long)l * L + s0, sv);
        const float4 c0 = *reinterpret_cast<const float4*>(csr + s0);
        const float4 c1 = *reinterpret_cast<const float4*>(csr + s0 + 4);
        const float cv[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const bool ok = (s0 + j <= l) && (!dr || dr[s0 + j] == dl);
          o[j] = ok ? sv[j] * __expf(cl - cv[j]) : 0.f;
        }
        out.x = pack_bf16(o[0], o[1]);
        out.y = pack_bf16(o[2], o[3]);
        out.z = pack_bf16(o[4], o[5]);
        out.w = pack_bf16(o[6], o[7]);
      }
      *reinterpret_cast<uint4*>(wr + (long long)l * L + s0) = out;
    }
  }
}

// dscores[b, c, g, l, s] += dw * K (fp32, summed over the heads of the group with atomics);
// dcs[l] += sum_s e[l, s], dcs[s] -= sum_l e[l, s] with e = dw * scores * K. grid (h, nc, b).
// dcs must be zero on entry; dscores must be zero on entry.
__global__ void __launch_bounds__(SSD_THREADS)
ssd_decay_bwd_kernel(const __nv_bfloat16* __restrict__ dw, const __nv_bfloat16* __restrict__ scores,
                     const float* __restrict__ cs, const int* __restrict__ doc, float* __restrict__ dscores,
                     float* __restrict__ dcs, int H, int G, int NC, int L) {
  extern __shared__ float col_acc[];  // [L] column sums of e
  const int h = blockIdx.x, c = blockIdx.y, b = blockIdx.z;
  const int g = h / (H / G);
  const long long tile = (((long long)b * NC + c) * G + g) * L * L;
  const __nv_bfloat16* sc = scores + tile;
  float* dsc = dscores + tile;
  const float* csr = cs + (((long long)b * H + h) * NC + c) * L;
  float* dcsr = dcs + (((long long)b * H + h) * NC + c) * L;
  const int* dr = doc ? doc + ((long long)b * NC + c) * L : nullptr;
  const __nv_bfloat16* dwr = dw + (((long long)b * NC + c) * H + h) * (long long)L * L;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nvec = L / 8;
  for (int i = threadIdx.x; i < L; i += SSD_THREADS) col_acc[i] = 0.f;
  __syncthreads();
  float colr[2][8];  // column sums of this lane's (at most two) 8-column groups over the rows of its warp
#pragma unroll
  for (int q = 0; q < 2; ++q)
#pragma unroll
    for (int j = 0; j < 8; ++j) colr[q][j] = 0.f;
  for (int l = warp; l < L; l += SSD_THREADS / 32) {
    const float cl = csr[l];
    const int dl = dr ? dr[l] : 0;
    float row = 0.f;
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      const int v = lane + 32 * q;
      const int s0 = v * 8;
      if (v >= nvec || s0 > l) continue;
      float sv[8], dv[8];
      ssd_ld8(sc + (long long)l * L + s0, sv);
      ssd_ld8(dwr + (long long)l * L + s0, dv);
      const float4 c0 = *reinterpret_cast<const float4*>(csr + s0);
      const float4 c1 = *reinterpret_cast<const float4*>(csr + s0 + 4);
      const float cv[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
      float ds[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const bool ok = (s0 + j <= l) && (!dr || dr[s0 + j] == dl);
        const float k = ok ? __expf(cl - cv[j]) : 0.f;
        ds[j] = dv[j] * k;
        const float e = ds[j] * sv[j];
        row += e;
        colr[q][j] += e;
      }
      float4* dst = reinterpret_cast<float4*>(dsc + (long long)l * L + s0);
      atomicAdd(dst, make_float4(ds[0], ds[1], ds[2], ds[3]));
      atomicAdd(dst + 1, make_float4(ds[4], ds[5], ds[6], ds[7]));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) row += __shfl_xor_sync(0xffffffffu, row, o);
    if (lane == 0) atomicAdd(&dcsr[l], row);
  }
#pragma unroll
  for (int q = 0; q < 2; ++q) {
    const int v = lane + 32 * q;
    if (v < nvec) {
#pragma unroll
      for (int j = 0; j < 8; ++j) atomicAdd(&col_acc[v * 8 + j], colr[q][j]);
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < L; i += SSD_THREADS) atomicAdd(&dcsr[i], -col_acc[i]);
}

}  // namespace lb

extern "C" int lb_ssd_decay_fwd(const void* scores, const float* cs, const int* doc, void* w, int B, int H, int G,
                                int NC, int L, void* stream) {
  if (B <= 0 || H <= 0 || NC <= 0) return 0;
  if (L % 8 != 0 || L > 512 || G <= 0 || H % G != 0) return 1;
  dim3 grid(H, NC, B);
  lb::ssd_decay_fwd_kernel<<<grid, lb::SSD_THREADS, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(scores), cs, doc, reinterpret_cast<__nv_bfloat16*>(w), H, G, NC, L);
  lb::g_launches.fetch_add(1, std::memory_order_relaxed);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}

extern "C" int lb_ssd_decay_bwd(const void* dw, const void* scores, const float* cs, const int* doc, float* dscores,
                                float* dcs, int B, int H, int G, int NC, int L, void* stream) {
  if (B <= 0 || H <= 0 || NC <= 0) return 0;
  if (L % 8 != 0 || L > 512 || G <= 0 || H % G != 0) return 1;
  dim3 grid(H, NC, B);
  lb::ssd_decay_bwd_kernel<<<grid, lb::SSD_THREADS, L * sizeof(float), reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(dw), reinterpret_cast<const __nv_bfloat16*>(scores), cs, doc, dscores,
      dcs, H, G, NC, L);
  lb::g_launches.fetch_add(1, std::memory_order_relaxed);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}
