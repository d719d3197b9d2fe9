// Float8 (e4m3) linear layers on tcgen05: row-wise scaled GEMM and the quantisation kernels.
//
//   C[m, n] = (sum_k A8[m, k] * B8[n, k]) * row_scale[m] * col_scale[n]
//
// A8 / B8 are e4m3 with K contiguous; the scales are the fp32 factors the operands were divided
// by before rounding ("row-wise scaling": one per row of the activation, one per output feature
// of the weight). This is the arithmetic of lingua/float8.py:44-78 (scale(), matmul() around
// torch._scaled_mm); there the product comes from a cuBLAS / CUTLASS kernel, here from
// tcgen05.mma kind::f8f6f4 with the two scale vectors applied while the accumulator is drained.
//
// Same pipeline as the bf16 kernel (gemm.cu): TMA warp -> 4-stage ring of 128 x 128-byte and
// 256 x 128-byte swizzled tiles (128 e4m3 along K per stage), one MMA thread, two TMEM
// accumulators, four epilogue warps.
//
// Quantisation:
//   lb_quant_rows       x bf16 [rows, K] -> e4m3 [rows, K], scale[r] = max(|x[r, :]|, eps) / 448
//   lb_quant_transpose  w bf16 [N, K]    -> e4m3 [K, N] with one scale for the whole tensor
//                       (the weight operand of the input-gradient product, float8.py:116-127)
#include "common.cuh"
#include "lingua_b200.h"

namespace lb {
namespace f8 {

constexpr int BM = 128, BN = 256, BK = 128, UMMA_K = 32, STAGES = 4;
constexpr int A_BYTES = BM * 128, B_BYTES = BN * 128, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int SMEM = STAGES * STAGE_BYTES + 1024 + 256;
constexpr int THREADS = 192;
constexpr float E4M3_MAX = 448.f;
constexpr float AMAX_EPS = 1e-12f;

struct Params {
  int M, N, K, tiles_m, tiles_n;
  long long ldc;
  const float* row_scale;
  const float* col_scale;
  void* C;
  uint32_t* status;
  uint32_t idesc;  // carries the operand formats (e4m3 / e5m2)
};

template <typename OutT>
__global__ void __launch_bounds__(THREADS, 1)
gemm_fp8_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                const Params p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ int abort_flag;
  __shared__ uint32_t tmem_base_slot;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar_base = smem_base + STAGES * STAGE_BYTES;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 4);
    }
    fence_mbar_init();
    tma_prefetch_desc(&tma_a);
    tma_prefetch_desc(&tma_b);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&tmem_base_slot), 2 * BN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  const int num_kb = (p.K + BK - 1) / BK;
  const int num_tiles = p.tiles_m * p.tiles_n;

  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0;
      for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
        const int m0 = (tile % p.tiles_m) * BM, n0 = (tile / p.tiles_m) * BN;
        bool ok = true;
        for (int kb = 0; kb < num_kb && ok; ++kb, ++it) {
          const int s = it % STAGES;
          ok = mbar_wait(empty_bar(s), ((it / STAGES) & 1u) ^ 1u, &abort_flag, p.status, 1);
          if (!ok) break;
          mbar_arrive_expect_tx(full_bar(s), STAGE_BYTES);
          const uint32_t sa = smem_base + s * STAGE_BYTES;
          tma_load_4d(sa, &tma_a, full_bar(s), kb * BK, m0, 0, 0);
          tma_load_4d(sa + A_BYTES, &tma_b, full_bar(s), kb * BK, n0, 0, 0);
        }
        if (!ok) break;
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = p.idesc;
      uint32_t it = 0, tile_iter = 0;
      for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++tile_iter) {
        const int acc = tile_iter & 1;
        if (!mbar_wait(tempty_bar(acc), ((tile_iter >> 1) & 1u) ^ 1u, &abort_flag, p.status, 2)) break;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * BN;
        bool ok = true;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          ok = mbar_wait(full_bar(s), (it / STAGES) & 1u, &abort_flag, p.status, 3);
          if (!ok) break;
          tc_fence_after();
          const uint32_t sa = smem_base + s * STAGE_BYTES, sb = sa + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            umma_f8(tmem_d, make_smem_desc(sa + k * 32u, 16u, 1024u), make_smem_desc(sb + k * 32u, 16u, 1024u), idesc,
                    (kb | k) != 0);
          umma_commit(empty_bar(s));
        }
        if (!ok) break;
        umma_commit(tfull_bar(acc));
      }
    }
  } else {
    const int quarter = warp & 3;
    uint32_t tile_iter = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++tile_iter) {
      const int acc = tile_iter & 1;
      const int m0 = (tile % p.tiles_m) * BM, n0 = (tile / p.tiles_m) * BN;
      const int row = m0 + quarter * 32 + lane;
      const float rs = (row < p.M && p.row_scale) ? __ldg(p.row_scale + row) : 1.f;
      if (!mbar_wait(tfull_bar(acc), (tile_iter >> 1) & 1u, &abort_flag, p.status, 4)) break;
      tc_fence_after();
      OutT* crow = reinterpret_cast<OutT*>(p.C) + static_cast<long long>(row) * p.ldc;
      const uint32_t taddr = tmem_base + acc * BN + (static_cast<uint32_t>(quarter * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        const int col0 = n0 + c * 32;
        if (col0 >= p.N) break;
        uint32_t r[32];
        tmem_ld32(taddr + c * 32, r);
        tmem_wait_ld();
        if (row < p.M) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            const int col = col0 + g * 8;
            if (col < p.N) {
              float f[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                const float cs = (p.col_scale && col + j < p.N) ? __ldg(p.col_scale + col + j) : 1.f;
                f[j] = __uint_as_float(r[g * 8 + j]) * rs * cs;
              }
              if (sizeof(OutT) == 2) {
                uint4 v;
                v.x = pack_bf16(f[0], f[1]); v.y = pack_bf16(f[2], f[3]);
                v.z = pack_bf16(f[4], f[5]); v.w = pack_bf16(f[6], f[7]);
                *reinterpret_cast<uint4*>(crow + col) = v;
              } else {
                float4* dst = reinterpret_cast<float4*>(crow + col);
                dst[0] = make_float4(f[0], f[1], f[2], f[3]);
                dst[1] = make_float4(f[4], f[5], f[6], f[7]);
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar(acc));
    }
  }
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (abort_flag) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * BN);
  }
}

template <typename OutT>
static int launch(const LbGemmFp8Args& a, cudaStream_t stream) {
  CUtensorMap ta, tb;
  int rc = make_tmap_4d(&ta, a.A, 1, a.K, a.M, a.lda, 1, 0, 1, 0, BK, BM);
  if (rc) return 100 + rc;
  rc = make_tmap_4d(&tb, a.B, 1, a.K, a.N, a.ldb, 1, 0, 1, 0, BK, BN);
  if (rc) return 200 + rc;
  Params p;
  p.M = a.M; p.N = a.N; p.K = a.K;
  p.tiles_m = (a.M + BM - 1) / BM;
  p.tiles_n = (a.N + BN - 1) / BN;
  p.ldc = a.ldc;
  p.row_scale = a.row_scale; p.col_scale = a.col_scale;
  p.C = a.C; p.status = a.status;
  p.idesc = make_idesc(BM, BN, (uint32_t)a.a_fmt, (uint32_t)a.b_fmt, 0, 0);
  const long long tiles = (long long)p.tiles_m * p.tiles_n;
  const int grid = (int)(tiles < num_sms() ? tiles : num_sms());
  auto kern = gemm_fp8_kernel<OutT>;
  if (ensure_dyn_smem<gemm_fp8_kernel<OutT>>(SMEM)) return 300;
  kern<<<grid, THREADS, SMEM, stream>>>(ta, tb, p);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}

// ------------------------------------------------------------------ quantisation
constexpr int Q_THREADS = 256;
constexpr int Q_MAXV = 8;  // 8-element vectors per thread held in registers: K <= 16384

template <int FMT = 0>
__device__ __forceinline__ uint32_t cvt_e4m3x4(float a, float b, float c, float d) {
  const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, FMT ? __NV_E5M2 : __NV_E4M3);
  const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, FMT ? __NV_E5M2 : __NV_E4M3);
  return lo | (hi << 16);
}
constexpr float E5M2_MAX = 57344.f;

template <int FMT>
__global__ void __launch_bounds__(Q_THREADS)
quant_rows_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, int K, uint8_t* __restrict__ out,
                  long long ldo, float* __restrict__ scale) {
  const long long row = blockIdx.x;
  const int nvec = K / 8;
  uint4 raw[Q_MAXV];
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < Q_MAXV; ++i) {
    const int v = threadIdx.x + i * Q_THREADS;
    if (v < nvec) {
      raw[i] = *reinterpret_cast<const uint4*>(x + row * ldx + v * 8);
      const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&raw[i]);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(b[j]);
        amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
      }
    }
  }
  __shared__ float red[Q_THREADS / 32];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = 0.f;
#pragma unroll
  for (int i = 0; i < Q_THREADS / 32; ++i) amax = fmaxf(amax, red[i]);
  const float sc = fmaxf(amax, AMAX_EPS) / (FMT ? E5M2_MAX : E4M3_MAX);
  const float inv = 1.f / sc;
  if (threadIdx.x == 0) scale[row] = sc;
#pragma unroll
  for (int i = 0; i < Q_MAXV; ++i) {
    const int v = threadIdx.x + i * Q_THREADS;
    if (v < nvec) {
      const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&raw[i]);
      const float2 f0 = __bfloat1622float2(b[0]), f1 = __bfloat1622float2(b[1]);
      const float2 f2 = __bfloat1622float2(b[2]), f3 = __bfloat1622float2(b[3]);
      uint2 o;
      o.x = cvt_e4m3x4<FMT>(f0.x * inv, f0.y * inv, f1.x * inv, f1.y * inv);
      o.y = cvt_e4m3x4<FMT>(f2.x * inv, f2.y * inv, f3.x * inv, f3.y * inv);
      *reinterpret_cast<uint2*>(out + row * ldo + v * 8) = o;
    }
  }
}

// Rows longer than the register budget of quant_rows_kernel: two passes over the row (the second one
// hits L2).
template <int FMT>
__global__ void __launch_bounds__(Q_THREADS)
quant_rows_long_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, int K, uint8_t* __restrict__ out,
                       long long ldo, float* __restrict__ scale) {
  const long long row = blockIdx.x;
  const int nvec = K / 8;
  float amax = 0.f;
  for (int v = threadIdx.x; v < nvec; v += Q_THREADS) {
    const uint4 q = *reinterpret_cast<const uint4*>(x + row * ldx + v * 8);
    const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __bfloat1622float2(b[j]);
      amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
    }
  }
  __shared__ float red[Q_THREADS / 32];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = 0.f;
#pragma unroll
  for (int i = 0; i < Q_THREADS / 32; ++i) amax = fmaxf(amax, red[i]);
  const float sc = fmaxf(amax, AMAX_EPS) / (FMT ? E5M2_MAX : E4M3_MAX);
  const float inv = 1.f / sc;
  if (threadIdx.x == 0) scale[row] = sc;
  for (int v = threadIdx.x; v < nvec; v += Q_THREADS) {
    const uint4 q = *reinterpret_cast<const uint4*>(x + row * ldx + v * 8);
    const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&q);
    const float2 f0 = __bfloat1622float2(b[0]), f1 = __bfloat1622float2(b[1]);
    const float2 f2 = __bfloat1622float2(b[2]), f3 = __bfloat1622float2(b[3]);
    uint2 o;
    o.x = cvt_e4m3x4<FMT>(f0.x * inv, f0.y * inv, f1.x * inv, f1.y * inv);
    o.y = cvt_e4m3x4<FMT>(f2.x * inv, f2.y * inv, f3.x * inv, f3.y * inv);
    *reinterpret_cast<uint2*>(out + row * ldo + v * 8) = o;
  }
}

// out[k, n] = e4m3(w[n, k] / *scale). 64 x 64 tiles through shared memory.
__global__ void __launch_bounds__(256)
quant_transpose_kernel(const __nv_bfloat16* __restrict__ w, int N, int K, const float* __restrict__ scale,
                       uint8_t* __restrict__ out, long long ldo) {
  __shared__ float tile[64][65];
  const float inv = 1.f / fmaxf(*scale, AMAX_EPS / E4M3_MAX);
  const int n0 = blockIdx.y * 64, k0 = blockIdx.x * 64;
  for (int i = threadIdx.x; i < 64 * 64; i += 256) {
    const int r = i >> 6, c = i & 63;
    const int n = n0 + r, k = k0 + c;
    tile[r][c] = (n < N && k < K) ? __bfloat162float(w[(long long)n * K + k]) * inv : 0.f;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < 64 * 16; i += 256) {
    const int kr = i >> 4, nq = (i & 15) * 4;
    const int k = k0 + kr, n = n0 + nq;
    if (k < K && n < N) {  // N % 4 == 0 is checked on the host
      const uint32_t v = cvt_e4m3x4(tile[nq][kr], tile[nq + 1][kr], tile[nq + 2][kr], tile[nq + 3][kr]);
      *reinterpret_cast<uint32_t*>(out + (long long)k * ldo + n) = v;
    }
  }
}

}  // namespace f8
}  // namespace lb

extern "C" int lb_quant_rows(const void* x, long long ldx, long long rows, int K, void* out, long long ldo,
                             float* scale, void* stream) {
  return lb_quant_rows_fmt(x, ldx, rows, K, out, ldo, scale, 0, stream);
}

extern "C" int lb_gemm_fp8(const LbGemmFp8Args* a, void* stream) {
  if (!a || a->M <= 0 || a->N <= 0 || a->K <= 0) return 1;
  if ((a->lda % 16) || (a->ldb % 16) || (a->K % 16)) return 2;  // TMA strides in bytes
  if ((a->ldc % 8) || (a->N % 8)) return 3;
  if (a->a_fmt < 0 || a->a_fmt > 1 || a->b_fmt < 0 || a->b_fmt > 1) return 4;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  // large problems run on SM pairs (256 x 256 tiles, epilogue through TMA stores), like the bf16 products
  const long long tiles2 = (long long)((a->M + 255) / 256) * ((a->N + 255) / 256);
  if (a->M >= 256 && a->N >= 256 && tiles2 >= lb::num_sms() / 2 && !getenv("LB_FP8_ONE_SM"))
    return lb::gemm2_fp8_dispatch(*a, s);
  if (a->out_dtype == LB_BF16) return lb::f8::launch<__nv_bfloat16>(*a, s);
  if (a->out_dtype == LB_F32) return lb::f8::launch<float>(*a, s);
  return 5;
}

extern "C" int lb_quant_rows_fmt(const void* x, long long ldx, long long rows, int K, void* out, long long ldo,
                                 float* scale, int fmt, void* stream) {
  if (!x || !out || !scale || rows <= 0 || fmt < 0 || fmt > 1) return 1;
  if (K % 8 != 0 || ldx % 8 != 0 || ldo % 8 != 0) return 2;
  using namespace lb::f8;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const __nv_bfloat16* xp = reinterpret_cast<const __nv_bfloat16*>(x);
  uint8_t* op = reinterpret_cast<uint8_t*>(out);
  const bool lng = K > 8 * Q_THREADS * Q_MAXV;
  if (fmt == 0) {
    if (lng) quant_rows_long_kernel<0><<<(unsigned)rows, Q_THREADS, 0, st>>>(xp, ldx, K, op, ldo, scale);
    else quant_rows_kernel<0><<<(unsigned)rows, Q_THREADS, 0, st>>>(xp, ldx, K, op, ldo, scale);
  } else {
    if (lng) quant_rows_long_kernel<1><<<(unsigned)rows, Q_THREADS, 0, st>>>(xp, ldx, K, op, ldo, scale);
    else quant_rows_kernel<1><<<(unsigned)rows, Q_THREADS, 0, st>>>(xp, ldx, K, op, ldo, scale);
  }
  lb::g_launches.fetch_add(1, std::memory_order_relaxed);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}

extern "C" int lb_quant_transpose(const void* w, int N, int K, const float* scale, void* out, long long ldo,
                                  void* stream) {
  if (!w || !out || !scale || N <= 0 || K <= 0) return 1;
  if (N % 4 != 0 || ldo % 4 != 0) return 2;
  dim3 grid((K + 63) / 64, (N + 63) / 64);
  lb::f8::quant_transpose_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(w), N, K, scale, reinterpret_cast<uint8_t*>(out), ldo);
  lb::g_launches.fetch_add(1, std::memory_order_relaxed);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}
