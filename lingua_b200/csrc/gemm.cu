// Persistent, warp-specialised tcgen05 GEMM for sm_100a.
//
//   C[b] (+)= alpha * A[b] * B[b]^T        A: M x K, B: N x K, C: M x N (row-major)
//
// Either operand may be stored "K-major" (K contiguous) or "MN-major" (M resp. N
// contiguous), which covers the three GEMMs of a linear layer without transposes:
//   forward  Y  = X  W^T   : A = X  (K-major),  B = W (K-major)
//   dgrad    dX = dY W     : A = dY (K-major),  B = W (MN-major, stored [K_red, N_out])
//   wgrad    dW = dY^T X   : A = dY (MN-major), B = X (MN-major)
// (It replaces the cuBLAS calls behind nn.Linear in lingua/transformer.py:357-359,406,469-471.)
//
// One CTA per SM loops over 128 x BN output tiles. Warp 0 feeds a ring of shared-memory
// stages with TMA; one thread of warp 1 issues tcgen05.mma into one of two TMEM
// accumulators; warps 2-5 drain the other accumulator (tcgen05.ld -> registers -> global),
// so the epilogue of tile i overlaps the main loop of tile i+1.
#include "common.cuh"
#include "lingua_b200.h"

namespace lb {

constexpr int BM = 128;
constexpr int BK_BYTES = 128;  // one swizzle row
constexpr int GEMM_THREADS = 192;

template <int BN, int ESZ>
struct GemmCfg {
  static constexpr int BK = BK_BYTES / ESZ;           // elements along K per stage
  static constexpr int UMMA_K = 32 / ESZ;             // elements along K per MMA
  static constexpr int A_BYTES = BM * BK_BYTES;       // 16 KB
  static constexpr int B_BYTES = BN * BK_BYTES;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (BN == 256) ? 4 : 6;
  static constexpr int SMEM = STAGES * STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/;
  static constexpr int TMEM_COLS = 2 * BN;
};

struct GemmParams {
  int M, N, K;
  int tiles_m, tiles_n, nb0, nb1;
  long long ldc, c_bs0, c_bs1;
  float alpha;
  int accumulate;
  void* C;
  uint32_t* status;
};

template <int BN, int ESZ, int AMAJ, int BMAJ, typename OutT>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
            const GemmParams p) {
  using Cfg = GemmCfg<BN, ESZ>;
  extern __shared__ uint8_t smem_raw[];
  __shared__ int abort_flag;
  __shared__ uint32_t tmem_base_slot;

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar_base = smem_base + Cfg::STAGES * Cfg::STAGE_BYTES;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (Cfg::STAGES + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * Cfg::STAGES + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * Cfg::STAGES + 2 + a); };

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < Cfg::STAGES; ++s) {
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
    tmem_alloc(smem_u32(&tmem_base_slot), Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;

  const int num_kb = (p.K + Cfg::BK - 1) / Cfg::BK;
  const int tiles_per_batch = p.tiles_m * p.tiles_n;
  const int num_tiles = tiles_per_batch * p.nb0 * p.nb1;

  if (warp == 0) {
    if (lane == 0) {
      // ------------------------------------------------ TMA producer
      uint32_t it = 0;
      for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
        const int batch = tile / tiles_per_batch;
        const int t = tile - batch * tiles_per_batch;
        const int m0 = (t % p.tiles_m) * BM;
        const int n0 = (t / p.tiles_m) * BN;
        const int b0 = batch % p.nb0, b1 = batch / p.nb0;
        bool ok = true;
        for (int kb = 0; kb < num_kb && ok; ++kb, ++it) {
          const int s = it % Cfg::STAGES;
          const uint32_t ph = (it / Cfg::STAGES) & 1u;
          ok = mbar_wait(empty_bar(s), ph ^ 1u, &abort_flag, p.status, 1);
          if (!ok) break;
          mbar_arrive_expect_tx(full_bar(s), Cfg::STAGE_BYTES);
          const uint32_t sa = smem_base + s * Cfg::STAGE_BYTES;
          const uint32_t sb = sa + Cfg::A_BYTES;
          const int k0 = kb * Cfg::BK;
          if (AMAJ == 0) {
            tma_load_4d(sa, &tma_a, full_bar(s), k0, m0, b0, b1);
          } else {
            constexpr int CH = BK_BYTES / ESZ;  // M elements per 128-byte row
#pragma unroll
            for (int c = 0; c < BM / CH; ++c)
              tma_load_4d(sa + c * (Cfg::BK * BK_BYTES), &tma_a, full_bar(s), m0 + c * CH, k0, b0, b1);
          }
          if (BMAJ == 0) {
            tma_load_4d(sb, &tma_b, full_bar(s), k0, n0, b0, b1);
          } else {
            constexpr int CH = BK_BYTES / ESZ;
#pragma unroll
            for (int c = 0; c < BN / CH; ++c)
              tma_load_4d(sb + c * (Cfg::BK * BK_BYTES), &tma_b, full_bar(s), n0 + c * CH, k0, b0, b1);
          }
        }
        if (!ok) break;
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ------------------------------------------------ MMA issuer
      constexpr uint32_t FMT = (ESZ == 2) ? 1u : 0u;  // bf16 | e4m3
      constexpr uint32_t idesc = make_idesc(BM, BN, FMT, FMT, AMAJ, BMAJ);
      // Descriptor strides. K-major: 8-row groups are 1024 B apart. MN-major: 8-k groups are
      // 1024 B apart and 64-element (128 B) column chunks are BK rows * 128 B apart.
      constexpr uint32_t SBO = 1024;
      constexpr uint32_t LBO_MN = Cfg::BK * BK_BYTES;
      constexpr uint32_t A_KSTEP = (AMAJ == 0) ? 32u : Cfg::UMMA_K * BK_BYTES;
      constexpr uint32_t B_KSTEP = (BMAJ == 0) ? 32u : Cfg::UMMA_K * BK_BYTES;
      uint32_t it = 0, tile_iter = 0;
      for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++tile_iter) {
        const int acc = tile_iter & 1;
        const uint32_t acc_ph = (tile_iter >> 1) & 1u;
        if (!mbar_wait(tempty_bar(acc), acc_ph ^ 1u, &abort_flag, p.status, 2)) break;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * BN;
        bool ok = true;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % Cfg::STAGES;
          const uint32_t ph = (it / Cfg::STAGES) & 1u;
          ok = mbar_wait(full_bar(s), ph, &abort_flag, p.status, 3);
          if (!ok) break;
          tc_fence_after();
          const uint32_t sa = smem_base + s * Cfg::STAGE_BYTES;
          const uint32_t sb = sa + Cfg::A_BYTES;
#pragma unroll
          for (int k = 0; k < Cfg::BK / Cfg::UMMA_K; ++k) {
            const uint64_t ad = make_smem_desc(sa + k * A_KSTEP, AMAJ ? LBO_MN : 16u, SBO);
            const uint64_t bd = make_smem_desc(sb + k * B_KSTEP, BMAJ ? LBO_MN : 16u, SBO);
            if (ESZ == 2)
              umma_f16(tmem_d, ad, bd, idesc, (kb | k) != 0);
            else
              umma_f8(tmem_d, ad, bd, idesc, (kb | k) != 0);
          }
          umma_commit(empty_bar(s));
        }
        if (!ok) break;
        umma_commit(tfull_bar(acc));
      }
    }
  } else {
    // -------------------------------------------------- epilogue (warps 2..5)
    const int quarter = warp & 3;  // TMEM lanes this warp may touch
    uint32_t tile_iter = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++tile_iter) {
      const int acc = tile_iter & 1;
      const uint32_t acc_ph = (tile_iter >> 1) & 1u;
      const int batch = tile / tiles_per_batch;
      const int t = tile - batch * tiles_per_batch;
      const int m0 = (t % p.tiles_m) * BM;
      const int n0 = (t / p.tiles_m) * BN;
      const int b0 = batch % p.nb0, b1 = batch / p.nb0;
      if (!mbar_wait(tfull_bar(acc), acc_ph, &abort_flag, p.status, 4)) break;
      tc_fence_after();
      const int row = m0 + quarter * 32 + lane;
      OutT* crow = reinterpret_cast<OutT*>(p.C) + b0 * p.c_bs0 + b1 * p.c_bs1 +
                   static_cast<long long>(row) * p.ldc;
      const uint32_t taddr = tmem_base + acc * BN + (static_cast<uint32_t>(quarter * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        const int col0 = n0 + c * 32;
        if (col0 >= p.N) break;  // warp-uniform
        uint32_t r[32];
        tmem_ld32(taddr + c * 32, r);
        tmem_wait_ld();
        if (row < p.M) {
          if (sizeof(OutT) == 2) {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              if (col0 + g * 8 < p.N) {
                uint4 v;
                v.x = pack_bf16(__uint_as_float(r[g * 8 + 0]) * p.alpha, __uint_as_float(r[g * 8 + 1]) * p.alpha);
                v.y = pack_bf16(__uint_as_float(r[g * 8 + 2]) * p.alpha, __uint_as_float(r[g * 8 + 3]) * p.alpha);
                v.z = pack_bf16(__uint_as_float(r[g * 8 + 4]) * p.alpha, __uint_as_float(r[g * 8 + 5]) * p.alpha);
                v.w = pack_bf16(__uint_as_float(r[g * 8 + 6]) * p.alpha, __uint_as_float(r[g * 8 + 7]) * p.alpha);
                *reinterpret_cast<uint4*>(crow + col0 + g * 8) = v;
              }
            }
          } else {
#pragma unroll
            for (int g = 0; g < 8; ++g) {
              if (col0 + g * 4 < p.N) {
                float4* dst = reinterpret_cast<float4*>(crow + col0 + g * 4);
                float4 v;
                v.x = __uint_as_float(r[g * 4 + 0]) * p.alpha;
                v.y = __uint_as_float(r[g * 4 + 1]) * p.alpha;
                v.z = __uint_as_float(r[g * 4 + 2]) * p.alpha;
                v.w = __uint_as_float(r[g * 4 + 3]) * p.alpha;
                if (p.accumulate) {
                  const float4 o = *dst;
                  v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
                }
                *dst = v;
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
    // Give copies that were already issued time to land before the CTA's memory goes away.
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
      return nullptr;
    fn = reinterpret_cast<EncodeTiledFn>(sym);
  }
  return fn;
}

// Build a 4-D map {inner, outer, batch0, batch1}; strides in elements; box {box_inner, box_outer, 1, 1}.
int make_tmap_4d(CUtensorMap* out, const void* base, int esz, long long inner, long long outer,
                 long long ld, int nb0, long long bs0, int nb1, long long bs1, int box_inner,
                 int box_outer) {
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return -1;
  cuuint64_t dims[4] = {(cuuint64_t)inner, (cuuint64_t)outer, (cuuint64_t)nb0, (cuuint64_t)nb1};
  // A batch dimension of extent 1 may carry any (valid, 16-byte multiple) stride.
  long long s1 = ld * esz;
  long long s2 = (nb0 > 1 ? bs0 : ld * outer) * esz;
  long long s3 = (nb1 > 1 ? bs1 : (nb0 > 1 ? bs0 * nb0 : ld * outer)) * esz;
  if (s2 <= 0) s2 = s1;
  if (s3 <= 0) s3 = s2;
  cuuint64_t strides[3] = {(cuuint64_t)s1, (cuuint64_t)s2, (cuuint64_t)s3};
  cuuint32_t box[4] = {(cuuint32_t)box_inner, (cuuint32_t)box_outer, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUtensorMapDataType dt = esz == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                           : esz == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                      : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  CUresult r = enc(out, dt, 4, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}

static int g_num_sms = 0;
int num_sms() {
  if (!g_num_sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  return g_num_sms;
}

std::atomic<long long> g_launches{0};

template <int BN, int ESZ, int AMAJ, int BMAJ, typename OutT>
static int launch_gemm(const LbGemmArgs& a, cudaStream_t stream) {
  using Cfg = GemmCfg<BN, ESZ>;
  constexpr int CH = BK_BYTES / ESZ;
  CUtensorMap ta, tb;
  int rc;
  if (AMAJ == 0)
    rc = make_tmap_4d(&ta, a.A, ESZ, a.K, a.M, a.lda, a.nb0, a.a_bs0, a.nb1, a.a_bs1, Cfg::BK, BM);
  else
    rc = make_tmap_4d(&ta, a.A, ESZ, a.M, a.K, a.lda, a.nb0, a.a_bs0, a.nb1, a.a_bs1, CH, Cfg::BK);
  if (rc) return 100 + rc;
  if (BMAJ == 0)
    rc = make_tmap_4d(&tb, a.B, ESZ, a.K, a.N, a.ldb, a.nb0, a.b_bs0, a.nb1, a.b_bs1, Cfg::BK, BN);
  else
    rc = make_tmap_4d(&tb, a.B, ESZ, a.N, a.K, a.ldb, a.nb0, a.b_bs0, a.nb1, a.b_bs1, CH, Cfg::BK);
  if (rc) return 200 + rc;

  GemmParams p;
  p.M = a.M; p.N = a.N; p.K = a.K;
  p.tiles_m = (a.M + BM - 1) / BM;
  p.tiles_n = (a.N + BN - 1) / BN;
  p.nb0 = a.nb0; p.nb1 = a.nb1;
  p.ldc = a.ldc; p.c_bs0 = a.c_bs0; p.c_bs1 = a.c_bs1;
  p.alpha = a.alpha; p.accumulate = a.accumulate;
  p.C = a.C; p.status = a.status;
  const long long tiles = (long long)p.tiles_m * p.tiles_n * a.nb0 * a.nb1;
  const int grid = (int)(tiles < num_sms() ? tiles : num_sms());
  auto kern = gemm_kernel<BN, ESZ, AMAJ, BMAJ, OutT>;
  if (ensure_dyn_smem<gemm_kernel<BN, ESZ, AMAJ, BMAJ, OutT>>(Cfg::SMEM)) return 300;
  kern<<<grid, GEMM_THREADS, Cfg::SMEM, stream>>>(ta, tb, p);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}

template <int BN, int ESZ, typename OutT>
static int dispatch_major(const LbGemmArgs& a, cudaStream_t s) {
  if (a.a_major == 0 && a.b_major == 0) return launch_gemm<BN, ESZ, 0, 0, OutT>(a, s);
  if (a.a_major == 0 && a.b_major == 1) return launch_gemm<BN, ESZ, 0, 1, OutT>(a, s);
  if (a.a_major == 1 && a.b_major == 0) return launch_gemm<BN, ESZ, 1, 0, OutT>(a, s);
  return launch_gemm<BN, ESZ, 1, 1, OutT>(a, s);
}

}  // namespace lb

extern "C" int lb_gemm(const LbGemmArgs* args, void* stream) {
  using namespace lb;
  const LbGemmArgs& a = *args;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (a.M <= 0 || a.N <= 0 || a.K <= 0 || a.nb0 <= 0 || a.nb1 <= 0) return 1;
  if (a.in_dtype != LB_BF16) return 2;  // fp8 operands go through lb_gemm_fp8
  // rows of C are written in 8-element vectors: a ragged N needs ldc >= N rounded up to 8
  if ((a.ldc % 8) || (a.lda % 8) || (a.ldb % 8) || a.ldc < ((a.N + 7) / 8) * 8) return 3;
  if (a.out_dtype == LB_BF16 && a.accumulate) return 4;
  // Large problems run on SM pairs (256 x 256 tiles); force_bn = 512 selects that explicitly,
  // 128 / 256 select the single-SM kernels.
  const long long tiles2 = (long long)((a.M + 255) / 256) * ((a.N + 255) / 256) * a.nb0 * a.nb1;
  if (a.force_bn == 512 || (a.force_bn == 0 && a.M >= 256 && a.N >= 256 && tiles2 >= num_sms() / 2))
    return gemm2_dispatch(a, s);
  // Narrow outputs use the 128-wide tile so that small N does not waste half of every MMA.
  // So do few-row problems (decode steps): they stream the weight once, and twice as many tiles keep
  // twice as many SMs pulling on memory.
  const long long tiles256 = (long long)((a.M + 127) / 128) * ((a.N + 255) / 256) * a.nb0 * a.nb1;
  const bool narrow = a.N <= 128 || a.force_bn == 128 || (a.force_bn == 0 && a.M <= 128 && tiles256 < num_sms());
  if (a.out_dtype == LB_BF16)
    return narrow ? dispatch_major<128, 2, __nv_bfloat16>(a, s) : dispatch_major<256, 2, __nv_bfloat16>(a, s);
  if (a.out_dtype == LB_F32)
    return narrow ? dispatch_major<128, 2, float>(a, s) : dispatch_major<256, 2, float>(a, s);
  return 5;
}

extern "C" long long lb_launch_count() { return lb::g_launches.load(); }
extern "C" void lb_launch_count_add(long long n) { lb::g_launches.fetch_add(n); }
