// Tensor-parallel GEMMs with the collective fused in (sm_100a, bf16, NVLink peer memory).
//
// A tensor-parallel transformer block with sequence-sharded activations needs two patterns
// (the reference gets both from torch DTensor + NCCL: lingua/transformer.py:560-640 applies
// ColwiseParallel / RowwiseParallel / SequenceParallel, each a separate all-gather or
// reduce-scatter kernel around the cuBLAS GEMM):
//
//   mode 1  all-gather -> GEMM     Y[M, N] = gather_r(A_r)[M, K] * W[N, K]^T
//           every rank holds a slab A_r of M / world rows in peer-visible memory. Tiles of the
//           local slab run first; meanwhile one extra warp per CTA pulls the remote slabs into a
//           local gather buffer in 16 KB pieces (bulk copies peer -> shared -> local, pieces
//           claimed from an atomic counter) and bumps a per-row-tile counter; the TMA producer
//           of a tile that needs remote rows waits on that counter. Each remote byte crosses
//           NVLink exactly once and the transfer hides behind the local slab's math.
//
//   mode 2  GEMM -> scatter        P[M, N] = A[M, K_local] * W[N, K_local]^T  (a partial sum)
//           rows [o * M/world, (o+1) * M/world) belong to rank o. The epilogue packs each
//           128 x 64 piece of the accumulator into shared memory and TMA-stores it straight
//           into slot `rank` of owner o's staging buffer over NVLink, remote owners first, so the
//           reduce-scatter's traffic overlaps the main loop. The sum over slots is taken by the
//           residual + RMSNorm kernel that has to read the data anyway (lb_reduce_norm).
//
// Neither mode contains a wait on another GPU: cross-rank ordering is the caller's job
// (lb_peer_barrier before / after). The only waits are on this kernel's own copies and are
// bounded (status word, see common.cuh). No load uses cluster multicast.
#include "common.cuh"
#include "lingua_b200.h"

namespace lb {
namespace tp {

constexpr int BM = 128, BN = 256, BK = 64, UMMA_K = 16, STAGES = 4;
constexpr int ROW_BYTES = 128;
constexpr int A_BYTES = BM * ROW_BYTES, B_BYTES = BN * ROW_BYTES, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int PIECE = 16384;         // bytes per all-gather copy
constexpr int AUX_BYTES = 2 * PIECE; // mode 1: two copy buffers; mode 2: two store staging tiles
constexpr int SMEM = STAGES * STAGE_BYTES + AUX_BYTES + 1024 + 256;
constexpr int THREADS = 224;  // TMA warp, MMA warp, 4 epilogue warps, copy warp

struct TmapSet {
  CUtensorMap m[LB_MAX_PEERS];
};

struct Params {
  int M, N, K;
  int tiles_n, tiles_per_slab, world, rank;
  long long ldc;
  float alpha;
  void* C;                             // mode 1 output
  const uint8_t* peer_a[LB_MAX_PEERS]; // mode 1: every rank's slab
  uint8_t* gather;                     // mode 1: [world][rows_per_slab][K] local copy of remote slabs
  uint32_t* flags;                     // mode 1: [world * tiles_per_slab] arrival counts, then the piece counter
  uint32_t* status;
};

__device__ __forceinline__ void epi_bar_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// Tile order: slabs (rows of one rank) in rotation starting at `first`, then column tiles, then
// the row tiles of the slab (fastest), so CTAs of a wave share the B tile through L2.
struct Tile { int slab, ml, nt; };
__device__ __forceinline__ Tile tile_of(int tile, const Params& p, int first) {
  const int per_slab = p.tiles_per_slab * p.tiles_n;
  const int si = tile / per_slab;
  const int rem = tile - si * per_slab;
  Tile t;
  t.slab = (first + si) % p.world;
  t.nt = rem / p.tiles_per_slab;
  t.ml = rem - t.nt * p.tiles_per_slab;
  return t;
}

template <int MODE, int BMAJ = 0>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tp_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_gather,
               const __grid_constant__ CUtensorMap tma_b, const __grid_constant__ TmapSet owners,
               const Params p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ int abort_flag;
  __shared__ uint32_t tmem_base_slot;

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t aux_base = smem_base + STAGES * STAGE_BYTES;
  const uint32_t bar_base = aux_base + AUX_BYTES;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };
  auto copy_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + 4 + b); };

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 4);
      mbar_init(copy_bar(a), 1);
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
  const int num_tiles = p.world * p.tiles_per_slab * p.tiles_n;
  // mode 1 starts with the rows it already has; mode 2 starts with the rows that have to travel
  const int first = (MODE == 1) ? p.rank : (p.rank + 1) % p.world;

  if (warp == 0) {
    if (lane == 0) {
      // ------------------------------------------------ TMA producer
      const uint32_t pieces_per_tile = static_cast<uint32_t>((long long)BM * p.K * 2 / PIECE);
      uint32_t it = 0;
      for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
        const Tile t = tile_of(tile, p, first);
        const int n0 = t.nt * BN;
        const CUtensorMap* amap = &tma_a;
        int m0 = (t.slab * p.tiles_per_slab + t.ml) * BM;
        bool ok = true;
        if (MODE == 1) {
          if (t.slab == p.rank) {
            m0 = t.ml * BM;  // own slab is read in place
          } else {
            amap = &tma_gather;
            ok = flag_wait_ge(p.flags + t.slab * p.tiles_per_slab + t.ml, pieces_per_tile, &abort_flag,
                              p.status, 5);
            fence_proxy_async_all();  // the rows were written by bulk copies of other CTAs
          }
        }
        for (int kb = 0; kb < num_kb && ok; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1u;
          ok = mbar_wait(empty_bar(s), ph ^ 1u, &abort_flag, p.status, 1);
          if (!ok) break;
          mbar_arrive_expect_tx(full_bar(s), STAGE_BYTES);
          const uint32_t sa = smem_base + s * STAGE_BYTES;
          tma_load_4d(sa, amap, full_bar(s), kb * BK, m0, 0, 0);
          if (BMAJ == 0) {
            tma_load_4d(sa + A_BYTES, &tma_b, full_bar(s), kb * BK, n0, 0, 0);
          } else {
            // B stored [K, N] (N contiguous): BK rows of 64-element chunks, one chunk column per load
#pragma unroll
            for (int c = 0; c < BN / 64; ++c)
              tma_load_4d(sa + A_BYTES + c * (BK * ROW_BYTES), &tma_b, full_bar(s), n0 + c * 64, kb * BK, 0, 0);
          }
        }
        if (!ok) break;
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ------------------------------------------------ MMA issuer
      constexpr uint32_t idesc = make_idesc(BM, BN, 1u, 1u, 0, BMAJ);
      uint32_t it = 0, tile_iter = 0;
      for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++tile_iter) {
        const int acc = tile_iter & 1;
        const uint32_t acc_ph = (tile_iter >> 1) & 1u;
        if (!mbar_wait(tempty_bar(acc), acc_ph ^ 1u, &abort_flag, p.status, 2)) break;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * BN;
        bool ok = true;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1u;
          ok = mbar_wait(full_bar(s), ph, &abort_flag, p.status, 3);
          if (!ok) break;
          tc_fence_after();
          const uint32_t sa = smem_base + s * STAGE_BYTES;
          const uint32_t sb = sa + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t ad = make_smem_desc(sa + k * 32u, 16u, 1024u);
            const uint64_t bd = BMAJ == 0 ? make_smem_desc(sb + k * 32u, 16u, 1024u)
                                          : make_smem_desc(sb + k * (16u * ROW_BYTES), BK * ROW_BYTES, 1024u);
            umma_f16(tmem_d, ad, bd, idesc, (kb | k) != 0);
          }
          umma_commit(empty_bar(s));
        }
        if (!ok) break;
        umma_commit(tfull_bar(acc));
      }
    }
  } else if (warp < 6) {
    // -------------------------------------------------- epilogue (warps 2..5)
    const int quarter = warp & 3;  // TMEM lanes this warp may touch
    const int trow = quarter * 32 + lane;
    const bool issuer = (warp == 2 && lane == 0);
    uint32_t tile_iter = 0, chunk_iter = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++tile_iter) {
      const int acc = tile_iter & 1;
      const uint32_t acc_ph = (tile_iter >> 1) & 1u;
      const Tile t = tile_of(tile, p, first);
      const int n0 = t.nt * BN;
      if (!mbar_wait(tfull_bar(acc), acc_ph, &abort_flag, p.status, 4)) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + acc * BN + (static_cast<uint32_t>(quarter * 32) << 16);
      if (MODE == 1) {
        const int row = (t.slab * p.tiles_per_slab + t.ml) * BM + trow;
        __nv_bfloat16* crow = reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<long long>(row) * p.ldc;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          const int col0 = n0 + c * 32;
          if (col0 >= p.N) break;  // warp-uniform
          uint32_t r[32];
          tmem_ld32(taddr + c * 32, r);
          tmem_wait_ld();
          if (row < p.M) {
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
          }
        }
      } else {
        // 128 x 64 pieces: TMEM -> registers -> 128B-swizzled shared tile -> TMA store into
        // slot `rank` of the owner's staging buffer (peer memory unless the owner is this rank).
#pragma unroll 1
        for (int c = 0; c < BN / 64; ++c) {
          const int col0 = n0 + c * 64;
          if (col0 >= p.N) break;  // uniform over the four warps
          const uint32_t buf = aux_base + (chunk_iter & 1u) * PIECE;
          if (issuer) tma_store_wait_read<1>();  // the store that last used this buffer has read it
          epi_bar_sync();
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            uint32_t r[32];
            tmem_ld32(taddr + c * 64 + h * 32, r);
            tmem_wait_ld();
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              const uint32_t unit = static_cast<uint32_t>(h * 4 + g) ^ static_cast<uint32_t>(trow & 7);
              const uint32_t dst = buf + trow * ROW_BYTES + unit * 16u;
              const uint32_t v0 = pack_bf16(__uint_as_float(r[g * 8 + 0]) * p.alpha, __uint_as_float(r[g * 8 + 1]) * p.alpha);
              const uint32_t v1 = pack_bf16(__uint_as_float(r[g * 8 + 2]) * p.alpha, __uint_as_float(r[g * 8 + 3]) * p.alpha);
              const uint32_t v2 = pack_bf16(__uint_as_float(r[g * 8 + 4]) * p.alpha, __uint_as_float(r[g * 8 + 5]) * p.alpha);
              const uint32_t v3 = pack_bf16(__uint_as_float(r[g * 8 + 6]) * p.alpha, __uint_as_float(r[g * 8 + 7]) * p.alpha);
              asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(v0), "r"(v1), "r"(v2), "r"(v3)
                           : "memory");
            }
          }
          fence_proxy_async_smem();
          epi_bar_sync();
          if (issuer) {
            tma_store_4d(&owners.m[t.slab], buf, col0, t.ml * BM, p.rank, 0);
            tma_store_commit();
          }
          ++chunk_iter;
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar(acc));
    }
    if (MODE == 2 && issuer) tma_store_wait<0>();
  } else if (MODE == 1 && lane == 0 && p.world > 1) {
    // -------------------------------------------------- all-gather copier (warp 6)
    const long long slab_bytes = (long long)p.tiles_per_slab * BM * p.K * 2;
    const long long tile_bytes = (long long)BM * p.K * 2;
    const uint32_t pieces_per_slab = static_cast<uint32_t>(slab_bytes / PIECE);
    const uint32_t total = pieces_per_slab * (p.world - 1);
    uint32_t* counter = p.flags + p.world * p.tiles_per_slab;
    auto claim = [&]() -> long long {
      const uint32_t i = atomicAdd(counter, 1u);
      return i < total ? (long long)i : -1ll;
    };
    auto locate = [&](long long piece, int& slab, long long& off) {
      const int si = 1 + static_cast<int>(piece / pieces_per_slab);
      slab = (p.rank + si) % p.world;
      off = (piece % pieces_per_slab) * PIECE;
    };
    uint32_t i = 0;
    long long cur = claim();
    if (cur >= 0) {
      int slab; long long off;
      locate(cur, slab, off);
      mbar_arrive_expect_tx(copy_bar(0), PIECE);
      bulk_load(aux_base, p.peer_a[slab] + off, PIECE, copy_bar(0));
    }
    uint32_t* pending = nullptr;  // counter of the piece whose store is in flight
    while (cur >= 0) {
      if (pending) {
        tma_store_wait<0>();  // landed in local memory (and its buffer is free again)
        fence_proxy_async_all();
        red_release_gpu_add(pending, 1u);
        pending = nullptr;
      }
      const long long nxt = claim();
      if (nxt >= 0) {
        int slab; long long off;
        locate(nxt, slab, off);
        const uint32_t b = (i + 1) & 1u;
        mbar_arrive_expect_tx(copy_bar(b), PIECE);
        bulk_load(aux_base + b * PIECE, p.peer_a[slab] + off, PIECE, copy_bar(b));
      }
      if (!mbar_wait(copy_bar(i & 1u), (i >> 1) & 1u, &abort_flag, p.status, 6)) break;
      int slab; long long off;
      locate(cur, slab, off);
      bulk_store(p.gather + slab * slab_bytes + off, aux_base + (i & 1u) * PIECE, PIECE);
      tma_store_commit();
      pending = p.flags + slab * p.tiles_per_slab + static_cast<int>(off / tile_bytes);
      cur = nxt;
      ++i;
    }
    tma_store_wait<0>();
    if (pending) {
      fence_proxy_async_all();
      red_release_gpu_add(pending, 1u);
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
    tmem_dealloc(tmem_base, 2 * BN);
  }
}

template <int MODE, int BMAJ = 0>
static int launch(const LbTpGemmArgs& a, cudaStream_t stream) {
  const int W = a.world;
  const int rows = a.M / W;
  CUtensorMap ta, tg, tb;
  TmapSet owners;
  int rc;
  if (MODE == 1) {
    rc = make_tmap_4d(&ta, a.a_peers[a.rank], 2, a.K, rows, a.K, 1, 0, 1, 0, BK, BM);
    if (rc) return 100 + rc;
    rc = make_tmap_4d(&tg, W > 1 ? a.gather : a.a_peers[a.rank], 2, a.K, (long long)rows * (W > 1 ? W : 1), a.K, 1, 0,
                      1, 0, BK, BM);
    if (rc) return 110 + rc;
    for (int r = 0; r < LB_MAX_PEERS; ++r) owners.m[r] = ta;
  } else {
    rc = make_tmap_4d(&ta, a.A, 2, a.K, a.M, a.lda, 1, 0, 1, 0, BK, BM);
    if (rc) return 100 + rc;
    tg = ta;
    for (int r = 0; r < LB_MAX_PEERS; ++r) {
      const int o = r < W ? r : 0;
      rc = make_tmap_4d(&owners.m[r], a.c_peers[o], 2, a.N, rows, a.ldc, W, a.slot_stride, 1, 0, 64, BM);
      if (rc) return 120 + rc;
    }
  }
  if (BMAJ == 0)
    rc = make_tmap_4d(&tb, a.B, 2, a.K, a.N, a.ldb, 1, 0, 1, 0, BK, BN);
  else
    rc = make_tmap_4d(&tb, a.B, 2, a.N, a.K, a.ldb, 1, 0, 1, 0, 64, BK);
  if (rc) return 200 + rc;

  Params p;
  p.M = a.M; p.N = a.N; p.K = a.K;
  p.tiles_n = (a.N + BN - 1) / BN;
  p.tiles_per_slab = rows / BM;
  p.world = W; p.rank = a.rank;
  p.ldc = a.ldc; p.alpha = a.alpha;
  p.C = a.C;
  for (int r = 0; r < LB_MAX_PEERS; ++r)
    p.peer_a[r] = reinterpret_cast<const uint8_t*>(MODE == 1 ? a.a_peers[r < W ? r : 0] : nullptr);
  p.gather = reinterpret_cast<uint8_t*>(a.gather);
  p.flags = a.flags;
  p.status = a.status;
  if (MODE == 1 && W > 1) {
    cudaError_t e = cudaMemsetAsync(a.flags, 0, sizeof(uint32_t) * (W * p.tiles_per_slab + 1), stream);
    if (e != cudaSuccess) return 500 + (int)e;
  }
  const long long tiles = (long long)W * p.tiles_per_slab * p.tiles_n;
  const int grid = (int)(tiles < num_sms() ? tiles : num_sms());
  auto kern = gemm_tp_kernel<MODE, BMAJ>;
  if (ensure_dyn_smem<gemm_tp_kernel<MODE, BMAJ>>(SMEM)) return 300;
  kern<<<grid, THREADS, SMEM, stream>>>(ta, tg, tb, owners, p);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}

}  // namespace tp
}  // namespace lb

extern "C" int lb_gemm_tp(const LbTpGemmArgs* a, void* stream) {
  if (!a || (a->mode != 1 && a->mode != 2)) return 1;
  if (a->world < 1 || a->world > LB_MAX_PEERS || a->rank < 0 || a->rank >= a->world) return 2;
  if (a->M <= 0 || a->N <= 0 || a->K <= 0) return 3;
  if (a->M % (a->world * lb::tp::BM) != 0) return 4;  // a row tile never straddles two ranks
  if (a->K % 64 != 0 || a->N % 8 != 0 || a->ldc % 8 != 0 || a->ldb % 8 != 0) return 5;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (a->mode == 1) {
    if (!a->C || (a->world > 1 && (!a->gather || !a->flags))) return 6;
    return a->b_major ? lb::tp::launch<1, 1>(*a, s) : lb::tp::launch<1, 0>(*a, s);
  }
  if (!a->A || a->lda % 8 != 0 || a->slot_stride % 8 != 0) return 7;
  return a->b_major ? lb::tp::launch<2, 1>(*a, s) : lb::tp::launch<2, 0>(*a, s);
}
