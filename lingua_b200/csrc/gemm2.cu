// Two-SM variant of the tcgen05 GEMM: a cluster of two CTAs (one per SM) computes one 256 x 256
// output tile with tcgen05.mma.cta_group::2. Each CTA TMA-loads its own 128 rows of A and its
// own 128-row half of B (no multicast: every byte of shared memory is written by the CTA that
// owns it), the leader CTA's MMA thread issues the paired MMA that reads both halves of B, and
// each CTA drains the 128 x 256 accumulator held in its own TMEM. Halving the B traffic per
// SM shrinks a stage to 32 KB, which buys a 6-deep TMA ring instead of 4.
//
// Same contract as gemm_kernel in gemm.cu (operand majors, alpha, fp32 accumulate, batching).
//
// Epilogue: the four epilogue warps of a CTA move the accumulator TMEM -> registers -> a
// 128-byte-swizzled shared-memory piece of 128 rows x 128 bytes, and one thread hands the piece
// to the TMA unit (cp.async.bulk.tensor store, or cp.reduce...add when accumulating into an fp32
// output, which needs no read of C by the SM). Every row of a piece is one full 128-byte line.
//
// Scatter mode (fp32 output, lb_gemm_scatter): the rows of the output are owned by the ranks of a
// data-parallel group in blocks of 128 rows. A table gives (owner, destination row) per block;
// the TMA store of a piece goes straight into the owner's buffer -- over NVLink when the owner is
// a peer -- so the reduce-scatter of a weight gradient (lingua/distributed.py:434-463 leaves it to
// FSDP2's post-backward NCCL reduce-scatter) travels tile by tile underneath the main loop of the
// following tiles. The kernel waits on no other GPU; cross-rank ordering is the caller's job.
//
// Tiles are walked in groups of `group_m` row tiles (all column tiles of a group before the next
// group), so the tiles in flight at any time share few distinct A and B panels in L2.
#include "common.cuh"
#include "lingua_b200.h"

namespace lb {

constexpr int G2_THREADS = 192;
constexpr int G2_THREADS_GATHER = 224;    // + the warp that pulls remote weight rows (gather mode)
constexpr int G2_BM = 256, G2_BN = 256;   // per cluster
constexpr int G2_ROWS = 128;              // A rows and B rows loaded by one CTA
constexpr int G2_BK = 64;                 // bf16 elements per stage (128 bytes)
constexpr int G2_A_BYTES = G2_ROWS * 128;
constexpr int G2_STAGE_BYTES = 2 * G2_A_BYTES;
constexpr int G2_STAGES = 6;
constexpr int G2_STAGES_GATHER = 5;       // gather mode trades one stage for the two copy buffers
constexpr int G2_PIECE = G2_ROWS * 128;   // one epilogue piece: 128 rows x 128 bytes
constexpr int G2_COPY = 16384;            // bytes per pulled piece of a remote weight block
constexpr int G2_SMEM = G2_STAGES * G2_STAGE_BYTES + 2 * G2_PIECE + 1024 + 256;
static_assert(G2_STAGES_GATHER * G2_STAGE_BYTES + 2 * G2_COPY <= G2_STAGES * G2_STAGE_BYTES, "gather buffers fit");

struct OwnerMaps {
  CUtensorMap m[LB_MAX_PEERS];
};

struct Gemm2Params {
  int M, N, K;
  int tiles_m, tiles_n, nb0, nb1;
  long long ldc, c_bs0, c_bs1;
  float alpha;
  int accumulate;
  int epi_tma;        // epilogue through shared memory + TMA (C meets the TMA alignment rules)
  int scatter;        // rows go to their owners' buffers (fp32 only)
  int group_m;        // row tiles per rasterisation group
  int m_rot;          // the walk over row tiles starts at this tile (scatter: rows that have to travel first)
  const int2* blocks; // scatter: (owner, destination row) per 128-row block of M
  void* C;
  uint32_t* status;
  // gather mode (lb_gemm_gather): B is a weight matrix whose 128-row blocks are owned by the ranks of a group; the
  // blocks of other ranks are pulled from their copy of the matrix into this one while the product runs
  // float8 operands (lb_gemm_fp8 on SM pairs): result scaled by row_scale[m] * col_scale[n] instead of alpha
  const float* row_scale;
  const float* col_scale;
  uint32_t idesc_f8;                   // instruction descriptor with the two operand formats (e4m3 / e5m2)
  int raster_n;                        // walk column tiles in groups instead of row tiles
  const int* n_order;                  // column tile visited at each position of the walk (own rows first)
  const int2* g_blocks;                // remote blocks in the order they are pulled: (block, owner)
  int g_n_remote;
  uint32_t g_ppb;                      // pieces per block
  const uint8_t* peer_b[LB_MAX_PEERS]; // every rank's copy of B
  uint8_t* local_b;
  uint32_t* flags;                     // [blocks of N] pieces landed, then the piece counter
  int n_blocks;
  // grouped products (lb_gemm_grouped): mode 1 = the B matrix of a row tile is chosen by grp_sel[row tile];
  // mode 2 = batch g contracts over the K range (grp_sel[2g], 64 * grp_sel[2g + 1]) of unbatched A and B
  int grp_mode, grp_n;
  const int* grp_sel;
  // Tail split: when the last wave of the persistent walk would keep at most half of the SM pairs busy, its tiles
  // are issued as two half-width tiles each (256 x 128), which halves the time the other pairs sit idle.
  int tail_first;        // first tile of the split region (= number of tiles when nothing is split)
  int num_work;          // work items of the walk: tail_first + 2 * split tiles
  uint32_t idesc_f8_half;
};

// work item of the persistent walk -> (tile, column offset inside the tile, tile width)
__device__ __forceinline__ void g2_work(int work, const Gemm2Params& p, int& tile, int& n_off, int& bn) {
  if (work < p.tail_first) {
    tile = work;
    n_off = 0;
    bn = G2_BN;
  } else {
    const int i = work - p.tail_first;
    tile = p.tail_first + (i >> 1);
    n_off = (i & 1) * (G2_BN / 2);
    bn = G2_BN / 2;
  }
}

// group of a row tile (mode 1), always checked: -1 marks a tile without rows (nothing is loaded, multiplied or
// stored for it), any other bad entry is reported and replaced by group 0
__device__ __forceinline__ int g2_row_group(const Gemm2Params& p, int mt) {
  const int g = __ldg(p.grp_sel + mt);
  if (g >= -1 && g < p.grp_n) return g;
  if (p.status) atomicOr(p.status, ST_BAD_ARG | 0x43);
  return 0;
}
// (first k, number of 64-wide k blocks) of batch g (mode 2), clamped to the operands' K extent
__device__ __forceinline__ int2 g2_k_range(const Gemm2Params& p, int g) {
  int2 r = make_int2(__ldg(p.grp_sel + 2 * g), __ldg(p.grp_sel + 2 * g + 1));
  if (r.x < 0 || r.y < 0 || (long long)r.x + 64ll * r.y > (long long)((p.K + 63) / 64) * 64) {
    if (p.status) atomicOr(p.status, ST_BAD_ARG | 0x44);
    r = make_int2(0, 0);
  }
  return r;
}

// tile index inside one batch -> (row tile, column tile)
__device__ __forceinline__ void g2_tile_coords(int t, const Gemm2Params& p, int& mt, int& nt) {
  if (p.raster_n) {
    // groups of group_m column tiles, all row tiles of a group before the next group: the weight rows are needed
    // in the order of p.n_order, which leaves the remote ones time to arrive
    const int per_group = p.group_m * p.tiles_m;
    const int grp = t / per_group;
    const int first = grp * p.group_m;
    const int gsz = min(p.group_m, p.tiles_n - first);
    const int r = t - grp * per_group;
    mt = r / gsz;
    nt = first + (r - mt * gsz);
    if (p.n_order) nt = p.n_order[nt];
    return;
  }
  const int per_group = p.group_m * p.tiles_n;
  const int grp = t / per_group;
  const int first = grp * p.group_m;
  const int gsz = min(p.group_m, p.tiles_m - first);
  const int r = t - grp * per_group;
  nt = r / gsz;
  mt = first + (r - nt * gsz) + p.m_rot;
  if (mt >= p.tiles_m) mt -= p.tiles_m;
}
__device__ __forceinline__ void g2_epi_bar_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// address of the same shared-memory location in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t mapa(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA load issued by either CTA of the pair; the transaction bytes are counted on an mbarrier that
// may live in the other CTA (cluster address).
__device__ __forceinline__ void tma_load_4d_pair(uint32_t dst_smem, const CUtensorMap* m, uint32_t bar_cluster,
                                                 int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(dst_smem), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc2(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma2_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma2_f8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t"
      "}\n"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrive on one mbarrier (cluster address, either CTA) when all MMAs issued so far have completed
__device__ __forceinline__ void umma2_commit(uint32_t bar_cluster) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster)
               : "memory");
}

template <int AMAJ, int BMAJ, typename OutT, bool GATHER = false, bool F8 = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GATHER ? G2_THREADS_GATHER : G2_THREADS, 1)
gemm2_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
             const __grid_constant__ CUtensorMap tma_c, const __grid_constant__ OwnerMaps owners,
             const Gemm2Params p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ int abort_flag;
  __shared__ uint32_t tmem_base_slot;

  constexpr int STAGES = GATHER ? G2_STAGES_GATHER : G2_STAGES;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t copy_base = smem_base + STAGES * G2_STAGE_BYTES;  // gather mode only: two copy buffers
  const uint32_t aux_base = smem_base + G2_STAGES * G2_STAGE_BYTES;
  const uint32_t bar_base = aux_base + 2 * G2_PIECE;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (G2_STAGES + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * G2_STAGES + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * G2_STAGES + 2 + a); };
  auto copy_bar = [&](int b) { return bar_base + 8u * (2 * G2_STAGES + 4 + b); };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < G2_STAGES; ++s) {
      mbar_init(full_bar(s), 1);   // the leader's producer arrives; bytes come from both CTAs
      mbar_init(empty_bar(s), 1);  // one commit from the leader's MMA thread
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 8);  // 4 epilogue warps x 2 CTAs (used in the leader only)
      mbar_init(copy_bar(a), 1);
    }
    fence_mbar_init();
    tma_prefetch_desc(&tma_a);
    tma_prefetch_desc(&tma_b);
  }
  if (warp == 1) {
    tmem_alloc2(smem_u32(&tmem_base_slot), 512);
    tmem_relinquish2();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // barriers of both CTAs are initialised before any remote arrive / TMA
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;

  constexpr int BK_ELEMS = F8 ? 128 : G2_BK;  // one 128-byte swizzle row along K per stage
  const int num_kb = (p.K + BK_ELEMS - 1) / BK_ELEMS;
  const int tiles_per_batch = p.tiles_m * p.tiles_n;

  if (warp == 0) {
    if (lane == 0) {
      // ------------------------------------------------ TMA producer (both CTAs)
      uint32_t it = 0;
      bool ok = true;
      for (int work = pair; ok && work < p.num_work; work += n_pairs) {
        int tile, n_off, bn;
        g2_work(work, p, tile, n_off, bn);
        const int batch = tile / tiles_per_batch;
        const int t = tile - batch * tiles_per_batch;
        int mt, nt;
        g2_tile_coords(t, p, mt, nt);
        const int m0 = mt * G2_BM + rank * G2_ROWS;
        // each CTA of the pair supplies half of the tile's B rows; a half-width tile still loads a full box per
        // CTA (the stage layout and byte count stay the same) and the MMA reads only its first bn / 2 rows
        const int n0 = nt * G2_BN + n_off + rank * (bn / 2);
        const int b0 = batch % p.nb0, b1 = batch / p.nb0;
        int ab0 = b0, bb0 = b0, k_first = 0, kb_n = num_kb;
        if (p.grp_mode == 1) {
          bb0 = g2_row_group(p, mt);
          if (bb0 < 0) kb_n = 0;
        } else if (p.grp_mode == 2) {
          const int2 kr = g2_k_range(p, b0);
          ab0 = bb0 = 0;
          k_first = kr.x;
          kb_n = kr.y;
        }
        if (GATHER && p.g_n_remote > 0) {
          // this CTA's half of the B tile is one 128-row block of the weight: if another rank owns it, its pieces
          // must have landed in the local copy (written by bulk copies of any CTA's gather warp)
          const int blk = n0 / G2_ROWS;
          if (blk < p.n_blocks) {
            ok = flag_wait_ge(p.flags + blk, p.g_ppb, &abort_flag, p.status, 0x35);
            if (!ok) break;
            fence_proxy_async_all();
          }
        }
        for (int kb = 0; kb < kb_n; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1u;
          ok = mbar_wait(empty_bar(s), ph ^ 1u, &abort_flag, p.status, 0x31);
          if (!ok) break;
          if (leader) mbar_arrive_expect_tx(full_bar(s), 2 * G2_STAGE_BYTES);
          const uint32_t lead_full = mapa(full_bar(s), 0);
          const uint32_t sa = smem_base + s * G2_STAGE_BYTES;
          const uint32_t sb = sa + G2_A_BYTES;
          const int k0 = k_first + kb * BK_ELEMS;
          if (AMAJ == 0) {
            tma_load_4d_pair(sa, &tma_a, lead_full, k0, m0, ab0, b1);
          } else {
#pragma unroll
            for (int c = 0; c < 2; ++c)
              tma_load_4d_pair(sa + c * (G2_BK * 128), &tma_a, lead_full, m0 + c * 64, k0, ab0, b1);
          }
          if (BMAJ == 0) {
            tma_load_4d_pair(sb, &tma_b, lead_full, k0, n0, bb0, b1);
          } else {
#pragma unroll
            for (int c = 0; c < 2; ++c)
              tma_load_4d_pair(sb + c * (G2_BK * 128), &tma_b, lead_full, n0 + c * 64, k0, bb0, b1);
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && leader) {
      // ------------------------------------------------ MMA issuer (leader CTA only)
      constexpr uint32_t idesc_full = make_idesc(G2_BM, G2_BN, 1, 1, AMAJ, BMAJ);
      constexpr uint32_t idesc_half = make_idesc(G2_BM, G2_BN / 2, 1, 1, AMAJ, BMAJ);
      constexpr uint32_t SBO = 1024, LBO_MN = G2_BK * 128;
      constexpr uint32_t A_KSTEP = (AMAJ == 0) ? 32u : 16u * 128u;
      constexpr uint32_t B_KSTEP = (BMAJ == 0) ? 32u : 16u * 128u;
      uint32_t it = 0, tile_iter = 0;
      bool ok = true;
      for (int work = pair; ok && work < p.num_work; work += n_pairs, ++tile_iter) {
        int tile, n_off, bn;
        g2_work(work, p, tile, n_off, bn);
        const uint32_t idesc = bn == G2_BN ? idesc_full : idesc_half;
        const uint32_t idesc8 = bn == G2_BN ? p.idesc_f8 : p.idesc_f8_half;
        const int acc = tile_iter & 1;
        const uint32_t acc_ph = (tile_iter >> 1) & 1u;
        ok = mbar_wait(tempty_bar(acc), acc_ph ^ 1u, &abort_flag, p.status, 0x32);
        if (!ok) break;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * G2_BN;
        int kb_n = num_kb;
        if (p.grp_mode == 2) kb_n = g2_k_range(p, (tile / tiles_per_batch) % p.nb0).y;
        if (p.grp_mode == 1) {
          int mt, nt;
          g2_tile_coords(tile % tiles_per_batch, p, mt, nt);
          if (g2_row_group(p, mt) < 0) kb_n = 0;
        }
        for (int kb = 0; kb < kb_n; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1u;
          ok = mbar_wait(full_bar(s), ph, &abort_flag, p.status, 0x33);
          if (!ok) break;
          tc_fence_after();
          const uint32_t sa = smem_base + s * G2_STAGE_BYTES;
          const uint32_t sb = sa + G2_A_BYTES;
#pragma unroll
          for (int k = 0; k < G2_BK / 16; ++k) {
            const uint64_t ad = make_smem_desc(sa + k * A_KSTEP, AMAJ ? LBO_MN : 16u, SBO);
            const uint64_t bd = make_smem_desc(sb + k * B_KSTEP, BMAJ ? LBO_MN : 16u, SBO);
            if (F8)
              umma2_f8(tmem_d, ad, bd, idesc8, (kb | k) != 0);
            else
              umma2_f16(tmem_d, ad, bd, idesc, (kb | k) != 0);
          }
          umma2_commit(mapa(empty_bar(s), 0));
          umma2_commit(mapa(empty_bar(s), 1));
        }
        if (!ok) break;
        umma2_commit(mapa(tfull_bar(acc), 0));
        umma2_commit(mapa(tfull_bar(acc), 1));
      }
    }
  } else if (warp < 6) {
    // -------------------------------------------------- epilogue (warps 2..5, both CTAs)
    const int quarter = warp & 3;
    const int trow = quarter * 32 + lane;
    const bool issuer = (warp == 2 && lane == 0);
    constexpr int PC = 128 / (int)sizeof(OutT);  // columns per piece: 32 fp32 or 64 bf16
    uint32_t tile_iter = 0, piece_iter = 0;
    for (int work = pair; work < p.num_work; work += n_pairs, ++tile_iter) {
      int tile, n_off, bn;
      g2_work(work, p, tile, n_off, bn);
      const int acc = tile_iter & 1;
      const uint32_t acc_ph = (tile_iter >> 1) & 1u;
      const int batch = tile / tiles_per_batch;
      const int t = tile - batch * tiles_per_batch;
      int mt, nt;
      g2_tile_coords(t, p, mt, nt);
      const int m0 = mt * G2_BM + rank * G2_ROWS;
      const int n0 = nt * G2_BN + n_off;
      const int b0 = batch % p.nb0, b1 = batch / p.nb0;
      // a group without rows issued no product: its accumulator holds whatever the previous tile left
      const bool empty = p.grp_mode == 2 && g2_k_range(p, b0).y == 0;
      const bool dead = p.grp_mode == 1 && g2_row_group(p, mt) < 0;  // a row tile past the last group
      if (!mbar_wait(tfull_bar(acc), acc_ph, &abort_flag, p.status, 0x34)) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + acc * G2_BN + (static_cast<uint32_t>(quarter * 32) << 16);
      // scale of this thread's row: alpha, or the row's quantisation scale for float8 operands
      float rs = p.alpha;
      if (F8) rs = (m0 + trow < p.M && p.row_scale) ? __ldg(p.row_scale + m0 + trow) : 1.f;
      auto cscale = [&](int col) -> float {
        return (F8 && p.col_scale && col < p.N) ? __ldg(p.col_scale + col) : 1.f;
      };
      if (p.epi_tma) {
        if (m0 < p.M && !dead) {
          const CUtensorMap* cmap = &tma_c;
          int drow = m0;
          bool table_ok = true;
          if (p.scatter) {
            const int2 e = p.blocks[m0 / G2_ROWS];
            table_ok = LB_CHECK_INDEX(e.x >= 0 && e.x < LB_MAX_PEERS && e.y >= 0 && (e.y % 8) == 0, p.status, 0x41);
            cmap = &owners.m[table_ok ? e.x : 0];
            drow = e.y;
          }
#pragma unroll 1
          for (int c = 0; c < G2_BN / PC; ++c) {
            const int col0 = n0 + c * PC;
            if (col0 >= p.N || c * PC >= bn || !table_ok) break;  // uniform over the four warps
            const uint32_t buf = aux_base + (piece_iter & 1u) * G2_PIECE;
            if (issuer) tma_store_wait_read<1>();  // the store that last used this buffer has read it
            g2_epi_bar_sync();
            const uint32_t rowbase = buf + trow * 128;
            const uint32_t sw = static_cast<uint32_t>(trow & 7);
            if (sizeof(OutT) == 4) {
              uint32_t r[32];
              tmem_ld32(taddr + c * 32, r);
              tmem_wait_ld();
              if (empty) {
#pragma unroll
                for (int i = 0; i < 32; ++i) r[i] = 0u;
              }
#pragma unroll
              for (int g = 0; g < 8; ++g) {
                const uint32_t dst = rowbase + ((static_cast<uint32_t>(g) ^ sw) << 4);
                const int cc = col0 + g * 4;
                const uint32_t v0 = __float_as_uint(__uint_as_float(r[g * 4 + 0]) * rs * cscale(cc + 0));
                const uint32_t v1 = __float_as_uint(__uint_as_float(r[g * 4 + 1]) * rs * cscale(cc + 1));
                const uint32_t v2 = __float_as_uint(__uint_as_float(r[g * 4 + 2]) * rs * cscale(cc + 2));
                const uint32_t v3 = __float_as_uint(__uint_as_float(r[g * 4 + 3]) * rs * cscale(cc + 3));
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(v0), "r"(v1), "r"(v2), "r"(v3)
                             : "memory");
              }
            } else {
#pragma unroll
              for (int h = 0; h < 2; ++h) {
                uint32_t r[32];
                tmem_ld32(taddr + c * 64 + h * 32, r);
                tmem_wait_ld();
                if (empty) {
#pragma unroll
                  for (int i = 0; i < 32; ++i) r[i] = 0u;
                }
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                  const uint32_t dst = rowbase + ((static_cast<uint32_t>(h * 4 + g) ^ sw) << 4);
                  const int cc = col0 + h * 32 + g * 8;
                  const uint32_t v0 = pack_bf16(__uint_as_float(r[g * 8 + 0]) * rs * cscale(cc + 0), __uint_as_float(r[g * 8 + 1]) * rs * cscale(cc + 1));
                  const uint32_t v1 = pack_bf16(__uint_as_float(r[g * 8 + 2]) * rs * cscale(cc + 2), __uint_as_float(r[g * 8 + 3]) * rs * cscale(cc + 3));
                  const uint32_t v2 = pack_bf16(__uint_as_float(r[g * 8 + 4]) * rs * cscale(cc + 4), __uint_as_float(r[g * 8 + 5]) * rs * cscale(cc + 5));
                  const uint32_t v3 = pack_bf16(__uint_as_float(r[g * 8 + 6]) * rs * cscale(cc + 6), __uint_as_float(r[g * 8 + 7]) * rs * cscale(cc + 7));
                  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(v0), "r"(v1), "r"(v2), "r"(v3)
                               : "memory");
                }
              }
            }
            fence_proxy_async_smem();
            g2_epi_bar_sync();
            if (issuer) {
              if (sizeof(OutT) == 4 && p.accumulate)
                tma_reduce_add_4d(cmap, buf, col0, drow, b0, b1);
              else
                tma_store_4d(cmap, buf, col0, drow, b0, b1);
              tma_store_commit();
            }
            ++piece_iter;
          }
        }
      } else {
        const int row = m0 + trow;
        OutT* crow = reinterpret_cast<OutT*>(p.C) + b0 * p.c_bs0 + b1 * p.c_bs1 + static_cast<long long>(row) * p.ldc;
#pragma unroll 1
        for (int c = 0; c < G2_BN / 32; ++c) {
          const int col0 = n0 + c * 32;
          if (col0 >= p.N || c * 32 >= bn) break;
          uint32_t r[32];
          tmem_ld32(taddr + c * 32, r);
          tmem_wait_ld();
          if (empty) {
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = 0u;
          }
          if (row < p.M && !dead) {
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
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa(tempty_bar(acc), 0));
    }
    if (issuer) tma_store_wait<0>();  // every piece has left shared memory and landed
  } else if (GATHER && lane == 0 && p.g_n_remote > 0) {
    // -------------------------------------------------- weight gather (warp 6, both CTAs)
    // Pieces of the remote blocks are claimed from one counter by all CTAs, pulled peer -> shared -> local with
    // bulk copies (two in flight), and counted per block once they have landed; every remote byte crosses NVLink
    // once. Blocks are pulled in the order the tile walk needs them.
    const uint32_t total = static_cast<uint32_t>(p.g_n_remote) * p.g_ppb;
    const long long block_bytes = (long long)p.g_ppb * G2_COPY;
    uint32_t* counter = p.flags + p.n_blocks;
    auto claim = [&]() -> long long {
      const uint32_t i = atomicAdd(counter, 1u);
      return i < total ? (long long)i : -1ll;
    };
    auto locate = [&](long long piece, int& blk, int& owner, long long& off) {
      int2 e = p.g_blocks[piece / p.g_ppb];
      if (!LB_CHECK_INDEX(e.x >= 0 && e.x < p.n_blocks && e.y >= 0 && e.y < LB_MAX_PEERS && p.peer_b[e.y], p.status, 0x42))
        e = make_int2(0, 0), abort_flag = 1;  // stop pulling: the producer's bounded wait reports the rest
      blk = e.x;
      owner = e.y;
      off = (long long)blk * block_bytes + (piece % p.g_ppb) * G2_COPY;
    };
    uint32_t i = 0;
    long long cur = claim();
    if (cur >= 0) {
      int blk, owner; long long off;
      locate(cur, blk, owner, off);
      mbar_arrive_expect_tx(copy_bar(0), G2_COPY);
      bulk_load(copy_base, p.peer_b[owner] + off, G2_COPY, copy_bar(0));
    }
    uint32_t* pending = nullptr;  // flag of the piece whose store is in flight
    while (cur >= 0) {
      if (pending) {
        tma_store_wait<0>();  // landed in local memory (and its buffer is free again)
        fence_proxy_async_all();
        red_release_gpu_add(pending, 1u);
        pending = nullptr;
      }
      const long long nxt = claim();
      if (nxt >= 0) {
        int blk, owner; long long off;
        locate(nxt, blk, owner, off);
        const uint32_t b = (i + 1) & 1u;
        mbar_arrive_expect_tx(copy_bar(b), G2_COPY);
        bulk_load(copy_base + b * G2_COPY, p.peer_b[owner] + off, G2_COPY, copy_bar(b));
      }
      if (!mbar_wait(copy_bar(i & 1u), (i >> 1) & 1u, &abort_flag, p.status, 0x36)) break;
      int blk, owner; long long off;
      locate(cur, blk, owner, off);
      bulk_store(p.local_b + off, copy_base + (i & 1u) * G2_COPY, G2_COPY);
      tma_store_commit();
      pending = p.flags + blk;
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
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  // Neither CTA may leave (or free tensor memory) while its partner can still signal its barriers
  // or while paired MMAs may still be writing into its TMEM.
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc2(tmem_base, 512);
  }
}

struct F8Extra {
  const float* row_scale;
  const float* col_scale;
  int a_fmt, b_fmt;  // 0 = e4m3, 1 = e5m2
};

template <int AMAJ, int BMAJ, typename OutT, bool GATHER = false, bool F8 = false>
static int launch_gemm2(const LbGemmArgs& a_in, const LbScatterArgs* sc, cudaStream_t stream,
                        const LbGatherArgs* ga = nullptr, const F8Extra* f8 = nullptr,
                        const LbGroupArgs* gr = nullptr) {
  CUtensorMap ta, tb, tc;
  OwnerMaps owners;
  int rc;
  constexpr int IN_ESZ = F8 ? 1 : 2;
  constexpr int BK_IN = 128 / IN_ESZ;
  LbGemmArgs a = a_in;
  // batch extents of the operands' maps: a grouped product batches only B (mode 1) or only C (mode 2)
  int a_nb0 = a.nb0, b_nb0 = a.nb0;
  long long a_bs0 = a.a_bs0, b_bs0 = a.b_bs0;
  if (gr && gr->mode == 1) {
    b_nb0 = gr->n_groups;
    b_bs0 = gr->group_stride;
  } else if (gr && gr->mode == 2) {
    a.nb0 = gr->n_groups;
    a.c_bs0 = gr->group_stride;
    a_nb0 = b_nb0 = 1;
    a_bs0 = b_bs0 = 0;
  }
  if (AMAJ == 0)
    rc = make_tmap_4d(&ta, a.A, IN_ESZ, a.K, a.M, a.lda, a_nb0, a_bs0, a.nb1, a.a_bs1, BK_IN, G2_ROWS);
  else
    rc = make_tmap_4d(&ta, a.A, 2, a.M, a.K, a.lda, a_nb0, a_bs0, a.nb1, a.a_bs1, 64, G2_BK);
  if (rc) return 100 + rc;
  if (BMAJ == 0)
    rc = make_tmap_4d(&tb, a.B, IN_ESZ, a.K, a.N, a.ldb, b_nb0, b_bs0, a.nb1, a.b_bs1, BK_IN, G2_ROWS);
  else
    rc = make_tmap_4d(&tb, a.B, 2, a.N, a.K, a.ldb, b_nb0, b_bs0, a.nb1, a.b_bs1, 64, G2_BK);
  if (rc) return 200 + rc;
  Gemm2Params p;
  p.grp_mode = gr ? gr->mode : 0;
  p.grp_n = gr ? gr->n_groups : 0;
  p.grp_sel = gr ? gr->sel : nullptr;
  p.row_scale = f8 ? f8->row_scale : nullptr;
  p.col_scale = f8 ? f8->col_scale : nullptr;
  p.idesc_f8 = f8 ? make_idesc(G2_BM, G2_BN, (uint32_t)f8->a_fmt, (uint32_t)f8->b_fmt, 0, 0) : 0u;
  p.M = a.M; p.N = a.N; p.K = a.K;
  p.tiles_m = (a.M + G2_BM - 1) / G2_BM;
  p.tiles_n = (a.N + G2_BN - 1) / G2_BN;
  p.nb0 = a.nb0; p.nb1 = a.nb1;
  p.ldc = a.ldc; p.c_bs0 = a.c_bs0; p.c_bs1 = a.c_bs1;
  p.alpha = a.alpha; p.accumulate = a.accumulate;
  p.C = a.C; p.status = a.status;
  // Row tiles per rasterisation group: the A rows of a group are re-used by every column tile and should stay in
  // L2 while B streams past them, so take the largest group whose slice of A stays under 48 MB. Measured under the
  // power cap at 8192 x 11008 x 4096: 16 tiles 1254 TFLOP/s, 8 tiles 1229, 32 tiles 1173; at K = 11008 eight tiles
  // are best. LB_GEMM_GROUP_M overrides the choice for tuning runs.
  int group_m = 32;
  while (group_m > 4 && (long long)group_m * G2_BM * a.K * IN_ESZ > (48ll << 20)) group_m >>= 1;
  if (const char* e = getenv("LB_GEMM_GROUP_M")) {
    const int v = atoi(e);
    if (v > 0) group_m = v;
  }
  p.group_m = p.tiles_m < group_m ? p.tiles_m : group_m;
  p.m_rot = 0;
  p.scatter = 0;
  p.blocks = nullptr;
  p.raster_n = 0;
  p.n_order = nullptr;
  p.g_blocks = nullptr;
  p.g_n_remote = 0;
  p.g_ppb = 0;
  p.local_b = nullptr;
  p.flags = nullptr;
  p.n_blocks = 0;
  for (int r = 0; r < LB_MAX_PEERS; ++r) p.peer_b[r] = nullptr;
  if (GATHER) {
    if (!ga) return 8;
    p.raster_n = 1;
    p.group_m = p.tiles_n < 8 ? p.tiles_n : 8;
    p.n_order = ga->n_order;
    p.g_blocks = reinterpret_cast<const int2*>(ga->remote_blocks);
    p.g_n_remote = ga->n_remote;
    p.g_ppb = static_cast<uint32_t>((long long)G2_ROWS * a.K * 2 / G2_COPY);
    p.local_b = reinterpret_cast<uint8_t*>(const_cast<void*>(a.B));
    p.flags = ga->flags;
    p.n_blocks = a.N / G2_ROWS;
    for (int r = 0; r < LB_MAX_PEERS; ++r)
      p.peer_b[r] = reinterpret_cast<const uint8_t*>(ga->b_peers[r < ga->world ? r : 0]);
    if (ga->n_remote > 0) {
      // own blocks start complete, remote ones at zero; the piece counter follows the block flags
      cudaError_t e = cudaMemcpyAsync(ga->flags, ga->flags_init, sizeof(uint32_t) * (p.n_blocks + 1),
                                      cudaMemcpyDeviceToDevice, stream);
      if (e != cudaSuccess) return 500 + (int)e;
    }
  }
  constexpr int ESZ = (int)sizeof(OutT);
  constexpr int PC = 128 / ESZ;
  // TMA stores need a 16-byte aligned base and pitches that are multiples of 16 bytes
  auto tma_ok = [&](const void* base) {
    return (reinterpret_cast<uintptr_t>(base) % 16 == 0) && (a.ldc * ESZ) % 16 == 0 &&
           (a.nb0 <= 1 || (a.c_bs0 * ESZ) % 16 == 0) && (a.nb1 <= 1 || (a.c_bs1 * ESZ) % 16 == 0);
  };
  if (sc) {
    if (ESZ != 4 || a.nb0 != 1 || a.nb1 != 1) return 6;
    for (int o = 0; o < LB_MAX_PEERS; ++o) {
      const int src = o < sc->world ? o : 0;
      if (!tma_ok(sc->dst[src]) || sc->dst_rows[src] < 0) return 7;
      // an owner without rows in this product still needs a valid map (it is never used)
      const long long rows = sc->dst_rows[src] > 0 ? sc->dst_rows[src] : 1;
      rc = make_tmap_4d(&owners.m[o], sc->dst[src], ESZ, a.N, rows, a.ldc, 1, 0, 1, 0, PC, G2_ROWS);
      if (rc) return 120 + rc;
    }
    tc = owners.m[0];
    p.scatter = 1;
    p.epi_tma = 1;
    p.blocks = reinterpret_cast<const int2*>(sc->blocks);
    p.m_rot = sc->m_rot >= 0 && sc->m_rot < p.tiles_m ? sc->m_rot : 0;
  } else {
    p.epi_tma = tma_ok(a.C) ? 1 : 0;
    if (p.epi_tma) {
      rc = make_tmap_4d(&tc, a.C, ESZ, a.N, a.M, a.ldc, a.nb0, a.c_bs0, a.nb1, a.c_bs1, PC, G2_ROWS);
      if (rc) return 110 + rc;
    } else {
      tc = ta;
    }
    for (int o = 0; o < LB_MAX_PEERS; ++o) owners.m[o] = tc;
  }
  const long long tiles = (long long)p.tiles_m * p.tiles_n * a.nb0 * a.nb1;
  const int max_pairs = num_sms() / 2;
  if (tiles > 0x3fffffffll) return 9;
  p.tail_first = (int)tiles;
  p.idesc_f8_half = f8 ? make_idesc(G2_BM, G2_BN / 2, (uint32_t)f8->a_fmt, (uint32_t)f8->b_fmt, 0, 0) : 0u;
  {
    // split the last wave when it would occupy at most half of the pairs (see Gemm2Params::tail_first); not in
    // gather mode, whose producer waits per 128-row block of B, nor for batched or grouped launches
    static const bool no_split = getenv("LB_GEMM_NO_TAIL_SPLIT") != nullptr;
    const int rem = (int)(tiles % max_pairs);
    if (!no_split && !GATHER && !gr && a.nb0 == 1 && a.nb1 == 1 && rem > 0 && 2 * rem <= max_pairs)
      p.tail_first = (int)tiles - rem;
  }
  p.num_work = p.tail_first + 2 * ((int)tiles - p.tail_first);
  const int pairs = p.num_work < max_pairs ? p.num_work : max_pairs;
  if (ensure_dyn_smem<gemm2_kernel<AMAJ, BMAJ, OutT, GATHER, F8>>(G2_SMEM)) return 300;
  gemm2_kernel<AMAJ, BMAJ, OutT, GATHER, F8>
      <<<2 * pairs, GATHER ? G2_THREADS_GATHER : G2_THREADS, G2_SMEM, stream>>>(ta, tb, tc, owners, p);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}

template <typename OutT>
static int dispatch2(const LbGemmArgs& a, const LbScatterArgs* sc, cudaStream_t s) {
  if (a.a_major == 0 && a.b_major == 0) return launch_gemm2<0, 0, OutT>(a, sc, s);
  if (a.a_major == 0 && a.b_major == 1) return launch_gemm2<0, 1, OutT>(a, sc, s);
  if (a.a_major == 1 && a.b_major == 0) return launch_gemm2<1, 0, OutT>(a, sc, s);
  return launch_gemm2<1, 1, OutT>(a, sc, s);
}

int gemm2_dispatch(const LbGemmArgs& a, cudaStream_t s) {
  if (a.out_dtype == LB_BF16) return dispatch2<__nv_bfloat16>(a, nullptr, s);
  if (a.out_dtype == LB_F32) return dispatch2<float>(a, nullptr, s);
  return 5;
}

// float8 operands on SM pairs: same contract as lb_gemm_fp8 (gemm_fp8.cu), which forwards large problems here
int gemm2_fp8_dispatch(const LbGemmFp8Args& f, cudaStream_t s) {
  LbGemmArgs a = {};
  a.A = f.A; a.B = f.B; a.C = f.C; a.status = f.status;
  a.M = f.M; a.N = f.N; a.K = f.K;
  a.nb0 = a.nb1 = 1;
  a.alpha = 1.f;
  a.lda = f.lda; a.ldb = f.ldb; a.ldc = f.ldc;
  F8Extra x = {f.row_scale, f.col_scale, f.a_fmt, f.b_fmt};
  if (f.out_dtype == LB_BF16) return launch_gemm2<0, 0, __nv_bfloat16, false, true>(a, nullptr, s, nullptr, &x);
  if (f.out_dtype == LB_F32) return launch_gemm2<0, 0, float, false, true>(a, nullptr, s, nullptr, &x);
  return 5;
}

}  // namespace lb

extern "C" int lb_gemm_scatter(const LbGemmArgs* args, const LbScatterArgs* sc, void* stream) {
  using namespace lb;
  if (!args || !sc) return 1;
  const LbGemmArgs& a = *args;
  if (a.M <= 0 || a.N <= 0 || a.K <= 0 || a.nb0 != 1 || a.nb1 != 1) return 1;
  if (a.in_dtype != LB_BF16 || a.out_dtype != LB_F32) return 2;
  if ((a.ldc % 4) || (a.lda % 8) || (a.ldb % 8) || a.ldc < a.N || (a.N % 4)) return 3;
  if (sc->world < 1 || sc->world > LB_MAX_PEERS || !sc->blocks) return 4;
  return dispatch2<float>(a, sc, reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int lb_gemm_grouped(const LbGemmArgs* args, const LbGroupArgs* gr, void* stream) {
  using namespace lb;
  if (!args || !gr || !gr->sel) return 1;
  const LbGemmArgs& a = *args;
  if (a.M <= 0 || a.N <= 0 || a.K <= 0 || a.nb0 != 1 || a.nb1 != 1) return 1;
  if (a.in_dtype != LB_BF16) return 2;
  if ((a.lda % 8) || (a.ldb % 8) || gr->n_groups < 1 || gr->group_stride % 8) return 3;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (gr->mode == 1) {
    if (a.a_major != 0 || a.out_dtype != LB_BF16 || a.accumulate) return 4;
    return a.b_major == 0 ? launch_gemm2<0, 0, __nv_bfloat16>(a, nullptr, s, nullptr, nullptr, gr)
                          : launch_gemm2<0, 1, __nv_bfloat16>(a, nullptr, s, nullptr, nullptr, gr);
  }
  if (gr->mode == 2) {
    if (a.a_major != 1 || a.b_major != 1 || a.out_dtype != LB_F32 || (a.ldc % 4)) return 5;
    return launch_gemm2<1, 1, float>(a, nullptr, s, nullptr, nullptr, gr);
  }
  return 6;
}

extern "C" int lb_gemm_gather(const LbGemmArgs* args, const LbGatherArgs* ga, void* stream) {
  using namespace lb;
  if (!args || !ga) return 1;
  const LbGemmArgs& a = *args;
  if (a.M <= 0 || a.N <= 0 || a.K <= 0 || a.nb0 != 1 || a.nb1 != 1) return 1;
  if (a.in_dtype != LB_BF16 || a.out_dtype != LB_BF16 || a.a_major != 0 || a.b_major != 0 || a.accumulate) return 2;
  if ((a.ldc % 8) || (a.lda % 8) || a.ldb != a.K || a.K % 64 || a.N % G2_ROWS) return 3;  // whole contiguous blocks
  if (ga->world < 1 || ga->world > LB_MAX_PEERS || ga->n_remote < 0) return 4;
  if (ga->n_remote > 0 && (!ga->remote_blocks || !ga->flags || !ga->flags_init || !ga->n_order)) return 5;
  return launch_gemm2<0, 0, __nv_bfloat16, true>(a, nullptr, reinterpret_cast<cudaStream_t>(stream), ga);
}
