// Flash attention forward / backward for head_dim 128 on tcgen05 (sm_100a).
//
// Causal, block-causal (documents packed in one sequence, given as doc_start[token]) and
// sliding-window masks; grouped-query attention without materialising repeated K/V heads.
// Replaces the SDPA / xformers / flex_attention calls of lingua/transformer.py:374-404 and
// the mask builders of lingua/transformer.py:142-217.
//
// Forward, one CTA per (pair of 128-query blocks, head, batch): warp 0 streams K and V tiles
// with TMA, one thread of warp 1 issues S = Q K^T and O += P V for both query tiles in turn, two
// groups of four warps (one thread per query row) run the online softmax on S straight out of
// TMEM, write P back into TMEM as the A operand of the second MMA, and rescale the TMEM-resident
// O only when a row maximum grew by more than 2^8.
//
// Backward, one CTA per (128-key block, kv head, batch), looping over the query blocks that
// can see it: S and dP are recomputed on the tensor cores, dV and dK accumulate in TMEM for
// the whole loop, and dQ tiles are added to an fp32 scratch buffer with TMA reductions.
#include "common.cuh"
#include "lingua_b200.h"

namespace lb {

constexpr int AT_THREADS = 192;
constexpr int BWD_THREADS = 320;  // TMA warp, MMA warp, 8 softmax warps (two per TMEM lane quarter)
constexpr int AT_TILE = 128 * 128 * 2;  // one 128 x 128 bf16 tile: two 16 KB halves of 64 columns
constexpr int AT_HALF = 128 * 64 * 2;
constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;

constexpr uint32_t IDESC_KK = make_idesc(128, 128, 1, 1, 0, 0);
constexpr uint32_t IDESC_KM = make_idesc(128, 128, 1, 1, 0, 1);
constexpr uint32_t IDESC_MM = make_idesc(128, 128, 1, 1, 1, 1);

// k-th 16-wide reduction slice of a tile whose 128-byte rows run along the reduction dim
__device__ __forceinline__ uint64_t desc_k(uint32_t tile, int k) {
  return make_smem_desc(tile + (k >> 2) * AT_HALF + (k & 3) * 32, 16, 1024);
}
// k-th 16-row reduction slice of a tile whose 128-byte rows run along M/N (one row per k)
__device__ __forceinline__ uint64_t desc_mn(uint32_t tile, int k) {
  return make_smem_desc(tile + k * 2048, AT_HALF, 1024);
}
// 32 bf16 of row r, columns [32c, 32c+32) into a 128 x 128 tile in the TMA 128-byte swizzle
__device__ __forceinline__ void st_tile_row32(uint32_t tile, int r, int c, const uint32_t (&pk)[16]) {
  const uint32_t base = tile + (c >> 1) * AT_HALF + r * 128;
  const int unit0 = (c & 1) * 4;
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const uint32_t addr = base + (((unit0 + u) ^ (r & 7)) << 4);
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(pk[4 * u]), "r"(pk[4 * u + 1]),
                 "r"(pk[4 * u + 2]), "r"(pk[4 * u + 3])
                 : "memory");
  }
}

// Optional timing trace (compile with -DLB_ATTN_TRACE): CTA (0,0,0) of the forward kernel records
// clock64() at fixed points of its softmax and MMA loops; lb_attn_trace_read copies them out.
#ifdef LB_ATTN_TRACE
__device__ long long g_attn_trace[4096];
#define LB_TRACE(slot) \
  do { if (trace_on) g_attn_trace[(slot) & 4095] = clock64(); } while (0)
#else
#define LB_TRACE(slot) do { } while (0)
#endif

struct AttnParams {
  int B, S, H, Hkv;
  int causal, window;
  float scale;
  const int* doc_start;  // [B*S]: first token of the document of each token, or null
  const int* doc_end;    // [B*S]: one past the last token of that document, or null
  __nv_bfloat16* O;      // [B,S,H,128] contiguous
  float* lse;            // [B,H,S] natural log
  const float* delta;    // [B,H,S]
  float* dq_acc;         // [B,S,H,128] fp32
  __nv_bfloat16 *dk, *dv;
  long long k_sb, k_ss, k_sh, v_sb, v_ss, v_sh;  // strides of dk / dv (same as k / v)
  uint32_t* status;
};

// ============================================================================ forward
// One CTA owns two consecutive 128-query tiles of one head and streams the K / V tiles both of
// them need through a 2-stage ring (each K / V tile is fetched once for 256 queries). Each query
// tile has its own S and O accumulators in tensor memory (4 x 128 columns); the eight softmax
// warps handle the tiles alternately, and the MMA thread interleaves them the same way:
//     ... O0 += P0 V(j) | S0 = Q0 K(j+1)^T | O1 += P1 V(j) | S1 = Q1 K(j+1)^T ...
// so the tensor pipe works on one tile while the other tile's softmax runs. P never touches
// shared memory: it is written as bf16 pairs over the first 64 columns of its S and read from
// there as the A operand of the second MMA.
constexpr int FWD_THREADS = 320;  // TMA warp, MMA warp, 8 softmax warps
constexpr int FWD_SMEM = 6 * AT_TILE /*Q0, Q1, K x 2, V x 2*/ + 1024 + 256;

__global__ void __launch_bounds__(FWD_THREADS, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk,
                const __grid_constant__ CUtensorMap tv, const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ int abort_flag;
  __shared__ uint32_t tmem_slot;
  __shared__ float xchg[2][128][2];  // row maximum / row sum halves exchanged between partner warps
  const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
  auto sQ = [&](int t) { return sbase + t * AT_TILE; };
  auto sK = [&](int s) { return sbase + 2 * AT_TILE + s * 2 * AT_TILE; };
  auto sV = [&](int s) { return sbase + 3 * AT_TILE + s * 2 * AT_TILE; };
  const uint32_t bars = sbase + 6 * AT_TILE;
  const uint32_t q_full = bars;
  auto k_full = [&](int s) { return bars + 8 + 8 * s; };
  auto v_full = [&](int s) { return bars + 24 + 8 * s; };
  auto kv_empty = [&](int s) { return bars + 40 + 8 * s; };
  auto s_full = [&](int t) { return bars + 56 + 8 * t; };
  auto p_full = [&](int t) { return bars + 72 + 8 * t; };
  auto o_done = [&](int t) { return bars + 88 + 8 * t; };
  auto pair_bar = [&](int q) { return bars + 104 + 8 * q; };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#ifdef LB_ATTN_TRACE
  const bool trace_on = blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && (threadIdx.x == 32 || threadIdx.x == 64);
#endif
  const int nqb = (p.S + 127) / 128;
  const int npair = (nqb + 1) / 2;
  const int pair = npair - 1 - blockIdx.x;  // longest rows first
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (p.H / p.Hkv);

  // kv block range [j0, j1] of each query tile; a tile past the end of the sequence has none
  auto tile_range = [&](int qb, int& j0, int& j1, int& lo_last_out) {
    j0 = 1; j1 = 0; lo_last_out = 0;
    if (qb >= nqb) return;
    const int row_first = qb * 128;
    const int row_last = min(qb * 128 + 127, p.S - 1);
    int lo_first = p.doc_start ? p.doc_start[(long long)b * p.S + row_first] : 0;
    int lo_last = p.doc_start ? p.doc_start[(long long)b * p.S + row_last] : 0;
    if (p.window > 0) {
      lo_first = max(lo_first, row_first - p.window + 1);
      lo_last = max(lo_last, row_last - p.window + 1);
    }
    j0 = lo_first / 128;
    j1 = p.causal ? qb : nqb - 1;
    lo_last_out = lo_last;
  };
  int a_j0, a_j1, a_lo, b_j0, b_j1, b_lo;
  tile_range(2 * pair, a_j0, a_j1, a_lo);
  tile_range(2 * pair + 1, b_j0, b_j1, b_lo);
  const bool two = b_j1 >= b_j0;
  const int jlo = two ? min(a_j0, b_j0) : a_j0;
  const int jhi = two ? max(a_j1, b_j1) : a_j1;
  const int n = jhi - jlo + 1;
  auto active = [&](int t, int j) { return t ? (j >= b_j0 && j <= b_j1) : (j >= a_j0 && j <= a_j1); };

  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(k_full(s), 1);
      mbar_init(v_full(s), 1);
      mbar_init(kv_empty(s), 1);
      mbar_init(s_full(s), 1);
      mbar_init(p_full(s), 8);
      mbar_init(o_done(s), 1);
    }
    for (int q = 0; q < 4; ++q) mbar_init(pair_bar(q), 64);
    fence_mbar_init();
    tma_prefetch_desc(&tq);
    tma_prefetch_desc(&tk);
    tma_prefetch_desc(&tv);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;
  auto tS = [&](int t) { return tmem + t * 128; };
  auto tO = [&](int t) { return tmem + 256 + t * 128; };

  if (warp == 0) {
    if (lane == 0) {
      mbar_arrive_expect_tx(q_full, two ? 2 * AT_TILE : AT_TILE);
      for (int t = 0; t < (two ? 2 : 1); ++t) {
        tma_load_4d(sQ(t), &tq, q_full, 0, (2 * pair + t) * 128, h, b);
        tma_load_4d(sQ(t) + AT_HALF, &tq, q_full, 64, (2 * pair + t) * 128, h, b);
      }
      for (int it = 0; it < n; ++it) {
        const int s = it & 1, kv0 = (jlo + it) * 128;
        if (!mbar_wait(kv_empty(s), ((it >> 1) & 1) ^ 1, &abort_flag, p.status, 0x11)) break;
        mbar_arrive_expect_tx(k_full(s), AT_TILE);
        tma_load_4d(sK(s), &tk, k_full(s), 0, kv0, hk, b);
        tma_load_4d(sK(s) + AT_HALF, &tk, k_full(s), 64, kv0, hk, b);
        mbar_arrive_expect_tx(v_full(s), AT_TILE);
        tma_load_4d(sV(s), &tv, v_full(s), 0, kv0, hk, b);
        tma_load_4d(sV(s) + AT_HALF, &tv, v_full(s), 64, kv0, hk, b);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // MMAs of one thread run in issue order: S_t(j+1) overwrites P_t(j) only after O_t += P_t V(j)
      // has read it, and a commit after S_t(j+1) also covers that product.
      auto issue_s = [&](int t, int s) {
#pragma unroll
        for (int k = 0; k < 8; ++k) umma_f16(tS(t), desc_k(sQ(t), k), desc_k(sK(s), k), IDESC_KK, k != 0);
        umma_commit(s_full(t));
      };
      uint32_t n_pv0 = 0, n_pv1 = 0;
      auto issue_pv = [&](int t, int s, int j) -> bool {
        uint32_t& cnt = t ? n_pv1 : n_pv0;
        if (!mbar_wait(p_full(t), cnt & 1, &abort_flag, p.status, 0x17)) return false;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < 8; ++k) umma_f16_ts(tO(t), tS(t) + k * 8, desc_mn(sV(s), k), IDESC_KM, (cnt | k) != 0);
        ++cnt;
        if (j == (t ? b_j1 : a_j1)) umma_commit(o_done(t));
        return true;
      };
      bool ok = n > 0 && mbar_wait(q_full, 0, &abort_flag, p.status, 0x12) &&
                mbar_wait(k_full(0), 0, &abort_flag, p.status, 0x13);
      if (ok) {
        tc_fence_after();
        if (active(0, jlo)) issue_s(0, 0);
        if (active(1, jlo)) issue_s(1, 0);
      }
      for (int it = 0; ok && it < n; ++it) {
        const int j = jlo + it, s = it & 1, s1 = s ^ 1;
        const bool more = it + 1 < n;
        const uint32_t ph = (it >> 1) & 1, ph1 = ((it + 1) >> 1) & 1;
        bool k_ready = false;
        if (active(0, j) || active(1, j)) {
          ok = mbar_wait(v_full(s), ph, &abort_flag, p.status, 0x16);
          if (!ok) break;
        }
        LB_TRACE(2048 + it * 8 + 0);
        if (active(0, j)) {
          ok = issue_pv(0, s, j);
          if (!ok) break;
        }
        LB_TRACE(2048 + it * 8 + 1);
        if (more && active(0, j + 1)) {
          ok = mbar_wait(k_full(s1), ph1, &abort_flag, p.status, 0x14);
          if (!ok) break;
          k_ready = true;
          tc_fence_after();
          LB_TRACE(2048 + it * 8 + 2);
          issue_s(0, s1);
        }
        LB_TRACE(2048 + it * 8 + 3);
        if (active(1, j)) {
          ok = issue_pv(1, s, j);
          if (!ok) break;
        }
        LB_TRACE(2048 + it * 8 + 4);
        umma_commit(kv_empty(s));
        if (more && active(1, j + 1)) {
          if (!k_ready) {
            ok = mbar_wait(k_full(s1), ph1, &abort_flag, p.status, 0x15);
            if (!ok) break;
            tc_fence_after();
          }
          issue_s(1, s1);
        }
        LB_TRACE(2048 + it * 8 + 5);
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax warps
    // All eight warps work on one query tile at a time, in the order the MMA thread issues the
    // S products (S0(j), S1(j), S0(j+1), ...). Two warps share each quarter of the TMEM lanes:
    // both own the same 32 query rows and `ch` selects which 64 of the 128 key columns a thread
    // handles, so one softmax step is half as long as with one thread per row; the tensor pipe
    // meanwhile runs the other tile's products.
    const int quarter = warp & 3;
    const int ch = (warp - 2) >> 2;
    const int r = quarter * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    const float sl2 = p.scale * LOG2E;
    // partner warps meet on an mbarrier (64 arrivals) so that this wait is bounded like every other
    uint32_t xph = 0;
    auto pair_sync = [&]() -> bool {
      mbar_arrive(pair_bar(quarter));
      const bool got = mbar_wait(pair_bar(quarter), xph, &abort_flag, p.status, 0x1C);
      xph ^= 1u;
      return got;
    };
    int lo0 = 0, lo1 = 0;
    {
      const int q0 = 2 * pair * 128 + r, q1 = q0 + 128;
      if (p.doc_start) {
        lo0 = p.doc_start[(long long)b * p.S + min(q0, p.S - 1)];
        lo1 = p.doc_start[(long long)b * p.S + min(q1, p.S - 1)];
      }
      if (p.window > 0) {
        lo0 = max(lo0, q0 - p.window + 1);
        lo1 = max(lo1, q1 - p.window + 1);
      }
    }
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    uint32_t cnt0 = 0, cnt1 = 0;
    bool ok = true;
    for (int step = 0; step < 2 * n && ok; ++step) {
      const int t = step & 1, j = jlo + (step >> 1);
      if (!active(t, j)) continue;
      const int qb = 2 * pair + t;
      const int q_idx = qb * 128 + r;
      const int lo = t ? lo1 : lo0;
      const int hi = p.causal ? min(q_idx, p.S - 1) : p.S - 1;  // last visible key
      const int lo_last = t ? b_lo : a_lo;
      const uint32_t cnt = t ? cnt1 : cnt0;
      float m_used = t ? m1 : m0, l = t ? l1 : l0;
      const int kv0 = j * 128 + ch * 64;
      // s_full was committed after O += P V of this tile's previous step was issued: O is quiescent
      LB_TRACE(step * 8 + 0);
      ok = mbar_wait(s_full(t), cnt & 1, &abort_flag, p.status, 0x18);
      if (!ok) break;
      tc_fence_after();
      LB_TRACE(step * 8 + 1);
      const bool need_mask = (p.causal && j == qb) || (j * 128 < lo_last) || (j * 128 + 128 > p.S);
      const uint32_t tSt = tS(t) + lane_off, tOt = tO(t) + lane_off + ch * 64;
      uint32_t sv[2][32];
      tmem_ld32(tSt + ch * 64, sv[0]);
      tmem_ld32(tSt + ch * 64 + 32, sv[1]);
      tmem_wait_ld();
      LB_TRACE(step * 8 + 2);
      float mx = -INFINITY;
      if (need_mask) {
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            const int kv = kv0 + c * 32 + e;
            if (kv < lo || kv > hi) sv[c][e] = 0xFF800000u;  // -inf
            mx = fmaxf(mx, __uint_as_float(sv[c][e]));
          }
      } else {
        // four independent chains instead of one serial one
        float mxa[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
          for (int e = 0; e < 32; e += 2)
            mxa[(e >> 1) & 3] = fmax3(mxa[(e >> 1) & 3], __uint_as_float(sv[c][e]), __uint_as_float(sv[c][e + 1]));
        mx = fmaxf(fmaxf(mxa[0], mxa[1]), fmaxf(mxa[2], mxa[3]));
      }
      // the other half of the row lives in the partner warp; this barrier also orders its TMEM
      // reads of S before this warp's P stores into the same columns
      xchg[t][r][ch] = mx;
      ok = pair_sync();
      if (!ok) break;
      LB_TRACE(step * 8 + 3);
      mx = fmaxf(mx, xchg[t][r][ch ^ 1]) * sl2;
      const float m_new = fmaxf(m_used, mx);
      if (cnt == 0) {
        m_used = m_new;
      } else {
        const bool need = m_new > m_used + 8.f;
        if (__any_sync(0xFFFFFFFFu, need)) {
          const float f = need ? exp2f(m_used - m_new) : 1.f;
#pragma unroll 1
          for (int c = 0; c < 2; ++c) {
            uint32_t rr[32];
            tmem_ld32(tOt + c * 32, rr);
            tmem_wait_ld();
#pragma unroll
            for (int e = 0; e < 32; ++e) rr[e] = __float_as_uint(__uint_as_float(rr[e]) * f);
            tmem_st32(tOt + c * 32, rr);
          }
          l *= f;
          if (need) m_used = m_new;
        }
      }
      const float m_eff = (m_used == -INFINITY) ? 0.f : m_used;
      // P = exp2(S * scale - m): this thread's 64 scores -> 32 packed columns [32 ch, 32 ch + 32)
      uint32_t pk[32];
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        if (need_mask) {
#pragma unroll
          for (int e = 0; e < 32; e += 2) {
            // masked scores are -inf and give exactly 0
            const float p0 = exp2f(__uint_as_float(sv[c][e]) * sl2 - m_eff);
            const float p1 = exp2f(__uint_as_float(sv[c][e + 1]) * sl2 - m_eff);
            l += p0 + p1;
            pk[c * 16 + (e >> 1)] = pack_bf16(p0, p1);
          }
        } else {
          // packed fp32 pairs for the scale / subtract and the row sum; two of every eight
          // exponentials run on the FMA pipe so that the MUFU unit is not the limit
          const uint64_t sl2_2 = pack_f2(sl2, sl2), negm2 = pack_f2(-m_eff, -m_eff);
          uint64_t ls2 = 0ull;
#pragma unroll
          for (int e = 0; e < 32; e += 8) {
            const uint64_t x01 = ffma2(pack_u2(sv[c][e], sv[c][e + 1]), sl2_2, negm2);
            const uint64_t x23 = ffma2(pack_u2(sv[c][e + 2], sv[c][e + 3]), sl2_2, negm2);
            const uint64_t x45 = ffma2(pack_u2(sv[c][e + 4], sv[c][e + 5]), sl2_2, negm2);
            const uint64_t x67 = ffma2(pack_u2(sv[c][e + 6], sv[c][e + 7]), sl2_2, negm2);
            float a0, a1, a2, a3, a4, a5, q6, q7;
            unpack_f2(x01, a0, a1);
            unpack_f2(x23, a2, a3);
            unpack_f2(x45, a4, a5);
            const float p0 = exp2f(a0), p1 = exp2f(a1), p2 = exp2f(a2), p3 = exp2f(a3), p4 = exp2f(a4), p5 = exp2f(a5);
            const uint64_t p67 = exp2_poly2(x67);
            unpack_f2(p67, q6, q7);
            ls2 = fadd2(ls2, fadd2(fadd2(pack_f2(p0, p1), pack_f2(p2, p3)), fadd2(pack_f2(p4, p5), p67)));
            pk[c * 16 + (e >> 1)] = pack_bf16(p0, p1);
            pk[c * 16 + (e >> 1) + 1] = pack_bf16(p2, p3);
            pk[c * 16 + (e >> 1) + 2] = pack_bf16(p4, p5);
            pk[c * 16 + (e >> 1) + 3] = pack_bf16(q6, q7);
          }
          float s0, s1;
          unpack_f2(ls2, s0, s1);
          l += s0 + s1;
        }
      }
      LB_TRACE(step * 8 + 4);
      tmem_st32(tSt + ch * 32, pk);
      tmem_wait_st();
      LB_TRACE(step * 8 + 5);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full(t));
      LB_TRACE(step * 8 + 6);
      if (t) { m1 = m_used; l1 = l; cnt1 = cnt + 1; } else { m0 = m_used; l0 = l; cnt0 = cnt + 1; }
    }
    // epilogue: each thread normalises and stores 64 of the 128 output columns of its row
#pragma unroll 1
    for (int t = 0; t < 2 && ok; ++t) {
      const int qb = 2 * pair + t;
      if (qb >= nqb) break;
      const int q_idx = qb * 128 + r;
      const uint32_t cnt = t ? cnt1 : cnt0;
      const float m_used = t ? m1 : m0;
      float l = t ? l1 : l0;
      if (cnt > 0) {
        ok = mbar_wait(o_done(t), 0, &abort_flag, p.status, 0x1A);
        if (!ok) break;
      }
      tc_fence_after();
      xchg[t][r][ch] = l;
      ok = pair_sync();
      if (!ok) break;
      l += xchg[t][r][ch ^ 1];
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* orow = p.O + (((long long)b * p.S + q_idx) * p.H + h) * 128 + ch * 64;
#pragma unroll 1
      for (int c = 0; c < 2; ++c) {
        uint32_t rr[32];
        if (cnt > 0) {
          tmem_ld32(tO(t) + lane_off + ch * 64 + c * 32, rr);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e) rr[e] = 0u;
        }
        if (q_idx < p.S) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 v;
            v.x = pack_bf16(__uint_as_float(rr[g * 8 + 0]) * inv, __uint_as_float(rr[g * 8 + 1]) * inv);
            v.y = pack_bf16(__uint_as_float(rr[g * 8 + 2]) * inv, __uint_as_float(rr[g * 8 + 3]) * inv);
            v.z = pack_bf16(__uint_as_float(rr[g * 8 + 4]) * inv, __uint_as_float(rr[g * 8 + 5]) * inv);
            v.w = pack_bf16(__uint_as_float(rr[g * 8 + 6]) * inv, __uint_as_float(rr[g * 8 + 7]) * inv);
            *reinterpret_cast<uint4*>(orow + c * 32 + g * 8) = v;
          }
        }
      }
      if (ch == 0 && q_idx < p.S && p.lse) {
        const float m_eff = (m_used == -INFINITY) ? 0.f : m_used;
        p.lse[((long long)b * p.H + h) * p.S + q_idx] = l > 0.f ? (m_eff + log2f(l)) * LN2 : INFINITY;
      }
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
    tmem_dealloc(tmem, 512);
  }
}

// ============================================================================ backward
// delta[b,h,s] = sum_d O[b,s,h,d] * dO[b,s,h,d]; one warp per (b,s,h)
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ O, const __nv_bfloat16* __restrict__ dO,
                                  float* __restrict__ delta, int B, int S, int H) {
  const long long w = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long long total = (long long)B * S * H;
  if (w >= total) return;
  const uint2 a = reinterpret_cast<const uint2*>(O + w * 128)[lane];
  const uint2 g = reinterpret_cast<const uint2*>(dO + w * 128)[lane];
  const float2 a0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&a.x));
  const float2 a1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&a.y));
  const float2 g0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&g.x));
  const float2 g1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&g.y));
  float s = a0.x * g0.x + a0.y * g0.y + a1.x * g1.x + a1.y * g1.y;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xFFFFFFFFu, s, o);
  if (lane == 0) {
    const int hh = w % H;
    const long long bs = w / H;
    const int s_i = bs % S;
    const int bb = bs / S;
    delta[((long long)bb * H + hh) * S + s_i] = s;
  }
}

// dq[b,s,h,:] (bf16, strided) = dq_acc[b,s,h,:] (fp32 contiguous)
__global__ void attn_dq_store_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dq, int B, int S,
                                     int H, long long sb, long long ss, long long sh) {
  const long long total = (long long)B * S * H * 16;  // 8-element vectors
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int v = i & 15;
    const long long row = i >> 4;
    const int hh = row % H;
    const long long bs = row / H;
    const int s_i = bs % S;
    const int bb = bs / S;
    const float4 x = reinterpret_cast<const float4*>(acc + row * 128)[2 * v];
    const float4 y = reinterpret_cast<const float4*>(acc + row * 128)[2 * v + 1];
    uint4 o;
    o.x = pack_bf16(x.x, x.y);
    o.y = pack_bf16(x.z, x.w);
    o.z = pack_bf16(y.x, y.y);
    o.w = pack_bf16(y.z, y.w);
    *reinterpret_cast<uint4*>(dq + bb * sb + s_i * ss + hh * sh + v * 8) = o;
  }
}

constexpr int BWD_SMEM = 2 * AT_TILE /*K,V*/ + 4 * AT_TILE /*Q,dO x 2*/ + AT_TILE /*P|dS*/ + 1024 + 256;

__global__ void __launch_bounds__(BWD_THREADS, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk,
                const __grid_constant__ CUtensorMap tv, const __grid_constant__ CUtensorMap tdo,
                const __grid_constant__ CUtensorMap tdq, const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ int abort_flag;
  __shared__ uint32_t tmem_slot;
  const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sK = sbase, sV = sbase + AT_TILE;
  auto sQ = [&](int s) { return sbase + 2 * AT_TILE + s * 2 * AT_TILE; };
  auto sdO = [&](int s) { return sbase + 3 * AT_TILE + s * 2 * AT_TILE; };
  const uint32_t sP = sbase + 6 * AT_TILE;
  const uint32_t bars = sbase + 7 * AT_TILE;
  const uint32_t kv_full = bars;
  auto qd_full = [&](int s) { return bars + 8 + 8 * s; };
  auto dq_staged = [&](int s, int half) { return bars + 120 + 16 * s + 8 * half; };  // half 0: over Q, 1: over dO
  const uint32_t s_full = bars + 40, p_full = bars + 48, dv_done = bars + 56, ds_full = bars + 64;
  const uint32_t dq_full = bars + 72, dq_drained = bars + 80, dp_full = bars + 88, s_free = bars + 96;
  auto do_full = [&](int s) { return bars + 104 + 8 * s; };  // dO of a stage lands separately from Q

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#ifdef LB_ATTN_TRACE
  const bool trace_on = blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && (threadIdx.x == 0 || threadIdx.x == 32 || threadIdx.x == 64);
#endif
  const int nqb = (p.S + 127) / 128;
  const int jb = blockIdx.x;  // kv block
  const int hk = blockIdx.y, b = blockIdx.z;
  const int group = p.H / p.Hkv;
  const int kv0 = jb * 128;
  const int kv_last = min(kv0 + 127, p.S - 1);

  // query blocks that can see this key block: [i0, i1]
  const int i0 = p.causal ? jb : 0;
  int i1 = nqb - 1;
  if (p.doc_end) i1 = min(i1, (p.doc_end[(long long)b * p.S + kv_last] - 1) / 128);
  if (p.window > 0) i1 = min(i1, (kv_last + p.window - 1) / 128);
  const int nq = max(i1 - i0 + 1, 0);
  const int n = nq * group;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(kv_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(qd_full(s), 1);
      mbar_init(do_full(s), 1);
      mbar_init(dq_staged(s, 0), 4);
      mbar_init(dq_staged(s, 1), 4);
    }
    mbar_init(s_full, 1);
    mbar_init(p_full, 8);
    mbar_init(dv_done, 1);
    mbar_init(ds_full, 8);
    mbar_init(dq_full, 1);
    mbar_init(dq_drained, 8);
    mbar_init(dp_full, 1);
    mbar_init(s_free, 8);
    fence_mbar_init();
    tma_prefetch_desc(&tq);
    tma_prefetch_desc(&tk);
    tma_prefetch_desc(&tv);
    tma_prefetch_desc(&tdo);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;
  const uint32_t tS = tmem, tdP = tmem + 128, tdV = tmem + 256, tdK = tmem + 384;

  if (warp == 0) {
    if (lane == 0) {
      mbar_arrive_expect_tx(kv_full, 2 * AT_TILE);
      tma_load_4d(sK, &tk, kv_full, 0, kv0, hk, b);
      tma_load_4d(sK + AT_HALF, &tk, kv_full, 64, kv0, hk, b);
      tma_load_4d(sV, &tv, kv_full, 0, kv0, hk, b);
      tma_load_4d(sV + AT_HALF, &tv, kv_full, 64, kv0, hk, b);
      // Stage s (Q and dO of query block `it`) is recycled in two steps: once dK and dQ of that block
      // are done, the softmax warps spill dQ (fp32, 64 KB) over the two tiles; this thread adds it to
      // the global accumulator with four TMA reductions and only then loads block it + 2.
      for (int it = 0; it < n + 2; ++it) {
        const int s = it & 1;
        if (it >= 2) {
          const int j = it - 2;
          // dQ of block j: columns [0,64) were spilled over Q's tile, [64,128) over dO's. Each half is
          // reduced as soon as it is there; the Q tile can be reloaded once the first half has been read.
          LB_TRACE(3072 + it * 4 + 0);
          const int hj = hk * group + j / nq;
          const int qj = (i0 + j % nq) * 128;
          if (!mbar_wait(dq_staged(s, 0), (j >> 1) & 1, &abort_flag, p.status, 0x21)) break;
          tma_reduce_add_4d(&tdq, sQ(s), 0, qj, hj, b);
          tma_reduce_add_4d(&tdq, sQ(s) + AT_HALF, 32, qj, hj, b);
          tma_store_commit();
          LB_TRACE(3072 + it * 4 + 1);
          if (!mbar_wait(dq_staged(s, 1), (j >> 1) & 1, &abort_flag, p.status, 0x2D)) break;
          tma_reduce_add_4d(&tdq, sdO(s), 64, qj, hj, b);
          tma_reduce_add_4d(&tdq, sdO(s) + AT_HALF, 96, qj, hj, b);
          tma_store_commit();
          LB_TRACE(3072 + it * 4 + 2);
          tma_store_wait_read<1>();
          LB_TRACE(3072 + it * 4 + 3);
        }
        if (it >= n) continue;
        const int h = hk * group + it / nq;
        const int q0 = (i0 + it % nq) * 128;
        // Q first: S of the next block only needs Q, dO is needed later (dP, dV)
        mbar_arrive_expect_tx(qd_full(s), AT_TILE);
        tma_load_4d(sQ(s), &tq, qd_full(s), 0, q0, h, b);
        tma_load_4d(sQ(s) + AT_HALF, &tq, qd_full(s), 64, q0, h, b);
        if (it >= 2) tma_store_wait_read<0>();
        mbar_arrive_expect_tx(do_full(s), AT_TILE);
        tma_load_4d(sdO(s), &tdo, do_full(s), 0, q0, h, b);
        tma_load_4d(sdO(s) + AT_HALF, &tdo, do_full(s), 64, q0, h, b);
      }
      tma_store_wait<0>();
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // Issue order per query block i (softmax warps work on i while the tensor cores already
      // run what does not depend on them):
      //   dV(i) | S(i+1) | dK(i), dQ(i) | dP(i+1)
      // dQ(i) lands in the TMEM columns of dP, so dP(i+1) waits until dQ(i) has been read out,
      // while S(i+1) only needs the softmax warps to have copied S(i) into registers.
      bool ok = mbar_wait(kv_full, 0, &abort_flag, p.status, 0x22);
      if (ok && n > 0) {
        ok = mbar_wait(qd_full(0), 0, &abort_flag, p.status, 0x23);
        if (ok) {
          tc_fence_after();
#pragma unroll
          for (int k = 0; k < 8; ++k) umma_f16(tS, desc_k(sQ(0), k), desc_k(sK, k), IDESC_KK, k != 0);
          umma_commit(s_full);
          ok = mbar_wait(do_full(0), 0, &abort_flag, p.status, 0x2C);
          if (ok) {
            tc_fence_after();
#pragma unroll
            for (int k = 0; k < 8; ++k) umma_f16(tdP, desc_k(sdO(0), k), desc_k(sV, k), IDESC_KK, k != 0);
            umma_commit(dp_full);
          }
        }
      }
      for (int it = 0; ok && it < n; ++it) {
        const int s = it & 1, s1 = s ^ 1;
        const bool more = it + 1 < n;
        LB_TRACE(2048 + it * 16 + 0);
        ok = mbar_wait(p_full, it & 1, &abort_flag, p.status, 0x25);
        if (!ok) break;
        tc_fence_after();
        LB_TRACE(2048 + it * 16 + 1);
        // dV[kv, d] += P^T dO : both operands read with one 128-byte row per query
#pragma unroll
        for (int k = 0; k < 8; ++k) umma_f16(tdV, desc_mn(sP, k), desc_mn(sdO(s), k), IDESC_MM, (it | k) != 0);
        umma_commit(dv_done);
        LB_TRACE(2048 + it * 16 + 2);
        if (more) {
          ok = mbar_wait(qd_full(s1), ((it + 1) >> 1) & 1, &abort_flag, p.status, 0x23) &&
               mbar_wait(s_free, it & 1, &abort_flag, p.status, 0x24);
          if (!ok) break;
          tc_fence_after();
          LB_TRACE(2048 + it * 16 + 3);
#pragma unroll
          for (int k = 0; k < 8; ++k) umma_f16(tS, desc_k(sQ(s1), k), desc_k(sK, k), IDESC_KK, k != 0);
          umma_commit(s_full);
        }
        LB_TRACE(2048 + it * 16 + 4);
        ok = mbar_wait(ds_full, it & 1, &abort_flag, p.status, 0x26);
        if (!ok) break;
        tc_fence_after();
        LB_TRACE(2048 + it * 16 + 5);
#pragma unroll
        for (int k = 0; k < 8; ++k) umma_f16(tdK, desc_mn(sP, k), desc_mn(sQ(s), k), IDESC_MM, (it | k) != 0);
        // dQ[q, d] = dS K, into the columns that held dP
#pragma unroll
        for (int k = 0; k < 8; ++k) umma_f16(tdP, desc_k(sP, k), desc_mn(sK, k), IDESC_KM, k != 0);
        umma_commit(dq_full);
        LB_TRACE(2048 + it * 16 + 6);
        if (more) {
          ok = mbar_wait(dq_drained, it & 1, &abort_flag, p.status, 0x2A) &&
               mbar_wait(do_full(s1), ((it + 1) >> 1) & 1, &abort_flag, p.status, 0x2C);
          if (!ok) break;
          tc_fence_after();
          LB_TRACE(2048 + it * 16 + 7);
#pragma unroll
          for (int k = 0; k < 8; ++k) umma_f16(tdP, desc_k(sdO(s1), k), desc_k(sV, k), IDESC_KK, k != 0);
          umma_commit(dp_full);
        }
        LB_TRACE(2048 + it * 16 + 8);
      }
    }
  } else {
    // Two warps share each quarter of the TMEM lanes: both own the same 32 rows, `ch` selects which
    // 64 of the 128 columns a thread handles. Two resident warps per scheduler hide each other's
    // latencies, and no reduction along a row is needed in the backward pass.
    const int quarter = warp & 3;
    const int ch = (warp - 2) >> 2;  // 0: columns [0,64), 1: columns [64,128)
    const int r = quarter * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t col_off = ch * 64;
    const float sl2 = p.scale * LOG2E;
    bool ok = true;

    auto drain_dq = [&](int it_done, bool release) -> bool {
      if (!mbar_wait(dq_full, it_done & 1, &abort_flag, p.status, 0x29)) return false;
      tc_fence_after();
      uint32_t qv[2][32];
      tmem_ld32(tdP + lane_off + col_off, qv[0]);
      tmem_ld32(tdP + lane_off + col_off + 32, qv[1]);
      tmem_wait_ld();
      if (release) {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(dq_drained);
      }
      // dK(it_done) and dQ(it_done) have completed, so nothing reads Q / dO of that block any more:
      // their 64 KB become four 128 x 32 fp32 boxes (128-byte swizzled rows) for the TMA reduction.
      const uint32_t stage = sQ(it_done & 1);
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        const uint32_t box = stage + (2 * ch + cc) * AT_HALF + r * 128;
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          const uint32_t dst = box + ((static_cast<uint32_t>(g) ^ static_cast<uint32_t>(r & 7)) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(qv[cc][4 * g]),
                       "r"(qv[cc][4 * g + 1]), "r"(qv[cc][4 * g + 2]), "r"(qv[cc][4 * g + 3]) : "memory");
        }
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(dq_staged(it_done & 1, ch));
      return true;
    };

    // per-row statistics of the next iteration are fetched one iteration ahead
    auto row_stats = [&](int it, float& lse2, float& dlt, int& lo) {
      const int h = hk * group + it / nq;
      const int q_idx = (i0 + it % nq) * 128 + r;
      const bool row_ok = q_idx < p.S;
      const long long stat_i = ((long long)b * p.H + h) * p.S + min(q_idx, p.S - 1);
      lse2 = row_ok ? p.lse[stat_i] * LOG2E : INFINITY;
      dlt = row_ok ? p.delta[stat_i] : 0.f;
      lo = 0;
      if (p.doc_start) lo = p.doc_start[(long long)b * p.S + min(q_idx, p.S - 1)];
      if (p.window > 0) lo = max(lo, q_idx - p.window + 1);
    };
    float lse2_n = 0.f, dlt_n = 0.f;
    int lo_n = 0;
    if (n > 0) row_stats(0, lse2_n, dlt_n, lo_n);

    for (int it = 0; it < n; ++it) {
      const int h = hk * group + it / nq;
      const int ib = i0 + it % nq;
      const int q_idx = ib * 128 + r;
      const bool row_ok = q_idx < p.S;
      const float lse2 = lse2_n, dlt = dlt_n;
      const int lo = lo_n;
      if (it + 1 < n) row_stats(it + 1, lse2_n, dlt_n, lo_n);
      const int hi = p.causal ? min(q_idx, p.S - 1) : p.S - 1;
      int lo_blk = 0;
      {
        const int rl = min(ib * 128 + 127, p.S - 1);
        if (p.doc_start) lo_blk = p.doc_start[(long long)b * p.S + rl];
        if (p.window > 0) lo_blk = max(lo_blk, rl - p.window + 1);
      }
      const bool need_mask = (p.causal && ib == jb) || (kv0 < lo_blk) || (kv0 + 128 > p.S) || (ib * 128 + 128 > p.S);

      LB_TRACE(it * 16 + 0);
      ok = mbar_wait(s_full, it & 1, &abort_flag, p.status, 0x27);
      if (!ok) break;
      tc_fence_after();
      LB_TRACE(it * 16 + 1);
      // P = exp(S - lse), packed to bf16 in registers; S's TMEM columns are released right away
      uint32_t pkP[32];
      {
        uint32_t sv[2][32];
        tmem_ld32(tS + lane_off + col_off, sv[0]);
        tmem_ld32(tS + lane_off + col_off + 32, sv[1]);
        tmem_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(s_free);
        LB_TRACE(it * 16 + 2);
        if (need_mask) {
#pragma unroll
          for (int cc = 0; cc < 2; ++cc) {
#pragma unroll
            for (int e = 0; e < 32; e += 2) {
              float p0 = exp2f(__uint_as_float(sv[cc][e]) * sl2 - lse2);
              float p1 = exp2f(__uint_as_float(sv[cc][e + 1]) * sl2 - lse2);
              const int kv = kv0 + col_off + cc * 32 + e;
              if (!row_ok || kv < lo || kv > hi) p0 = 0.f;
              if (!row_ok || kv + 1 < lo || kv + 1 > hi) p1 = 0.f;
              pkP[cc * 16 + (e >> 1)] = pack_bf16(p0, p1);
            }
          }
        } else {
          // interior block: packed fp32 pairs for the scale / subtract, and two of every eight
          // exponentials on the FMA pipe
          const uint64_t sl2_2 = pack_f2(sl2, sl2), nl2 = pack_f2(-lse2, -lse2);
#pragma unroll
          for (int cc = 0; cc < 2; ++cc) {
#pragma unroll
            for (int e = 0; e < 32; e += 8) {
              const uint64_t x01 = ffma2(pack_u2(sv[cc][e], sv[cc][e + 1]), sl2_2, nl2);
              const uint64_t x23 = ffma2(pack_u2(sv[cc][e + 2], sv[cc][e + 3]), sl2_2, nl2);
              const uint64_t x45 = ffma2(pack_u2(sv[cc][e + 4], sv[cc][e + 5]), sl2_2, nl2);
              const uint64_t x67 = ffma2(pack_u2(sv[cc][e + 6], sv[cc][e + 7]), sl2_2, nl2);
              float a0, a1, a2, a3, a4, a5, q6, q7;
              unpack_f2(x01, a0, a1);
              unpack_f2(x23, a2, a3);
              unpack_f2(x45, a4, a5);
              unpack_f2(exp2_poly2(x67), q6, q7);
              pkP[cc * 16 + (e >> 1)] = pack_bf16(exp2f(a0), exp2f(a1));
              pkP[cc * 16 + (e >> 1) + 1] = pack_bf16(exp2f(a2), exp2f(a3));
              pkP[cc * 16 + (e >> 1) + 2] = pack_bf16(exp2f(a4), exp2f(a5));
              pkP[cc * 16 + (e >> 1) + 3] = pack_bf16(q6, q7);
            }
          }
        }
      }
      // The shared P|dS tile is free once dK(i-1) and dQ(i-1) have completed; reading dQ(i-1) out
      // here also lets the tensor cores start dP(i).
      LB_TRACE(it * 16 + 3);
      if (it > 0) {
        ok = drain_dq(it - 1, true);
        if (!ok) break;
      }
      LB_TRACE(it * 16 + 4);
#pragma unroll
      for (int cc = 0; cc < 2; ++cc)
        st_tile_row32(sP, r, 2 * ch + cc, *reinterpret_cast<const uint32_t(*)[16]>(&pkP[cc * 16]));
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
      LB_TRACE(it * 16 + 5);

      // dS = P * (dP - delta) * scale
      ok = mbar_wait(dp_full, it & 1, &abort_flag, p.status, 0x2B);
      if (!ok) break;
      tc_fence_after();
      LB_TRACE(it * 16 + 6);
      {
        uint32_t dd[2][32];
        tmem_ld32(tdP + lane_off + col_off, dd[0]);
        tmem_ld32(tdP + lane_off + col_off + 32, dd[1]);
        tmem_wait_ld();
        const uint64_t sc2 = pack_f2(p.scale, p.scale), ndl2 = pack_f2(-dlt, -dlt);
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
#pragma unroll
          for (int e = 0; e < 32; e += 2) {
            const uint32_t pp = pkP[cc * 16 + (e >> 1)];
            const uint64_t ps = fmul2(pack_u2(pp << 16, pp & 0xFFFF0000u), sc2);
            const uint64_t dm = fadd2(pack_u2(dd[cc][e], dd[cc][e + 1]), ndl2);
            float d0, d1;
            unpack_f2(fmul2(ps, dm), d0, d1);
            pkP[cc * 16 + (e >> 1)] = pack_bf16(d0, d1);
          }
        }
      }
      LB_TRACE(it * 16 + 7);
      ok = mbar_wait(dv_done, it & 1, &abort_flag, p.status, 0x28);
      if (!ok) break;
      LB_TRACE(it * 16 + 8);
#pragma unroll
      for (int cc = 0; cc < 2; ++cc)
        st_tile_row32(sP, r, 2 * ch + cc, *reinterpret_cast<const uint32_t(*)[16]>(&pkP[cc * 16]));
      tc_fence_before();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(ds_full);
      LB_TRACE(it * 16 + 9);
    }
    if (ok && n > 0) ok = drain_dq(n - 1, false);
    // epilogue: dK (warps with ch == 0) and dV (ch == 1) rows of this key block; every MMA has
    // completed because the last dq_full was the last commit.
    if (ok) {
      tc_fence_after();
      const int kv_idx = kv0 + r;
      __nv_bfloat16* drow = ch == 0 ? p.dk + b * p.k_sb + (long long)kv_idx * p.k_ss + hk * p.k_sh
                                    : p.dv + b * p.v_sb + (long long)kv_idx * p.v_ss + hk * p.v_sh;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t rr[32];
        if (n > 0) {
          tmem_ld32((ch == 0 ? tdK : tdV) + lane_off + c * 32, rr);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e) rr[e] = 0u;
        }
        if (kv_idx < p.S) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 v;
            v.x = pack_bf16(__uint_as_float(rr[g * 8 + 0]), __uint_as_float(rr[g * 8 + 1]));
            v.y = pack_bf16(__uint_as_float(rr[g * 8 + 2]), __uint_as_float(rr[g * 8 + 3]));
            v.z = pack_bf16(__uint_as_float(rr[g * 8 + 4]), __uint_as_float(rr[g * 8 + 5]));
            v.w = pack_bf16(__uint_as_float(rr[g * 8 + 6]), __uint_as_float(rr[g * 8 + 7]));
            *reinterpret_cast<uint4*>(drow + c * 32 + g * 8) = v;
          }
        }
      }
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
    tmem_dealloc(tmem, 512);
  }
}

static int make_qkv_map(CUtensorMap* m, const void* ptr, int B, int S, int H, long long sb, long long ss,
                        long long sh) {
  return make_tmap_4d(m, ptr, 2, 128, S, ss, H, sh, B, sb, 64, 128);
}

}  // namespace lb

using namespace lb;

extern "C" int lb_attn_fwd(const LbAttnArgs* a, void* stream) {
  if (a->D != 128) return 1;
  if (a->H % a->Hkv) return 2;
  if (a->doc_start && !a->causal) return 3;
  if (a->B <= 0 || a->S <= 0) return 0;
  CUtensorMap tq, tk, tv;
  if (make_qkv_map(&tq, a->q, a->B, a->S, a->H, a->q_sb, a->q_ss, a->q_sh)) return 10;
  if (make_qkv_map(&tk, a->k, a->B, a->S, a->Hkv, a->k_sb, a->k_ss, a->k_sh)) return 11;
  if (make_qkv_map(&tv, a->v, a->B, a->S, a->Hkv, a->v_sb, a->v_ss, a->v_sh)) return 12;
  AttnParams p = {};
  p.B = a->B; p.S = a->S; p.H = a->H; p.Hkv = a->Hkv;
  p.causal = a->causal; p.window = a->window; p.scale = a->scale;
  p.doc_start = a->doc_start; p.doc_end = a->doc_end;
  p.O = (__nv_bfloat16*)a->o; p.lse = a->lse; p.status = a->status;
  if (ensure_dyn_smem<attn_fwd_kernel>(FWD_SMEM)) return 20;
  dim3 grid(((a->S + 127) / 128 + 1) / 2, a->H, a->B);
  attn_fwd_kernel<<<grid, FWD_THREADS, FWD_SMEM, (cudaStream_t)stream>>>(tq, tk, tv, p);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}

// Needs a->delta ([B,H,S] fp32) and a->dq_acc ([B,S,H,128] fp32) as scratch; dq_acc is cleared here.
extern "C" int lb_attn_bwd(const LbAttnArgs* a, void* stream) {
  if (a->D != 128) return 1;
  if (a->H % a->Hkv) return 2;
  if (a->doc_start && !a->causal) return 3;
  if (!a->delta || !a->dq_acc || !a->lse) return 4;
  if (a->B <= 0 || a->S <= 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  CUtensorMap tq, tk, tv, tdo, tdq;
  // dq_acc [B, S, H, 128] fp32, reduced into in boxes of 32 columns (one 128-byte swizzle row) x 128 rows
  if (make_tmap_4d(&tdq, a->dq_acc, 4, 128, a->S, (long long)a->H * 128, a->H, 128, a->B, (long long)a->S * a->H * 128,
                   32, 128))
    return 14;
  if (make_qkv_map(&tq, a->q, a->B, a->S, a->H, a->q_sb, a->q_ss, a->q_sh)) return 10;
  if (make_qkv_map(&tk, a->k, a->B, a->S, a->Hkv, a->k_sb, a->k_ss, a->k_sh)) return 11;
  if (make_qkv_map(&tv, a->v, a->B, a->S, a->Hkv, a->v_sb, a->v_ss, a->v_sh)) return 12;
  if (make_qkv_map(&tdo, a->dout, a->B, a->S, a->H, (long long)a->S * a->H * 128, (long long)a->H * 128, 128)) return 13;
  const long long rows = (long long)a->B * a->S * a->H;
  attn_delta_kernel<<<(unsigned)((rows * 32 + 255) / 256), 256, 0, st>>>(
      (const __nv_bfloat16*)a->o, (const __nv_bfloat16*)a->dout, a->delta, a->B, a->S, a->H);
  if (cudaMemsetAsync(a->dq_acc, 0, rows * 128 * sizeof(float), st) != cudaSuccess) return 21;
  AttnParams p = {};
  p.B = a->B; p.S = a->S; p.H = a->H; p.Hkv = a->Hkv;
  p.causal = a->causal; p.window = a->window; p.scale = a->scale;
  p.doc_start = a->doc_start; p.doc_end = a->doc_end;
  p.lse = a->lse; p.delta = a->delta; p.dq_acc = a->dq_acc;
  p.dk = (__nv_bfloat16*)a->dk; p.dv = (__nv_bfloat16*)a->dv;
  p.k_sb = a->k_sb; p.k_ss = a->k_ss; p.k_sh = a->k_sh;
  p.v_sb = a->v_sb; p.v_ss = a->v_ss; p.v_sh = a->v_sh;
  p.status = a->status;
  if (ensure_dyn_smem<attn_bwd_kernel>(BWD_SMEM)) return 20;
  dim3 grid((a->S + 127) / 128, a->Hkv, a->B);
  attn_bwd_kernel<<<grid, BWD_THREADS, BWD_SMEM, st>>>(tq, tk, tv, tdo, tdq, p);
  long long total = rows * 16;
  int blocks = (int)((total + 255) / 256 < (long long)num_sms() * 8 ? (total + 255) / 256 : (long long)num_sms() * 8);
  attn_dq_store_kernel<<<blocks, 256, 0, st>>>(a->dq_acc, (__nv_bfloat16*)a->dq, a->B, a->S, a->H, a->q_sb, a->q_ss, a->q_sh);
  g_launches.fetch_add(4, std::memory_order_relaxed);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}

// ---------------------------------------------------------------------------------------------
// Attention backward for callers that must not allocate device memory (see lingua_b200.h).
// The two scratch buffers of lb_attn_bwd live in one fixed array inside the library image.
namespace lb {
constexpr long long NOALLOC_MAX_ROWS = 65536;  // B * S * H
constexpr int NOALLOC_MAX_DEVICES = 64;
// [0, ROWS*128): dQ accumulator; [ROWS*128, ROWS*129): per-row delta. 33,816,576 bytes per GPU.
static __device__ __align__(256) float g_attn_bwd_scratch[NOALLOC_MAX_ROWS * 129];
// Device address of the array for each device that has been set up (the symbol itself is only a
// host-side handle and must never be handed to a kernel).
static float* g_attn_bwd_scratch_addr[NOALLOC_MAX_DEVICES] = {nullptr};
}  // namespace lb

extern "C" long long lb_attn_bwd_noalloc_max_rows(void) { return lb::NOALLOC_MAX_ROWS; }

extern "C" int lb_attn_bwd_noalloc(const LbAttnArgs* a, void* stream) {
  using namespace lb;
  if (!a) return 1;
  const long long rows = (long long)a->B * a->S * a->H;
  if (a->B < 0 || a->S < 0 || a->H < 0 || rows > NOALLOC_MAX_ROWS) return 30;  // beyond the fixed scratch
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= NOALLOC_MAX_DEVICES) return 31;
  if (!g_attn_bwd_scratch_addr[dev]) {
    // once per device, with that device current: resolve the array's address on this device
    float* p = nullptr;
    if (cudaGetSymbolAddress((void**)&p, g_attn_bwd_scratch) != cudaSuccess || !p) return 32;
    g_attn_bwd_scratch_addr[dev] = p;
  }
  LbAttnArgs b = *a;
  b.dq_acc = g_attn_bwd_scratch_addr[dev];
  b.delta = g_attn_bwd_scratch_addr[dev] + NOALLOC_MAX_ROWS * 128;
  return lb_attn_bwd(&b, stream);  // clears dq_acc with a memset on `stream`, then launches
}

#ifdef LB_ATTN_TRACE
extern "C" int lb_attn_trace_read(long long* host, int n) {
  if (n > 4096) n = 4096;
  return (int)cudaMemcpyFromSymbol(host, lb::g_attn_trace, sizeof(long long) * n);
}
#endif
