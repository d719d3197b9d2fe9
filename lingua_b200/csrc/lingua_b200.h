// C ABI of liblingua_b200.so. Every entry point takes raw device pointers and a CUDA
// stream (as void*), launches asynchronously on that stream and returns 0 on success or a
// small positive error code for a rejected argument / failed launch. Python binds these
// with ctypes (lingua_b200/ops/_lib.py).
#pragma once
#include <stdint.h>
#ifdef __cplusplus
#include <atomic>
extern "C" {
#endif

enum { LB_BF16 = 0, LB_F32 = 1, LB_E4M3 = 2, LB_E5M2 = 3 };

// C[b0,b1] (+)= alpha * A[b0,b1] * B[b0,b1]^T with A: M x K, B: N x K.
// a_major / b_major: 0 = K contiguous (lda/ldb = stride between rows of M resp. N),
//                    1 = M resp. N contiguous (lda/ldb = stride between consecutive k).
// All strides are in elements. Batch strides are ignored for a batch extent of 1.
typedef struct LbGemmArgs {
  const void* A;
  const void* B;
  void* C;
  uint32_t* status;  // device word, OR'ed with an error code if a wait times out (may be NULL)
  int M, N, K;
  int a_major, b_major;
  int in_dtype, out_dtype;  // LB_*
  int accumulate;           // fp32 output only: C += result
  int nb0, nb1;
  int force_bn;             // 0 = automatic, 128 or 256
  float alpha;
  long long lda, ldb, ldc;
  long long a_bs0, a_bs1, b_bs0, b_bs1, c_bs0, c_bs1;
} LbGemmArgs;

int lb_gemm(const LbGemmArgs* args, void* stream);

// Flash attention, head_dim 128. q/k/v (and dq/dk/dv, which use the same strides) are
// [B,S,H,128] views given by element strides; o and dout are contiguous [B,S,H,128].
// lse: [B,H,S] fp32. doc_start / doc_end: [B*S] int32 or NULL (block-causal masking).
// Backward scratch, supplied by the caller: delta [B,H,S] fp32, dq_acc [B,S,H,128] fp32.
typedef struct LbAttnArgs {
  const void *q, *k, *v;
  void* o;
  float* lse;
  const void* dout;
  void *dq, *dk, *dv;
  float* delta;
  float* dq_acc;
  const int* doc_start;
  const int* doc_end;
  uint32_t* status;
  int B, S, H, Hkv, D;
  int causal, window;
  float scale;
  long long q_sb, q_ss, q_sh, k_sb, k_ss, k_sh, v_sb, v_ss, v_sh;
} LbAttnArgs;
int lb_attn_fwd(const LbAttnArgs* a, void* stream);
int lb_attn_bwd(const LbAttnArgs* a, void* stream);

// lb_attn_bwd for hosts that cannot allocate device memory at call time -- for example a
// serving or training process that has handed every byte of the GPU to its own arena, or a
// latency-critical loop that cannot afford the device-wide synchronisation a cudaMalloc /
// cudaFree implies. This entry point has no counterpart in the reference implementation.
//
// Same arguments and results as lb_attn_bwd, except that a->delta and a->dq_acc are ignored:
// the scratch comes from a fixed array compiled into the library (about 32.3 MB, resident on
// every GPU that loads the library until the process exits). It allocates nothing: no
// cudaMalloc / cudaFree, no allocating library call. Limits and rules:
//   * B * S * H must not exceed lb_attn_bwd_noalloc_max_rows() (65536); larger problems are
//     rejected with return code 30 and nothing is launched.
//   * The first call on each device looks up the array's device address (with that device
//     current). Make that first call outside any stream capture.
//   * `stream` must belong to the device that is current when the call is made: the scratch
//     address is chosen by the current device, not by the stream.
//   * All calls on one GPU share the array. Each call clears the part that must start at zero
//     on its own stream, but two calls that overlap in time on the same GPU (different streams,
//     threads or processes sharing the context) race on it: serialise them.
int lb_attn_bwd_noalloc(const LbAttnArgs* a, void* stream);
long long lb_attn_bwd_noalloc_max_rows(void);

// Float8 linear layers (gemm_fp8.cu). C[m,n] = (A8[m,:] . B8[n,:]) * row_scale[m] * col_scale[n];
// A8 [M, K], B8 [N, K] e4m3 with K contiguous (lda, ldb, K multiples of 16), scales fp32 or NULL.
typedef struct LbGemmFp8Args {
  const void* A;
  const void* B;
  void* C;
  const float* row_scale;
  const float* col_scale;
  uint32_t* status;
  int M, N, K;
  int out_dtype;  // LB_BF16 or LB_F32
  long long lda, ldb, ldc;
  int a_fmt, b_fmt;  // 0 = e4m3, 1 = e5m2 (the reference's choice for gradients is configurable the same way)
} LbGemmFp8Args;
int lb_gemm_fp8(const LbGemmFp8Args* a, void* stream);
// x bf16 [rows, K] (row pitch ldx) -> out e4m3 [rows, K] (pitch ldo bytes), scale[r] = max(amax_r, 1e-12) / 448.
int lb_quant_rows(const void* x, long long ldx, long long rows, int K, void* out, long long ldo, float* scale,
                  void* stream);
// Same with the target format chosen: fmt 0 = e4m3 (largest value 448), 1 = e5m2 (57344).
int lb_quant_rows_fmt(const void* x, long long ldx, long long rows, int K, void* out, long long ldo, float* scale,
                      int fmt, void* stream);
// w bf16 [N, K] contiguous -> out e4m3 [K, N] (pitch ldo bytes), every element divided by *scale (device fp32).
int lb_quant_transpose(const void* w, int N, int K, const float* scale, void* out, long long ldo, void* stream);

// Tensor-parallel GEMM with the collective fused in (bf16, K-contiguous operands, head of
// gemm_tp.cu for the algorithm). `world` ranks, this one is `rank`; M is the row count of the
// whole problem and must be a multiple of 128 * world; K % 64 == 0, N % 8 == 0.
//   mode 1: C[M, N] = gather(a_peers[r] : [M/world, K] contiguous) * B[N, K]^T. a_peers[] are
//           peer-visible addresses of every rank's slab (own included); gather is a local
//           [M, K] bf16 buffer, flags a local uint32 array of M/128 + 1 words (world > 1 only).
//   mode 2: partial = A[M, K] * B[N, K]^T; rows of owner o are stored into
//           c_peers[o] + rank * slot_stride (row pitch ldc), i.e. every rank's staging buffer
//           has one [M/world, N] slot per source rank.
// The kernel never waits on another GPU; order the ranks with lb_peer_barrier.
#define LB_MAX_PEERS 8
typedef struct LbTpGemmArgs {
  int mode;
  int world, rank;
  int M, N, K;
  float alpha;
  const void* B;
  long long ldb;
  uint32_t* status;
  // mode 1
  const void* a_peers[LB_MAX_PEERS];
  void* gather;
  uint32_t* flags;
  void* C;
  long long ldc;  // row pitch of C (mode 1) or of a staging slot (mode 2)
  // mode 2
  const void* A;
  long long lda;
  void* c_peers[LB_MAX_PEERS];
  long long slot_stride;
  // 0: B is [N, K] with K contiguous (ldb = row pitch); 1: B is stored [K, N] with N contiguous (ldb = pitch between
  // consecutive k), which is how a weight [out, in] enters the products of its backward pass without a transpose
  int b_major;
} LbTpGemmArgs;
int lb_gemm_tp(const LbTpGemmArgs* a, void* stream);

// Weight-gradient GEMM with the reduce-scatter's transfer fused into its epilogue (gemm2.cu): the product
// args->A * args->B^T (bf16 operands, fp32 result, no batching; args->C is ignored) is not written to one
// local matrix; its rows belong to the ranks of a data-parallel group in blocks of 128 rows. `blocks` holds
// one (owner, destination row) pair of ints per 128-row block of M; rows of owner o go to the matrix at dst[o]
// (dst_rows[o] rows of N floats, row pitch args->ldc), a peer-visible address when o is another rank -- usually
// this rank's slot in o's staging area, and this rank's own gradient shard for o == rank. args->accumulate adds
// to the destination (TMA reduction) instead of overwriting it. m_rot: index of the 256-row tile the walk over
// M starts at (the first rows that have to travel). The kernel waits on no other GPU: order the ranks with
// lb_peer_barrier before the destinations are read and before they are written again.
typedef struct LbScatterArgs {
  int world;
  int m_rot;
  const int* blocks;
  void* dst[LB_MAX_PEERS];
  long long dst_rows[LB_MAX_PEERS];
} LbScatterArgs;
int lb_gemm_scatter(const LbGemmArgs* args, const LbScatterArgs* sc, void* stream);

// Forward GEMM with the parameter all-gather fused in (gemm2.cu): C[M, N] = A[M, K] * B[N, K]^T (bf16, both
// K-contiguous) where B is this rank's copy of a weight matrix whose 128-row blocks are owned by the ranks of a
// data-parallel group. Only the own blocks of the local copy are current when the call is made; the kernel pulls
// every other block out of its owner's copy (b_peers[owner], the same matrix in that rank's peer-visible buffer) into
// the local one while it multiplies, own blocks first, and leaves the local copy complete for later kernels.
//   n_order        [ceil(N / 256)] column tiles in the order they are computed (device)
//   remote_blocks  n_remote (block, owner) int pairs in the order they are pulled (device)
//   flags_init     [N / 128 + 1] uint32: K / 64 for own blocks, 0 for remote ones, 0 for the trailing counter (device)
//   flags          workspace of the same size, overwritten by every call (device)
// N % 128 == 0, K % 64 == 0, ldb == K. The owners' copies must be final before the call (lb_peer_barrier) and
// must not change before every reader has finished.
typedef struct LbGatherArgs {
  int world, rank;
  int n_remote;
  const int* n_order;
  const int* remote_blocks;
  const uint32_t* flags_init;
  uint32_t* flags;
  const void* b_peers[LB_MAX_PEERS];
} LbGatherArgs;
int lb_gemm_gather(const LbGemmArgs* args, const LbGatherArgs* ga, void* stream);

// Grouped products on the SM-pair kernel: one launch for a bank of matrices, with the grouping read from device
// memory (no host copy of group sizes). bf16 operands, no batch dims in `args` (nb0 = nb1 = 1).
//   mode 1, grouped rows: C[m, :] = A[m, :] x B_g^T with g = sel[m / 256]: every 256-row tile of A uses the
//           matrix of its group; B_g = args->B + g * group_stride elements (K- or N-contiguous as args->b_major
//           says). Callers lay rows out group by group, each group padded to a multiple of 256 rows.
//           sel = -1 marks a row tile without rows: it is skipped and its output rows are left untouched.
//   mode 2, grouped contraction: C_g = A[:, rows_g]^T-style product over a range of K only:
//           C_g (+)= sum over k in [sel[2g], sel[2g] + 64 * sel[2g+1]) of A[k, m] B[k, n], C_g = args->C +
//           g * group_stride elements; a_major = b_major = 1 (K is the row index of both operands). A group with
//           zero blocks writes zeros (adds nothing when args->accumulate).
// sel is int32 device memory: [ceil(M / 256)] in mode 1, [n_groups][2] in mode 2; group indices are checked
// against n_groups in the kernel (out of range: status word, tile computed with group 0).
typedef struct LbGroupArgs {
  int mode;
  int n_groups;
  long long group_stride;
  const int* sel;
} LbGroupArgs;
int lb_gemm_grouped(const LbGemmArgs* args, const LbGroupArgs* gr, void* stream);

// Barrier over the ranks of a group. pads[r] is the peer-visible address of rank r's pad
// (uint32[world], zero before first use); epoch is the number of this barrier on these pads,
// counted from 1 by every rank alike. Bounded wait: on timeout the status word is set.
int lb_peer_barrier(void* const* pads, int world, int rank, uint32_t epoch, uint32_t* status, void* stream);
// Same with the wait limit given in nanoseconds (the default is 2 s).
int lb_peer_barrier_limit(void* const* pads, int world, int rank, uint32_t epoch, uint32_t* status,
                          unsigned long long limit_ns, void* stream);
// out[i] = scale * (own[i] + sum_s slots[s * slot_stride + i]), *sumsq += sum out[i]^2 (fp32, n elements):
// the reduction half of a reduce-scatter whose slots were filled by peer copies.
int lb_reduce_slots(const float* own, const float* slots, int n_slots, long long slot_stride, float* out,
                    long long n, float scale, float* sumsq, void* stream);
// Same with the grid capped at max_blocks blocks of 256 threads (0 = default): a small grid lets the reduction trickle
// beside compute kernels instead of competing with them.
int lb_reduce_slots_grid(const float* own, const float* slots, int n_slots, long long slot_stride, float* out,
                         long long n, float scale, float* sumsq, int max_blocks, void* stream);

// dst[i] += src[i] (fp32, n elements) with reductions that are atomic at the destination, which may be peer memory.
int lb_red_add(float* dst, const float* src, long long n, void* stream);

// out[i] = scale * sum_r srcs[r][i], *sumsq += sum out[i]^2 (fp32, n elements, n_src <= LB_MAX_PEERS): a
// reduce-scatter without staging. srcs[r] is this rank's slice inside rank r's buffer (peer-visible addresses,
// read with plain loads); order the ranks with lb_peer_barrier before (sources final) and after (readers done).
int lb_reduce_peers(const void* const* srcs, int n_src, float* out, long long n, float scale, float* sumsq,
                    void* stream);

// h = resid + sum_s slots[s] (bf16 [rows, D] each, slot_stride elements apart), y = RMSNorm(h) * w.
// resid, h_out, y_out (with w) and rstd_out are optional. D % 8 == 0, D <= 8192.
int lb_reduce_norm(const void* slots, int n_slots, long long slot_stride, const void* resid, const void* w,
                   float eps, void* h_out, void* y_out, float* rstd_out, long long rows, int D, void* stream);

// Decoding-step and gate kernels of the recurrent models (recurrent_step.cu). bf16 tensors unless noted.
// conv1d_update: x [N, C] (row pitch ldx), state [N, C, W] updated in place (window shifted, x appended),
//   w [C, W], out [N, C] (row pitch ldo) = (SiLU of) the weighted window. W in {2, 3, 4}.
int lb_conv1d_update(const void* x, long long ldx, void* state, const void* w, void* out, long long ldo, int N, int C,
                     int W, int act, void* stream);
// conv_states: x [T, C] packed documents (row pitch ldx), document d covers rows [starts[d], ends[d]) (int64 on the
//   device); out [n_docs, C, W] = the last W inputs of every document, zero where the document is shorter.
int lb_conv_states(const void* x, long long ldx, const long long* starts, const long long* ends, void* out, int n_docs,
                   int C, int W, void* stream);
// ssm_state_update: state fp32 [n, H, P, N] in place: state = exp(dt A) state + dt x B^T; y [n, H, P] = state . C
//   (+ D x). x [n, H*P] (pitch ldx), dt fp32 [n, H], A fp32 [H], B / C [n, G, N] (pitches ldb / ldc), D fp32 [H] or
//   [H, P] (d_has_p) or NULL. N % 4 == 0.
int lb_ssm_state_update(float* state, const void* x, long long ldx, const float* dt, const float* A, const void* B,
                        long long ldb, const void* Cm, long long ldc, const float* D, int d_has_p, void* y, int nseq,
                        int H, int P, int N, int G, void* stream);
// rnn_step: state fp32 [n] = a * state + b; out = bf16(state).
int lb_rnn_step(const void* a, const void* b, float* state, void* out, long long n, void* stream);
// RG-LRU gates on contiguous [rows, C] tensors (C % 8 == 0), sp = softplus(lambda) per channel (fp32 [C]):
//   a = exp(-8 sigmoid(ga) sp), b = sqrt(1 - a^2) sigmoid(gx) x. The backward also accumulates d sp into dsp (fp32 [C]).
int lb_rglru_gates_fwd(const void* gx, const void* ga, const void* x, const float* sp, void* a_out, void* b_out,
                       long long rows, int C, void* stream);
int lb_rglru_gates_bwd(const void* gx, const void* ga, const void* x, const float* sp, const void* da, const void* db,
                       void* dgx, void* dga, void* dx, float* dsp, long long rows, int C, void* stream);

// Number of kernels launched by this library in this process so far.
long long lb_launch_count(void);
void lb_launch_count_add(long long n);

#ifdef __cplusplus
}
#include <cuda.h>
#include <cuda_runtime.h>
namespace lb {
extern std::atomic<long long> g_launches;
int num_sms();
struct LbGemmArgsFwd;
// 4-D TMA map {inner, outer, batch0, batch1} with the 128-byte swizzle; strides in elements.
int make_tmap_4d(CUtensorMap* out, const void* base, int esz, long long inner, long long outer,
                 long long ld, int nb0, long long bs0, int nb1, long long bs1, int box_inner,
                 int box_outer);
// Opt a kernel in to `bytes` of dynamic shared memory. The attribute belongs to the (function, device) pair,
// so it is set once per device that launches the kernel, with that device current. Returns 0 on success.
template <auto Kern>
int ensure_dyn_smem(int bytes) {
  static bool done[64] = {};
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 1;
  if (!done[dev]) {
    if (cudaFuncSetAttribute(Kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess) return 2;
    done[dev] = true;
  }
  return 0;
}
// two-SM (cta_group::2) 256 x 256-tile variant, gemm2.cu
int gemm2_dispatch(const LbGemmArgs& a, cudaStream_t s);
int gemm2_fp8_dispatch(const LbGemmFp8Args& a, cudaStream_t s);
}
#endif
