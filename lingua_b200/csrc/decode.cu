// Single-token decode attention over a packed KV cache, head_dim 128.
//
// Every sequence of a generation batch owns a contiguous span of cache slots
// [start[i], start[i] + len[i]); a query token attends to exactly that span, so no dense
// (n_seqs x cache) mask is built (apps/main/generate.py:299-320 builds one and calls SDPA).
// The new token's K and V are appended to the cache by the same kernel before it attends.
//
// grid (n_seqs, n_heads); 4 warps stride over the keys, each lane owns 4 of the 128 channels,
// per-warp online softmax, merged through shared memory at the end.
#include "common.cuh"
#include "lingua_b200.h"

namespace lb {

__global__ void __launch_bounds__(128) decode_attn_kernel(
    const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_new,
    const __nv_bfloat16* __restrict__ v_new, __nv_bfloat16* __restrict__ k_cache,
    __nv_bfloat16* __restrict__ v_cache, const int* __restrict__ start, const int* __restrict__ len,
    __nv_bfloat16* __restrict__ out, int H, int Hkv, long long q_stride, long long kv_new_stride, float scale) {
  const int seq = blockIdx.x, h = blockIdx.y;
  const int hk = h / (H / Hkv);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int s0 = start[seq];
  const int n = len[seq];  // keys visible to this query, the new token included
  const long long row = (long long)Hkv * 128;
  // append the new token (one block per kv head does it: the first query head of the group)
  if (k_new && h % (H / Hkv) == 0 && warp == 0) {
    const long long dst = (long long)(s0 + n - 1) * row + hk * 128 + lane * 4;
    const long long src = (long long)seq * kv_new_stride + hk * 128 + lane * 4;
    *reinterpret_cast<uint2*>(k_cache + dst) = *reinterpret_cast<const uint2*>(k_new + src);
    *reinterpret_cast<uint2*>(v_cache + dst) = *reinterpret_cast<const uint2*>(v_new + src);
  }
  float qf[4];
  {
    const uint2 u = *reinterpret_cast<const uint2*>(q + (long long)seq * q_stride + h * 128 + lane * 4);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
    qf[0] = a.x * scale; qf[1] = a.y * scale; qf[2] = b.x * scale; qf[3] = b.y * scale;
  }
  float m = -INFINITY, l = 0.f, acc[4] = {0.f, 0.f, 0.f, 0.f};
  const int last = n - 1;
  for (int j = warp; j < n; j += 4) {
    uint2 ku, vu;
    if (j == last && k_new) {  // not yet visible through the cache for the other blocks of the group
      const long long src = (long long)seq * kv_new_stride + hk * 128 + lane * 4;
      ku = *reinterpret_cast<const uint2*>(k_new + src);
      vu = *reinterpret_cast<const uint2*>(v_new + src);
    } else {
      const long long off = (long long)(s0 + j) * row + hk * 128 + lane * 4;
      ku = *reinterpret_cast<const uint2*>(k_cache + off);
      vu = *reinterpret_cast<const uint2*>(v_cache + off);
    }
    const float2 k0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&ku.x));
    const float2 k1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&ku.y));
    float s = qf[0] * k0.x + qf[1] * k0.y + qf[2] * k1.x + qf[3] * k1.y;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xFFFFFFFFu, s, o);
    const float m_new = fmaxf(m, s);
    const float corr = __expf(m - m_new), p = __expf(s - m_new);
    const float2 v0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&vu.x));
    const float2 v1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&vu.y));
    acc[0] = acc[0] * corr + p * v0.x;
    acc[1] = acc[1] * corr + p * v0.y;
    acc[2] = acc[2] * corr + p * v1.x;
    acc[3] = acc[3] * corr + p * v1.y;
    l = l * corr + p;
    m = m_new;
  }
  __shared__ float sm_m[4], sm_l[4], sm_acc[4][128];
  if (lane == 0) { sm_m[warp] = m; sm_l[warp] = l; }
#pragma unroll
  for (int i = 0; i < 4; ++i) sm_acc[warp][lane * 4 + i] = acc[i];
  __syncthreads();
  if (warp == 0) {
    float M = fmaxf(fmaxf(sm_m[0], sm_m[1]), fmaxf(sm_m[2], sm_m[3]));
    float L = 0.f, o[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float c = sm_m[w] == -INFINITY ? 0.f : __expf(sm_m[w] - M);
      L += sm_l[w] * c;
#pragma unroll
      for (int i = 0; i < 4; ++i) o[i] += sm_acc[w][lane * 4 + i] * c;
    }
    const float inv = L > 0.f ? 1.f / L : 0.f;
    uint2 u;
    u.x = pack_bf16(o[0] * inv, o[1] * inv);
    u.y = pack_bf16(o[2] * inv, o[3] * inv);
    *reinterpret_cast<uint2*>(out + ((long long)seq * H + h) * 128 + lane * 4) = u;
  }
}

}  // namespace lb

// q: [n_seqs, H, 128] (row stride q_stride), k_new / v_new: [n_seqs, Hkv, 128] (row stride
// kv_new_stride) or NULL when the cache already holds the token; caches: [slots, Hkv, 128];
// start / len: int32 [n_seqs]; out: [n_seqs, H, 128] contiguous.
extern "C" int lb_decode_attn(const void* q, const void* k_new, const void* v_new, void* k_cache, void* v_cache,
                              const int* start, const int* len, void* out, int n_seqs, int H, int Hkv, int D,
                              long long q_stride, long long kv_new_stride, float scale, void* stream) {
  using namespace lb;
  if (D != 128 || H % Hkv) return 1;
  if (n_seqs <= 0) return 0;
  dim3 grid(n_seqs, H);
  decode_attn_kernel<<<grid, 128, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_new, (const __nv_bfloat16*)v_new, (__nv_bfloat16*)k_cache,
      (__nv_bfloat16*)v_cache, start, len, (__nv_bfloat16*)out, H, Hkv, q_stride, kv_new_stride, scale);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}
