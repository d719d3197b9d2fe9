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

// Number of kernels launched by this library in this process so far.
long long lb_launch_count(void);
void lb_launch_count_add(long long n);

#ifdef __cplusplus
}
namespace lb {
extern std::atomic<long long> g_launches;
int num_sms();
}
#endif
