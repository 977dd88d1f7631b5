// out[M,N] = x[M,K] * w[N,K]^T on the CUDA cores with 32-bit multiply-adds: the
// true 32-bit matrix product (no tensor-core mode of reduced precision), also
// usable with bfloat16 operands as the plain stand-in of the tensor-core kernel.
// Every output element is one chain of fused multiply-adds over k = 0..K-1 in
// order, so a row's result does not depend on which other rows are in the batch.
#include "api.h"
#include "common.cuh"

namespace {
constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

template <typename TX, typename TW, typename TO>
__global__ void __launch_bounds__(256) gemm_simt_kernel(TO* __restrict__ out, const TX* __restrict__ x,
                                                        const TW* __restrict__ w, int M, int N, int K, int ldx,
                                                        int ldw, int ldo) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float xs[BK][BM + 4];
  __shared__ float ws[BK][BN + 4];
  const int tid = threadIdx.x;
  const int tx = tid % 16, ty = tid / 16;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
    // each thread loads 4 elements of each tile: row = e / BK, k = e % BK
#pragma unroll
    for (int e = tid; e < BM * BK; e += 256) {
      const int r = e / BK, kk = e % BK;
      const int m = m0 + r, k = k0 + kk;
      xs[kk][r] = (m < M && k < K) ? to_f32(x[(size_t)m * ldx + k]) : 0.f;
    }
#pragma unroll
    for (int e = tid; e < BN * BK; e += 256) {
      const int r = e / BK, kk = e % BK;
      const int n = n0 + r, k = k0 + kk;
      ws[kk][r] = (n < N && k < K) ? to_f32(w[(size_t)n * ldw + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[TM], b[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = xs[kk][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) b[j] = ws[kk][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int m = m0 + ty * TM + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int n = n0 + tx * TN + j;
      if (n < N) out[(size_t)m * ldo + n] = from_f32<TO>(acc[i][j]);
    }
  }
}

template <typename TX, typename TW, typename TO>
int launch(void* out, const void* x, const void* w, int M, int N, int K, int ldx, int ldw, int ldo,
           cudaStream_t stream) {
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  zi_launch(gemm_simt_kernel<TX, TW, TO>, dim3(grid), dim3(256), 0, stream, (TO*)out, (const TX*)x, (const TW*)w, M, N, K, ldx, ldw, ldo);
  return zi_check_launch("gemm_simt");
}
}  // namespace

extern "C" int zi_gemm_simt(void* out, int out_dtype, const void* x, int x_dtype, const void* w, int w_dtype, int M,
                            int N, int K, int ldx, int ldw, int ldo, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0) return zi_refuse("gemm: K must be positive, got %d", K);
  using bf = __nv_bfloat16;
  const int key = x_dtype * 4 + w_dtype * 2 + out_dtype;
  switch (key) {
    case 0: return launch<float, float, float>(out, x, w, M, N, K, ldx, ldw, ldo, stream);
    case 1: return launch<float, float, bf>(out, x, w, M, N, K, ldx, ldw, ldo, stream);
    case 2: return launch<float, bf, float>(out, x, w, M, N, K, ldx, ldw, ldo, stream);
    case 3: return launch<float, bf, bf>(out, x, w, M, N, K, ldx, ldw, ldo, stream);
    case 4: return launch<bf, float, float>(out, x, w, M, N, K, ldx, ldw, ldo, stream);
    case 5: return launch<bf, float, bf>(out, x, w, M, N, K, ldx, ldw, ldo, stream);
    case 6: return launch<bf, bf, float>(out, x, w, M, N, K, ldx, ldw, ldo, stream);
    case 7: return launch<bf, bf, bf>(out, x, w, M, N, K, ldx, ldw, ldo, stream);
  }
  return zi_refuse("gemm: unknown dtype tags x=%d w=%d out=%d", x_dtype, w_dtype, out_dtype);
}

ZI_TRACE_SETTER(gemm_simt)
