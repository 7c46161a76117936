// y = x W^T (+ bias) for any sizes, on CUDA cores, float32 accumulation in a fixed order.
//
// This is the whole linear layer of the true 32-bit path (no tensor-core mode of reduced
// precision anywhere), and the fallback of the bfloat16 path for shapes the tensor-core
// kernels refuse.  W is row-major [N][K] as stored in the file: y[m][n] = sum_k x[m][k] W[n][k]
// (stratum/native/stratum_linear.h:491-507).  Each output element is one chain of fused
// multiply-adds over k = 0..K-1, so its value does not depend on M, on the tile it falls in,
// or on what else is in the step.
//
// Epilogues: 0 store as T; 1 add into a float32 tensor in place (the residual stream);
//            2 store as float32 (logits).
#include "common.cuh"

#define LS_BM 64
#define LS_BN 64
#define LS_BK 16
#define LS_TM 4
#define LS_TN 4

template <typename T, int EPI>
__global__ void __launch_bounds__(256)
linear_simple_kernel(const T* __restrict__ x, const T* __restrict__ w, const float* __restrict__ bias,
                     void* __restrict__ out, int M, int N, int K, int ldx, int ldo) {
  __shared__ float xs[LS_BK][LS_BM + 1];
  __shared__ float ws[LS_BK][LS_BN + 1];
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * LS_BM, n0 = blockIdx.x * LS_BN;
  const int tm = (tid / 16) * LS_TM, tn = (tid % 16) * LS_TN;
  float acc[LS_TM][LS_TN];
#pragma unroll
  for (int i = 0; i < LS_TM; i++)
#pragma unroll
    for (int j = 0; j < LS_TN; j++) acc[i][j] = 0.f;

  // each thread loads 4 elements of each tile per step: row = tid / 4, k = (tid % 4) * 4 .. +3
  const int lr = tid / 4, lk = (tid % 4) * 4;
  for (int k0 = 0; k0 < K; k0 += LS_BK) {
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int k = k0 + lk + j;
      const int m = m0 + lr, n = n0 + lr;
      xs[lk + j][lr] = (m < M && k < K) ? to_float(x[(size_t)m * ldx + k]) : 0.f;
      ws[lk + j][lr] = (n < N && k < K) ? to_float(w[(size_t)n * K + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < LS_BK; kk++) {
      float a[LS_TM], b[LS_TN];
#pragma unroll
      for (int i = 0; i < LS_TM; i++) a[i] = xs[kk][tm + i];
#pragma unroll
      for (int j = 0; j < LS_TN; j++) b[j] = ws[kk][tn + j];
#pragma unroll
      for (int i = 0; i < LS_TM; i++)
#pragma unroll
        for (int j = 0; j < LS_TN; j++) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < LS_TM; i++) {
    const int m = m0 + tm + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < LS_TN; j++) {
      const int n = n0 + tn + j;
      if (n >= N) continue;
      float v = acc[i][j];
      if (bias) v += bias[n];
      const size_t o = (size_t)m * ldo + n;
      if (EPI == 0) ((T*)out)[o] = from_float<T>(v);
      else if (EPI == 1) ((float*)out)[o] += v;
      else ((float*)out)[o] = v;
    }
  }
}

template <typename T>
static int launch_linear_simple(const void* x, const void* w, const float* bias, void* out, int epilogue,
                                int M, int N, int K, int ldx, int ldo, cudaStream_t stream) {
  dim3 grid((N + LS_BN - 1) / LS_BN, (M + LS_BM - 1) / LS_BM);
  if (epilogue == 0)
    linear_simple_kernel<T, 0><<<grid, 256, 0, stream>>>((const T*)x, (const T*)w, bias, out, M, N, K, ldx, ldo);
  else if (epilogue == 1)
    linear_simple_kernel<T, 1><<<grid, 256, 0, stream>>>((const T*)x, (const T*)w, bias, out, M, N, K, ldx, ldo);
  else if (epilogue == 2)
    linear_simple_kernel<T, 2><<<grid, 256, 0, stream>>>((const T*)x, (const T*)w, bias, out, M, N, K, ldx, ldo);
  else
    return STRATUM_ERR_SHAPE;
  return launch_status();
}

// x: [M][ldx] T (first K columns used); w: [N][K] T; bias: float32 [N] or null; out: [M][ldo].
STRATUM_EXPORT int stratum_linear_simple(const void* x, const void* w, const float* bias, void* out, int dtype,
                                         int epilogue, int M, int N, int K, int ldx, int ldo,
                                         cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || ldx < K || ldo < N) return STRATUM_ERR_SHAPE;
  if ((M + LS_BM - 1) / LS_BM > 65535) return STRATUM_ERR_LIMIT;
  if (dtype == STRATUM_DT_F32) return launch_linear_simple<float>(x, w, bias, out, epilogue, M, N, K, ldx, ldo, stream);
  if (dtype == STRATUM_DT_BF16) return launch_linear_simple<bf16>(x, w, bias, out, epilogue, M, N, K, ldx, ldo, stream);
  return STRATUM_ERR_DTYPE;
}
