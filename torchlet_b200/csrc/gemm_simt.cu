// Plain CUDA-core matrix product  out[M, N] (+)= x[M, K] . w[N, K]^T + bias[N].
//
// This is the true 32-bit path (float operands, IEEE fused multiply-add, no tensor
// cores, no reduced-precision mode) and the any-size path for bfloat16 operands
// that the tensor-core kernels refuse.  Each output element is the sum over k in
// ascending order of x[m, k] * w[n, k]: the order depends on K alone, so a row's
// result does not depend on which other rows are in the batch.
//
// Reference counterparts: nn.Linear in v10_triton_paged_gqa/layer/gqa.py:122-124,84
// and model/qwen2_5.py:83-87; down_kernel / swiglu_kernel GEMMs in
// v10_triton_paged_gqa/kernel/ffn_swiglu.py:5-164.
#include "common.cuh"

namespace {

using namespace tl;

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

template <typename T, typename OutT, bool ACCUM>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const T* __restrict__ x, const T* __restrict__ w, const float* __restrict__ bias,
                 OutT* __restrict__ out, int M, int N, int K, int ldx, int ldw, int ldo) {
  tl::pdl_wait();               // everything before us in the stream is complete and visible
  tl::pdl_launch_dependents();  // the next kernel may start its own prologue

  __shared__ float xs[BK][BM + 1];
  __shared__ float ws[BK][BN + 1];
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int tx = tid % 16, ty = tid / 16;  // 16 x 16 threads, each TM x TN outputs
  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
    // 64 rows x 16 k-values per operand, 4 per thread
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int e = tid + i * 256;
      const int r = e / BK, c = e % BK;
      const int k = k0 + c;
      float xv = 0.f, wv = 0.f;
      if (k < K) {
        if (m0 + r < M) xv = to_float(x[(size_t)(m0 + r) * ldx + k]);
        if (n0 + r < N) wv = to_float(w[(size_t)(n0 + r) * ldw + k]);
      }
      xs[c][r] = xv;
      ws[c][r] = wv;
    }
    __syncthreads();
#pragma unroll
    for (int c = 0; c < BK; ++c) {
      float xa[TM], wb[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) xa[i] = xs[c][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) wb[j] = ws[c][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(xa[i], wb[j], acc[i][j]);
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
      if (n >= N) continue;
      float v = acc[i][j];
      if (bias) v += bias[n];
      OutT* o = out + (size_t)m * ldo + n;
      if (ACCUM)
        *o = from_float<OutT>(to_float(*o) + v);
      else
        *o = from_float<OutT>(v);
    }
  }
}

template <typename T, typename OutT>
int launch(const void* x, const void* w, const float* bias, void* out, int accumulate, int M, int N,
           int K, int ldx, int ldw, int ldo, cudaStream_t stream) {
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  if (grid.y > 65535) return TL_ERR_UNSUPPORTED;
  if (accumulate)
    tl::launch_kernel(gemm_simt_kernel<T, OutT, true>, grid, 256, 0, stream, (const T*)x, (const T*)w, bias, (OutT*)out, M, N, K, ldx, ldw, ldo);
  else
    tl::launch_kernel(gemm_simt_kernel<T, OutT, false>, grid, 256, 0, stream, (const T*)x, (const T*)w, bias, (OutT*)out, M, N, K, ldx, ldw, ldo);
  return TL_LAUNCH_CHECK();
}

}  // namespace

extern "C" int tl_gemm_simt(const void* x, const void* w, int in_dtype, const float* bias, void* out,
                            int out_dtype, int accumulate, int M, int N, int K, int ldx, int ldw,
                            int ldo, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0) return TL_ERR_UNSUPPORTED;
  if (in_dtype == TL_DTYPE_F32) {
    if (out_dtype != TL_DTYPE_F32) return TL_ERR_UNSUPPORTED;
    return launch<float, float>(x, w, bias, out, accumulate, M, N, K, ldx, ldw, ldo, stream);
  }
  if (out_dtype == TL_DTYPE_F32)
    return launch<__nv_bfloat16, float>(x, w, bias, out, accumulate, M, N, K, ldx, ldw, ldo, stream);
  return launch<__nv_bfloat16, __nv_bfloat16>(x, w, bias, out, accumulate, M, N, K, ldx, ldw, ldo, stream);
}
