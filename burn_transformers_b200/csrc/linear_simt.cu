// out[M,N] = act(A[M,K] @ W + bias) (+ residual), accumulated in 32-bit with plain fused
// multiply-adds (no tensor cores, no reduced-precision matrix mode).  This is the matrix
// product of the true 32-bit path and the fallback for shapes the tensor-core kernels refuse.
// W is either [K,N] with N contiguous (a Conv1D weight as stored) or [N,K] with K contiguous
// (an embedding table used as a tied readout).  Every output element is one sequential sum over
// k, so a row's result does not depend on which other rows are in the call.
#include "common.cuh"

namespace bt {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

template <typename TIn, typename TOut, bool W_IS_NK>
__global__ void __launch_bounds__(256)
linear_simt_kernel(const TIn* __restrict__ A, const TIn* __restrict__ W, const float* __restrict__ bias,
                   const float* residual, TOut* out, int M, int N, int K, int act) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Bs[BK][BN + 4];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
    {  // A tile: thread -> row tid/4, four consecutive k
      const int r = tid >> 2, kq = (tid & 3) * 4;
      const int gm = m0 + r;
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int gk = k0 + kq + u;
        As[kq + u][r] = (gm < M && gk < K) ? to_float(A[(long long)gm * K + gk]) : 0.f;
      }
    }
    if (W_IS_NK) {  // thread -> n tid/4, four consecutive k
      const int c = tid >> 2, kq = (tid & 3) * 4;
      const int gn = n0 + c;
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int gk = k0 + kq + u;
        Bs[kq + u][c] = (gn < N && gk < K) ? to_float(W[(long long)gn * K + gk]) : 0.f;
      }
    } else {  // thread -> k tid/16, four consecutive n
      const int kr = tid >> 4, nq = (tid & 15) * 4;
      const int gk = k0 + kr;
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int gn = n0 + nq + u;
        Bs[kr][nq + u] = (gn < N && gk < K) ? to_float(W[(long long)gk * N + gn]) : 0.f;
      }
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[TM], b[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) b[j] = Bs[kk][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int gm = m0 + ty * TM + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int gn = n0 + tx * TN + j;
      if (gn >= N) continue;
      float v = acc[i][j];
      if (bias) v += bias[gn];
      v = apply_activation(v, act);
      if (residual) v += residual[(long long)gm * N + gn];
      out[(long long)gm * N + gn] = from_float<TOut>(v);
    }
  }
}

template <typename TIn, typename TOut>
static void launch(const void* A, const void* W, const float* bias, const float* residual, void* out, int M, int N,
                   int K, int w_is_nk, int act, cudaStream_t stream) {
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  if (w_is_nk)
    linear_simt_kernel<TIn, TOut, true><<<grid, 256, 0, stream>>>((const TIn*)A, (const TIn*)W, bias, residual,
                                                                  (TOut*)out, M, N, K, act);
  else
    linear_simt_kernel<TIn, TOut, false><<<grid, 256, 0, stream>>>((const TIn*)A, (const TIn*)W, bias, residual,
                                                                   (TOut*)out, M, N, K, act);
}

}  // namespace bt

// in_dtype: type of A and W.  out_dtype: type of out (32-bit when it is the residual stream or logits).
extern "C" int bt_linear_simt(const void* A, const void* W, const float* bias, const float* residual, void* out,
                              int M, int N, int K, int w_is_nk, int act, int in_dtype, int out_dtype,
                              cudaStream_t stream) {
  using namespace bt;
  BT_CHECK(M >= 0 && N > 0 && K > 0, "linear: bad sizes M=%d N=%d K=%d", M, N, K);
  BT_CHECK(act >= 0 && act <= 2, "linear: unknown activation %d", act);
  BT_CHECK((long long)((M + BM - 1) / BM) <= 65535, "linear: M=%d needs more than 65535 row tiles", M);
  BT_CHECK(!(residual && out_dtype != kF32), "linear: a residual needs a 32-bit output");
  if (M == 0) return 0;
  if (in_dtype == kF32 && out_dtype == kF32)
    launch<float, float>(A, W, bias, residual, out, M, N, K, w_is_nk, act, stream);
  else if (in_dtype == kBF16 && out_dtype == kF32)
    launch<__nv_bfloat16, float>(A, W, bias, residual, out, M, N, K, w_is_nk, act, stream);
  else if (in_dtype == kBF16 && out_dtype == kBF16)
    launch<__nv_bfloat16, __nv_bfloat16>(A, W, bias, residual, out, M, N, K, w_is_nk, act, stream);
  else
    return fail("linear: unsupported dtypes in=%d out=%d", in_dtype, out_dtype);
  BT_LAUNCH_OK("linear_simt");
  return 0;
}
