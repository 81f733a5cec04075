// LayerNorm over the last axis of 32-bit rows: statistics and normalisation in 32-bit,
// the result rounded once to the output type.  mean, then the mean of squared deviations
// (two passes, no E[x^2]-E[x]^2 cancellation).  `rows` (optional) picks the input rows.
#include "common.cuh"

namespace bt {

template <typename TOut, int THREADS>
__global__ void __launch_bounds__(THREADS)
layernorm_kernel(const float* __restrict__ x, const int* __restrict__ rows, const float* __restrict__ gamma,
                 const float* __restrict__ beta, TOut* __restrict__ out, int width, float eps) {
  __shared__ float scratch[33];
  extern __shared__ float row_cache[];  // width floats
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x;
  const float* src = x + (long long)(rows ? rows[r] : r) * width;
  float s = 0.f;
  for (int c = threadIdx.x; c < width; c += THREADS) {
    const float v = src[c];
    row_cache[c] = v;
    s += v;
  }
  const float mean = block_sum(s, scratch) / (float)width;
  float q = 0.f;
  for (int c = threadIdx.x; c < width; c += THREADS) {
    const float d = row_cache[c] - mean;
    q += d * d;
  }
  const float var = block_sum(q, scratch) / (float)width;
  const float rstd = 1.f / sqrtf(var + eps);
  TOut* dst = out + (long long)r * width;
  for (int c = threadIdx.x; c < width; c += THREADS) {
    float v = (row_cache[c] - mean) * rstd;
    v = v * gamma[c] + (beta ? beta[c] : 0.f);
    dst[c] = from_float<TOut>(v);
  }
}

}  // namespace bt

extern "C" int bt_layernorm(const float* x, const int* rows, const float* gamma, const float* beta, void* out,
                            int n_rows, int width, float eps, int out_dtype, cudaStream_t stream) {
  using namespace bt;
  BT_CHECK(n_rows >= 0 && width > 0, "layernorm: bad sizes rows=%d width=%d", n_rows, width);
  BT_CHECK(width <= 12000, "layernorm: width %d exceeds the supported 12000", width);
  if (n_rows == 0) return 0;
  constexpr int T = 256;
  const size_t smem = (size_t)width * sizeof(float);
  if (out_dtype == kF32)
    BT_PDL_OK("layernorm", launch_pdl(layernorm_kernel<float, T>, dim3(n_rows), dim3(T), smem, stream, 1, x, rows, gamma,
                                      beta, (float*)out, width, eps));
  else if (out_dtype == kBF16)
    BT_PDL_OK("layernorm", launch_pdl(layernorm_kernel<__nv_bfloat16, T>, dim3(n_rows), dim3(T), smem, stream, 1, x, rows,
                                      gamma, beta, (__nv_bfloat16*)out, width, eps));
  else
    return fail("layernorm: unknown dtype %d", out_dtype);
  return 0;
}
