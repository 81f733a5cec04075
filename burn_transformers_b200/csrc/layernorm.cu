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

// The same for many rows that are not long: a warp holds one row in registers (J vectors of four per lane), so the
// row is read once and nothing is handed over between warps.  width is a multiple of 4, at most 128 J.
template <typename TOut, int J>
__global__ void __launch_bounds__(256)
layernorm_rows_kernel(const float* __restrict__ x, const int* __restrict__ rows, const float* __restrict__ gamma,
                      const float* __restrict__ beta, TOut* __restrict__ out, int n_rows, int width, float eps) {
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int r = blockIdx.x * (blockDim.x >> 5) + warp;
  if (r >= n_rows) return;
  const float* src = x + (long long)(rows ? rows[r] : r) * width;
  float4 v[J];
#pragma unroll
  for (int j = 0; j < J; ++j) {
    const int c = (j * 32 + lane) * 4;
    v[j] = c < width ? *reinterpret_cast<const float4*>(src + c) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  float s = 0.f;
#pragma unroll
  for (int j = 0; j < J; ++j) s += (v[j].x + v[j].y) + (v[j].z + v[j].w);
  const float mean = warp_sum(s) / (float)width;
  float q = 0.f;
#pragma unroll
  for (int j = 0; j < J; ++j)
    if ((j * 32 + lane) * 4 < width) {
      const float a = v[j].x - mean, b = v[j].y - mean, c = v[j].z - mean, d = v[j].w - mean;
      q += (a * a + b * b) + (c * c + d * d);
    }
  const float rstd = 1.f / sqrtf(warp_sum(q) / (float)width + eps);
  TOut* dst = out + (long long)r * width;
#pragma unroll
  for (int j = 0; j < J; ++j) {
    const int c = (j * 32 + lane) * 4;
    if (c < width) {
      const float4 g = *reinterpret_cast<const float4*>(gamma + c);
      float4 b = make_float4(0.f, 0.f, 0.f, 0.f);
      if (beta) b = *reinterpret_cast<const float4*>(beta + c);
      const float o0 = (v[j].x - mean) * rstd * g.x + b.x, o1 = (v[j].y - mean) * rstd * g.y + b.y;
      const float o2 = (v[j].z - mean) * rstd * g.z + b.z, o3 = (v[j].w - mean) * rstd * g.w + b.w;
      if constexpr (sizeof(TOut) == 4) {
        *reinterpret_cast<float4*>(dst + c) = make_float4(o0, o1, o2, o3);
      } else {
        __nv_bfloat162 lo = __floats2bfloat162_rn(o0, o1), hi = __floats2bfloat162_rn(o2, o3);
        uint2 packed;
        packed.x = *reinterpret_cast<unsigned*>(&lo);
        packed.y = *reinterpret_cast<unsigned*>(&hi);
        *reinterpret_cast<uint2*>(dst + c) = packed;
      }
    }
  }
}

template <typename TOut>
static int launch_layernorm(const float* x, const int* rows, const float* gamma, const float* beta, TOut* out, int n_rows,
                            int width, float eps, cudaStream_t stream) {
  constexpr int T = 256;
  const bool aligned = width % 4 == 0 && ((unsigned long long)x % 16) == 0 && ((unsigned long long)gamma % 16) == 0 &&
                       ((unsigned long long)beta % 16) == 0 && ((unsigned long long)out % (sizeof(TOut) == 4 ? 16 : 8)) == 0;
  // (the choice must not depend on the number of rows: a row's result is the same alone and in a batch)
  if (aligned && width <= 2048) {
    // (a warp's arithmetic does not depend on how many warps share its block: few rows are spread over more SMs)
    const int warps = n_rows >= 1024 ? 8 : 2;
    const dim3 grid((n_rows + warps - 1) / warps), block(warps * 32);
    if (width <= 1024)
      BT_PDL_OK("layernorm", launch_pdl(layernorm_rows_kernel<TOut, 8>, grid, block, 0, stream, 1, x, rows, gamma, beta, out,
                                        n_rows, width, eps));
    else
      BT_PDL_OK("layernorm", launch_pdl(layernorm_rows_kernel<TOut, 16>, grid, block, 0, stream, 1, x, rows, gamma, beta, out,
                                        n_rows, width, eps));
    return 0;
  }
  const size_t smem = (size_t)width * sizeof(float);
  BT_PDL_OK("layernorm", launch_pdl(layernorm_kernel<TOut, T>, dim3(n_rows), dim3(T), smem, stream, 1, x, rows, gamma, beta, out,
                                    width, eps));
  return 0;
}

}  // namespace bt

extern "C" int bt_layernorm(const float* x, const int* rows, const float* gamma, const float* beta, void* out,
                            int n_rows, int width, float eps, int out_dtype, cudaStream_t stream) {
  using namespace bt;
  BT_CHECK(n_rows >= 0 && width > 0, "layernorm: bad sizes rows=%d width=%d", n_rows, width);
  BT_CHECK(width <= 12000, "layernorm: width %d exceeds the supported 12000", width);
  if (n_rows == 0) return 0;
  if (out_dtype == kF32) return launch_layernorm<float>(x, rows, gamma, beta, (float*)out, n_rows, width, eps, stream);
  if (out_dtype == kBF16)
    return launch_layernorm<__nv_bfloat16>(x, rows, gamma, beta, (__nv_bfloat16*)out, n_rows, width, eps, stream);
  return fail("layernorm: unknown dtype %d", out_dtype);
}
