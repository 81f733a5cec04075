// Matrix products for steps with few rows (decode: one row per sequence, at most 64 rows): bfloat16
// operands, 32-bit accumulation, weights stored [N, K] with K contiguous.
//
// Such a product reads every weight once and does almost no arithmetic; the kernel is a weight stream.
// A warp owns 8 output columns, i.e. 8 weight rows, and reads them straight from global memory into the
// registers that mma.sync m16n8k16 wants as its B operand: lane (n = lane/4, q = lane%4) loads the 16 bytes
// W[n][32b + 8q .. 32b + 8q + 7] of every 32-wide block b of k.  Those 8 values feed two mma steps.  The
// tensor-core instruction does not care which k a register pair stands for as long as A uses the same
// assignment, so the A operand is loaded the same way (16 bytes of row lane/4, and of row lane/4 + 8):
// no shared-memory staging, no transposes, 16-byte loads only, and many of them in flight per lane.
//
// The 4 warps of a block either take 4 different column groups (WK = 1) or split K among them
// (WK = 2, 4) and add their partial sums through shared memory in a fixed order, so narrow outputs
// (N = 768) still spread over the whole GPU.  Results do not depend on what other rows are in the call.
//
// Optionally the rows are LayerNorm-ed on the way in: the block computes mean and 1/std of the 32-bit
// rows first (two passes), and the A loads normalise, scale and shift before rounding to bfloat16.
// The epilogue adds the bias, applies GELU, adds the 32-bit residual and writes 32-bit or bfloat16.
#include "common.cuh"

namespace bt {

constexpr int LS_WARPS = 4;
constexpr int LS_UNROLL = 8;   // 32-wide k blocks in flight per warp and iteration

struct StreamParams {
  const __nv_bfloat16* a;   // [M, K] bfloat16 rows; null: rows are LayerNorm(x32[rows[r] or r])
  const float* x32;
  const int* rows;
  const float* gamma;
  const float* beta;
  float eps;
  const __nv_bfloat16* w;   // [N, K]
  const float* bias;
  const float* residual;    // [M, N] 32-bit or null (may be `out`)
  void* out;
  int M, N, K, act, out_is_f32;
};

__device__ __forceinline__ uint4 ld_stream16(const void* p) {   // read once: do not keep in L1
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ uint4 ld_cached16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ void mma16816(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0,
                                         unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}

// 8 normalised values of one 32-bit row as 4 packed bfloat16 pairs
__device__ __forceinline__ uint4 normed_chunk(const float* x, const float* gamma, const float* beta, float mean, float rstd) {
  const float4 x0 = *reinterpret_cast<const float4*>(x), x1 = *reinterpret_cast<const float4*>(x + 4);
  const float4 g0 = *reinterpret_cast<const float4*>(gamma), g1 = *reinterpret_cast<const float4*>(gamma + 4);
  float4 b0 = make_float4(0.f, 0.f, 0.f, 0.f), b1 = b0;
  if (beta) {
    b0 = *reinterpret_cast<const float4*>(beta);
    b1 = *reinterpret_cast<const float4*>(beta + 4);
  }
  uint4 r;
  r.x = pack_bf16((x0.x - mean) * rstd * g0.x + b0.x, (x0.y - mean) * rstd * g0.y + b0.y);
  r.y = pack_bf16((x0.z - mean) * rstd * g0.z + b0.z, (x0.w - mean) * rstd * g0.w + b0.w);
  r.z = pack_bf16((x1.x - mean) * rstd * g1.x + b1.x, (x1.y - mean) * rstd * g1.y + b1.y);
  r.w = pack_bf16((x1.z - mean) * rstd * g1.z + b1.z, (x1.w - mean) * rstd * g1.w + b1.w);
  return r;
}

// MT: 16-row tiles (1..4).  WK: warps that split K (1, 2, 4).  FUSE_LN: rows come through LayerNorm (MT == 1).
template <int MT, int WK, bool FUSE_LN>
__global__ void __launch_bounds__(LS_WARPS * 32)
linear_stream_kernel(StreamParams p) {
  constexpr int WN = LS_WARPS / WK;                 // column groups per block
  __shared__ float stats[16][2];                    // mean, 1/std of the rows (fused LayerNorm)
  __shared__ float partial[WK > 1 ? LS_WARPS : 1][MT][32][4];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int wn = warp / WK, wk = warp % WK;
  const int n0 = (blockIdx.x * WN + wn) * 8;        // first of this warp's 8 columns
  const int g = lane >> 2, q = lane & 3;
  const int n = n0 + g;
  const bool n_ok = n < p.N;
  const int k_blocks = (p.K + 31) / 32;
  pdl_trigger();
  pdl_wait();

  if (FUSE_LN) {
    for (int r = warp; r < 16; r += LS_WARPS) {
      float mean = 0.f, rstd = 0.f;
      if (r < p.M) {
        const float* src = p.x32 + (long long)(p.rows ? p.rows[r] : r) * p.K;
        float s = 0.f;
        for (int c = lane * 4; c < p.K; c += 128) {
          const float4 v = *reinterpret_cast<const float4*>(src + c);
          s += (v.x + v.y) + (v.z + v.w);
        }
        mean = warp_sum(s) / (float)p.K;
        float d2 = 0.f;
        for (int c = lane * 4; c < p.K; c += 128) {
          const float4 v = *reinterpret_cast<const float4*>(src + c);
          const float a = v.x - mean, b = v.y - mean, cc = v.z - mean, d = v.w - mean;
          d2 += (a * a + b * b) + (cc * cc + d * d);
        }
        rstd = 1.f / sqrtf(warp_sum(d2) / (float)p.K + p.eps);
      }
      if (lane == 0) {
        stats[r][0] = mean;
        stats[r][1] = rstd;
      }
    }
    __syncthreads();
  }

  float acc[MT][4];
#pragma unroll
  for (int t = 0; t < MT; ++t)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[t][i] = 0.f;

  const __nv_bfloat16* wrow = p.w + (long long)(n_ok ? n : 0) * p.K;
  // rows of A this lane feeds: g and g + 8 of every 16-row tile
  const float* xrow[2] = {nullptr, nullptr};
  float mean[2] = {0.f, 0.f}, rstd[2] = {0.f, 0.f};
  if (FUSE_LN) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int r = g + 8 * h;
      if (r < p.M) {
        xrow[h] = p.x32 + (long long)(p.rows ? p.rows[r] : r) * p.K;
        mean[h] = stats[r][0];
        rstd[h] = stats[r][1];
      }
    }
  }

  for (int b0 = wk * LS_UNROLL; b0 < k_blocks; b0 += WK * LS_UNROLL) {
    uint4 wv[LS_UNROLL];
#pragma unroll
    for (int u = 0; u < LS_UNROLL; ++u) {
      const int kc = (b0 + u) * 32 + q * 8;
      wv[u] = (n_ok && kc < p.K) ? ld_stream16(wrow + kc) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < LS_UNROLL; ++u) {
      const int kc = (b0 + u) * 32 + q * 8;
      const bool k_ok = kc < p.K;
#pragma unroll
      for (int t = 0; t < MT; ++t) {
        uint4 lo = make_uint4(0, 0, 0, 0), hi = lo;
        if (FUSE_LN) {
          if (k_ok && xrow[0]) lo = normed_chunk(xrow[0] + kc, p.gamma + kc, p.beta ? p.beta + kc : nullptr, mean[0], rstd[0]);
          if (k_ok && xrow[1]) hi = normed_chunk(xrow[1] + kc, p.gamma + kc, p.beta ? p.beta + kc : nullptr, mean[1], rstd[1]);
        } else {
          const int r0 = t * 16 + g, r1 = r0 + 8;
          if (k_ok && r0 < p.M) lo = ld_cached16(p.a + (long long)r0 * p.K + kc);
          if (k_ok && r1 < p.M) hi = ld_cached16(p.a + (long long)r1 * p.K + kc);
        }
        mma16816(acc[t], lo.x, hi.x, lo.y, hi.y, wv[u].x, wv[u].y);
        mma16816(acc[t], lo.z, hi.z, lo.w, hi.w, wv[u].z, wv[u].w);
      }
    }
  }

  if (WK > 1) {
#pragma unroll
    for (int t = 0; t < MT; ++t)
#pragma unroll
      for (int i = 0; i < 4; ++i) partial[warp][t][lane][i] = acc[t][i];
    __syncthreads();
    if (wk != 0) return;
#pragma unroll
    for (int t = 0; t < MT; ++t)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float v = acc[t][i];
#pragma unroll
        for (int j = 1; j < WK; ++j) v += partial[warp + j][t][lane][i];
        acc[t][i] = v;
      }
  }
  // accumulator layout: c0, c1 -> row g, columns 2q, 2q+1; c2, c3 -> row g + 8
#pragma unroll
  for (int t = 0; t < MT; ++t)
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = t * 16 + g + (i >> 1) * 8;
      const int c = n0 + 2 * q + (i & 1);
      if (r >= p.M || c >= p.N) continue;
      float v = acc[t][i];
      if (p.bias) v += p.bias[c];
      v = apply_activation(v, p.act);
      const long long o = (long long)r * p.N + c;
      if (p.residual) v += p.residual[o];
      if (p.out_is_f32)
        reinterpret_cast<float*>(p.out)[o] = v;
      else
        reinterpret_cast<__nv_bfloat16*>(p.out)[o] = __float2bfloat16_rn(v);
    }
}

template <int MT, int WK, bool LN>
static int launch_stream(const StreamParams& p, cudaStream_t stream) {
  constexpr int WN = LS_WARPS / WK;
  const int groups = (p.N + 7) / 8;
  const int blocks = (groups + WN - 1) / WN;
  BT_PDL_OK("linear_stream", launch_pdl(linear_stream_kernel<MT, WK, LN>, dim3(blocks), dim3(LS_WARPS * 32), 0, stream, 1, p));
  return 0;
}

template <int WK, bool LN>
static int launch_stream_mt(const StreamParams& p, cudaStream_t stream) {
  switch ((p.M + 15) / 16) {
    case 1: return launch_stream<1, WK, LN>(p, stream);
    case 2: if (!LN) return launch_stream<2, WK, false>(p, stream); break;
    case 3: if (!LN) return launch_stream<3, WK, false>(p, stream); break;
    case 4: if (!LN) return launch_stream<4, WK, false>(p, stream); break;
  }
  return fail("linear_stream: %d rows are not supported%s", p.M, LN ? " with a fused LayerNorm" : "");
}

}  // namespace bt

// Whether bt_linear_stream takes these sizes (the caller picks another kernel otherwise).
extern "C" int bt_linear_stream_supports(int M, int N, int K, int fuse_ln) {
  if (M < 1 || M > 64 || N < 1 || K < 8) return 0;
  if (K % 8 != 0) return 0;                 // 16-byte chunks of weight rows and of bfloat16 rows
  if (fuse_ln && M > 16) return 0;
  return 1;
}

// w: [N, K] bfloat16.  a: bfloat16 rows, or null with (x32, gamma, beta, eps, rows) to normalise on the way in.
// warps_k: warps of a block that split K (1, 2, 4); 0 lets the library choose.
extern "C" int bt_linear_stream(const void* a, const float* x32, const int* rows, const float* gamma,
                                const float* beta, float eps, const void* w, const float* bias,
                                const float* residual, void* out, int M, int N, int K, int act, int out_is_f32,
                                int warps_k, cudaStream_t stream) {
  using namespace bt;
  const int fuse_ln = a == nullptr;
  BT_CHECK(bt_linear_stream_supports(M, N, K, fuse_ln), "linear_stream: sizes M=%d N=%d K=%d are not supported", M, N, K);
  BT_CHECK(!fuse_ln || (x32 && gamma), "linear_stream: fused LayerNorm needs 32-bit rows and a gain");
  BT_CHECK(act >= 0 && act <= 2, "linear_stream: unknown activation %d", act);
  BT_CHECK(!(residual && !out_is_f32), "linear_stream: a residual needs a 32-bit output");
  if (warps_k <= 0) {
    // one block per 8 columns unless that makes many more blocks than the GPU holds at once
    const int groups = (N + 7) / 8;
    const int sms = sm_count();
  BT_CHECK(sms > 0, "linear_stream: cannot read the number of multiprocessors of the current device");
    warps_k = groups >= sms * 8 ? 1 : (groups >= sms * 4 ? 2 : 4);
    while (warps_k > 1 && K / warps_k < 32 * LS_UNROLL) warps_k /= 2;
  }
  BT_CHECK(warps_k == 1 || warps_k == 2 || warps_k == 4, "linear_stream: warps_k %d must be 1, 2 or 4", warps_k);
  StreamParams p{(const __nv_bfloat16*)a, x32, rows, gamma, beta, eps, (const __nv_bfloat16*)w, bias, residual, out,
                 M, N, K, act, out_is_f32};
  if (fuse_ln) {
    if (warps_k == 1) return launch_stream_mt<1, true>(p, stream);
    if (warps_k == 2) return launch_stream_mt<2, true>(p, stream);
    return launch_stream_mt<4, true>(p, stream);
  }
  if (warps_k == 1) return launch_stream_mt<1, false>(p, stream);
  if (warps_k == 2) return launch_stream_mt<2, false>(p, stream);
  return launch_stream_mt<4, false>(p, stream);
}
