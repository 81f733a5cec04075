// Matrix products for steps with few rows (decode: one row per sequence, at most 64 rows), bfloat16
// operands, 32-bit accumulation.  Such a product reads every weight once and does almost no arithmetic, so
// the kernel is built to have the whole weight matrix in flight at once:
//   * the grid is (split, column tiles): each block owns BN output columns and one slice of K, and loads its
//     whole [K slice x BN] weight panel with 16-byte asynchronous copies issued back to back;
//   * the blocks that share a column tile form a thread-block cluster along K; their partial sums are added
//     through distributed shared memory in a fixed order (rank 0, 1, ...), so the result is deterministic and
//     needs neither atomics nor scratch memory;
//   * optionally the rows (at most 16) are LayerNorm-ed on the way in (32-bit statistics over the full row,
//     two passes), which saves a kernel and a round trip of the normalised rows;
//   * the weight panel is requested before the kernel waits for its predecessor (programmatic dependent
//     launch), so weights stream while the previous kernel is still finishing;
//   * the epilogue adds the bias, applies GELU, adds the 32-bit residual and writes 32-bit or bfloat16.
// The products themselves use mma.sync m16n8k16: with at most 64 rows the tensor pipe is idle either way.
#include <cooperative_groups.h>
#include <cuda_pipeline.h>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace bt {

constexpr int SK_THREADS = 128;
constexpr int SK_BN = 32;          // output columns per block: 4 warps x 8

struct SkinnyParams {
  const __nv_bfloat16* a;      // [M, K] bfloat16 rows, or null when the rows come from `x32` through LayerNorm
  const float* x32;            // [*, K] 32-bit rows to normalise (fused LayerNorm), row r = rows ? rows[r] : r
  const int* rows;
  const float* gamma;
  const float* beta;
  float eps;
  const __nv_bfloat16* w;      // [K, N] (N contiguous) or [N, K] (K contiguous)
  const float* bias;           // [N] or null
  const float* residual;       // [M, N] 32-bit or null (may be `out`)
  void* out;                   // [M, N] 32-bit or bfloat16
  int M, N, K, k_slice, act, out_is_f32;
};

__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* p) {
  const unsigned a = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x2(unsigned (&r)[2], const void* p) {
  const unsigned a = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];\n" : "=r"(r[0]), "=r"(r[1]) : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x2_trans(unsigned (&r)[2], const void* p) {
  const unsigned a = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];\n" : "=r"(r[0]), "=r"(r[1]) : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const unsigned (&a)[4], const unsigned (&b)[2]) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem));
}

// Shared memory: A panel [16*MT][k_slice + 8] bf16, W panel (KN: [k_slice][BN + 8]; NK: [BN][k_slice + 8]) bf16,
// then (reused after the products) the partial tile [16*MT][BN] 32-bit.
template <int MT, bool W_IS_NK, bool FUSE_LN>
__global__ void __launch_bounds__(SK_THREADS)
linear_skinny_kernel(SkinnyParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  cg::cluster_group cluster = cg::this_cluster();
  const int split = (int)cluster.num_blocks();
  const int rank = (int)cluster.block_rank();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int n0 = blockIdx.y * SK_BN;
  const int k0 = rank * p.k_slice;
  const int k_len = max(0, min(p.k_slice, p.K - k0));       // valid k of this slice (the rest is zero)
  const int ks = p.k_slice;
  const int a_stride = ks + 8;                              // elements; +16 bytes keeps ldmatrix conflict-free
  __nv_bfloat16* As = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  __nv_bfloat16* Ws = As + 16 * MT * a_stride;
  const int w_stride = W_IS_NK ? ks + 8 : SK_BN + 8;

  // ---- weights first: they do not depend on the previous kernel's result -------------------------------
  if (W_IS_NK) {
    const int chunks_per_row = ks / 8;
    for (int i = tid; i < SK_BN * chunks_per_row; i += SK_THREADS) {
      const int r = i / chunks_per_row, c = (i - r * chunks_per_row) * 8;
      __nv_bfloat16* dst = Ws + r * w_stride + c;
      if (n0 + r < p.N && c < k_len)      // K is a multiple of 8, so a chunk is inside or outside as a whole
        cp_async16(dst, p.w + (long long)(n0 + r) * p.K + k0 + c);
      else
        *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
    }
  } else {
    constexpr int chunks_per_row = SK_BN / 8;
    for (int i = tid; i < ks * chunks_per_row; i += SK_THREADS) {
      const int r = i / chunks_per_row, c = (i - r * chunks_per_row) * 8;
      __nv_bfloat16* dst = Ws + r * w_stride + c;
      if (r < k_len && n0 + c < p.N)      // N is a multiple of 8
        cp_async16(dst, p.w + (long long)(k0 + r) * p.N + n0 + c);
      else
        *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
    }
  }
  asm volatile("cp.async.commit_group;\n" ::);
  pdl_trigger();   // the next kernel may start fetching its own weights
  pdl_wait();      // from here on the rows (and the residual) of the previous kernel are read

  // ---- rows ----------------------------------------------------------------------------------------
  if (FUSE_LN) {
    // Statistics of all rows at once: the block's 128 threads are dealt out 16 (at most 8 rows) or 8 (at most
    // 16 rows) to a row, so every row's loads are in flight together and one memory round trip serves them all.
    // Pass 1 sums the row; pass 2 re-reads it (from L1 now) and sums the squared deviations.
    __shared__ float stats[16][2];
    {
      const int lanes_per_row = p.M <= 8 ? 16 : 8;
      const int r = tid / lanes_per_row, li = tid % lanes_per_row;
      const bool live = r < p.M;
      const float* src = p.x32 + (long long)(live ? (p.rows ? p.rows[r] : r) : 0) * p.K;
      float s = 0.f;
      if (live)
        for (int c = li * 4; c < p.K; c += lanes_per_row * 4) {
          const float4 v = *reinterpret_cast<const float4*>(src + c);
          s += (v.x + v.y) + (v.z + v.w);
        }
      for (int o = lanes_per_row >> 1; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
      const float mean = s / (float)p.K;
      float d2 = 0.f;
      if (live)
        for (int c = li * 4; c < p.K; c += lanes_per_row * 4) {
          const float4 v = *reinterpret_cast<const float4*>(src + c);
          const float a = v.x - mean, b = v.y - mean, cc = v.z - mean, d = v.w - mean;
          d2 += (a * a + b * b) + (cc * cc + d * d);
        }
      for (int o = lanes_per_row >> 1; o > 0; o >>= 1) d2 += __shfl_xor_sync(0xffffffffu, d2, o);
      if (li == 0 && r < 16) {
        stats[r][0] = live ? mean : 0.f;
        stats[r][1] = live ? 1.f / sqrtf(d2 / (float)p.K + p.eps) : 0.f;
      }
    }
    __syncthreads();
    const int chunks_per_row = ks / 8;
    for (int i = tid; i < 16 * chunks_per_row; i += SK_THREADS) {
      const int r = i / chunks_per_row, c = (i - r * chunks_per_row) * 8;
      uint4 packed = make_uint4(0, 0, 0, 0);
      if (r < p.M && c < k_len) {
        const float* x = p.x32 + (long long)(p.rows ? p.rows[r] : r) * p.K + k0 + c;
        const float* gm = p.gamma + k0 + c;
        const float mean = stats[r][0], rstd = stats[r][1];
        const float4 x0 = *reinterpret_cast<const float4*>(x), x1 = *reinterpret_cast<const float4*>(x + 4);
        const float4 g0 = *reinterpret_cast<const float4*>(gm), g1 = *reinterpret_cast<const float4*>(gm + 4);
        float4 b0 = make_float4(0.f, 0.f, 0.f, 0.f), b1 = b0;
        if (p.beta) {
          b0 = *reinterpret_cast<const float4*>(p.beta + k0 + c);
          b1 = *reinterpret_cast<const float4*>(p.beta + k0 + c + 4);
        }
        auto pack = [](float lo, float hi) {
          __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
          return *reinterpret_cast<unsigned*>(&v);
        };
        packed.x = pack((x0.x - mean) * rstd * g0.x + b0.x, (x0.y - mean) * rstd * g0.y + b0.y);
        packed.y = pack((x0.z - mean) * rstd * g0.z + b0.z, (x0.w - mean) * rstd * g0.w + b0.w);
        packed.z = pack((x1.x - mean) * rstd * g1.x + b1.x, (x1.y - mean) * rstd * g1.y + b1.y);
        packed.w = pack((x1.z - mean) * rstd * g1.z + b1.z, (x1.w - mean) * rstd * g1.w + b1.w);
      }
      *reinterpret_cast<uint4*>(As + r * a_stride + c) = packed;
    }
  } else {
    const int chunks_per_row = ks / 8;
    for (int i = tid; i < 16 * MT * chunks_per_row; i += SK_THREADS) {
      const int r = i / chunks_per_row, c = (i - r * chunks_per_row) * 8;
      __nv_bfloat16* dst = As + r * a_stride + c;
      if (r < p.M && c < k_len)
        cp_async16(dst, p.a + (long long)r * p.K + k0 + c);
      else
        *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
    }
    asm volatile("cp.async.commit_group;\n" ::);
  }
  asm volatile("cp.async.wait_all;\n" ::);
  __syncthreads();

  // ---- products: warp w owns columns n0 + 8w .. +7 for all rows ----------------------------------------
  float acc[MT][4];
#pragma unroll
  for (int t = 0; t < MT; ++t)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[t][i] = 0.f;
  const int nw = warp * 8;
  for (int kk = 0; kk < ks; kk += 16) {
    unsigned b[2];
    if (W_IS_NK)
      ldmatrix_x2(b, Ws + (nw + (lane & 7)) * w_stride + kk + ((lane >> 3) & 1) * 8);
    else
      ldmatrix_x2_trans(b, Ws + (kk + (lane & 15)) * w_stride + nw);
#pragma unroll
    for (int t = 0; t < MT; ++t) {
      unsigned a[4];
      ldmatrix_x4(a, As + (t * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * a_stride + kk + (lane >> 4) * 8);
      mma_bf16(acc[t], a, b);
    }
  }

  // ---- reduce over the cluster and finish -----------------------------------------------------------
  const int row_in = lane >> 2, col_in = (lane & 3) * 2;
  auto finish = [&](int r, int c, float v) {
    const int gn = n0 + c;
    if (r >= p.M || gn >= p.N) return;
    if (p.bias) v += p.bias[gn];
    v = apply_activation(v, p.act);
    const long long o = (long long)r * p.N + gn;
    if (p.residual) v += p.residual[o];
    if (p.out_is_f32)
      reinterpret_cast<float*>(p.out)[o] = v;
    else
      reinterpret_cast<__nv_bfloat16*>(p.out)[o] = __float2bfloat16_rn(v);
  };
  if (split == 1) {
#pragma unroll
    for (int t = 0; t < MT; ++t) {
      finish(t * 16 + row_in, nw + col_in, acc[t][0]);
      finish(t * 16 + row_in, nw + col_in + 1, acc[t][1]);
      finish(t * 16 + row_in + 8, nw + col_in, acc[t][2]);
      finish(t * 16 + row_in + 8, nw + col_in + 1, acc[t][3]);
    }
    return;
  }
  __syncthreads();   // the panels are no longer read: reuse their memory for the partial tile
  float* part = reinterpret_cast<float*>(smem_raw);   // [16*MT][SK_BN]
#pragma unroll
  for (int t = 0; t < MT; ++t) {
    part[(t * 16 + row_in) * SK_BN + nw + col_in] = acc[t][0];
    part[(t * 16 + row_in) * SK_BN + nw + col_in + 1] = acc[t][1];
    part[(t * 16 + row_in + 8) * SK_BN + nw + col_in] = acc[t][2];
    part[(t * 16 + row_in + 8) * SK_BN + nw + col_in + 1] = acc[t][3];
  }
  cluster.sync();
  const int total = 16 * MT * SK_BN;
  const int per = (total + split - 1) / split;
  for (int e = rank * per + tid; e < min(total, (rank + 1) * per); e += SK_THREADS) {
    float from[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) from[j] = j < split ? cluster.map_shared_rank(part, j)[e] : 0.f;   // all in flight
    float v = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) v += from[j];
    finish(e / SK_BN, e % SK_BN, v);
  }
  cluster.sync();    // nobody leaves while a peer may still read its partial tile
}

template <int MT, bool NK, bool LN>
static int launch_skinny(const SkinnyParams& p, int split, cudaStream_t stream) {
  const int ks = p.k_slice;
  const size_t panels = sizeof(__nv_bfloat16) * ((size_t)16 * MT * (ks + 8) + (NK ? (size_t)SK_BN * (ks + 8) : (size_t)ks * (SK_BN + 8)));
  const size_t partial = sizeof(float) * 16 * MT * SK_BN;
  const size_t smem = panels > partial ? panels : partial;
  auto kern = linear_skinny_kernel<MT, NK, LN>;
  BT_CHECK(smem <= 200 * 1024, "linear_skinny: a K slice of %d needs %zu bytes of shared memory", ks, smem);
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  BT_CHECK(e == cudaSuccess, "linear_skinny: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
  e = launch_pdl(kern, dim3(split, (p.N + SK_BN - 1) / SK_BN, 1), dim3(SK_THREADS, 1, 1), smem, stream, split, p);
  BT_CHECK(e == cudaSuccess, "linear_skinny: launch failed: %s", cudaGetErrorString(e));
  count_launch();
  return 0;
}

template <bool NK, bool LN>
static int launch_skinny_mt(const SkinnyParams& p, int split, cudaStream_t stream) {
  const int mt = (p.M + 15) / 16;
  switch (mt) {
    case 1: return launch_skinny<1, NK, LN>(p, split, stream);
    case 2: if (!LN) return launch_skinny<2, NK, false>(p, split, stream); break;
    case 3: if (!LN) return launch_skinny<3, NK, false>(p, split, stream); break;
    case 4: if (!LN) return launch_skinny<4, NK, false>(p, split, stream); break;
  }
  return fail("linear_skinny: %d rows exceed 64", p.M);
}

}  // namespace bt

// Whether bt_linear_skinny takes these sizes (the caller falls back to another kernel otherwise).
extern "C" int bt_linear_skinny_supports(int M, int N, int K, int w_is_nk, int fuse_ln) {
  if (M < 1 || M > 64 || N < 1 || K < 16) return 0;
  if (K % 8 != 0) return 0;                       // 16-byte chunks of rows (and of [N,K] weight rows)
  if (!w_is_nk && N % 8 != 0) return 0;           // 16-byte chunks of [K,N] weight rows
  if (fuse_ln && M > 16) return 0;                // the fused LayerNorm handles one 16-row tile
  return 1;
}

// a: bfloat16 rows, or null with (x32, gamma, beta, eps, rows) to normalise 32-bit rows on the way in.
// split: blocks per cluster along K (1..8); 0 lets the library choose.
extern "C" int bt_linear_skinny(const void* a, const float* x32, const int* rows, const float* gamma,
                                const float* beta, float eps, const void* w, const float* bias,
                                const float* residual, void* out, int M, int N, int K, int w_is_nk, int act,
                                int out_is_f32, int split, cudaStream_t stream) {
  using namespace bt;
  const int fuse_ln = a == nullptr;
  BT_CHECK(bt_linear_skinny_supports(M, N, K, w_is_nk, fuse_ln), "linear_skinny: sizes M=%d N=%d K=%d are not supported", M, N, K);
  BT_CHECK(!fuse_ln || (x32 && gamma), "linear_skinny: fused LayerNorm needs 32-bit rows and a gain");
  BT_CHECK(act >= 0 && act <= 2, "linear_skinny: unknown activation %d", act);
  BT_CHECK(!(residual && !out_is_f32), "linear_skinny: a residual needs a 32-bit output");
  const int n_tiles = (N + SK_BN - 1) / SK_BN;
  BT_CHECK(n_tiles <= 65535, "linear_skinny: N=%d needs too many column tiles", N);
  if (split <= 0) {
    // enough blocks to fill the GPU about once, slices of at least 64 and at most 1024 k
    split = 1;
    const int sms = sm_count();
  BT_CHECK(sms > 0, "linear_skinny: cannot read the number of multiprocessors of the current device");
    while (split < 8 && n_tiles * split < sms && K / (split * 2) >= 64) split *= 2;
    while ((K + split - 1) / split > 1024 && split < 8) split *= 2;
  }
  BT_CHECK(split >= 1 && split <= 8, "linear_skinny: split %d is outside 1..8", split);
  int k_slice = ((K + split - 1) / split + 15) / 16 * 16;
  SkinnyParams p{(const __nv_bfloat16*)a, x32, rows, gamma, beta, eps, (const __nv_bfloat16*)w, bias, residual, out,
                 M, N, K, k_slice, act, out_is_f32};
  if (w_is_nk) return fuse_ln ? launch_skinny_mt<true, true>(p, split, stream) : launch_skinny_mt<true, false>(p, split, stream);
  return fuse_ln ? launch_skinny_mt<false, true>(p, split, stream) : launch_skinny_mt<false, false>(p, split, stream);
}
