// Matrix products for steps with 17 to 64 rows (decode of a larger batch), bfloat16 operands, 32-bit accumulation:
//   out[M, N] = act(A[M, K] @ W[N, K]^T + bias) (+ residual),  W stored [N, K] (K contiguous).
//
// A classic shared-memory tile product on mma.sync, kept short because the step is a chain of latencies:
//   * the grid is (split, column tiles): a block owns all (at most 64) rows, 64 output columns and one slice of K;
//     the blocks that share a column tile form a thread-block cluster along K, and their partial sums are added
//     through distributed shared memory in a fixed order (no atomics, no scratch memory: the result does not
//     depend on timing);
//   * a block copies its whole [64 x K slice] panels of A and W into shared memory with 16-byte asynchronous
//     copies issued back to back (chunks of at most 384 k), rows of 128 bytes with the 16-byte chunks swizzled
//     (chunk ^ row & 7) so that ldmatrix reads without bank conflicts; the weight panel is asked for before the
//     kernel waits for its predecessor (programmatic dependent launch);
//   * four warps take a 32 x 32 quarter of the tile each: per 16 k two ldmatrix.x4 for A, two for W, eight
//     mma.sync.m16n8k16;
//   * the epilogue adds the bias, applies GELU, adds the 32-bit residual and writes 32-bit or bfloat16.
#include <cooperative_groups.h>

#include "api.h"
#include "common.cuh"

namespace cg = cooperative_groups;

namespace bt {

constexpr int LM_THREADS = 128;
constexpr int LM_BM = 64, LM_BN = 64, LM_BK = 64;     // rows, columns, k of one shared-memory tile
constexpr int LM_CHUNK_BLOCKS = 6;                    // k tiles in shared memory at a time (6 x 16 KB)

struct MidParams {
  const __nv_bfloat16* a;      // [M, K]
  const __nv_bfloat16* w;      // [N, K]
  const float* bias;           // [N] or null
  const float* residual;       // [M, N] 32-bit or null (may be `out`)
  void* out;                   // [M, N] 32-bit or bfloat16
  int M, N, K, k_slice, act, out_is_f32;
};

__device__ __forceinline__ unsigned lm_smem(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void lm_cp16(void* smem, const void* gmem) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(lm_smem(smem)), "l"(gmem) : "memory");
}
__device__ __forceinline__ void lm_ldmatrix_x4(unsigned (&r)[4], unsigned addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void lm_mma(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// Byte offset of the 16-byte chunk `chunk` (8 k) of row `row` in a 64 x 64 tile of bfloat16.
__device__ __forceinline__ unsigned lm_swizzled(int row, int chunk) { return (unsigned)(row * 128 + ((chunk ^ (row & 7)) << 4)); }

// One 64-row panel (of A or of W) of k tiles [kb0, kb1) of this block's slice into shared memory; rows at or
// beyond `n_rows` and k at or beyond K are zero.
__device__ __forceinline__ void lm_load_panel(unsigned char* tiles, const __nv_bfloat16* src, int row0, int n_rows, int K, int k0, int n_kb) {
  // 64 rows x 8 chunks per k tile
  for (int i = threadIdx.x; i < n_kb * 512; i += LM_THREADS) {
    const int kb = i >> 9, r = (i >> 3) & 63, c = i & 7;
    const int k = k0 + kb * LM_BK + c * 8;
    unsigned char* dst = tiles + kb * (LM_BM * 128) + lm_swizzled(r, c);
    if (row0 + r < n_rows && k < K)
      lm_cp16(dst, src + (long long)(row0 + r) * K + k);
    else
      *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
  }
}

__global__ void __launch_bounds__(LM_THREADS)
linear_mid_kernel(MidParams p) {
  extern __shared__ __align__(128) unsigned char lm_smem_raw[];
  pdl_trigger();
  cg::cluster_group cluster = cg::this_cluster();
  const int split = (int)cluster.num_blocks(), rank = (int)cluster.block_rank();
  const int n0 = blockIdx.y * LM_BN;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int wm = warp & 1, wn = warp >> 1;          // the warp's 32 x 32 quarter
  unsigned char* a_tiles = lm_smem_raw;                                  // [LM_CHUNK_BLOCKS][64 x 128 B]
  unsigned char* w_tiles = a_tiles + LM_CHUNK_BLOCKS * LM_BM * 128;      // [LM_CHUNK_BLOCKS][64 x 128 B]
  float* part = reinterpret_cast<float*>(w_tiles + LM_CHUNK_BLOCKS * LM_BN * 128);   // [64][64] partial sums
  const int k_begin = rank * p.k_slice, k_end = min(p.K, k_begin + p.k_slice);
  const int n_kb_all = k_end > k_begin ? (k_end - k_begin + LM_BK - 1) / LM_BK : 0;

  float acc[2][4][4];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[i][j][e] = 0.f;

  bool waited = false;
  for (int kb0 = 0; kb0 < n_kb_all; kb0 += LM_CHUNK_BLOCKS) {
    const int n_kb = min(LM_CHUNK_BLOCKS, n_kb_all - kb0);
    const int k0 = k_begin + kb0 * LM_BK;
    if (kb0 > 0) __syncthreads();      // everyone has read the chunk before
    // weights first: nothing of this step writes them, so they may travel before the predecessor has finished
    lm_load_panel(w_tiles, p.w, n0, p.N, p.K, k0, n_kb);
    if (!waited) {
      pdl_wait();
      waited = true;
    }
    lm_load_panel(a_tiles, p.a, 0, p.M, p.K, k0, n_kb);
    asm volatile("cp.async.wait_all;\n" ::: "memory");
    __syncthreads();
    const unsigned a_base = lm_smem(a_tiles), w_base = lm_smem(w_tiles);
    // ldmatrix.x4: lane L gives the address of row L % 8 of block L / 8.  A: blocks (rows 0-7 | 8-15) x (k 0-7 | 8-15)
    // of a 16 x 16 tile; W: blocks (columns 0-7 | 8-15) x (k 0-7 | 8-15) of two 8-column tiles.
    const int blk = lane >> 3, r8 = lane & 7;
    for (int kb = 0; kb < n_kb; ++kb) {
#pragma unroll
      for (int ks = 0; ks < LM_BK / 16; ++ks) {
        unsigned af[2][4], bf[2][4];
#pragma unroll
        for (int i = 0; i < 2; ++i)
          lm_ldmatrix_x4(af[i], a_base + kb * (LM_BM * 128) + lm_swizzled(wm * 32 + i * 16 + (blk & 1) * 8 + r8, ks * 2 + (blk >> 1)));
#pragma unroll
        for (int j = 0; j < 2; ++j)
          lm_ldmatrix_x4(bf[j], w_base + kb * (LM_BN * 128) + lm_swizzled(wn * 32 + j * 16 + (blk >> 1) * 8 + r8, ks * 2 + (blk & 1)));
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            // bf[j]: {columns 0-7: k 0-7, k 8-15; columns 8-15: k 0-7, k 8-15}
            lm_mma(acc[i][2 * j], af[i][0], af[i][1], af[i][2], af[i][3], bf[j][0], bf[j][1]);
            lm_mma(acc[i][2 * j + 1], af[i][0], af[i][1], af[i][2], af[i][3], bf[j][2], bf[j][3]);
          }
      }
    }
  }
  if (!waited) pdl_wait();

  // ---- the block's partial tile; with a split, the cluster adds its members' tiles in the order of their ranks ----
  const int g = lane >> 2, q = lane & 3;
  if (split > 1) {
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int r = wm * 32 + i * 16 + g + (e >> 1) * 8, c = wn * 32 + j * 8 + 2 * q + (e & 1);
          part[r * LM_BN + c] = acc[i][j][e];
        }
    cluster.sync();
    // rank r finishes the elements e with e / 4 % split == r (four consecutive columns at a time)
    for (int v = rank + tid * split; v < LM_BM * LM_BN / 4; v += LM_THREADS * split) {
      const int r = (v * 4) / LM_BN, c = (v * 4) % LM_BN;
      float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int j = 0; j < split; ++j) {
        const float4 x = *reinterpret_cast<const float4*>(cluster.map_shared_rank(part, j) + v * 4);
        sum.x += x.x; sum.y += x.y; sum.z += x.z; sum.w += x.w;
      }
      const float s4[4] = {sum.x, sum.y, sum.z, sum.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int col = n0 + c + e;
        if (r < p.M && col < p.N) {
          const long long o = (long long)r * p.N + col;
          float x = apply_activation(s4[e] + (p.bias ? p.bias[col] : 0.f), p.act);
          if (p.residual) x += p.residual[o];
          if (p.out_is_f32)
            reinterpret_cast<float*>(p.out)[o] = x;
          else
            reinterpret_cast<__nv_bfloat16*>(p.out)[o] = __float2bfloat16_rn(x);
        }
      }
    }
    cluster.sync();    // nobody leaves while a peer may still read its partial tile
    return;
  }
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int r = wm * 32 + i * 16 + g + (e >> 1) * 8, col = n0 + wn * 32 + j * 8 + 2 * q + (e & 1);
        if (r < p.M && col < p.N) {
          const long long o = (long long)r * p.N + col;
          float x = apply_activation(acc[i][j][e] + (p.bias ? p.bias[col] : 0.f), p.act);
          if (p.residual) x += p.residual[o];
          if (p.out_is_f32)
            reinterpret_cast<float*>(p.out)[o] = x;
          else
            reinterpret_cast<__nv_bfloat16*>(p.out)[o] = __float2bfloat16_rn(x);
        }
      }
}

}  // namespace bt

extern "C" int bt_linear_mid_supports(int M, int N, int K) { return M >= 1 && M <= 64 && N >= 1 && K >= 8 && K % 8 == 0; }

// a: [M, K] bfloat16 (M <= 64); w: [N, K] bfloat16; out: [M, N] 32-bit (out_is_f32) or bfloat16.
// split: blocks per cluster along K (1..8); 0 lets the library choose.
extern "C" int bt_linear_mid(const void* a, const void* w, const float* bias, const float* residual, void* out, int M, int N,
                             int K, int act, int out_is_f32, int split, cudaStream_t stream) {
  using namespace bt;
  BT_CHECK(bt_linear_mid_supports(M, N, K), "linear_mid: sizes M=%d N=%d K=%d are not supported", M, N, K);
  BT_CHECK(act >= 0 && act <= 2, "linear_mid: unknown activation %d", act);
  BT_CHECK(!(residual && !out_is_f32), "linear_mid: a residual needs a 32-bit output");
  BT_CHECK(((unsigned long long)a % 16) == 0 && ((unsigned long long)w % 16) == 0, "linear_mid: operands must lie on 16-byte boundaries");
  const int n_tiles = (N + LM_BN - 1) / LM_BN;
  BT_CHECK(n_tiles <= 65535, "linear_mid: N=%d needs too many column tiles", N);
  const int k_blocks = (K + LM_BK - 1) / LM_BK;
  if (split <= 0) {
    // the fewest slices that fill most of the GPU; if none does, the most that divide K's tiles evenly
    const int sms = sm_count() > 0 ? sm_count() : 148;
    split = 0;
    for (int s = 1; s <= 8 && split == 0; ++s)
      if (s <= k_blocks && n_tiles * s * 5 >= sms * 4) split = s;
    for (int s = 8; s >= 1 && split == 0; --s)
      if (s <= k_blocks && k_blocks % s == 0) split = s;
  }
  BT_CHECK(split >= 1 && split <= 8, "linear_mid: split %d is outside 1..8", split);
  const int k_slice = (k_blocks + split - 1) / split * LM_BK;
  MidParams p{(const __nv_bfloat16*)a, (const __nv_bfloat16*)w, bias, residual, out, M, N, K, k_slice, act, out_is_f32};
  const size_t smem = (size_t)LM_CHUNK_BLOCKS * (LM_BM + LM_BN) * 128 + (size_t)LM_BM * LM_BN * sizeof(float);
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(linear_mid_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    BT_CHECK(e == cudaSuccess, "linear_mid: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
    configured = true;
  }
  BT_PDL_OK("linear_mid", launch_pdl(linear_mid_kernel, dim3(split, n_tiles), dim3(LM_THREADS), smem, stream, split, p));
  return 0;
}
