// Matrix products for steps with 17 to 64 rows (decode of a larger batch), bfloat16 operands, 32-bit accumulation:
//   out[M, N] = act(A[M, K] @ W[N, K]^T + bias) (+ residual),  W stored [N, K] (K contiguous).
//
// Such a step is a chain of latencies, so the kernel is one short chain per block and nothing between blocks:
//   * a block owns all (at most 64) rows and BN = 16 output columns, over the whole of K when K is short: then there
//     is no sum across blocks at all.  A long K is split over the blocks of a thread-block cluster, whose partial
//     sums are added through distributed shared memory in the order of their ranks (no atomics, no scratch
//     memory: the result does not depend on timing);
//   * a producer warp asks the tensor memory accelerator for 64 x 64 boxes of A and 16 x 64 boxes of W (128-byte
//     swizzle, so that ldmatrix reads without bank conflicts) into a ring of stages; the boxes of W are asked for
//     before the kernel waits for its predecessor (programmatic dependent launch): nothing of the step writes
//     weights, so they travel while the previous kernel finishes;
//   * four warps take 16 rows each: per 16 k one ldmatrix.x4 for A, one for W, two mma.sync.m16n8k16; a warp that
//     has read a stage hands it back to the producer;
//   * the epilogue adds the bias, applies GELU, adds the 32-bit residual and writes 32-bit or bfloat16.
// Every wait for a stage is bounded; a wait that runs out sets the status word and the block returns.
#include <cooperative_groups.h>

#include "api.h"
#include "common.cuh"
#include "tma.cuh"

namespace cg = cooperative_groups;

namespace bt {

constexpr int LM_WARPS = 4;                           // consumer warps (16 rows each); one more warp produces
constexpr int LM_THREADS = (LM_WARPS + 1) * 32;
constexpr int LM_BM = 64, LM_BK = 64;                 // rows and k of one stage; its columns BN are 16 or 64
constexpr int LM_MAX_STAGES = 8;
constexpr int LM_A_BYTES = LM_BM * LM_BK * 2;
constexpr int lm_stages(int bn) { return bn <= 32 ? 8 : 6; }
constexpr int LM_WAIT_LIMIT = 1 << 20;

struct MidParams {
  const float* bias;           // [N] or null
  const float* residual;       // [M, N] 32-bit or null (may be `out`)
  void* out;                   // [M, N] 32-bit or bfloat16
  int* status;
  int M, N, K, k_slice, act, out_is_f32;      // k_slice: the k (a multiple of 64) a block of a cluster takes
  int rows16;                                 // M rounded up to 16: the rows of a box of A
};

__device__ __forceinline__ unsigned lm_smem(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void lm_ldmatrix_x4(unsigned (&r)[4], unsigned addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void lm_mma(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// Byte offset of the 16-byte chunk `chunk` (8 k) of row `row` in a tile of 128-byte rows with the 128-byte swizzle.
__device__ __forceinline__ unsigned lm_swizzled(int row, int chunk) { return (unsigned)(row * 128 + ((chunk ^ (row & 7)) << 4)); }
__device__ __forceinline__ bool lm_wait(unsigned long long* bar, unsigned parity) {
  for (int i = 0; i < LM_WAIT_LIMIT; ++i) {
    unsigned done;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(done) : "r"(lm_smem(bar)), "r"(parity) : "memory");
    if (done) return true;
  }
  return false;
}
__device__ __forceinline__ void lm_tma(void* dst, const CUtensorMap* map, int col, int row, unsigned long long* bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n" ::"r"(
                   lm_smem(dst)),
               "l"(map), "r"(col), "r"(row), "r"(lm_smem(bar))
               : "memory");
}

template <int LM_BN>
__global__ void __launch_bounds__(LM_THREADS)
linear_mid_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w, MidParams p) {
  constexpr int LM_STAGES = lm_stages(LM_BN), LM_W_BYTES = LM_BN * LM_BK * 2;
  extern __shared__ unsigned char lm_smem_raw[];
  __shared__ __align__(8) unsigned long long full[LM_MAX_STAGES], empty[LM_MAX_STAGES];
  __shared__ int failed;
  pdl_trigger();
  cg::cluster_group cluster = cg::this_cluster();
  const int split = (int)cluster.num_blocks(), rank = (int)cluster.block_rank();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int n0 = blockIdx.y * LM_BN;
  unsigned char* tiles = lm_smem_raw + ((1024u - (lm_smem(lm_smem_raw) & 1023u)) & 1023u);     // [stage][A 8 KB | W]
  // behind the ring, in a cluster only: this block's partial sums [64][BN], read by its cluster peers
  float* part = reinterpret_cast<float*>(tiles + (size_t)LM_STAGES * (LM_A_BYTES + LM_W_BYTES));
  const int k_begin = rank * p.k_slice, k_end = min(p.K, k_begin + p.k_slice);
  const int k_blocks = k_end > k_begin ? (k_end - k_begin + LM_BK - 1) / LM_BK : 0;
  if (tid == 0) {
    for (int s = 0; s < LM_STAGES; ++s) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(lm_smem(&full[s])), "r"(1));
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(lm_smem(&empty[s])), "r"(p.rows16 / 16));
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    failed = 0;
  }
  __syncthreads();

  const unsigned stage_bytes = (unsigned)(p.rows16 * LM_BK * 2 + LM_W_BYTES);
  if (warp == LM_WARPS) {
    // ---- producer: one lane asks for the boxes ----
    if (lane == 0) {
      // the first stages' weights before the wait for the predecessor; their rows of A after it
      const int early = min(k_blocks, LM_STAGES);
      for (int kb = 0; kb < early; ++kb) {
        unsigned char* st = tiles + (size_t)kb * (LM_A_BYTES + LM_W_BYTES);
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(lm_smem(&full[kb])), "r"(stage_bytes) : "memory");
        lm_tma(st + LM_A_BYTES, &map_w, k_begin + kb * LM_BK, n0, &full[kb]);
      }
      pdl_wait();
      for (int kb = 0; kb < early; ++kb) lm_tma(tiles + (size_t)kb * (LM_A_BYTES + LM_W_BYTES), &map_a, k_begin + kb * LM_BK, 0, &full[kb]);
      for (int kb = early; kb < k_blocks; ++kb) {
        const int s = kb % LM_STAGES;
        if (!lm_wait(&empty[s], ((kb / LM_STAGES) - 1) & 1)) {      // every consumer warp has read the stage's last use
          failed = 1;
          break;
        }
        unsigned char* st = tiles + (size_t)s * (LM_A_BYTES + LM_W_BYTES);
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(lm_smem(&full[s])), "r"(stage_bytes) : "memory");
        lm_tma(st, &map_a, k_begin + kb * LM_BK, 0, &full[s]);
        lm_tma(st + LM_A_BYTES, &map_w, k_begin + kb * LM_BK, n0, &full[s]);
      }
    }
  } else {
    // ---- consumers: warp w owns rows 16 w .. 16 w + 15 and the block's 16 columns ----
    pdl_wait();
    float acc[LM_BN / 8][4];
#pragma unroll
    for (int j = 0; j < LM_BN / 8; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[j][e] = 0.f;
    // ldmatrix.x4: lane L gives the address of row L % 8 of block L / 8.  A: blocks (rows 0-7 | 8-15) x (k 0-7 | 8-15);
    // W: blocks (columns 0-7: k 0-7, k 8-15; columns 8-15: k 0-7, k 8-15).
    const int blk = lane >> 3, r8 = lane & 7;
    const int my_blocks = warp * 16 < p.M ? k_blocks : 0;      // a warp without rows takes no part in the ring
    const int g = lane >> 2, q = lane & 3;
    // what the epilogue adds travels while the products run (a block that sums over a cluster reads it there)
    float pre_bias[LM_BN / 8][2], pre_res[LM_BN / 8][4];
    if (split == 1) {
#pragma unroll
      for (int j = 0; j < LM_BN / 8; ++j) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int col = n0 + j * 8 + 2 * q + e;
          pre_bias[j][e] = (p.bias && col < p.N) ? __ldg(p.bias + col) : 0.f;
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int r = warp * 16 + g + (e >> 1) * 8, col = n0 + j * 8 + 2 * q + (e & 1);
          pre_res[j][e] = (p.residual && r < p.M && col < p.N) ? p.residual[(long long)r * p.N + col] : 0.f;
        }
      }
    }
    bool ok = true;
    for (int kb = 0; kb < my_blocks && ok; ++kb) {
      const int s = kb % LM_STAGES;
      if (!lm_wait(&full[s], (kb / LM_STAGES) & 1)) {
        ok = false;
        break;
      }
      const unsigned a_base = lm_smem(tiles + (size_t)s * (LM_A_BYTES + LM_W_BYTES)), w_base = a_base + LM_A_BYTES;
#pragma unroll
      for (int ks = 0; ks < LM_BK / 16; ++ks) {
        unsigned af[4];
        lm_ldmatrix_x4(af, a_base + lm_swizzled(warp * 16 + (blk & 1) * 8 + r8, ks * 2 + (blk >> 1)));
#pragma unroll
        for (int nb = 0; nb < LM_BN / 16; ++nb) {
          unsigned bf[4];
          lm_ldmatrix_x4(bf, w_base + lm_swizzled(nb * 16 + (blk >> 1) * 8 + r8, ks * 2 + (blk & 1)));
          lm_mma(acc[2 * nb], af[0], af[1], af[2], af[3], bf[0], bf[1]);
          lm_mma(acc[2 * nb + 1], af[0], af[1], af[2], af[3], bf[2], bf[3]);
        }
      }
      __syncwarp();
      if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(lm_smem(&empty[s])) : "memory");
    }
    if (!ok) failed = 1;
    if (split > 1) {
      // (a block that failed leaves NaN, which its peers' sums keep)
#pragma unroll
      for (int j = 0; j < LM_BN / 8; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e)
          part[(warp * 16 + g + (e >> 1) * 8) * LM_BN + j * 8 + 2 * q + (e & 1)] = ok ? acc[j][e] : NAN;
    } else if (ok) {
#pragma unroll
      for (int j = 0; j < LM_BN / 8; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int r = warp * 16 + g + (e >> 1) * 8, col = n0 + j * 8 + 2 * q + (e & 1);
          if (r < p.M && col < p.N) {
            const long long o = (long long)r * p.N + col;
            const float x = apply_activation(acc[j][e] + pre_bias[j][e & 1], p.act) + pre_res[j][e];
            if (p.out_is_f32)
              reinterpret_cast<float*>(p.out)[o] = x;
            else
              reinterpret_cast<__nv_bfloat16*>(p.out)[o] = __float2bfloat16_rn(x);
          }
        }
    }
  }
  if (split > 1) {
    // the cluster adds its members' tiles in the order of their ranks; rank r finishes every split-th group of four
    cluster.sync();
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
  }
  __syncthreads();
  if (tid == 0 && failed && p.status) atomicExch(p.status, 5);
}

}  // namespace bt

extern "C" int bt_linear_mid_supports(int M, int N, int K) { return M >= 1 && M <= 64 && N >= 1 && K >= 8 && K % 8 == 0; }

// a: [M, K] bfloat16 (M <= 64); w: [N, K] bfloat16; out: [M, N] 32-bit (out_is_f32) or bfloat16.
// status: optional int that is set to 5 if a block's wait for a stage ran out.
// split: blocks per cluster along K (1, 2, 4 or 8); 0 lets the library choose from the shape
// alone (at most 1024 of K per block; two blocks per tile when the tiles are fewer than half the multiprocessors).
extern "C" int bt_linear_mid(const void* a, const void* w, const float* bias, const float* residual, void* out, int* status, int M,
                             int N, int K, int act, int out_is_f32, int split, cudaStream_t stream) {
  using namespace bt;
  BT_CHECK(bt_linear_mid_supports(M, N, K), "linear_mid: sizes M=%d N=%d K=%d are not supported", M, N, K);
  BT_CHECK(act >= 0 && act <= 2, "linear_mid: unknown activation %d", act);
  BT_CHECK(!(residual && !out_is_f32), "linear_mid: a residual needs a 32-bit output");
  const int k_blocks = (K + LM_BK - 1) / LM_BK;
  if (split <= 0) {
    split = 1;
    while (split < 8 && (k_blocks + split - 1) / split > 16) split *= 2;
  }
  // Every block reads all rows of A (from L2) for its columns of W: the wider a block's share of columns, the less
  // often the rows are read.  So: the widest of 64, 32 and 16 columns that still leaves a block (or more) for
  // every multiprocessor; a readout (N >= 8192) takes 64 in any case.
  const int want_blocks = sm_count();
  int bn = 16;
  if (N >= 8192) bn = 64;
  else
    for (int cand = 64; cand > 16; cand /= 2)
      if (((N + cand - 1) / cand) * split >= want_blocks) {
        bn = cand;
        break;
      }
  const int n_tiles = (N + bn - 1) / bn;
  const int rows16 = (M + 15) / 16 * 16;
  CUtensorMap ma, mw;
  if (int rc = tensor_map_2d_bf16(&ma, a, (unsigned long long)M, (unsigned long long)K, (unsigned long long)K, rows16)) return rc;
  if (int rc = tensor_map_2d_bf16(&mw, w, (unsigned long long)N, (unsigned long long)K, (unsigned long long)K, bn)) return rc;
  if (split == 1 && k_blocks >= 8 && 2 * n_tiles <= sm_count()) split = 2;      // too few blocks to fill the device
  BT_CHECK(split == 1 || split == 2 || split == 4 || split == 8, "linear_mid: split %d is not 1, 2, 4 or 8", split);
  const int k_slice = (k_blocks + split - 1) / split * LM_BK;
  MidParams p{bias, residual, out, status, M, N, K, k_slice, act, out_is_f32, rows16};
  BT_CHECK(n_tiles <= 65535, "linear_mid: N=%d needs too many column tiles", N);
  auto launch = [&](auto kernel, int bn_) -> int {
    const size_t smem = (size_t)lm_stages(bn_) * (LM_A_BYTES + bn_ * LM_BK * 2) + 1024 + (split > 1 ? (size_t)LM_BM * bn_ * 4 : 0);
    static bool configured[3] = {false, false, false};
    const int which = bn_ == 64 ? 2 : (bn_ == 32 ? 1 : 0);
    if (!configured[which]) {
      const size_t most = (size_t)lm_stages(bn_) * (LM_A_BYTES + bn_ * LM_BK * 2) + 1024 + (size_t)LM_BM * bn_ * 4;
      cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)most);
      BT_CHECK(e == cudaSuccess, "linear_mid: cannot reserve %zu bytes of shared memory: %s", most, cudaGetErrorString(e));
      configured[which] = true;
    }
    BT_PDL_OK("linear_mid", launch_pdl(kernel, dim3(split, n_tiles), dim3(LM_THREADS), smem, stream, split, ma, mw, p));
    return 0;
  };
  if (bn == 64) return launch(linear_mid_kernel<64>, 64);
  if (bn == 32) return launch(linear_mid_kernel<32>, 32);
  return launch(linear_mid_kernel<16>, 16);
}
