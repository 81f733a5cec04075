// Matrix products for steps with few rows (decode of up to 128 sequences) over large weights with a long K,
// bfloat16 operands, 32-bit accumulation, on the fifth-generation tensor cores:
//   out[M, N] = act(X[M, K] @ W[N, K]^T + bias) (+ residual),  M <= 128,  W stored [N, K] (K contiguous).
//
// Such a product is the time its weights take to arrive, and a multiprocessor pulls them at about 50 GB/s whatever
// the kernel does (a 128 x 64 box of W with its rows of X lands every 0.37 us), so the shape has to be spread over
// as many multiprocessors as it can keep busy without reading the rows of X too often:
//   * the operands change places: 128 rows of W are the tensor cores' M side, the step's rows (rounded up to 16)
//     the N side.  No tensor-core row is spent on padding, and a block's share of the traffic is its 128 x 64 boxes
//     of W (16 KB) beside R x 64 boxes of X (2 to 16 KB, from L2);
//   * a block owns 128 output columns and a slice of K; the blocks of a thread-block cluster share a column tile
//     and add their partial sums through distributed shared memory in the order of their ranks (no atomics, no
//     scratch memory: the result does not depend on timing).  The number of slices is chosen so that one wave of
//     blocks covers the device;
//   * warp 0 asks the tensor memory accelerator for the boxes (cp.async.bulk.tensor, 128-byte swizzle) into a ring
//     of stages, the boxes of W for the whole ring before the kernel waits for its predecessor (programmatic
//     dependent launch): nothing of a step writes weights, so they travel while the previous kernel finishes;
//   * one thread of warp 1 issues tcgen05.mma (M = 128, N = R, K = 16, four per stage) into an accumulator in tensor
//     memory and commits each stage back to the producer;
//   * warps 2-9 read the accumulator with tcgen05.ld (a thread holds one output column for 32 rows) and put it into
//     a tile in shared memory, over the ring, which nobody needs any more;
//   * all threads then finish groups of 8 columns of a row: the sum over the cluster's tiles, bias, GELU, the 32-bit
//     residual, 16- and 32-byte stores.  (With few warps on a multiprocessor this part is bound by the instructions
//     a warp can issue, hence eight warps and nothing per element that can be settled per thread.)
// Every wait is bounded; a wait that runs out sets the status word, the block still takes part in its cluster's
// barriers, frees its tensor memory and returns.
#include <cooperative_groups.h>

#include "api.h"
#include "common.cuh"
#include "tcgen05.cuh"
#include "tma.cuh"

namespace cg = cooperative_groups;

namespace bt {

constexpr int TF_BN = 128;                // rows of W (output columns) of a block: the tensor cores' M
constexpr int TF_THREADS = 10 * 32;       // producer, issuer, eight epilogue warps (two per quarter of the lanes)
constexpr int TF_MAX_STAGES = 8;
constexpr int TF_MAX_ROWS = 128;
constexpr unsigned TF_W_BYTES = TF_BN * TC_BK * 2;
constexpr size_t TF_RING_BUDGET = 200 * 1024;    // the ring of stages, one block on a multiprocessor
constexpr size_t TF_RING_PAIRED = 104 * 1024;    // the ring when two blocks share one

struct FewParams {
  const float* bias;           // [N] or null
  const float* residual;       // [M, N] 32-bit or null (may be `out`)
  void* out;                   // [M, N] 32-bit or bfloat16
  int* status;
  int M, N, K, k_slice, act, out_is_f32;      // k_slice: the k (a multiple of 64) a block of a cluster takes
  int rows16;                                 // M rounded up to 16: the rows of a box of X, the tensor cores' N
  int stages, tmem_cols;
};

__global__ void __launch_bounds__(TF_THREADS)
linear_few_tcgen05_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w, FewParams p) {
  extern __shared__ unsigned char tf_smem_raw[];
  __shared__ __align__(8) unsigned long long full[TF_MAX_STAGES], empty[TF_MAX_STAGES], acc_full;
  __shared__ unsigned tmem_base;
  __shared__ int failed;
  pdl_trigger();     // the next kernel may set itself up (and fetch its weights) while this one runs
  cg::cluster_group cluster = cg::this_cluster();
  const int split = (int)cluster.num_blocks(), rank = (int)cluster.block_rank();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int n0 = blockIdx.y * TF_BN;
  unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<unsigned long long>(tf_smem_raw) + 1023ull) & ~1023ull);
  const unsigned x_bytes = (unsigned)p.rows16 * TC_BK * 2, stage_bytes = TF_W_BYTES + x_bytes;     // [stage][W 16 KB | X]
  // a block's partial sums [rows16][128] for its cluster peers lie over the ring: they are written when every
  // product has read its stage
  float* part = reinterpret_cast<float*>(tiles);
  const int k_begin = rank * p.k_slice, k_end = min(p.K, k_begin + p.k_slice);
  const int k_blocks = k_end > k_begin ? (k_end - k_begin + TC_BK - 1) / TC_BK : 0;
  const int stages = p.stages;

  if (tid == 0) {
    for (int s = 0; s < stages; ++s) {
      tc_bar_init(&full[s], 1);
      tc_bar_init(&empty[s], 1);
    }
    tc_bar_init(&acc_full, 1);
    failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(tc_smem(&tmem_base)), "r"(p.tmem_cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  const unsigned tmem_acc = tmem_base;
  // What a thread finishes at the end are groups of 8 columns of a row, rank + split (tid + 192 i): the step is a
  // multiple of the 16 groups of a row, so a thread keeps its columns, and their bias (a weight) can be read now.
  const bool exact = p.residual != nullptr || p.out_is_f32 != 0;
  const bool vec_ok = p.N % 8 == 0;
  const int groups = p.rows16 * (TF_BN / 8), step = TF_THREADS * split;
  const int my_col = n0 + ((rank + tid * split) % (TF_BN / 8)) * 8;
  float my_bias[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) my_bias[e] = (p.bias && my_col + e < p.N) ? __ldg(p.bias + my_col + e) : 0.f;

  if (warp == 0) {
    if (lane == 0) {
      // ---- producer: the ring's boxes of W first, then the wait for the predecessor, then the rows ----
      const int early = min(k_blocks, stages);
      for (int kb = 0; kb < early; ++kb) {
        tc_bar_expect(&full[kb], stage_bytes);
        tc_tma_load(tiles + (size_t)kb * stage_bytes, &map_w, k_begin + kb * TC_BK, n0, &full[kb]);
      }
      pdl_wait();
      for (int kb = 0; kb < early; ++kb)
        tc_tma_load(tiles + (size_t)kb * stage_bytes + TF_W_BYTES, &map_x, k_begin + kb * TC_BK, 0, &full[kb]);
      for (int kb = early; kb < k_blocks; ++kb) {
        const int s = kb % stages;
        if (!tc_bar_wait(&empty[s], ((kb / stages) - 1) & 1)) {      // the products of the stage's last use have read it
          failed = 1;
          break;
        }
        tc_bar_expect(&full[s], stage_bytes);
        tc_tma_load(tiles + (size_t)s * stage_bytes, &map_w, k_begin + kb * TC_BK, n0, &full[s]);
        tc_tma_load(tiles + (size_t)s * stage_bytes + TF_W_BYTES, &map_x, k_begin + kb * TC_BK, 0, &full[s]);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---- issuer.  Instruction descriptor: 32-bit accumulator, bfloat16 operands, both K-major, N = rows16, M = 128
      const unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(p.rows16 >> 3) << 17) | ((unsigned)(TF_BN >> 4) << 24);
      bool ok = true;
      for (int kb = 0; kb < k_blocks; ++kb) {
        const int s = kb % stages;
        if (!tc_bar_wait(&full[s], (kb / stages) & 1)) {
          failed = 1;
          ok = false;
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        unsigned char* w_tile = tiles + (size_t)s * stage_bytes;
        const unsigned long long dw = tc_desc(w_tile), dx = tc_desc(w_tile + TF_W_BYTES);
#pragma unroll
        for (int k = 0; k < TC_BK / 16; ++k)     // 16 bfloat16 = 32 bytes further along the row: +2 in 16-byte units
          tc_mma(tmem_acc, dw + 2ull * k, dx + 2ull * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
        tc_commit(&empty[s]);                    // arrives when these products have read the stage
      }
      if (ok && k_blocks > 0) tc_commit(&acc_full);          // arrives when every product has finished
    }
  } else {
    // ---- the accumulator leaves tensor memory: warp w reaches lanes 32 (w % 4) .. + 31, the block's columns of that
    // quarter; a thread holds one column for all rows and writes it into the tile `part` [rows16][128] ----
    const int quarter = warp & 3, half = (warp - 2) >> 2;      // the two warps of a quarter take every other 32 rows
    bool ok = true;
    if (k_blocks > 0) {
      ok = __all_sync(0xffffffffu, tc_bar_wait(&acc_full, 0));      // (the reads below are collective)
      asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    }
#pragma unroll 1
    for (int m0 = 32 * half; m0 < p.rows16; m0 += 64) {
      float v[32];
      // (the allocation is a multiple of 32 columns: a last chunk of 16 rows reads 16 columns nobody wrote and drops them)
      if (ok && k_blocks > 0) {
        tc_ld32(tmem_acc + ((unsigned)(quarter * 32) << 16) + (unsigned)m0, v);
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = ok ? 0.f : NAN;      // (a block that failed leaves NaN, which its peers' sums keep)
      }
      const int live = min(32, p.rows16 - m0);
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (i < live) part[(m0 + i) * TF_BN + quarter * 32 + lane] = v[i];
    }
    if (!ok) failed = 1;
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  }
  // ---- every thread finishes groups of 8 columns of a row: the sum over the cluster's tiles in the order of the
  // ranks (rank r takes every split-th group), bias, activation, residual; 16- and 32-byte accesses ----
  if (split > 1) cluster.sync(); else __syncthreads();
  pdl_wait();      // the residual is read and the output written only when the previous kernel has finished
  {
    constexpr int U = 2;      // groups whose loads are in flight together (a store may not pass a load of the residual)
    for (int g0 = rank + tid * split; g0 < groups; g0 += U * step) {
      float acc[U][8], res[U][8];
      long long o[U];
      bool live[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int g = g0 + u * step;
        const int r = g / (TF_BN / 8);
        live[u] = g < groups && r < p.M && my_col < p.N;
        o[u] = (long long)r * p.N + my_col;
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[u][e] = 0.f, res[u][e] = 0.f;
        if (!live[u]) continue;
        if (split == 1) {
          const float4 x = *reinterpret_cast<const float4*>(part + g * 8), y = *reinterpret_cast<const float4*>(part + g * 8 + 4);
          acc[u][0] = x.x; acc[u][1] = x.y; acc[u][2] = x.z; acc[u][3] = x.w;
          acc[u][4] = y.x; acc[u][5] = y.y; acc[u][6] = y.z; acc[u][7] = y.w;
        } else {
          for (int j = 0; j < split; ++j) {
            const float* peer = cluster.map_shared_rank(part, j) + g * 8;
            const float4 x = *reinterpret_cast<const float4*>(peer), y = *reinterpret_cast<const float4*>(peer + 4);
            acc[u][0] += x.x; acc[u][1] += x.y; acc[u][2] += x.z; acc[u][3] += x.w;
            acc[u][4] += y.x; acc[u][5] += y.y; acc[u][6] += y.z; acc[u][7] += y.w;
          }
        }
        if (p.residual) {
          if (vec_ok) {
            const float4 x = *reinterpret_cast<const float4*>(p.residual + o[u]), y = *reinterpret_cast<const float4*>(p.residual + o[u] + 4);
            res[u][0] = x.x; res[u][1] = x.y; res[u][2] = x.z; res[u][3] = x.w;
            res[u][4] = y.x; res[u][5] = y.y; res[u][6] = y.z; res[u][7] = y.w;
          } else {
#pragma unroll
            for (int e = 0; e < 8; ++e)
              if (my_col + e < p.N) res[u][e] = p.residual[o[u] + e];
          }
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (!live[u]) continue;
        float x[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) x[e] = tc_activation(acc[u][e] + my_bias[e], p.act, exact) + res[u][e];
        if (vec_ok) {
          if (p.out_is_f32) {
            float* dst = reinterpret_cast<float*>(p.out) + o[u];
            *reinterpret_cast<float4*>(dst) = make_float4(x[0], x[1], x[2], x[3]);
            *reinterpret_cast<float4*>(dst + 4) = make_float4(x[4], x[5], x[6], x[7]);
          } else {
            uint4 packed;
            packed.x = tc_pack(x[0], x[1]); packed.y = tc_pack(x[2], x[3]);
            packed.z = tc_pack(x[4], x[5]); packed.w = tc_pack(x[6], x[7]);
            *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.out) + o[u]) = packed;
          }
        } else {
#pragma unroll
          for (int e = 0; e < 8; ++e)
            if (my_col + e < p.N) {
              if (p.out_is_f32)
                reinterpret_cast<float*>(p.out)[o[u] + e] = x[e];
              else
                reinterpret_cast<__nv_bfloat16*>(p.out)[o[u] + e] = __float2bfloat16_rn(x[e]);
            }
        }
      }
    }
  }
  if (split > 1) cluster.sync();    // nobody leaves while a peer may still read its partial tile
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_acc), "r"(p.tmem_cols) : "memory");
  }
  if (tid == 0 && failed && p.status) atomicExch(p.status, 7);
}

// The split of K over a cluster for a shape: the one with the shortest estimated time, from
// (waves of blocks over the places for a block) x (a block's k-blocks x the time of one + what a block costs at all);
// every block of a cluster has some of K.
static int tf_choose_split(int n_tiles, int k_blocks, int places) {
  int best = 1;
  double best_cost = -1.0;
  for (int s = 1; s <= 8; ++s) {
    const int per = (k_blocks + s - 1) / s;
    if ((s - 1) * per >= k_blocks) continue;          // a rank would be left without k
    const long long blocks = (long long)n_tiles * s;
    const long long waves = (blocks + places - 1) / places;
    const double cost = (double)waves * (per * 0.25 + 2.0 + 0.15 * (s > 1 ? s : 0));
    if (best_cost < 0 || cost < best_cost - 1e-9) {
      best_cost = cost;
      best = s;
    }
  }
  return best;
}

}  // namespace bt

extern "C" int bt_linear_few_tcgen05_supports(int M, int N, int K) {
  return M >= 1 && M <= bt::TF_MAX_ROWS && N >= 8 && K >= 8 && K % 8 == 0;   // rows of X and W are 16-byte multiples
}

// x: [M, K] bfloat16 (M <= 128); w: [N, K] bfloat16; out: [M, N] 32-bit (out_is_f32) or bfloat16.
// status: optional int that is set to 7 if a block's bounded wait ran out.
// split: blocks per cluster along K (1 to 8); 0 lets the library choose from the shape.
extern "C" int bt_linear_few_tcgen05(const void* x, const void* w, const float* bias, const float* residual, void* out, int* status,
                                     int M, int N, int K, int act, int out_is_f32, int split, cudaStream_t stream) {
  using namespace bt;
  BT_CHECK(bt_linear_few_tcgen05_supports(M, N, K), "linear_few_tcgen05: sizes M=%d N=%d K=%d are not supported", M, N, K);
  BT_CHECK(act >= 0 && act <= 2, "linear_few_tcgen05: unknown activation %d", act);
  BT_CHECK(!(residual && !out_is_f32), "linear_few_tcgen05: a residual needs a 32-bit output");
  BT_CHECK(split >= 0 && split <= 8, "linear_few_tcgen05: split %d is not between 0 and 8", split);
  const int sms = sm_count();
  BT_CHECK(sms > 0, "linear_few_tcgen05: cannot read the number of multiprocessors of the current device");
  const int k_blocks = (K + TC_BK - 1) / TC_BK;
  const int n_tiles = (N + TF_BN - 1) / TF_BN;
  BT_CHECK(n_tiles <= 65535, "linear_few_tcgen05: N=%d needs too many column tiles", N);
  // With at most 16 rows a stage is 18 KB: a ring of 104 KB holds what a block needs, two blocks share a multiprocessor,
  // and the next product of a step streams its weights while this one sums and finishes (measured at 8 rows, 4800 x
  // 1600: 7.5 against 9.5 us a launch in a graph).  More rows take the whole of shared memory for a long K's stages.
  const int rows16 = (M + 15) / 16 * 16;
  const bool paired = rows16 <= 16;
  const size_t budget = paired ? TF_RING_PAIRED : TF_RING_BUDGET;
  if (split == 0) split = tf_choose_split(n_tiles, k_blocks, paired ? 2 * sms : sms);
  const int per = (k_blocks + split - 1) / split;
  BT_CHECK((split - 1) * per < k_blocks, "linear_few_tcgen05: split %d leaves a block without any of K=%d", split, K);
  const size_t stage_bytes = TF_W_BYTES + (size_t)rows16 * TC_BK * 2;
  int stages = (int)(budget / stage_bytes);
  if (stages > TF_MAX_STAGES) stages = TF_MAX_STAGES;
  if (stages > per) stages = per;
  size_t ring = (size_t)stages * stage_bytes;
  const size_t part_bytes = (size_t)rows16 * TF_BN * 4;
  if (ring < part_bytes) ring = part_bytes;
  const size_t smem = ring + 1024;
  CUtensorMap mx, mw;
  if (int rc = tensor_map_2d_bf16(&mx, x, (unsigned long long)M, (unsigned long long)K, (unsigned long long)K, (unsigned)rows16)) return rc;
  if (int rc = tensor_map_2d_bf16(&mw, w, (unsigned long long)N, (unsigned long long)K, (unsigned long long)K, TF_BN)) return rc;
  const int tmem_cols = rows16 <= 32 ? 32 : (rows16 <= 64 ? 64 : 128);
  FewParams p{bias, residual, out, status, M, N, K, per * TC_BK, act, out_is_f32, rows16, stages, tmem_cols};
  static bool configured = false;
  if (!configured) {
    const size_t most = TF_RING_BUDGET + 1024;
    cudaError_t e = cudaFuncSetAttribute(linear_few_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)most);
    BT_CHECK(e == cudaSuccess, "linear_few_tcgen05: cannot reserve %zu bytes of shared memory: %s", most, cudaGetErrorString(e));
    configured = true;
  }
  BT_PDL_OK("linear_few_tcgen05", launch_pdl(linear_few_tcgen05_kernel, dim3(split, n_tiles), dim3(TF_THREADS), smem, stream, split, mx, mw, p));
  return 0;
}
