// Matrix products for steps with many rows (prefill), bfloat16 operands, 32-bit accumulation, on the
// fifth-generation tensor cores:  out[M,N] = act(A[M,K] @ W[N,K]^T + bias) (+ residual).
//
// A block computes 128 x BN tiles of the output, one after another (one block per SM).  Its ten warps have fixed jobs:
//   warp 0    asks the tensor memory accelerator (TMA) for the next 128 x 64 tile of A and BN x 64 tile of W
//             (cp.async.bulk.tensor, 128-byte swizzle) into a ring of shared-memory stages;
//   warp 1    one elected thread issues tcgen05.mma (M = 128, N = BN, K = 16, four per stage) whose accumulator
//             lives in tensor memory (TMEM), and commits each stage back to the producer when it has been read;
//   warps 2-9 wait for a tile's last commit and read the accumulator with tcgen05.ld (a warp reaches the 32 TMEM lanes
//             of its quarter; the two warps of a quarter take half of the columns each).  A thread then holds 32
//             consecutive columns of one row: it adds the bias, applies GELU and writes the segment with 16-byte
//             stores (bfloat16 or 32-bit); with a 32-bit residual the warp first turns its patch through shared
//             memory, so that four lanes read and write 64 contiguous bytes of a row.  There are two
//             accumulators, so this runs while the next tile's products are already being issued.
// Both operands are K-major (K contiguous): A as the activations are stored, W as [N, K].
// The kernel is launched as a programmatic dependent: it sets itself up (barriers, tensor memory) and asks for its
// first tiles of W while its predecessor still runs, and waits for it only before it touches activations.
// Stages hand over through mbarriers; every wait is bounded, and a wait that runs out marks the call as failed
// (status word) instead of hanging: the block still frees its tensor memory and returns.
// Rows and columns beyond M, N, K are zero-filled by the TMA on the way in and skipped on the way out.
#include "common.cuh"
#include "tcgen05.cuh"
#include "tma.cuh"

namespace bt {

constexpr int TC_BM = 128;
constexpr int TC_EPI_WARPS = 8;                    // two per quarter of the accumulator's rows, half the columns each
constexpr int TC_THREADS = (2 + TC_EPI_WARPS) * 32;
constexpr int TC_PATCH_STRIDE = 20;       // floats between rows of an epilogue warp's 32 x 16 patch in shared memory

struct TcParams {
  const float* bias;        // [N] or null
  const float* residual;    // [M, N] 32-bit or null (may be `out`)
  void* out;                // [M, N] 32-bit or bfloat16
  int* status;              // set to 1 when a bounded wait ran out
  int M, N, K, act, out_is_f32;
};


// Persistent: a block walks over output tiles (tile, tile + grid, ...).  The accumulator is double-buffered in
// tensor memory (2 x BN columns), so the epilogue of one tile runs while the products of the next are issued.
// Shared memory: STAGES x (A tile 128 x 64, W tile BN x 64), each tile 1024-byte aligned, then a 32 x 20 float
// patch per epilogue warp through which accumulator rows are turned into coalesced global rows.
template <int BN, int STAGES>
__global__ void __launch_bounds__(TC_THREADS)
linear_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w, TcParams p) {
  extern __shared__ unsigned char tc_smem_raw[];
  __shared__ __align__(8) unsigned long long full[STAGES], empty[STAGES], acc_full[2], acc_empty[2];
  __shared__ unsigned tmem_base;
  __shared__ int failed;
  constexpr unsigned A_BYTES = TC_BM * TC_BK * 2, W_BYTES = BN * TC_BK * 2;
  // columns of tensor memory from one accumulator to the other: a power of two, as the allocation has to be
  constexpr int ACC = BN <= 64 ? 64 : (BN <= 128 ? 128 : 256);
  unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<unsigned long long>(tc_smem_raw) + 1023ull) & ~1023ull);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  pdl_trigger();     // the next kernel may set itself up (and fetch its weights) while this one runs
  const int tiles_m = (p.M + TC_BM - 1) / TC_BM, tiles_n = (p.N + BN - 1) / BN;
  const int n_tiles = tiles_m * tiles_n;
  const int k_blocks = (p.K + TC_BK - 1) / TC_BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      tc_bar_init(&full[s], 1);
      tc_bar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      tc_bar_init(&acc_full[b], 1);
      tc_bar_init(&acc_empty[b], TC_EPI_WARPS);       // one arrival per epilogue warp
    }
    failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 1) {
    // two accumulators of BN 32-bit columns each (the count is a power of two of at least 32)
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(tc_smem(&tmem_base)), "r"(2 * ACC) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  const unsigned tmem_acc = tmem_base;

  if (warp == 0) {
    if (lane == 0) {
      // The first stages' tiles of W are asked for before the kernel waits for its predecessor (programmatic dependent
      // launch): nothing of a step writes weights, so they travel while the previous kernel finishes.  Their tiles
      // of A follow after the wait.
      const int pre = (int)blockIdx.x < n_tiles ? (k_blocks < STAGES ? k_blocks : STAGES) : 0;
      {
        const int m0 = ((int)blockIdx.x % tiles_m) * TC_BM, n0 = ((int)blockIdx.x / tiles_m) * BN;
        for (int kb = 0; kb < pre; ++kb) {
          tc_bar_expect(&full[kb], A_BYTES + W_BYTES);
          tc_tma_load(tiles + (size_t)kb * (A_BYTES + W_BYTES) + A_BYTES, &map_w, kb * TC_BK, n0, &full[kb]);
        }
        pdl_wait();
        for (int kb = 0; kb < pre; ++kb) tc_tma_load(tiles + (size_t)kb * (A_BYTES + W_BYTES), &map_a, kb * TC_BK, m0, &full[kb]);
      }
      int it = 0;                          // k-blocks loaded so far, over all tiles
      for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        const int m0 = (tile % tiles_m) * TC_BM, n0 = (tile / tiles_m) * BN;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          if (it < pre) continue;          // asked for above
          const int s = it % STAGES;
          if (it >= STAGES && !tc_bar_wait(&empty[s], ((it / STAGES) - 1) & 1)) {
            failed = 1;
            tile = n_tiles;
            break;
          }
          tc_bar_expect(&full[s], A_BYTES + W_BYTES);
          unsigned char* a_tile = tiles + (size_t)s * (A_BYTES + W_BYTES);
          tc_tma_load(a_tile, &map_a, kb * TC_BK, m0, &full[s]);
          tc_tma_load(a_tile + A_BYTES, &map_w, kb * TC_BK, n0, &full[s]);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // instruction descriptor: 32-bit accumulator, bfloat16 operands, both K-major, N = BN, M = 128
      const unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(BN >> 3) << 17) | ((unsigned)(TC_BM >> 4) << 24);
      int it = 0, local = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++local) {
        const int buf = local & 1;
        // the epilogue must have emptied this accumulator (it was last used two tiles ago)
        if (local >= 2 && !tc_bar_wait(&acc_empty[buf], ((local >> 1) - 1) & 1)) {
          failed = 1;
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        const unsigned d_tmem = tmem_acc + (unsigned)(buf * ACC);
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          if (!tc_bar_wait(&full[s], (it / STAGES) & 1)) {
            failed = 1;
            ok = false;
            break;
          }
          asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
          unsigned char* a_tile = tiles + (size_t)s * (A_BYTES + W_BYTES);
          const unsigned long long da = tc_desc(a_tile), dw = tc_desc(a_tile + A_BYTES);
#pragma unroll
          for (int k = 0; k < TC_BK / 16; ++k)   // 16 bfloat16 = 32 bytes further along the row: +2 in 16-byte units
            tc_mma(d_tmem, da + 2ull * k, dw + 2ull * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          tc_commit(&empty[s]);                  // arrives when these products have read the stage
        }
        tc_commit(&acc_full[buf]);               // arrives when every product issued so far has finished
      }
    }
  } else {
    // epilogue: warp w reaches TMEM lanes 32 * (w % 4) .. + 31, i.e. the tile's rows of that quarter; the two warps
    // of a quarter take half of the tile's columns each.  A thread holds 32 consecutive columns of its row: bias,
    // activation and residual are applied there and the row segment is written with 16-byte stores.
    const int quarter = warp & 3, half = (warp - 2) >> 2;
    float* patch = reinterpret_cast<float*>(tiles + (size_t)STAGES * (A_BYTES + W_BYTES)) + (warp - 2) * (32 * TC_PATCH_STRIDE);
    pdl_wait();      // the residual is read and the output written only when the previous kernel has finished
    const bool vec_ok = p.out_is_f32 ? (p.N % 4 == 0) : (p.N % 8 == 0);
    int local = 0;
    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++local) {
      const int buf = local & 1;
      const int m0 = (tile % tiles_m) * TC_BM, n0 = (tile / tiles_m) * BN;
      const bool ok = tc_bar_wait(&acc_full[buf], (local >> 1) & 1);
      if (!ok) {
        failed = 1;
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
      const int row = m0 + quarter * 32 + lane;
      const bool row_ok = row < p.M;
      // (the first warp of a quarter takes the larger part when the 32-column chunks are an odd number)
      constexpr int SPLIT = (BN / 32 + 1) / 2 * 32;
#pragma unroll 1
      for (int c0 = half ? SPLIT : 0; c0 < (half ? BN : SPLIT); c0 += 32) {
        float v[32];
        tc_ld32(tmem_acc + ((unsigned)(quarter * 32) << 16) + (unsigned)(buf * ACC + c0), v);
        const int col0 = n0 + c0;
        if (col0 >= p.N) continue;                 // (uniform in the warp; the load above is collective)
        const long long o0 = (long long)row * p.N + col0;
        if (vec_ok && col0 + 32 <= p.N && p.residual != nullptr) {
          // 32-bit output with a residual (the residual stream itself, as a rule): the warp's patch goes through
          // shared memory, 16 columns at a time, so that global memory is reached row by row: a thread writes its
          // row (rows 20 floats apart: no bank conflicts for 16-byte accesses), then lane 4 r + c takes columns
          // 4 c .. 4 c + 3 of rows r, r + 8, ..., so that four lanes cover 64 contiguous bytes of a row of the
          // residual and of the output.  (With a lane per row every instruction touches 32 lines, and the
          // load/store unit takes them one by one: 1.8 us per 32 columns each way.)
          const int cq = lane & 3, rq = lane >> 2;
          const int row_base = m0 + quarter * 32 + rq;
#pragma unroll
          for (int h16 = 0; h16 < 2; ++h16) {
            const long long o_base = (long long)row_base * p.N + col0 + 16 * h16 + 4 * cq;
            float4 res[4];
#pragma unroll
            for (int k = 0; k < 4; ++k)
              if (row_base + 8 * k < p.M) res[k] = *reinterpret_cast<const float4*>(p.residual + o_base + (long long)(8 * k) * p.N);
#pragma unroll
            for (int j = 0; j < 4; ++j)
              *reinterpret_cast<float4*>(patch + lane * TC_PATCH_STRIDE + 4 * j) =
                  make_float4(v[16 * h16 + 4 * j], v[16 * h16 + 4 * j + 1], v[16 * h16 + 4 * j + 2], v[16 * h16 + 4 * j + 3]);
            __syncwarp();
            float4 b4 = make_float4(0.f, 0.f, 0.f, 0.f);
            if (p.bias) b4 = __ldg(reinterpret_cast<const float4*>(p.bias + col0 + 16 * h16 + 4 * cq));
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              float4 x = *reinterpret_cast<const float4*>(patch + (rq + 8 * k) * TC_PATCH_STRIDE + 4 * cq);
              x.x = tc_activation(x.x + b4.x, p.act, true) + res[k].x;
              x.y = tc_activation(x.y + b4.y, p.act, true) + res[k].y;
              x.z = tc_activation(x.z + b4.z, p.act, true) + res[k].z;
              x.w = tc_activation(x.w + b4.w, p.act, true) + res[k].w;
              if (row_base + 8 * k < p.M) *reinterpret_cast<float4*>(reinterpret_cast<float*>(p.out) + o_base + (long long)(8 * k) * p.N) = x;
            }
            __syncwarp();      // the patch is free again
          }
        } else if (vec_ok && col0 + 32 <= p.N) {
          float4 res[8];
          if (p.residual && row_ok) {
            // the whole segment of the residual first, so that the latencies overlap (the output may be the
            // residual itself, which keeps the compiler from moving these loads above the stores on its own)
#pragma unroll
            for (int j = 0; j < 8; ++j) res[j] = *reinterpret_cast<const float4*>(p.residual + o0 + 4 * j);
          }
          if (p.bias) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float4 b4 = __ldg(reinterpret_cast<const float4*>(p.bias + col0 + 4 * j));
              v[4 * j] += b4.x; v[4 * j + 1] += b4.y; v[4 * j + 2] += b4.z; v[4 * j + 3] += b4.w;
            }
          }
          const bool exact = p.residual != nullptr || p.out_is_f32 != 0;
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = tc_activation(v[i], p.act, exact);
          if (p.out_is_f32) {
            if (!row_ok) continue;
            float* dst = reinterpret_cast<float*>(p.out) + o0;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              float4 x = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
              if (p.residual) { x.x += res[j].x; x.y += res[j].y; x.z += res[j].z; x.w += res[j].w; }
              *reinterpret_cast<float4*>(dst + 4 * j) = x;
            }
          } else {
            // bfloat16: the thread's 64-byte row goes into the patch (rows 80 bytes apart: no bank conflicts), then
            // lane 4 r + c writes 16 bytes of rows r, r + 8, r + 16, r + 24: four lanes cover a row's 64 bytes,
            // an instruction 8 lines instead of 32
            unsigned char* patch8 = reinterpret_cast<unsigned char*>(patch);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint4 x;
              x.x = tc_pack(v[8 * j], v[8 * j + 1]);
              x.y = tc_pack(v[8 * j + 2], v[8 * j + 3]);
              x.z = tc_pack(v[8 * j + 4], v[8 * j + 5]);
              x.w = tc_pack(v[8 * j + 6], v[8 * j + 7]);
              *reinterpret_cast<uint4*>(patch8 + lane * (TC_PATCH_STRIDE * 4) + 16 * j) = x;
            }
            __syncwarp();
            const int cq = lane & 3, rq = lane >> 2;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const int r = rq + 8 * k, grow = m0 + quarter * 32 + r;
              const uint4 x = *reinterpret_cast<const uint4*>(patch8 + r * (TC_PATCH_STRIDE * 4) + 16 * cq);
              if (grow < p.M) *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.out) + (long long)grow * p.N + col0 + 8 * cq) = x;
            }
            __syncwarp();      // the patch is free again
          }
        } else if (row_ok) {
          // a ragged edge, or rows that are no multiple of 16 bytes: one element at a time
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            if (col0 + i >= p.N) break;
            float x = tc_activation(v[i] + (p.bias ? p.bias[col0 + i] : 0.f), p.act, p.residual != nullptr || p.out_is_f32 != 0);
            if (p.residual) x += p.residual[o0 + i];
            if (p.out_is_f32)
              reinterpret_cast<float*>(p.out)[o0 + i] = x;
            else
              reinterpret_cast<__nv_bfloat16*>(p.out)[o0 + i] = __float2bfloat16_rn(x);
          }
        }
      }
      // this warp has read its part of the accumulator: hand the buffer back to the issuer
      asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
      __syncwarp();
      if (lane == 0) tc_bar_arrive(&acc_empty[buf]);
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_acc), "r"(2 * ACC) : "memory");
  }
  if (threadIdx.x == 0 && failed && p.status) atomicExch(p.status, 2);
}

template <int BN, int STAGES>
static int launch_tc(const CUtensorMap& ma, const CUtensorMap& mw, const TcParams& p, cudaStream_t stream) {
  constexpr size_t smem = (size_t)STAGES * (TC_BM * TC_BK * 2 + BN * TC_BK * 2) + 1024 + (size_t)TC_EPI_WARPS * 32 * TC_PATCH_STRIDE * 4;
  auto kern = linear_tcgen05_kernel<BN, STAGES>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    BT_CHECK(e == cudaSuccess, "linear_tcgen05: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
    configured = true;
  }
  const int n_tiles = ((p.N + BN - 1) / BN) * ((p.M + TC_BM - 1) / TC_BM);
  const int sms = sm_count();
  BT_CHECK(sms > 0, "linear_tcgen05: cannot read the number of multiprocessors of the current device");
  const int blocks = n_tiles < sms ? n_tiles : sms;     // one persistent block per SM
  BT_PDL_OK("linear_tcgen05", launch_pdl(kern, dim3(blocks), dim3(TC_THREADS), smem, stream, 1, ma, mw, p));
  return 0;
}

}  // namespace bt

extern "C" int bt_linear_tcgen05_supports(int M, int N, int K) {
  return M >= 1 && N >= 8 && K >= 8 && K % 8 == 0;   // rows of A and W are 16-byte multiples
}

// a: [M, K] bfloat16; w: [N, K] bfloat16; out: [M, N] 32-bit (out_is_f32) or bfloat16.
extern "C" int bt_linear_tcgen05(const void* a, const void* w, const float* bias, const float* residual, void* out,
                                 int* status, int M, int N, int K, int act, int out_is_f32, cudaStream_t stream) {
  using namespace bt;
  BT_CHECK(bt_linear_tcgen05_supports(M, N, K), "linear_tcgen05: sizes M=%d N=%d K=%d are not supported", M, N, K);
  BT_CHECK(act >= 0 && act <= 2, "linear_tcgen05: unknown activation %d", act);
  BT_CHECK(!(residual && !out_is_f32), "linear_tcgen05: a residual needs a 32-bit output");
  // The tile's width: wide tiles reuse every loaded row of A for more columns, narrow ones cover the GPU with fewer
  // idle multiprocessors and fewer rounds.  Cost of a width = rounds of tiles over the multiprocessors x the time of
  // a k-block at that width (measured: 0.31 us at 128 columns, 0.55 us at 256: about 37 + width); ties go to the wider.
  const long long rows = (M + TC_BM - 1) / TC_BM;
  const int sms = sm_count();
  BT_CHECK(sms > 0, "linear_tcgen05: cannot read the number of multiprocessors of the current device");
  int bn = 256;
  long long best = -1;
  for (int width : {256, 192, 128, 96, 64}) {
    const long long tiles = rows * ((N + width - 1) / width);
    const long long cost = ((tiles + sms - 1) / sms) * (37 + width);
    if (best < 0 || cost < best) {
      best = cost;
      bn = width;
    }
  }
  CUtensorMap ma, mw;
  if (int rc = tensor_map_2d_bf16(&ma, a, (unsigned long long)M, (unsigned long long)K, (unsigned long long)K, TC_BM)) return rc;
  if (int rc = tensor_map_2d_bf16(&mw, w, (unsigned long long)N, (unsigned long long)K, (unsigned long long)K, (unsigned)bn)) return rc;
  TcParams p{bias, residual, out, status, M, N, K, act, out_is_f32};
  if (bn == 64) return launch_tc<64, 6>(ma, mw, p, stream);
  if (bn == 96) return launch_tc<96, 6>(ma, mw, p, stream);
  if (bn == 128) return launch_tc<128, 6>(ma, mw, p, stream);
  if (bn == 192) return launch_tc<192, 5>(ma, mw, p, stream);
  return launch_tc<256, 4>(ma, mw, p, stream);
}
