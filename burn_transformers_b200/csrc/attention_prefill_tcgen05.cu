// Causal attention for steps that bring many tokens per sequence (prefill), bfloat16, on the fifth-generation
// tensor cores: both products of a tile, S = Q K^T and O += P V, are tcgen05.mma with accumulators in tensor
// memory (TMEM); the S x S score plane is never stored.
//
// A block (one per multiprocessor) owns 128 queries of one (sequence, head) and walks over that sequence's keys in
// tiles of 128.
//   warps 0-7  softmax: query row r is TMEM lane r, and two threads share it (a warp reaches the lanes of quarter
//              warp % 4; warps 0-3 take keys 0-63 of a tile and the lower half of the output channels, warps 4-7
//              the rest).  A thread reads its part of S with tcgen05.ld, the pair agree on the row's maximum through
//              shared memory, keep running maximum and sum in 32-bit (scores in base 2), write P = exp2(S - max) as
//              bfloat16 into shared memory in the layout the tensor core reads (K-major, 128-byte swizzle), then
//              add the tile's P V, read from TMEM, to their part of the row of the output, which lives in registers;
//   warp 8     one lane asks the tensor memory accelerator (TMA) for the queries once and for each tile's keys and
//              values (64 x 64 boxes, 128-byte swizzle) into two stages each;
//   warp 9     one lane issues the products: S = Q K^T (both operands K-major) into one of two accumulators, so that
//              the next tile's scores are computed while this tile's are weighed, and O_tile = P V (P K-major, V as
//              it lies in memory: "MN-major", head channels contiguous) when P is written.  P and O_tile are
//              double too: the softmax warps take a tile's P V only after they have written the next tile's P, so
//              that the product runs while they compute.
// Blocks are numbered by falling length (every sequence and head of the last query tile first).
// Keys and values come either from the rows of the step's own projections (sequences that start at position 0)
// or from the pages of the cache (a page is one 64-row box).  Query t of sequence s sits at position
// past[s] + (t - seq_start[s]); key j is visible when j <= position (causal) and j > position - window
// (window > 0).  A query that sees no key yields zeros.  Masked keys get the weight 0 exactly; what lies beyond
// a sequence's end in a tile is finite (rows of the next sequence, zero fill past the tensor, old page contents).
// All hand-overs go through mbarriers; every wait is bounded, and a wait that runs out sets the status word:
// the block still frees its tensor memory and returns.
#include "api.h"
#include "common.cuh"
#include "tma.cuh"

namespace bt {

constexpr int TA_BQ = 128, TA_BK = 128;
constexpr int TA_SOFTMAX_WARPS = 8;              // two threads per query row
constexpr int TA_THREADS = (TA_SOFTMAX_WARPS + 2) * 32;
constexpr int TA_STAGES = 2;                     // (the issuer's code is written out for two)
constexpr int TA_WAIT_LIMIT = 1 << 22;
constexpr int TA_BOX_BYTES = 64 * 128;            // a 64-row x 64-column bfloat16 box

struct TaParams {
  __nv_bfloat16* out;          // [tokens, n_heads * HD]
  const int* seq_start;
  const int* past_len;
  const int* table;            // null: keys and values are rows of the projections
  int table_stride, table_len;
  int* status;
  int n_heads, n_kv_heads;
  int k_col, v_col;            // packed: first column of the keys / values in a row of the projections
  float scale_log2;            // scale * log2(e)
  int causal, window;
};

__device__ __forceinline__ unsigned ta_smem(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void ta_bar_init(unsigned long long* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(ta_smem(bar)), "r"(count));
}
__device__ __forceinline__ void ta_bar_expect(unsigned long long* bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(ta_smem(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void ta_bar_arrive(unsigned long long* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(ta_smem(bar)) : "memory");
}
__device__ __forceinline__ bool ta_bar_wait(unsigned long long* bar, unsigned parity) {
  for (int i = 0; i < TA_WAIT_LIMIT; ++i) {
    unsigned done;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(done) : "r"(ta_smem(bar)), "r"(parity) : "memory");
    if (done) return true;
  }
  return false;
}
__device__ __forceinline__ void ta_tma(void* dst, const CUtensorMap* map, int col, int row, unsigned long long* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n" ::"r"(
          ta_smem(dst)),
      "l"(map), "r"(col), "r"(row), "r"(ta_smem(bar))
      : "memory");
}
// Shared-memory operand descriptor for tiles of 128-byte rows with the 128-byte swizzle.  K-major operands (Q, K, P):
// groups of 8 rows lie 1024 bytes apart (stride offset); the leading offset is not used.  The MN-major operand (V:
// rows are keys, the 64 head channels of a row are contiguous): 8 keys are 1024 bytes (stride offset) and the next
// 64 channels lie `leading` bytes further.
__device__ __forceinline__ unsigned long long ta_desc(const void* tile, unsigned leading) {
  unsigned long long d = 0;
  d |= (unsigned long long)((ta_smem(tile) & 0x3FFFFu) >> 4);
  d |= (unsigned long long)((leading >> 4) & 0x3FFFu) << 16;
  d |= (unsigned long long)(1024 >> 4) << 32;
  d |= (unsigned long long)1 << 46;
  d |= (unsigned long long)2 << 61;
  return d;
}
__device__ __forceinline__ void ta_mma(unsigned tmem_d, unsigned long long a, unsigned long long b, unsigned idesc, unsigned accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_d),
      "l"(a), "l"(b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void ta_commit(unsigned long long* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(ta_smem(bar)) : "memory");
}
// A load of 32 columns of this thread's TMEM lane without the wait, and the wait with the registers as operands
// (so that nothing that uses them is moved before it): two loads in flight halve the exposed latency.
__device__ __forceinline__ void ta_ld32_issue(unsigned taddr, unsigned (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,"
      "%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}
__device__ __forceinline__ void ta_ld_wait(unsigned (&a)[32], unsigned (&b)[32]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;\n"
               : "+r"(a[0]), "+r"(a[1]), "+r"(a[2]), "+r"(a[3]), "+r"(a[4]), "+r"(a[5]), "+r"(a[6]), "+r"(a[7]), "+r"(a[8]),
                 "+r"(a[9]), "+r"(a[10]), "+r"(a[11]), "+r"(a[12]), "+r"(a[13]), "+r"(a[14]), "+r"(a[15]), "+r"(a[16]),
                 "+r"(a[17]), "+r"(a[18]), "+r"(a[19]), "+r"(a[20]), "+r"(a[21]), "+r"(a[22]), "+r"(a[23]), "+r"(a[24]),
                 "+r"(a[25]), "+r"(a[26]), "+r"(a[27]), "+r"(a[28]), "+r"(a[29]), "+r"(a[30]), "+r"(a[31]), "+r"(b[0]),
                 "+r"(b[1]), "+r"(b[2]), "+r"(b[3]), "+r"(b[4]), "+r"(b[5]), "+r"(b[6]), "+r"(b[7]), "+r"(b[8]), "+r"(b[9]),
                 "+r"(b[10]), "+r"(b[11]), "+r"(b[12]), "+r"(b[13]), "+r"(b[14]), "+r"(b[15]), "+r"(b[16]), "+r"(b[17]),
                 "+r"(b[18]), "+r"(b[19]), "+r"(b[20]), "+r"(b[21]), "+r"(b[22]), "+r"(b[23]), "+r"(b[24]), "+r"(b[25]),
                 "+r"(b[26]), "+r"(b[27]), "+r"(b[28]), "+r"(b[29]), "+r"(b[30]), "+r"(b[31])
               :
               : "memory");
}
__device__ __forceinline__ float ta_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ unsigned ta_pack(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}
__device__ __forceinline__ void ta_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void ta_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }

// Tensor memory of a block: two S accumulators (2 x 128 columns) and two P V accumulators (2 x HD columns), at most
// 512 columns: the whole of a multiprocessor's, which one block has to itself.
constexpr int TA_TMEM_COLS = 512;

// Shared memory (the dynamic region, which must start on a 1024-byte boundary):
//   Q      [HD / 64][128 rows][128 bytes]
//   K, V   [stage][HD / 64][128 keys][128 bytes] each, two stages
//   P      [tile parity][2][128 rows][128 bytes]    (keys 0-63 | 64-127 of the tile)
//   the row maxima the two threads of a row exchange [tile parity][2 halves][128] (at the end: their sums)
//   barriers, the tensor-memory address, the failure flag
template <int HD>
constexpr size_t ta_smem_bytes() {
  return (size_t)(HD / 64) * 2 * TA_BOX_BYTES * (1 + 2 * TA_STAGES) + 2 * 2 * 2 * TA_BOX_BYTES + 4 * 128 * 4 + 256;
}

template <int HD>
__global__ void __launch_bounds__(TA_THREADS, 1)
attention_prefill_tcgen05_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap k_map,
                                 const __grid_constant__ CUtensorMap v_map, TaParams p) {
  constexpr int CB = HD / 64;                              // 64-column boxes per row of a head
  constexpr int TILE_BYTES = CB * 2 * TA_BOX_BYTES;        // 128 rows of a head
  constexpr int HH = HD / 2;                               // output channels of one of the two threads of a row
  extern __shared__ __align__(1024) unsigned char ta_raw[];
  unsigned char* Qs = ta_raw;
  unsigned char* Ks = Qs + TILE_BYTES;                     // [stage]
  unsigned char* Vs = Ks + TA_STAGES * TILE_BYTES;         // [stage]
  unsigned char* Ps = Vs + TA_STAGES * TILE_BYTES;                         // [tile parity][2 boxes]
  float* x_max = reinterpret_cast<float*>(Ps + 2 * 2 * 2 * TA_BOX_BYTES);  // [tile parity][half][row]
  unsigned long long* bars = reinterpret_cast<unsigned long long*>(x_max + 4 * 128);
  unsigned long long* q_full = bars;                       // 1
  unsigned long long* k_full = bars + 1;                   // [stage]
  unsigned long long* k_empty = k_full + TA_STAGES;        // [stage]
  unsigned long long* v_full = k_empty + TA_STAGES;        // [stage]
  unsigned long long* v_empty = v_full + TA_STAGES;        // [stage]
  unsigned long long* s_full = v_empty + TA_STAGES;        // [2]: the two S accumulators
  unsigned long long* p_ready = s_full + 2;                // [2]: the two P tiles
  unsigned long long* o_full = p_ready + 2;                // [2]: the two P V accumulators
  unsigned long long* o_free = o_full + 2;                 // [2]
  unsigned* tmem_base = reinterpret_cast<unsigned*>(o_free + 2);
  int* failed = reinterpret_cast<int*>(tmem_base + 1);

  // The next kernel's blocks come in once every block of this one has started; on multiprocessors that have run out
  // of query tiles they set themselves up while the longest tiles are still being worked on.
  pdl_trigger();
  // Blocks are numbered by falling length: every (sequence, head) of the last query tile first, so that the
  // multiprocessors that finish early pick up the short ones.
  const int seq = (int)blockIdx.x / p.n_heads, head = (int)blockIdx.x % p.n_heads;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // (sequence starts and lengths were written before the previous kernel started: safe to read before the wait)
  const int t0 = p.seq_start[seq], n_new = p.seq_start[seq + 1] - t0;
  const int q_tile = (int)gridDim.y - 1 - (int)blockIdx.y;
  const int q0 = q_tile * TA_BQ;
  if (q0 >= n_new) return;
  if ((ta_smem(ta_raw) & 1023u) != 0) {      // the swizzled layouts need the alignment: refuse rather than compute nonsense
    if (threadIdx.x == 0 && p.status) atomicExch(p.status, 6);
    return;
  }
  const int past = p.past_len[seq];
  const int kv_len = past + n_new;
  const int kv_head = head / (p.n_heads / p.n_kv_heads);
  const int nq = min(TA_BQ, n_new - q0);
  const int pos_first = past + q0, pos_last = past + q0 + nq - 1;
  int key_lo = 0, key_hi = kv_len - 1;                                   // keys any query of the block can see
  if (p.causal) key_hi = min(key_hi, pos_last);
  if (p.window > 0) key_lo = max(0, pos_first - p.window + 1);
  const int kt_lo = key_lo / TA_BK, kt_hi = key_hi / TA_BK;
  const int n_tiles = kt_hi - kt_lo + 1;

  if (threadIdx.x == 0) {
    ta_bar_init(q_full, 1);
    for (int s = 0; s < TA_STAGES; ++s) {
      ta_bar_init(&k_full[s], 1);
      ta_bar_init(&k_empty[s], 1);
      ta_bar_init(&v_full[s], 1);
      ta_bar_init(&v_empty[s], 1);
    }
    ta_bar_init(&s_full[0], 1);
    ta_bar_init(&s_full[1], 1);
    for (int b = 0; b < 2; ++b) {
      ta_bar_init(&p_ready[b], TA_SOFTMAX_WARPS);
      ta_bar_init(&o_full[b], 1);
      ta_bar_init(&o_free[b], TA_SOFTMAX_WARPS);
    }
    *failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == TA_SOFTMAX_WARPS + 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(ta_smem(tmem_base)), "r"(TA_TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  ta_fence_before();
  __syncthreads();
  ta_fence_after();
  const unsigned tmem_s = *tmem_base, tmem_o = tmem_s + 2 * TA_BK;
  pdl_wait();      // the projections (and the pages) of this step are complete from here on

  if (warp == TA_SOFTMAX_WARPS) {
    if (lane == 0) {
      // ---- producer ----
      ta_bar_expect(q_full, TILE_BYTES);
      for (int cb = 0; cb < CB; ++cb)
        for (int h = 0; h < 2; ++h)
          ta_tma(Qs + cb * 2 * TA_BOX_BYTES + h * TA_BOX_BYTES, &q_map, head * HD + cb * 64, t0 + q0 + h * 64, q_full);
      // where the 64 keys of half h of tile `it` lie: their row in the tensor and the first columns of K and V
      auto where = [&](int it, int h, int& row, int& col_k, int& col_v) {
        const int kt = kt_lo + it;
        if (p.table) {
          // a page is one box; a half tile beyond the sequence's end repeats its last page (masked, but finite)
          const int key = min(kt * TA_BK + h * 64, kv_len - 1);
          const int page = p.table[(long long)seq * p.table_stride + (key / 64) % p.table_len];
          row = (page * p.n_kv_heads + kv_head) * 64;
          col_k = col_v = 0;
        } else {
          row = t0 + kt * TA_BK + h * 64;
          col_k = p.k_col + kv_head * HD;
          col_v = p.v_col + kv_head * HD;
        }
      };
      auto load = [&](int it, bool values) {
        const int s = it % TA_STAGES;
        unsigned long long* bar = values ? &v_full[s] : &k_full[s];
        unsigned char* dst = (values ? Vs : Ks) + s * TILE_BYTES;
        ta_bar_expect(bar, TILE_BYTES);
        for (int h = 0; h < 2; ++h) {
          int row, col_k, col_v;
          where(it, h, row, col_k, col_v);
          for (int cb = 0; cb < CB; ++cb)
            ta_tma(dst + cb * 2 * TA_BOX_BYTES + h * TA_BOX_BYTES, values ? &v_map : &k_map, (values ? col_v : col_k) + cb * 64, row, bar);
        }
      };
      for (int it = 0; it < min(n_tiles, TA_STAGES); ++it) {
        load(it, false);
        load(it, true);
      }
      // a stage of K is free when S of its tile is computed, a stage of V when its P V is
      for (int it = 0; it + TA_STAGES < n_tiles; ++it) {
        const int s = it % TA_STAGES;
        const unsigned parity = (unsigned)(it / TA_STAGES) & 1u;
        if (!ta_bar_wait(&k_empty[s], parity)) {
          *failed = 1;
          break;
        }
        load(it + TA_STAGES, false);
        if (!ta_bar_wait(&v_empty[s], parity)) {
          *failed = 1;
          break;
        }
        load(it + TA_STAGES, true);
      }
    }
  } else if (warp == TA_SOFTMAX_WARPS + 1) {
    if (lane == 0) {
      // ---- issuer ----
      // instruction descriptors: 32-bit accumulator, bfloat16 operands, M = 128; S: N = 128, both K-major;
      // P V: N = HD, the second operand MN-major
      const unsigned idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(TA_BK >> 3) << 17) | ((unsigned)(TA_BQ >> 4) << 24);
      const unsigned idesc_o = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((unsigned)(HD >> 3) << 17) | ((unsigned)(TA_BQ >> 4) << 24);
      // operand descriptors, made once: Q and K per 16 channels, P per 16 keys, V per 16 keys (and stage)
      unsigned long long dq[HD / 16], dk[TA_STAGES][HD / 16], dp[TA_BK / 16], dv[TA_STAGES][TA_BK / 16];
#pragma unroll
      for (int k = 0; k < HD / 16; ++k) {
        dq[k] = ta_desc(Qs + (k / 4) * 2 * TA_BOX_BYTES, 16) + 2ull * (k % 4);
#pragma unroll
        for (int s = 0; s < TA_STAGES; ++s) dk[s][k] = ta_desc(Ks + s * TILE_BYTES + (k / 4) * 2 * TA_BOX_BYTES, 16) + 2ull * (k % 4);
      }
#pragma unroll
      for (int j = 0; j < TA_BK / 16; ++j) {
        dp[j] = ta_desc(Ps + (j / 4) * 2 * TA_BOX_BYTES, 16) + 2ull * (j % 4);      // (the second P tile: 32 KB further)
        // 16 keys further: 16 rows of 128 bytes; the next 64 channels: a whole 128-row box further
#pragma unroll
        for (int s = 0; s < TA_STAGES; ++s) dv[s][j] = ta_desc(Vs + s * TILE_BYTES + j * 16 * 128, 2 * TA_BOX_BYTES);
      }
      // S of tile `it` = Q K^T into accumulator it % 2, when the tile's keys have landed.  (The accumulator is free:
      // the softmax warps had read tile it - 2's before they announced its P.)
      auto scores = [&](int it) -> bool {
        const int s = it % TA_STAGES;
        if (!ta_bar_wait(&k_full[s], (it / TA_STAGES) & 1)) return false;
        ta_fence_after();
        const unsigned d = tmem_s + (unsigned)((it & 1) * TA_BK);
        if (s == 0) {
#pragma unroll
          for (int k = 0; k < HD / 16; ++k) ta_mma(d, dq[k], dk[0][k], idesc_s, k > 0 ? 1u : 0u);
        } else {
#pragma unroll
          for (int k = 0; k < HD / 16; ++k) ta_mma(d, dq[k], dk[1][k], idesc_s, k > 0 ? 1u : 0u);
        }
        ta_commit(&s_full[it & 1]);
        ta_commit(&k_empty[s]);
        return true;
      };
      bool ok = ta_bar_wait(q_full, 0);
      ok = ok && scores(0);
      if (n_tiles > 1) ok = ok && scores(1);
      for (int it = 0; it < n_tiles && ok; ++it) {
        const int s = it % TA_STAGES;
        // O_tile = P V into accumulator it % 2, when P and V lie in shared memory and that accumulator's last
        // contents (tile it - 2) have been taken
        if (!ta_bar_wait(&v_full[s], (it / TA_STAGES) & 1) || !ta_bar_wait(&p_ready[it & 1], (it >> 1) & 1) ||
            (it >= 2 && !ta_bar_wait(&o_free[it & 1], ((it - 2) >> 1) & 1))) {
          ok = false;
          break;
        }
        ta_fence_after();
        if (s == 0) {
#pragma unroll
          for (int j = 0; j < TA_BK / 16; ++j) ta_mma(tmem_o, dp[j], dv[0][j], idesc_o, j > 0 ? 1u : 0u);      // (tile parity 0)
        } else {
#pragma unroll
          for (int j = 0; j < TA_BK / 16; ++j)
            ta_mma(tmem_o + (unsigned)HD, dp[j] + (unsigned long long)((2 * 2 * TA_BOX_BYTES) >> 4), dv[1][j], idesc_o, j > 0 ? 1u : 0u);
        }
        ta_commit(&o_full[it & 1]);
        ta_commit(&v_empty[s]);
        if (it + 2 < n_tiles) ok = scores(it + 2);      // its accumulator was read before P of tile `it` was announced
      }
      if (!ok) *failed = 1;
    }
  } else {
    // ---- softmax: two threads per query row.  Warp w reaches the TMEM lanes of quarter w % 4 (rows 32 (w % 4) ..);
    // warps 0-3 take keys 0-63 of a tile and the lower half of the output channels, warps 4-7 the rest ----
    const int half = warp >> 2;
    const int r = (warp & 3) * 32 + lane;
    const int pos = past + q0 + r;
    const unsigned lane_base = (unsigned)((warp & 3) * 32) << 16;
    float m = -INFINITY, l = 0.f;
    float o[HH];
#pragma unroll
    for (int i = 0; i < HH; ++i) o[i] = 0.f;
    bool ok = true;
    // adds the P V of tile `t` (accumulator t % 2) to this thread's channels and hands the accumulator back
    auto take_o = [&](int t) {
      unsigned a[32], b[32];
      const unsigned addr = tmem_o + (unsigned)((t & 1) * HD) + lane_base + (unsigned)(half * HH);
      if constexpr (HH == 32) {
        ta_ld32_issue(addr, a);
        ta_ld32_issue(addr, b);
        ta_ld_wait(a, b);
#pragma unroll
        for (int i = 0; i < 32; ++i) o[i] += __uint_as_float(a[i]);
      } else {
        ta_ld32_issue(addr, a);
        ta_ld32_issue(addr + 32u, b);
        ta_ld_wait(a, b);
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          o[i] += __uint_as_float(a[i]);
          o[32 + i] += __uint_as_float(b[i]);
        }
      }
      ta_fence_before();
      __syncwarp();
      if (lane == 0) ta_bar_arrive(&o_free[t & 1]);
    };
    // (after a wait has run out the remaining waits are skipped, but every warp still runs every tile: the two
    // warps of a row meet at a barrier in each)
    for (int it = 0; it < n_tiles; ++it) {
      const int key0 = (kt_lo + it) * TA_BK;
      const unsigned s_addr = tmem_s + lane_base + (unsigned)((it & 1) * TA_BK + half * 64);
      if (ok && !ta_bar_wait(&s_full[it & 1], (it >> 1) & 1)) ok = false;
      ta_fence_after();
      // every key of the tile visible to every query of the block?  Then nothing is masked (the common tile).
      const bool whole = key0 + TA_BK <= kv_len && (!p.causal || key0 + TA_BK - 1 <= pos_first) &&
                         (p.window <= 0 || key0 > pos_last - p.window) && p.scale_log2 > 0.f;
      int lo = 0, hi = kv_len - 1;          // this row's visible keys, then relative to this thread's 64 keys
      if (p.causal) hi = min(hi, pos);
      if (p.window > 0) lo = max(0, pos - p.window + 1);
      lo -= key0 + half * 64;
      hi -= key0 + half * 64;
      unsigned a[32], b[32];
      ta_ld32_issue(s_addr, a);
      ta_ld32_issue(s_addr + 32u, b);
      ta_ld_wait(a, b);
      // the row's maximum over this thread's keys, then over the row (the other thread's through shared memory)
      float tile_max = -INFINITY;
      if (whole) {
#pragma unroll
        for (int i = 0; i < 32; ++i) tile_max = fmaxf(tile_max, fmaxf(__uint_as_float(a[i]), __uint_as_float(b[i])));
        tile_max *= p.scale_log2;       // (the scale is positive on this path)
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          tile_max = fmaxf(tile_max, (i >= lo && i <= hi) ? __uint_as_float(a[i]) * p.scale_log2 : -INFINITY);
          tile_max = fmaxf(tile_max, (i + 32 >= lo && i + 32 <= hi) ? __uint_as_float(b[i]) * p.scale_log2 : -INFINITY);
        }
      }
      x_max[((it & 1) * 2 + half) * 128 + r] = tile_max;
      // the two warps of a quarter meet at a barrier of their own (64 threads); both run every tile, see below
      asm volatile("bar.sync %0, 64;\n" ::"r"(1 + (warp & 3)) : "memory");
      tile_max = fmaxf(tile_max, x_max[((it & 1) * 2 + (half ^ 1)) * 128 + r]);
      const float m_new = fmaxf(m, tile_max);
      const float m_use = m_new == -INFINITY ? 0.f : m_new;
      const float alpha = ta_exp2(m - m_use);         // 0 for a row that had seen nothing yet
      // weights, their sum, and P in shared memory: this thread's 64 keys are one box's row of 128 bytes
      float sum = 0.f;
      float va[32], vb[32];
      if (whole) {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          va[i] = ta_exp2(fmaf(__uint_as_float(a[i]), p.scale_log2, -m_use));
          vb[i] = ta_exp2(fmaf(__uint_as_float(b[i]), p.scale_log2, -m_use));
          sum += va[i] + vb[i];
        }
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          va[i] = (i >= lo && i <= hi) ? ta_exp2(fmaf(__uint_as_float(a[i]), p.scale_log2, -m_use)) : 0.f;
          vb[i] = (i + 32 >= lo && i + 32 <= hi) ? ta_exp2(fmaf(__uint_as_float(b[i]), p.scale_log2, -m_use)) : 0.f;
          sum += va[i] + vb[i];
        }
      }
      // (this P tile is free: its last products, of tile it - 2, were waited for before that tile's O was taken)
      unsigned char* box = Ps + (it & 1) * 2 * 2 * TA_BOX_BYTES + half * 2 * TA_BOX_BYTES + r * 128;
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) {
        uint4 x, y;
        x.x = ta_pack(va[8 * ch], va[8 * ch + 1]);
        x.y = ta_pack(va[8 * ch + 2], va[8 * ch + 3]);
        x.z = ta_pack(va[8 * ch + 4], va[8 * ch + 5]);
        x.w = ta_pack(va[8 * ch + 6], va[8 * ch + 7]);
        y.x = ta_pack(vb[8 * ch], vb[8 * ch + 1]);
        y.y = ta_pack(vb[8 * ch + 2], vb[8 * ch + 3]);
        y.z = ta_pack(vb[8 * ch + 4], vb[8 * ch + 5]);
        y.w = ta_pack(vb[8 * ch + 6], vb[8 * ch + 7]);
        *reinterpret_cast<uint4*>(box + ((ch ^ (r & 7)) << 4)) = x;
        *reinterpret_cast<uint4*>(box + (((ch + 4) ^ (r & 7)) << 4)) = y;
      }
      l = l * alpha + sum;
      m = m_new;
      // P is written (generic proxy) and S is read: the issuer may go on
      asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
      ta_fence_before();
      __syncwarp();
      if (lane == 0) ta_bar_arrive(&p_ready[it & 1]);
      // the last tile's P V was computed while this tile's weights were: take it now, then age the sum by this
      // tile's factor
      if (it > 0) {
        if (ok && !ta_bar_wait(&o_full[(it - 1) & 1], ((it - 1) >> 1) & 1)) ok = false;
        ta_fence_after();
        take_o(it - 1);
      }
#pragma unroll
      for (int i = 0; i < HH; ++i) o[i] *= alpha;
    }
    if (ok && !ta_bar_wait(&o_full[(n_tiles - 1) & 1], ((n_tiles - 1) >> 1) & 1)) ok = false;
    ta_fence_after();
    take_o(n_tiles - 1);
    // the row's sum is the two threads' (both hold the same maximum)
    // (through the exchange buffer that the last tile did not use: nobody reads that one any more)
    float* x_sum = x_max + (n_tiles & 1) * 2 * 128;
    x_sum[half * 128 + r] = l;
    asm volatile("bar.sync %0, 64;\n" ::"r"(1 + (warp & 3)) : "memory");
    l += x_sum[(half ^ 1) * 128 + r];
    if (!ok) *failed = 1;
    if (ok && r < nq) {
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* dst = p.out + (long long)(t0 + q0 + r) * ((long long)p.n_heads * HD) + head * HD + half * HH;
#pragma unroll
      for (int c = 0; c < HH; c += 8) {
        uint4 x;
        x.x = ta_pack(o[c] * inv, o[c + 1] * inv);
        x.y = ta_pack(o[c + 2] * inv, o[c + 3] * inv);
        x.z = ta_pack(o[c + 4] * inv, o[c + 5] * inv);
        x.w = ta_pack(o[c + 6] * inv, o[c + 7] * inv);
        *reinterpret_cast<uint4*>(dst + c) = x;
      }
    }
  }
  ta_fence_before();
  __syncthreads();
  if (warp == TA_SOFTMAX_WARPS + 1) {
    ta_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_s), "r"(TA_TMEM_COLS) : "memory");
  }
  if (threadIdx.x == 0 && *failed && p.status) atomicExch(p.status, 6);
}

template <int HD>
static int launch_ta(const CUtensorMap& qm, const CUtensorMap& km, const CUtensorMap& vm, const TaParams& p, int n_seqs, int max_new,
                     cudaStream_t stream) {
  constexpr size_t smem = ta_smem_bytes<HD>();
  auto kern = attention_prefill_tcgen05_kernel<HD>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    BT_CHECK(e == cudaSuccess, "attention_prefill_tcgen05: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
    configured = true;
  }
  const int q_tiles = (max_new + TA_BQ - 1) / TA_BQ;
  BT_CHECK(q_tiles <= 65535, "attention_prefill_tcgen05: %d new tokens in one sequence are too many for one launch", max_new);
  dim3 grid(n_seqs * p.n_heads, q_tiles);
  BT_PDL_OK("attention_prefill_tcgen05", launch_pdl(kern, grid, dim3(TA_THREADS), smem, stream, 1, qm, km, vm, p));
  return 0;
}

}  // namespace bt

// Head sizes and page size the tcgen05 kernel is built for (bfloat16 only).
extern "C" int bt_attention_prefill_tcgen05_supports(int head_dim, int page_size) {
  return (head_dim == 64 || head_dim == 128) && page_size == 64;
}

// q: the step's projections, `q_rows` rows of `q_row_stride` bfloat16; query head h at columns h * head_dim.
// Packed (kv_table null): k and v point at the first key / value column of the same rows.  Paged: k and v are the
// pools [pool_pages][n_kv_heads][64][head_dim].  status: optional int that is set to 6 if a bounded wait ran out.
extern "C" int bt_attention_prefill_tcgen05(const void* q, long long q_rows, long long q_row_stride, const void* k, const void* v,
                                            long long pool_pages, const int* kv_table, int table_stride, int table_len,
                                            int page_size, void* out, int* status, const int* seq_start, const int* past_len,
                                            int n_seqs, int max_new, int n_heads, int n_kv_heads, int head_dim, float scale,
                                            int causal, int window, cudaStream_t stream) {
  using namespace bt;
  BT_CHECK(bt_attention_prefill_tcgen05_supports(head_dim, page_size > 0 ? page_size : 64),
           "attention_prefill_tcgen05: head_dim %d (page size %d) is not supported", head_dim, page_size);
  BT_CHECK(n_heads > 0 && n_kv_heads > 0 && n_heads % n_kv_heads == 0,
           "attention_prefill_tcgen05: %d query heads cannot share %d key heads", n_heads, n_kv_heads);
  BT_CHECK(n_seqs <= 65535 && n_heads <= 65535, "attention_prefill_tcgen05: too many sequences or heads for one launch");
  BT_CHECK(q_row_stride % 8 == 0 && q_rows >= 1, "attention_prefill_tcgen05: rows must be 16-byte aligned");
  if (n_seqs == 0 || max_new == 0) return 0;
  CUtensorMap qm, km, vm;
  if (int rc = tensor_map_2d_bf16(&qm, q, (unsigned long long)q_rows, (unsigned long long)q_row_stride,
                                  (unsigned long long)q_row_stride, 64))
    return rc;
  int k_col = 0, v_col = 0;
  if (kv_table == nullptr) {
    const long long ko = (const __nv_bfloat16*)k - (const __nv_bfloat16*)q, vo = (const __nv_bfloat16*)v - (const __nv_bfloat16*)q;
    BT_CHECK(ko >= 0 && vo >= 0 && ko + (long long)n_kv_heads * head_dim <= q_row_stride && vo + (long long)n_kv_heads * head_dim <= q_row_stride &&
                 ko % 8 == 0 && vo % 8 == 0,
             "attention_prefill_tcgen05: packed keys and values must be 16-byte aligned columns of the query rows");
    k_col = (int)ko;
    v_col = (int)vo;
    km = qm;
    vm = qm;
  } else {
    BT_CHECK(pool_pages >= 1 && table_len >= 1, "attention_prefill_tcgen05: needs the pools' size and the table's length");
    const unsigned long long rows = (unsigned long long)pool_pages * n_kv_heads * 64;
    if (int rc = tensor_map_2d_bf16(&km, k, rows, head_dim, head_dim, 64)) return rc;
    if (int rc = tensor_map_2d_bf16(&vm, v, rows, head_dim, head_dim, 64)) return rc;
  }
  TaParams p{(__nv_bfloat16*)out, seq_start, past_len, kv_table, table_stride, table_len > 0 ? table_len : 1, status,
             n_heads, n_kv_heads, k_col, v_col, scale * 1.4426950408889634f, causal, window};
  if (head_dim == 64) return launch_ta<64>(qm, km, vm, p, n_seqs, max_new, stream);
  return launch_ta<128>(qm, km, vm, p, n_seqs, max_new, stream);
}
