// A whole decode step (at most 16 sequences, one token each, bfloat16) as ONE persistent kernel.
//
// A decode step of a small model is a chain of some sixty short dependent operations; launched one by one each
// costs a launch, a cold start of its weight stream and a tail.  Here one block per SM stays resident for the
// whole step and walks a list of phases that the host wrote once ("phase program"): embedding, then per layer
// [LayerNorm + projection] -> [attention over the pages] -> [merge + projection + residual] ->
// [LayerNorm + feed-forward up + GELU] -> [feed-forward down + residual], then [final norm + readout] and
// token selection.  Between phases the blocks meet at a grid barrier (an atomic counter; the launch is
// cooperative, so all blocks are resident, and the spin is bounded: if it runs out every block records the
// failure and returns).  Before it goes to the barrier a block already asks for what its next phase needs and
// nobody writes during the step: its first weight tiles (into registers) and the parameters of a LayerNorm, or
// its pages of keys and values (tensor-map copies into shared memory) -- so after the barrier the data is there.
// Attention is tensor-core work too (see the attention section below); the readout leaves per-block softmax
// partials so that greedy selection does not read the logits again.
//
// Matrix products: a phase's output columns are dealt out in tiles of 8 to the blocks; the 8 warps of a block
// split K, read their weights [N, K] straight into mma.sync B fragments (16 bytes per lane, see
// linear_stream.cu for the k permutation), take A fragments from a shared-memory panel of the (at most 16) rows,
// and add their partial sums through shared memory in a fixed order.  The rows' panel is built once per block
// and phase: copied, LayerNorm-ed (32-bit statistics, two passes), or merged from the attention phase's partial
// results.  Nothing is accumulated with atomics: results do not depend on timing.
#include "common.cuh"
#include "sampling.cuh"
#include "tma.cuh"
#include "decode_mma.cuh"

namespace bt {

constexpr int DS_THREADS = 256, DS_WARPS = 8;
constexpr int DS_SPIN_LIMIT = 1 << 22;      // polls of the grid barrier's counter before a block gives up
constexpr int DS_NB = 12;            // 32-wide k blocks a warp holds in registers at a time
constexpr int DS_MAX_SLOTS = 16;     // page slots (keys and values of a page) of a block's ring, at most
constexpr int DS_SLOT_BYTES_TOTAL = 128 * 1024;   // (shared memory is taken from the L1 cache, which the streamed weights need)
constexpr int DS_COPY_SPIN_LIMIT = 1 << 18;       // tries of a copy barrier (each may itself wait a while) before a warp gives up
constexpr int DS_TABLE_CACHE = 64;   // page-table entries per sequence the block keeps in shared memory

enum { PH_EMBED = 0, PH_LINEAR = 1, PH_ATTENTION = 2, PH_SAMPLE = 3 };
enum { A_ROWS = 0, A_LAYERNORM = 1, A_MERGE = 2 };

struct Phase {
  int type;
  // ---- linear: out[M,N] = act(A @ w^T + bias) (+ residual) ----
  int a_kind, M, N, K, act, out_is_f32;
  const __nv_bfloat16* a;        // A_ROWS: [M, K]
  const float* x32;              // A_LAYERNORM: rows to normalise, row r = rows ? rows[r] : r
  const int* rows;
  const float* gamma;
  const float* beta;
  float eps;
  const float* part;             // A_MERGE: [M * n_heads * n_splits][head_dim + 4] (values, max, sum, 2 unused) from the attention phase
  int n_splits, n_heads, head_dim;
  const __nv_bfloat16* w;        // [N, K]
  const float* bias;
  const float* residual;
  void* out;
  float* track;                  // optional [M][blocks][4]: every block's (max, sum of exp(. - max), first argmax) of the rows of `out`
  // ---- attention (writes `part_out` in the A_MERGE layout) ----
  const __nv_bfloat16* q;        // rows of the projections: query head h at q + h * head_dim
  long long q_stride;
  const __nv_bfloat16* new_k;    // the new token's key / value channels in the same rows (null: already filed)
  const __nv_bfloat16* new_v;
  __nv_bfloat16* k_pool;         // [page][kv_head][64][head_dim]
  __nv_bfloat16* v_pool;
  const int* table;
  int table_stride, table_len;
  const int* ctx_len;
  int n_kv_heads;
  float scale_log2;
  int window;
  float* part_out;
  // ---- embed ----
  const int* tokens;
  const int* positions;
  const __nv_bfloat16* wte;
  const __nv_bfloat16* wpe;
  float* resid_out;
  int width, vocab, n_positions;
  // ---- sample (and advance) ----
  const float* logits;
  int do_sample;
  float temperature;
  int top_k;
  float top_p, min_p;
  const unsigned long long* seeds;
  int* counters;
  int* out_ids;
  float* out_logp;
  int* adv_tokens;
  int* adv_positions;
  int* adv_past;
  int* adv_ctx;
  const float* partials;         // greedy selection from the readout's `track` instead of from the logits
  int n_partials;
  int pad0_;
  long long pad1_;
  // ---- attention: tensor maps of the layer's key and value pools, seen as [pages * kv_heads * 64 rows][head_dim] ----
  alignas(64) CUtensorMap k_map;
  CUtensorMap v_map;
};
static_assert(sizeof(Phase) % 64 == 0, "tensor maps in an array of phases stay on 64-byte boundaries");

__device__ __forceinline__ unsigned ds_ld_acquire(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float ds_ld_cg(const float* p) { return __ldcg(p); }
__device__ __forceinline__ uint4 ds_ld_stream16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ void ds_unpack8(const uint4& v, float (&f)[8]) {
  const unsigned w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}

constexpr int DS_MAX_ITEMS = 8;      // (sequence, head, split) items of an attention phase a block takes, at most
struct AttnItem {
  int seq, head, split, L, lo, pg_first, pg_end;   // pages [pg_first, pg_end)
};
struct AttnWork {
  AttnItem it[DS_MAX_ITEMS];
  int start[DS_MAX_ITEMS + 2];     // where each item's pages begin in the block's stream of pages; [n]: their number
  int n;
  // what the list was made for: the layers of a model ask for the same list again and again within a step
  const int* for_ctx;
  const int* for_table;
  int for_shape[6];
};

struct StepShared {
  int ok;                          // result of the last bounded wait
  float red[DS_WARPS][4][32][4];   // partial sums of the warps, per tile of a group
  float stats[16][2];
  float ml[2][DS_WARPS][2];
  SampleShared sample;
  alignas(64) Phase phase[2];
  AttnWork work;
  // lengths and page tables of the step's sequences (the same in every layer of a cache group), read once
  const int* ctx_src;
  const int* table_src;
  int ctx_cache[16];
  int table_cache[16][DS_TABLE_CACHE];
  float trk[4][16][3];             // the finishing warps' (max, sum, argmax) of every row
  unsigned long long bars[DS_MAX_SLOTS];   // completion of the bulk copies into each page slot
  long long* trace;
};

// Optional timeline of block 0: slot 0 a phase's begin, 1 its end, 2.. points inside it (nanoseconds).
constexpr int DS_TRACE_SLOTS = 8;
__device__ __forceinline__ void ds_stamp(StepShared& sh, int slot) {
  if (threadIdx.x == 0 && sh.trace) {
    long long t;
    asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t));
    sh.trace[slot] = t;
  }
}

// All blocks meet here.  `target`: how many arrivals the counter shows when everyone of this barrier has come.
// In two halves, so that a block can ask for the next phase's constants between its arrival and its wait: the
// release of the arrival then does not have to wait for those loads.
__device__ __forceinline__ void ds_grid_arrive(unsigned* counter) {
  __syncthreads();
  // release: everything this block wrote is visible before its arrival is
  if (threadIdx.x == 0) asm volatile("red.release.gpu.global.add.u32 [%0], 1;\n" ::"l"(counter) : "memory");
}
__device__ bool ds_grid_wait(unsigned* counter, unsigned target, StepShared& sh) {
  if (threadIdx.x == 0) {
    int ok = 1, spins = 0;      // acquire on the way out
    while (ds_ld_acquire(counter) < target) {
      if (++spins > DS_SPIN_LIMIT) {
        ok = 0;
        break;
      }
    }
    sh.ok = ok;
  }
  __syncthreads();
  return sh.ok != 0;
}

// Stride (in elements) of the rows' panel: rows 64 bytes apart modulo 128, so that the 16-byte fragment reads
// of two neighbouring rows fall into different halves of the banks.
__device__ __forceinline__ int ds_panel_stride(int K) {
  int bytes = K * 2;
  bytes += (64 - (bytes % 128) + 128) % 128;
  return bytes / 2;
}

// The kernel exists in several builds.  The general one holds the code for every length of product and every head
// size; the others hold only what a common model shape needs (PWA, PWB: the two values of ds_blocks_per_warp its
// products have; HDMAX: its largest head size), which keeps the code a step runs through small and close
// together: the instruction cache is a measurable part of the step.  PWA < 0: everything.
template <int PWA, int PWB>
__device__ __forceinline__ constexpr bool ds_built(int pw) { return PWA < 0 || pw == PWA || pw == PWB; }

// ---- the rows' panel -------------------------------------------------------------------------------------
// Asynchronous 16-byte copies from global memory (through the L2 cache only: other blocks wrote the data during
// this launch) into shared memory: all of a thread's copies are in flight together.
__device__ __forceinline__ void ds_cp16(const void* smem_dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(ds_smem(smem_dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void ds_cp_wait() { asm volatile("cp.async.wait_all;\n" ::: "memory"); }

// Shared memory of a linear phase: the panel (8 or 16 rows of bfloat16), then what the panel is made from
// (LayerNorm: the rows in 32-bit, gamma, beta; merge: the attention phase's partials).
__device__ __host__ __forceinline__ long long ds_panel_bytes(int K, int M) {
  long long row = (long long)K * 2;
  row += (64 - (row % 128) + 128) % 128;
  return (M > 8 ? 16 : 8) * row;        // the second eight rows are read only when there are more than eight
}
__device__ __host__ __forceinline__ long long ds_linear_smem(const Phase& ph) {
  long long bytes = ds_panel_bytes(ph.K, ph.M);
  if (ph.a_kind == A_LAYERNORM) bytes += ((long long)ph.M + 2) * ph.K * 4;
  if (ph.a_kind == A_MERGE) bytes += (long long)ph.M * ph.n_heads * ph.n_splits * (ph.head_dim + 4) * 4;
  return bytes;
}
__device__ __forceinline__ float* ds_norm_params(const Phase& ph, unsigned char* smem) {   // gamma[K], beta[K]
  return reinterpret_cast<float*>(smem + ds_panel_bytes(ph.K, ph.M)) + (long long)ph.M * ph.K;
}
// gamma and beta never change: they can be asked for before the grid barrier that precedes the phase
__device__ __forceinline__ void ds_prefetch_norm_params(const Phase& ph, unsigned char* smem) {
  float* gs = ds_norm_params(ph, smem);
  const int vecs = ph.K / 4;
  for (int i = threadIdx.x; i < vecs; i += DS_THREADS) {
    ds_cp16(gs + i * 4, ph.gamma + i * 4);
    if (ph.beta) ds_cp16(gs + ph.K + i * 4, ph.beta + i * 4);
  }
}

// LayerNorm of one row per warp, the row held in registers (J vectors of four per lane): mean, then the variance
// about it, then the normalised row goes into the panel as bfloat16.
template <int J>
__device__ __forceinline__ void ds_layernorm_row(const float* __restrict__ src, bool live, int K, float eps, const float* gs,
                                                 const float* bs, __nv_bfloat16* dst) {
  const int lane = threadIdx.x & 31;
  float4 v[J];
#pragma unroll
  for (int j = 0; j < J; ++j) {
    const int c = lane * 4 + j * 128;
    v[j] = (live && c < K) ? __ldcg(reinterpret_cast<const float4*>(src + c)) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  float s = 0.f;
#pragma unroll
  for (int j = 0; j < J; ++j) s += (v[j].x + v[j].y) + (v[j].z + v[j].w);
  const float mean = warp_sum(s) / (float)K;
  float d2 = 0.f;
#pragma unroll
  for (int j = 0; j < J; ++j) {
    if (lane * 4 + j * 128 < K) {
      const float a = v[j].x - mean, b = v[j].y - mean, c = v[j].z - mean, d = v[j].w - mean;
      d2 += (a * a + b * b) + (c * c + d * d);
    }
  }
  const float rs = 1.f / sqrtf(warp_sum(d2) / (float)K + eps);
  if (!live) return;
#pragma unroll
  for (int j = 0; j < J; ++j) {
    const int c = lane * 4 + j * 128;
    if (c < K) {
      const float4 g4 = *reinterpret_cast<const float4*>(gs + c);
      float4 b4 = make_float4(0.f, 0.f, 0.f, 0.f);
      if (bs) b4 = *reinterpret_cast<const float4*>(bs + c);
      uint2 packed;
      packed.x = ds_pack((v[j].x - mean) * rs * g4.x + b4.x, (v[j].y - mean) * rs * g4.y + b4.y);
      packed.y = ds_pack((v[j].z - mean) * rs * g4.z + b4.z, (v[j].w - mean) * rs * g4.w + b4.w);
      *reinterpret_cast<uint2*>(dst + c) = packed;
    }
  }
}

template <int PWA, int PWB>
__device__ void ds_build_panel(const Phase& ph, unsigned char* smem, StepShared& sh, bool params_asked) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int K = ph.K, KP = ds_panel_stride(K), M = ph.M;
  __nv_bfloat16* As = reinterpret_cast<__nv_bfloat16*>(smem);
  float* stage = reinterpret_cast<float*>(smem + ds_panel_bytes(K, M));
  // rows at and beyond M are never written: their products land in rows of the result that are not stored
  if (ph.a_kind == A_ROWS) {
    const __nv_bfloat16* a = ph.a;
    for (int r = warp; r < M; r += DS_WARPS) {
#pragma unroll 4
      for (int c = lane * 8; c < K; c += 256) ds_cp16(As + r * KP + c, a + (long long)r * K + c);
    }
    ds_cp_wait();
  } else if (ph.a_kind == A_LAYERNORM) {
    if (!params_asked) ds_prefetch_norm_params(ph, smem);
    const float* x32 = ph.x32;
    const int* rows = ph.rows;
    const float eps = ph.eps;
    const float* gs = stage + (long long)M * K;
    const float* bs = ph.beta ? gs + K : nullptr;
    if (K <= 13 * 128) {
      // the parameters were asked for long ago; the rows go from global memory straight into registers
      ds_cp_wait();
      __syncthreads();
      for (int r0 = 0; r0 < M; r0 += DS_WARPS) {
        const int r = r0 + warp;
        const bool live = r < M;
        const float* src = x32 + (long long)(live ? (rows ? rows[r] : r) : 0) * K;
        // (rows of K <= 512, <= 1024, <= 1664 have products of 1..2, 3..4, 6..12 blocks per warp)
        if constexpr (ds_built<PWA, PWB>(1) || ds_built<PWA, PWB>(2))
          if (K <= 4 * 128) ds_layernorm_row<4>(src, live, K, eps, gs, bs, As + r * KP);
        if constexpr (ds_built<PWA, PWB>(3) || ds_built<PWA, PWB>(4))
          if (K > 4 * 128 && K <= 8 * 128) ds_layernorm_row<8>(src, live, K, eps, gs, bs, As + r * KP);
        if constexpr (ds_built<PWA, PWB>(6) || ds_built<PWA, PWB>(12))
          if (K > 8 * 128) ds_layernorm_row<13>(src, live, K, eps, gs, bs, As + r * KP);
      }
    } else {
      // rows too long for registers: staged in shared memory, one warp to a row
      for (int r = warp; r < M; r += DS_WARPS) {
        const float* src = x32 + (long long)(rows ? rows[r] : r) * K;
#pragma unroll 4
        for (int c = lane * 4; c < K; c += 128) ds_cp16(stage + r * K + c, src + c);
      }
      ds_cp_wait();
      __syncthreads();
      for (int r = warp; r < M; r += DS_WARPS) {
        const float* src = stage + r * K;
        float s = 0.f;
        for (int c = lane * 4; c < K; c += 128) {
          const float4 v = *reinterpret_cast<const float4*>(src + c);
          s += (v.x + v.y) + (v.z + v.w);
        }
        const float mean = warp_sum(s) / (float)K;
        float d2 = 0.f;
        for (int c = lane * 4; c < K; c += 128) {
          const float4 v = *reinterpret_cast<const float4*>(src + c);
          const float a = v.x - mean, b = v.y - mean, cc = v.z - mean, d = v.w - mean;
          d2 += (a * a + b * b) + (cc * cc + d * d);
        }
        const float rs = 1.f / sqrtf(warp_sum(d2) / (float)K + eps);
        for (int c = lane * 4; c < K; c += 128) {
          const float4 v = *reinterpret_cast<const float4*>(src + c);
          const float4 g4 = *reinterpret_cast<const float4*>(gs + c);
          float4 b4 = make_float4(0.f, 0.f, 0.f, 0.f);
          if (bs) b4 = *reinterpret_cast<const float4*>(bs + c);
          uint2 packed;
          packed.x = ds_pack((v.x - mean) * rs * g4.x + b4.x, (v.y - mean) * rs * g4.y + b4.y);
          packed.y = ds_pack((v.z - mean) * rs * g4.z + b4.z, (v.w - mean) * rs * g4.w + b4.w);
          *reinterpret_cast<uint2*>(As + r * KP + c) = packed;
        }
      }
    }
  } else {  // A_MERGE: the attention phase's partial (weighted values, max, sum) of every split, added up
    const int hd = ph.head_dim, S = ph.n_splits, H = ph.n_heads, unit_floats = hd + 4;   // a multiple of four floats: units stay 16-byte aligned
    const float* part = ph.part;
    const int cpr = hd / 8, per_row = H * cpr;                 // 16-byte chunks of a head, of a row
    if (S <= 4) {
      // few splits: a thread loads everything its 8 dims need straight from global memory, all loads in flight
      // together (one trip to the L2 cache instead of a copy, two passes and their hand-overs)
      for (int i = tid; i < M * per_row; i += DS_THREADS) {
        const int r = i / per_row, j = i - r * per_row;
        const int h = j / cpr, ch = j - h * cpr;
        const float* base = part + ((long long)(r * H + h) * S) * unit_floats;
        float ms[4], ls[4];
        float4 p0[4], p1[4];
#pragma unroll
        for (int s2 = 0; s2 < 4; ++s2) {
          if (s2 < S) {
            const float2 ml = __ldcg(reinterpret_cast<const float2*>(base + s2 * unit_floats + hd));
            ms[s2] = ml.x;
            ls[s2] = ml.y;
            p0[s2] = __ldcg(reinterpret_cast<const float4*>(base + s2 * unit_floats + ch * 8));
            p1[s2] = __ldcg(reinterpret_cast<const float4*>(base + s2 * unit_floats + ch * 8 + 4));
          } else {
            ms[s2] = -INFINITY;
            ls[s2] = 0.f;
            p0[s2] = p1[s2] = make_float4(0.f, 0.f, 0.f, 0.f);
          }
        }
        const float mx = fmaxf(fmaxf(ms[0], ms[1]), fmaxf(ms[2], ms[3]));
        float L = 0.f, wgt[4];
#pragma unroll
        for (int s2 = 0; s2 < 4; ++s2) {
          wgt[s2] = ms[s2] == -INFINITY ? 0.f : ds_exp2(ms[s2] - mx);
          L += ls[s2] * wgt[s2];
        }
        const float inv = L > 0.f ? 1.f / L : 0.f;
        float o[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int s2 = 0; s2 < 4; ++s2) {
          const float w2 = wgt[s2] * inv;
          o[0] += p0[s2].x * w2; o[1] += p0[s2].y * w2; o[2] += p0[s2].z * w2; o[3] += p0[s2].w * w2;
          o[4] += p1[s2].x * w2; o[5] += p1[s2].y * w2; o[6] += p1[s2].z * w2; o[7] += p1[s2].w * w2;
        }
        uint4 packed;
        packed.x = ds_pack(o[0], o[1]);
        packed.y = ds_pack(o[2], o[3]);
        packed.z = ds_pack(o[4], o[5]);
        packed.w = ds_pack(o[6], o[7]);
        *reinterpret_cast<uint4*>(As + r * KP + h * hd + ch * 8) = packed;
      }
      __syncthreads();
      return;
    }
    const int vecs = M * H * S * (unit_floats / 4);
#pragma unroll 4
    for (int i = tid; i < vecs; i += DS_THREADS) ds_cp16(stage + i * 4, part + i * 4);
    ds_cp_wait();
    __syncthreads();
    // the weight of every split (exp2(max - row max) / sum) replaces its maximum; then the weighted values are added
    for (int u = tid; u < M * H; u += DS_THREADS) {
      float* base = stage + (long long)u * S * unit_floats;
      float mx = -INFINITY;
      for (int s2 = 0; s2 < S; ++s2) mx = fmaxf(mx, base[s2 * unit_floats + hd]);
      float L = 0.f;
      for (int s2 = 0; s2 < S; ++s2) {
        const float ms = base[s2 * unit_floats + hd];
        if (ms != -INFINITY) L += base[s2 * unit_floats + hd + 1] * ds_exp2(ms - mx);
      }
      const float inv = L > 0.f ? 1.f / L : 0.f;
      for (int s2 = 0; s2 < S; ++s2) {
        const float ms = base[s2 * unit_floats + hd];
        base[s2 * unit_floats + hd] = ms == -INFINITY ? 0.f : ds_exp2(ms - mx) * inv;
      }
    }
    __syncthreads();
    for (int i = tid; i < M * per_row; i += DS_THREADS) {
      const int r = i / per_row, j = i - r * per_row;
      const int h = j / cpr, ch = j - h * cpr;
      const float* base = stage + ((long long)(r * H + h) * S) * unit_floats;
      float o[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int s2 = 0; s2 < S; ++s2) {
        const float wgt = base[s2 * unit_floats + hd];
        const float4 p0 = *reinterpret_cast<const float4*>(base + s2 * unit_floats + ch * 8);
        const float4 p1 = *reinterpret_cast<const float4*>(base + s2 * unit_floats + ch * 8 + 4);
        o[0] += p0.x * wgt; o[1] += p0.y * wgt; o[2] += p0.z * wgt; o[3] += p0.w * wgt;
        o[4] += p1.x * wgt; o[5] += p1.y * wgt; o[6] += p1.z * wgt; o[7] += p1.w * wgt;
      }
      uint4 packed;
      packed.x = ds_pack(o[0], o[1]);
      packed.y = ds_pack(o[2], o[3]);
      packed.z = ds_pack(o[4], o[5]);
      packed.w = ds_pack(o[6], o[7]);
      *reinterpret_cast<uint4*>(As + r * KP + h * hd + ch * 8) = packed;
    }
  }
  __syncthreads();
}

// Weights of a group of 8-column tiles: this warp's k blocks (wk, wk + 8, ...) of each tile, 16 bytes per lane.
// PW: k blocks per warp and tile; TPG tiles per group; register i * TPG + t holds block i of tile t.
template <int PW, int TPG, int NREG>
__device__ __forceinline__ void ds_load_group(const Phase& ph, int first_tile, int tile_stride, int n_tiles, int first_block,
                                              uint4 (&wv)[NREG]) {
  const int lane = threadIdx.x & 31, wk = threadIdx.x >> 5;
  const int g = lane >> 2, q = lane & 3;
#pragma unroll
  for (int t = 0; t < TPG; ++t) {
    const int tile = first_tile + t * tile_stride;
    const int n = tile * 8 + g;
    const bool n_ok = tile < n_tiles && n < ph.N;
    const __nv_bfloat16* wrow = ph.w + (long long)(n_ok ? n : 0) * ph.K;
#pragma unroll
    for (int i = 0; i < PW; ++i) {
      const int kc = (wk + 8 * (first_block + i)) * 32 + q * 8;
      wv[i * TPG + t] = (n_ok && kc < ph.K) ? ds_ld_stream16(wrow + kc) : make_uint4(0, 0, 0, 0);
    }
  }
}

// Running (max, sum of exp(value - max), first index of the max) of the values a thread has finished, for two rows.
struct Track {
  float m[2], l[2];
  int idx[2];
};
__device__ __forceinline__ void ds_track_merge(float& m, float& l, int& idx, float m2, float l2, int idx2) {
  if (m2 > m || (m2 == m && idx2 < idx)) idx = idx2;
  const float mm = fmaxf(m, m2);
  l = mm == -INFINITY ? 0.f : l * expf(m - mm) + l2 * expf(m2 - mm);
  m = mm;
}

// Bias and residual of the elements warp t will finish in tile t of a group: asked for before the products.
template <int TPG>
__device__ __forceinline__ void ds_finish_operands(const Phase& ph, int first_tile, int tile_stride, int n_tiles,
                                                   float (&bias)[4], float (&res)[4]) {
  const int lane = threadIdx.x & 31, wk = threadIdx.x >> 5;
  const int g = lane >> 2, q = lane & 3;
#pragma unroll
  for (int i = 0; i < 4; ++i) bias[i] = res[i] = 0.f;
  if (wk < TPG) {
    const int tile = first_tile + wk * tile_stride;
    if (tile < n_tiles) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int r = g + (i >> 1) * 8;
        const int c = tile * 8 + 2 * q + (i & 1);
        if (r < ph.M && c < ph.N) {
          if (ph.bias) bias[i] = ph.bias[c];
          if (ph.residual) res[i] = ds_ld_cg(ph.residual + (long long)r * ph.N + c);
        }
      }
    }
  }
}

// Sum of the warps' partial tiles, bias, activation, residual, store: warp t finishes tile t of the group.
template <int TPG>
__device__ __forceinline__ void ds_finish_group(const Phase& ph, StepShared& sh, int first_tile, int tile_stride, int n_tiles,
                                                const float (&bias)[4], const float (&res)[4], Track& trk) {
  const int lane = threadIdx.x & 31, wk = threadIdx.x >> 5;
  const int g = lane >> 2, q = lane & 3;
  if (wk < TPG) {
    const int tile = first_tile + wk * tile_stride;
    if (tile < n_tiles) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int r = g + (i >> 1) * 8;
        const int c = tile * 8 + 2 * q + (i & 1);
        if (r < ph.M && c < ph.N) {
          const long long o = (long long)r * ph.N + c;
          float v = 0.f;
#pragma unroll
          for (int w = 0; w < DS_WARPS; ++w) v += sh.red[w][wk][lane][i];
          v = apply_activation(v + bias[i], ph.act) + res[i];
          if (ph.track) {          // columns come to a thread in rising order: the first maximum stays
            float& m = trk.m[i >> 1];
            if (v > m) {
              trk.l[i >> 1] = trk.l[i >> 1] * expf(m - v) + 1.f;
              m = v;
              trk.idx[i >> 1] = c;
            } else if (m != -INFINITY) {
              trk.l[i >> 1] += expf(v - m);
            }
          }
          if (ph.out_is_f32)
            reinterpret_cast<float*>(ph.out)[o] = v;
          else
            reinterpret_cast<__nv_bfloat16*>(ph.out)[o] = __float2bfloat16_rn(v);
        }
      }
    }
  }
}

// A block's tiles are blockIdx.x, blockIdx.x + grid, ...; TPG of them are computed together: their weights are in
// flight together and the rows' fragments are read once for all of them.  The first group's finishing operands
// (`bias0`, `res0`) were asked for before the panel was built.
template <int PW>
__device__ void ds_linear_tiles(const Phase& ph, const __nv_bfloat16* As, StepShared& sh, uint4 (&wpre)[DS_NB], bool have_pre,
                                float (&bias)[4], float (&res)[4], Track& trk) {
  constexpr int TPG = (DS_NB / PW) < 4 ? (DS_NB / PW) : 4;
  const int lane = threadIdx.x & 31, wk = threadIdx.x >> 5;
  const int g = lane >> 2, q = lane & 3;
  const int KP = ds_panel_stride(ph.K);
  const int n_tiles = (ph.N + 7) / 8;
  const int stride = gridDim.x;
  const bool two_rows = ph.M > 8;
  uint4 (&wv)[DS_NB] = wpre;       // the prefetched group is multiplied where it is
  if (!have_pre) ds_load_group<PW, TPG>(ph, blockIdx.x, stride, n_tiles, 0, wv);
  for (int first = blockIdx.x; first < n_tiles; first += TPG * stride) {
    if (first != (int)blockIdx.x) ds_finish_operands<TPG>(ph, first, stride, n_tiles, bias, res);
    float acc[TPG][4];
#pragma unroll
    for (int t = 0; t < TPG; ++t)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[t][i] = 0.f;
#pragma unroll
    for (int i = 0; i < PW; ++i) {
      const int kc = (wk + 8 * i) * 32 + q * 8;
      uint4 lo = make_uint4(0, 0, 0, 0), hi = lo;
      if (kc < ph.K) {
        lo = *reinterpret_cast<const uint4*>(As + g * KP + kc);
        if (two_rows) hi = *reinterpret_cast<const uint4*>(As + (g + 8) * KP + kc);
      }
#pragma unroll
      for (int t = 0; t < TPG; ++t) {
        ds_mma(acc[t], lo.x, hi.x, lo.y, hi.y, wv[i * TPG + t].x, wv[i * TPG + t].y);
        ds_mma(acc[t], lo.z, hi.z, lo.w, hi.w, wv[i * TPG + t].z, wv[i * TPG + t].w);
      }
    }
    // the registers of the weights are free again: the next group's travel while this one is finished
    if (first + TPG * stride < n_tiles) ds_load_group<PW, TPG>(ph, first + TPG * stride, stride, n_tiles, 0, wv);
#pragma unroll
    for (int t = 0; t < TPG; ++t)
#pragma unroll
      for (int i = 0; i < 4; ++i) sh.red[wk][t][lane][i] = acc[t][i];
    __syncthreads();
    ds_stamp(sh, 3);
    ds_finish_group<TPG>(ph, sh, first, stride, n_tiles, bias, res, trk);
    __syncthreads();
    ds_stamp(sh, 4);
  }
}

// K so long that a warp's share of a tile does not fit in registers at once: one tile at a time, K in pieces.
__device__ void ds_linear_tiles_long(const Phase& ph, const __nv_bfloat16* As, StepShared& sh, Track& trk) {
  const int lane = threadIdx.x & 31, wk = threadIdx.x >> 5;
  const int g = lane >> 2, q = lane & 3;
  const int KP = ds_panel_stride(ph.K);
  const int n_tiles = (ph.N + 7) / 8;
  const int per_warp = ((ph.K + 31) / 32 + DS_WARPS - 1) / DS_WARPS;
  const bool two_rows = ph.M > 8;
  for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
    float bias[4], res[4];
    ds_finish_operands<1>(ph, tile, 1, n_tiles, bias, res);
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int first = 0; first < per_warp; first += DS_NB) {
      uint4 wv[DS_NB];
      ds_load_group<DS_NB, 1>(ph, tile, 1, n_tiles, first, wv);
#pragma unroll
      for (int i = 0; i < DS_NB; ++i) {
        const int kc = (wk + 8 * (first + i)) * 32 + q * 8;
        uint4 lo = make_uint4(0, 0, 0, 0), hi = lo;
        if (kc < ph.K) {
          lo = *reinterpret_cast<const uint4*>(As + g * KP + kc);
          if (two_rows) hi = *reinterpret_cast<const uint4*>(As + (g + 8) * KP + kc);
        }
        ds_mma(acc, lo.x, hi.x, lo.y, hi.y, wv[i].x, wv[i].y);
        ds_mma(acc, lo.z, hi.z, lo.w, hi.w, wv[i].z, wv[i].w);
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) sh.red[wk][0][lane][i] = acc[i];
    __syncthreads();
    ds_finish_group<1>(ph, sh, tile, 1, n_tiles, bias, res, trk);
    __syncthreads();
  }
}

// k blocks per warp and tile, rounded up to a size the tiles are built for (0: too long for registers)
__device__ __forceinline__ int ds_blocks_per_warp(int K) {
  const int pw = ((K + 31) / 32 + DS_WARPS - 1) / DS_WARPS;
  return pw <= 1 ? 1 : pw <= 2 ? 2 : pw <= 3 ? 3 : pw <= 4 ? 4 : pw <= 6 ? 6 : pw <= 12 ? 12 : 0;
}

// The first group of weights of a phase, asked for before the phase's grid barrier.
template <int PWA, int PWB>
__device__ __forceinline__ bool ds_prefetch_weights(const Phase& ph, uint4 (&wpre)[DS_NB]) {
  const int n_tiles = (ph.N + 7) / 8;
  if ((int)blockIdx.x >= n_tiles) return false;
  const int pw = ds_blocks_per_warp(ph.K);
  if constexpr (ds_built<PWA, PWB>(1)) if (pw == 1) { ds_load_group<1, 4>(ph, blockIdx.x, gridDim.x, n_tiles, 0, wpre); return true; }
  if constexpr (ds_built<PWA, PWB>(2)) if (pw == 2) { ds_load_group<2, 4>(ph, blockIdx.x, gridDim.x, n_tiles, 0, wpre); return true; }
  if constexpr (ds_built<PWA, PWB>(3)) if (pw == 3) { ds_load_group<3, 4>(ph, blockIdx.x, gridDim.x, n_tiles, 0, wpre); return true; }
  if constexpr (ds_built<PWA, PWB>(4)) if (pw == 4) { ds_load_group<4, 3>(ph, blockIdx.x, gridDim.x, n_tiles, 0, wpre); return true; }
  if constexpr (ds_built<PWA, PWB>(6)) if (pw == 6) { ds_load_group<6, 2>(ph, blockIdx.x, gridDim.x, n_tiles, 0, wpre); return true; }
  if constexpr (ds_built<PWA, PWB>(12)) if (pw == 12) { ds_load_group<12, 1>(ph, blockIdx.x, gridDim.x, n_tiles, 0, wpre); return true; }
  return false;
}

// The block's (max, sum, argmax) of every row: the four lanes that share a row, then the finishing warps.
__device__ void ds_track_write(const Phase& ph, StepShared& sh, Track& trk) {
  const int lane = threadIdx.x & 31, wk = threadIdx.x >> 5;
  const int g = lane >> 2, q = lane & 3;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
#pragma unroll
    for (int o = 1; o <= 2; o <<= 1) {
      const float m2 = __shfl_xor_sync(0xffffffffu, trk.m[h], o);
      const float l2 = __shfl_xor_sync(0xffffffffu, trk.l[h], o);
      const int i2 = __shfl_xor_sync(0xffffffffu, trk.idx[h], o);
      ds_track_merge(trk.m[h], trk.l[h], trk.idx[h], m2, l2, i2);
    }
    if (wk < 4 && q == 0) {
      sh.trk[wk][g + 8 * h][0] = trk.m[h];
      sh.trk[wk][g + 8 * h][1] = trk.l[h];
      sh.trk[wk][g + 8 * h][2] = __int_as_float(trk.idx[h]);
    }
  }
  __syncthreads();
  if ((int)threadIdx.x < ph.M && threadIdx.x < 16) {
    const int r = threadIdx.x;
    float m = sh.trk[0][r][0], l = sh.trk[0][r][1];
    int idx = __float_as_int(sh.trk[0][r][2]);
    for (int w = 1; w < 4; ++w) ds_track_merge(m, l, idx, sh.trk[w][r][0], sh.trk[w][r][1], __float_as_int(sh.trk[w][r][2]));
    float* dst = ph.track + ((long long)r * gridDim.x + blockIdx.x) * 4;
    dst[0] = m;
    dst[1] = l;
    dst[2] = __int_as_float(idx);
  }
  __syncthreads();
}

// tiles of a group for a K of this many blocks per warp
__device__ __forceinline__ int ds_tiles_per_group(int pw) { return pw == 0 ? 1 : (DS_NB / pw < 4 ? DS_NB / pw : 4); }

template <int PWA, int PWB>
__device__ void ds_linear_phase(const Phase& ph, unsigned char* smem, StepShared& sh, uint4 (&wpre)[DS_NB], bool have_pre,
                                bool params_asked) {
  const __nv_bfloat16* As = reinterpret_cast<const __nv_bfloat16*>(smem);
  const int n_tiles = (ph.N + 7) / 8;
  Track trk;
  trk.m[0] = trk.m[1] = -INFINITY;
  trk.l[0] = trk.l[1] = 0.f;
  trk.idx[0] = trk.idx[1] = 0x7fffffff;
  if ((int)blockIdx.x >= n_tiles) {      // nothing to do in this phase (uniform for the block)
    if (params_asked) ds_cp_wait();
    if (ph.track) ds_track_write(ph, sh, trk);
    return;
  }
  const int pw = ds_blocks_per_warp(ph.K);
  float bias[4], res[4];
  // the first group's finishing operands travel while the panel is built (4, 4, 4, 3, 2, 1 tiles to a group)
  if constexpr (ds_built<PWA, PWB>(1) || ds_built<PWA, PWB>(2) || ds_built<PWA, PWB>(3))
    if (pw >= 1 && pw <= 3) ds_finish_operands<4>(ph, blockIdx.x, gridDim.x, n_tiles, bias, res);
  if constexpr (ds_built<PWA, PWB>(4)) if (pw == 4) ds_finish_operands<3>(ph, blockIdx.x, gridDim.x, n_tiles, bias, res);
  if constexpr (ds_built<PWA, PWB>(6)) if (pw == 6) ds_finish_operands<2>(ph, blockIdx.x, gridDim.x, n_tiles, bias, res);
  if constexpr (ds_built<PWA, PWB>(12)) if (pw == 12) ds_finish_operands<1>(ph, blockIdx.x, gridDim.x, n_tiles, bias, res);
  ds_build_panel<PWA, PWB>(ph, smem, sh, params_asked);
  ds_stamp(sh, 2);
  if constexpr (ds_built<PWA, PWB>(1)) if (pw == 1) ds_linear_tiles<1>(ph, As, sh, wpre, have_pre, bias, res, trk);
  if constexpr (ds_built<PWA, PWB>(2)) if (pw == 2) ds_linear_tiles<2>(ph, As, sh, wpre, have_pre, bias, res, trk);
  if constexpr (ds_built<PWA, PWB>(3)) if (pw == 3) ds_linear_tiles<3>(ph, As, sh, wpre, have_pre, bias, res, trk);
  if constexpr (ds_built<PWA, PWB>(4)) if (pw == 4) ds_linear_tiles<4>(ph, As, sh, wpre, have_pre, bias, res, trk);
  if constexpr (ds_built<PWA, PWB>(6)) if (pw == 6) ds_linear_tiles<6>(ph, As, sh, wpre, have_pre, bias, res, trk);
  if constexpr (ds_built<PWA, PWB>(12)) if (pw == 12) ds_linear_tiles<12>(ph, As, sh, wpre, have_pre, bias, res, trk);
  if constexpr (ds_built<PWA, PWB>(0)) if (pw == 0) ds_linear_tiles_long(ph, As, sh, trk);
  if (ph.track) ds_track_write(ph, sh, trk);
}

// ---- attention -------------------------------------------------------------------------------------------
// One query per (sequence, head): the tensor cores take it as row 0 of a 16-row tile, and the pages of keys and
// values, as they lie in shared memory, give the other operands:
//   scores   S[row][key]  = sum_d Q[row][d] K[key][d]     B fragment: lane (g, q) holds K[key 8t + g][32i + 8q .. + 8)
//   result   O[row][dim]  = sum_k P[row][key] V[key][dim]  B fragment: 8 x 8 blocks of V read transposed (ldmatrix)
// (the 16 bytes a lane loads of K serve two products: dims 32i + 8q + {0,1 | 2,3} and {4,5 | 6,7}; Q is loaded
// with the same pattern, so the pairing of the reduction index is the same on both sides).  Whole pages are copied
// asynchronously into a ring of page slots in shared memory (one bulk copy each for a page's keys and values,
// the first ones before the grid barrier), every slot with a completion barrier of its own; a warp takes chunks
// of 8 T keys of a landed page by itself, so nothing is synchronised inside a page.  The block's warps (and,
// with splits, its blocks) are merged afterwards.
// A page slot holds the page's keys, then its values, each as ceil(head_dim / 64) tiles of 64 rows x 128 bytes
// in the tensor memory accelerator's 128-byte swizzle: the 16-byte chunk c of row r lies at chunk c ^ (r & 7).
__device__ __host__ __forceinline__ int ds_col_blocks(int head_dim) { return (head_dim + 63) / 64; }
__device__ __host__ __forceinline__ int ds_slot_bytes(int head_dim) { return 2 * ds_col_blocks(head_dim) * DS_PAGE * 128; }
__device__ __host__ __forceinline__ int ds_attn_slots(int head_dim) {
  const int fit = DS_SLOT_BYTES_TOTAL / ds_slot_bytes(head_dim);
  int slots = 1;                      // a power of two
  while (2 * slots <= fit && 2 * slots <= DS_MAX_SLOTS) slots *= 2;
  return slots;
}
__device__ __host__ __forceinline__ long long ds_attn_smem(int head_dim) {
  return 1024 + (long long)ds_attn_slots(head_dim) * ds_slot_bytes(head_dim) + 2ll * DS_WARPS * head_dim * 4 +
         (long long)DS_MAX_ITEMS * 3 * head_dim * 2;      // alignment, page slots, the warps' results, the items' new rows
}
__device__ __forceinline__ unsigned char* ds_ring_base(unsigned char* smem) {
  return smem + ((1024u - (ds_smem(smem) & 1023u)) & 1023u);      // the swizzle pattern repeats every 1024 bytes
}

// Work items are (sequence, head, split); a split owns a run of pages.
__device__ __forceinline__ int ds_ctx_len(const Phase& ph, const StepShared& sh, int seq) {
  return sh.ctx_src == ph.ctx_len ? sh.ctx_cache[seq] : ph.ctx_len[seq];
}
__device__ __forceinline__ int ds_table_entry(const Phase& ph, const StepShared& sh, int seq, int index) {
  return sh.table_src == ph.table ? sh.table_cache[seq][index] : ph.table[(long long)seq * ph.table_stride + index];
}
// Every thread calls this: the phase's lengths and page tables come into shared memory unless they are there.
__device__ void ds_cache_tables(const Phase& ph, StepShared& sh) {
  if (sh.ctx_src == ph.ctx_len && sh.table_src == ph.table) return;       // (uniform: shared memory)
  const bool fits = ph.M <= 16 && ph.table_len <= DS_TABLE_CACHE;
  __syncthreads();            // nobody still reads the old copies
  if (fits) {
    for (int i = threadIdx.x; i < ph.M * ph.table_len; i += DS_THREADS) {
      const int seq = i / ph.table_len, index = i - seq * ph.table_len;
      sh.table_cache[seq][index] = ph.table[(long long)seq * ph.table_stride + index];
    }
    if ((int)threadIdx.x < ph.M) sh.ctx_cache[threadIdx.x] = ph.ctx_len[threadIdx.x];
  }
  if (threadIdx.x == 0) {
    sh.ctx_src = fits ? ph.ctx_len : nullptr;
    sh.table_src = fits ? ph.table : nullptr;
  }
  __syncthreads();
}
__device__ __forceinline__ AttnItem ds_attn_item(const Phase& ph, const StepShared& sh, int item) {
  AttnItem it;
  const int S = ph.n_splits;
  it.split = item % S;
  const int unit = item / S;
  it.head = unit % ph.n_heads;
  it.seq = unit / ph.n_heads;
  it.L = ds_ctx_len(ph, sh, it.seq);
  it.lo = ph.window > 0 ? max(0, it.L - ph.window) : 0;
  // (a sequence without keys, L <= 0, owns no page, files nothing and yields zeros)
  const int first = it.lo / DS_PAGE, last = it.L > 0 ? (it.L - 1) / DS_PAGE : first - 1;
  const int per = (last - first + 1 + S - 1) / S;
  it.pg_first = first + it.split * per;
  it.pg_end = min(last + 1, it.pg_first + per);
  return it;
}
// The block's items of an attention phase (blockIdx.x, blockIdx.x + grid, ...) and where each one's pages begin in
// the stream of all the block's pages.  Every thread calls this.
__device__ void ds_attn_plan(const Phase& ph, StepShared& sh) {
  const int tid = threadIdx.x;
  const int shape[6] = {ph.M, ph.n_heads, ph.n_kv_heads, ph.n_splits, ph.window, ph.table_len};
  bool same = sh.work.for_ctx == ph.ctx_len && sh.work.for_table == ph.table;      // (uniform: shared memory)
#pragma unroll
  for (int i = 0; i < 6; ++i) same = same && sh.work.for_shape[i] == shape[i];
  if (same) return;
  ds_cache_tables(ph, sh);
  const int n_items = ph.M * ph.n_heads * ph.n_splits;
  if (tid < DS_MAX_ITEMS) {
    const int item = blockIdx.x + tid * gridDim.x;
    int pages = -1;
    if (item < n_items) {
      const AttnItem it = ds_attn_item(ph, sh, item);
      sh.work.it[tid] = it;
      pages = max(it.pg_end - it.pg_first, 0);
    }
    sh.work.start[tid + 1] = pages;
  }
  __syncthreads();
  if (tid == 0) {
    int n = 0, total = 0;
    while (n < DS_MAX_ITEMS && sh.work.start[n + 1] >= 0) {
      const int pages = sh.work.start[n + 1];
      sh.work.start[n] = total;
      total += pages;
      ++n;
    }
    sh.work.start[n] = total;
    sh.work.n = n;
    sh.work.for_ctx = ph.ctx_len;
    sh.work.for_table = ph.table;
#pragma unroll
    for (int i = 0; i < 6; ++i) sh.work.for_shape[i] = shape[i];
  }
  __syncthreads();
}

// Warp 0 asks for the pages [ka, kb) of the block's stream, at most 32 of them: each lane looks one page up and
// issues its copies (a 64 x 64 box per tile).  Pages are numbered through the whole launch (`base` is the number of
// the phase's first page): number n lies in slot n % slots, and its completion is phase (n / slots) & 1 of that
// slot's barrier.  `maps`: the phase in global memory (tensor maps are read from there).
__device__ __forceinline__ void ds_issue_stream(const Phase& ph, const Phase* maps, int ka, int kb, unsigned base,
                                               unsigned char* ring, StepShared& sh) {
  const int lane = threadIdx.x & 31;
  const int cbs = ds_col_blocks(ph.head_dim);
  const unsigned slots = (unsigned)ds_attn_slots(ph.head_dim), slot_bytes = (unsigned)ds_slot_bytes(ph.head_dim);
  // the shared memory may just have been read or written by ordinary instructions: order them before the copies
  asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  const int k = ka + lane;
  if (k < kb) {
    int j = 0;
    while (j + 1 < sh.work.n && sh.work.start[j + 1] <= k) ++j;
    const AttnItem it = sh.work.it[j];
    const int pg = it.pg_first + (k - sh.work.start[j]);
    const int kv_head = it.head / (ph.n_heads / ph.n_kv_heads);
    const unsigned slot = (base + (unsigned)k) % slots;
    unsigned char* dst = ring + (size_t)slot * slot_bytes;
    const unsigned bar = ds_smem(&sh.bars[slot]);
    const int page = ds_table_entry(ph, sh, it.seq, pg % ph.table_len);
    const int row = (page * ph.n_kv_heads + kv_head) * DS_PAGE;
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(slot_bytes) : "memory");
    for (int cb = 0; cb < cbs; ++cb) {
      asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n" ::"r"(
                       ds_smem(dst + cb * DS_PAGE * 128)),
                   "l"(&maps->k_map), "r"(cb * 64), "r"(row), "r"(bar)
                   : "memory");
      asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n" ::"r"(
                       ds_smem(dst + (cbs + cb) * DS_PAGE * 128)),
                   "l"(&maps->v_map), "r"(cb * 64), "r"(row), "r"(bar)
                   : "memory");
    }
  }
}
// Every lane of a warp waits (with a limit) until the slot's copies of this use have landed.
__device__ __forceinline__ bool ds_wait_slot(StepShared& sh, unsigned slot, unsigned parity) {
  for (int i = 0; i < DS_COPY_SPIN_LIMIT; ++i) {
    unsigned done;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(done) : "r"(ds_smem(&sh.bars[slot])), "r"(parity) : "memory");
    if (done) return true;
  }
  return false;
}

// `page_seq`: the number the next page to be asked for gets (see ds_issue_stream).
// `asked`: how many pages of the block's stream were asked for before the grid barrier.
template <int I, int T>
__device__ bool ds_attention_items(const Phase& ph, const Phase* maps, unsigned char* smem, StepShared& sh, unsigned& page_seq,
                                   int asked) {
  constexpr int CK = 8 * T, CPP = DS_PAGE / CK;       // keys of a chunk, chunks of a page
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, q = lane & 3;
  const int hd = ph.head_dim, page_elems = DS_PAGE * hd;
  const float scale_log2 = ph.scale_log2;
  const int slots = ds_attn_slots(hd), slot_bytes = ds_slot_bytes(hd), cbs = ds_col_blocks(hd);
  unsigned char* ring = ds_ring_base(smem);                                                       // [slots][keys | values][tile][64][128 B]
  float* s_acc = reinterpret_cast<float*>(ring + (size_t)slots * slot_bytes);                     // [2][DS_WARPS][hd]
  __nv_bfloat16* rows = reinterpret_cast<__nv_bfloat16*>(s_acc + 2 * DS_WARPS * hd);                  // [items][query, new key, new value][hd]
  const int n_mine = sh.work.n, total = sh.work.start[n_mine];
  {
    // every item's query and new key and value come into shared memory while the pages travel
    const int vecs = hd / 8, has_new = ph.new_k ? 3 : 1;
    for (int i = tid; i < n_mine * has_new * vecs; i += DS_THREADS) {
      const int j = i / (has_new * vecs), r = (i / vecs) % has_new, c = i % vecs;
      const AttnItem it = sh.work.it[j];
      const int kv_head = it.head / (ph.n_heads / ph.n_kv_heads);
      const __nv_bfloat16* src = r == 0 ? ph.q + (long long)it.seq * ph.q_stride + it.head * hd
                                        : (r == 1 ? ph.new_k : ph.new_v) + (long long)it.seq * ph.q_stride + kv_head * hd;
      ds_cp16(rows + (j * 3 + r) * hd + c * 8, src + c * 8);
    }
  }
  const unsigned base = page_seq;
  page_seq += (unsigned)total;
  // pages travel in waves of as many as there are slots; the first wave may have been asked for already
  int wave_end = min(total, slots);
  if (asked < wave_end && warp == 0) ds_issue_stream(ph, maps, asked, wave_end, base, ring, sh);
  ds_cp_wait();
  __syncthreads();
  bool ok = true;
  for (int mine = 0; mine < n_mine; ++mine) {
    const AttnItem it = sh.work.it[mine];
    const __nv_bfloat16* my_rows = rows + mine * 3 * hd;
    const int k0 = sh.work.start[mine], n_pages = sh.work.start[mine + 1] - k0;
    const int kv_head = it.head / (ph.n_heads / ph.n_kv_heads);
    const int lo = max(it.lo, it.pg_first * DS_PAGE), hi = min(it.L, it.pg_end * DS_PAGE);
    // the query in the layout of the keys' loads; only row 0 of the tile (lanes with g = 0) is a query
    unsigned qa[I * 4];          // per 16 dims: dims 2q, 2q + 1 and 8 + 2q, 9 + 2q
#pragma unroll
    for (int j = 0; j < I * 4; ++j) {
      const int d = 16 * (j >> 1) + 8 * (j & 1) + 2 * q;
      qa[j] = (g == 0 && d < hd) ? *reinterpret_cast<const unsigned*>(my_rows + d) : 0u;
    }
    if (ph.new_k && it.L > 0 && it.split == 0 && it.head == kv_head * (ph.n_heads / ph.n_kv_heads)) {
      // this block also files the new token's key and value in the sequence's page
      const __nv_bfloat16* nk = my_rows + hd;
      const __nv_bfloat16* nv = my_rows + 2 * hd;
      const int pos = it.L - 1;
      const long long page = ds_table_entry(ph, sh, it.seq, (pos / DS_PAGE) % ph.table_len);
      const long long off = (page * ph.n_kv_heads + kv_head) * (long long)page_elems + (long long)(pos % DS_PAGE) * hd;
      for (int c = tid; c < hd / 8; c += DS_THREADS) {
        *reinterpret_cast<uint4*>(ph.k_pool + off + c * 8) = *reinterpret_cast<const uint4*>(nk + c * 8);
        *reinterpret_cast<uint4*>(ph.v_pool + off + c * 8) = *reinterpret_cast<const uint4*>(nv + c * 8);
      }
    }
    float m = -INFINITY, l = 0.f;
    float acc[I * 4][4];
#pragma unroll
    for (int n = 0; n < I * 4; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[n][e] = 0.f;
    // One chunk of the block's stream of chunks (CPP to a page), if it holds keys of this item's range.
    auto take_chunk = [&](int c) {
      const int k = c / CPP, h = c % CPP;
      const int key0 = (it.pg_first + (k - k0)) * DS_PAGE + h * CK;
      if (key0 >= hi || key0 + CK <= lo) return;
      const unsigned n = base + (unsigned)k, slot = n & (unsigned)(slots - 1);
      unsigned char* Kt = ring + (size_t)slot * slot_bytes;          // the page's key tiles; its value tiles follow
      const unsigned Ks = ds_smem(Kt), Vs = Ks + (unsigned)(cbs * DS_PAGE * 128);
      if (!ds_wait_slot(sh, slot, (n / (unsigned)slots) & 1u)) ok = false;
      if (ph.new_k && it.L - 1 >= key0 && it.L - 1 < key0 + CK) {
        // the newest key and value are not in their page yet (or only just): they come from the projections.
        // (No other warp touches this chunk's rows; the rows beyond are masked and hold old, finite numbers.)
        const int row = (it.L - 1) % DS_PAGE;
        for (int ch = lane; ch < hd / 8; ch += 32) {
          const unsigned off = (unsigned)((ch >> 3) * DS_PAGE * 128 + row * 128 + (((ch & 7) ^ (row & 7)) << 4));
          *reinterpret_cast<uint4*>(Kt + off) = *reinterpret_cast<const uint4*>(my_rows + hd + ch * 8);
          *reinterpret_cast<uint4*>(Kt + cbs * DS_PAGE * 128 + off) = *reinterpret_cast<const uint4*>(my_rows + 2 * hd + ch * 8);
        }
        __syncwarp();
      }
      ds_attn_chunk<I, T>(qa, Ks, Vs, hd, h * CK, key0, lo, hi, scale_log2, m, l, acc, lane);
    };
    // chunks go round the warps, counted through the block's stream so that every warp gets some
    if (total <= slots) {          // (uniform in the block) all pages are on their way: a warp goes straight to its chunks
      const int c_lo = k0 * CPP, c_hi = (k0 + n_pages) * CPP;
      for (int c = c_lo + ((warp - c_lo) & (DS_WARPS - 1)); c < c_hi; c += DS_WARPS) take_chunk(c);
    } else {
      for (int p = 0; p < n_pages; ++p) {
        const int k = k0 + p;
        if (k == wave_end) {       // everyone is done with the slots: the next wave can come
          __syncthreads();
          wave_end = min(total, k + slots);
          if (warp == 0) ds_issue_stream(ph, maps, k, wave_end, base, ring, sh);
        }
#pragma unroll 1
        for (int h = 0; h < CPP; ++h)
          if ((k * CPP + h) % DS_WARPS == warp) take_chunk(k * CPP + h);
      }
    }
    ds_stamp(sh, 2 + min(mine, 5));      // (when the item's chunks were done)
    // the four lanes of a row each summed their own keys' weights
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    // lane q of row 0 holds dims 8 n + 2 q + {0, 1} of value tile n.  (Two sets of the warps' results, used in
    // turn: the block-wide hand-over of the next item orders this item's reads before the item after that writes.)
    float* my_acc = s_acc + (mine & 1) * DS_WARPS * hd;
    float (*my_ml)[2] = sh.ml[mine & 1];
    if (g == 0) {
#pragma unroll
      for (int n = 0; n < I * 4; ++n) {
        const int d = 8 * n + 2 * q;
        if (d < hd) *reinterpret_cast<float2*>(my_acc + warp * hd + d) = make_float2(acc[n][0], acc[n][1]);
      }
      if (q == 0) {
        my_ml[warp][0] = m;
        my_ml[warp][1] = l;
      }
    }
    __syncthreads();
    if (tid < hd) {
      float Mb = -INFINITY;
#pragma unroll
      for (int w = 0; w < DS_WARPS; ++w) Mb = fmaxf(Mb, my_ml[w][0]);
      float Lb = 0.f, o = 0.f;
#pragma unroll
      for (int w = 0; w < DS_WARPS; ++w) {
        const float wg = Mb == -INFINITY ? 0.f : ds_exp2(my_ml[w][0] - Mb);
        Lb += my_ml[w][1] * wg;
        o += my_acc[w * hd + tid] * wg;
      }
      float* dst = ph.part_out + ((long long)(it.seq * ph.n_heads + it.head) * ph.n_splits + it.split) * (hd + 4);
      dst[tid] = o;
      if (tid == 0) {
        dst[hd] = Mb;
        dst[hd + 1] = Lb;
      }
    }
  }
  return __syncthreads_and(ok ? 1 : 0) != 0;
}

// 32-dim blocks of a head and 8-key tiles of a chunk for a head size (a multiple of 16, at most 128).
// `asked` < 0: the block's items have not even been listed yet.
template <int HDMAX>
__device__ bool ds_attention_phase(const Phase& ph, const Phase* maps, unsigned char* smem, StepShared& sh, unsigned& page_seq,
                                   int asked) {
  if (asked < 0) {
    ds_attn_plan(ph, sh);
    asked = 0;
  }
  const int hd = ph.head_dim;
  if (hd <= 64) return ds_attention_items<2, 4>(ph, maps, smem, sh, page_seq, asked);       // chunks of 32 keys
  if constexpr (HDMAX > 64) return ds_attention_items<4, 2>(ph, maps, smem, sh, page_seq, asked);      // chunks of 16 keys
  return false;
}

template <int PWA, int PWB, int HDMAX, bool SAMPLES>
__global__ void __launch_bounds__(DS_THREADS, 1)
decode_step_kernel(const Phase* __restrict__ phases, int n_phases, unsigned* counter, int* status, long long* trace) {
  extern __shared__ __align__(128) unsigned char ds_smem_raw[];
  __shared__ StepShared sh;
  const int tid = threadIdx.x, warp = tid >> 5;
  if (tid == 0) {
    for (int i = 0; i < DS_MAX_SLOTS; ++i)
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(ds_smem(&sh.bars[i])), "r"(1));
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    sh.ok = 1;
    sh.ctx_src = nullptr;
    sh.table_src = nullptr;
    sh.work.for_ctx = nullptr;
  }
  __syncthreads();
  // The phase being run lies in shared memory (its successor is copied in before the grid barrier): reading its
  // fields from global memory would cost a trip to the L2 cache after every barrier, several in a row.
  static_assert(sizeof(Phase) % 16 == 0, "phases are copied 16 bytes at a time");
  constexpr int PHASE_VECS = (int)(sizeof(Phase) / 16);
  if (tid < PHASE_VECS) reinterpret_cast<uint4*>(&sh.phase[0])[tid] = reinterpret_cast<const uint4*>(phases)[tid];
  __syncthreads();
  unsigned page_seq = 0;
  uint4 wpre[DS_NB];
  bool have_pre = false, params_pre = false, failed = false;
  int pages_pre = -1;
  for (int pi = 0; pi < n_phases && !failed; ++pi) {
    const Phase& ph = sh.phase[pi & 1];
    // the next phase's description travels meanwhile (nobody reads that buffer before the next block-wide sync)
    if (pi + 1 < n_phases && tid < PHASE_VECS)
      ds_cp16(reinterpret_cast<uint4*>(&sh.phase[(pi + 1) & 1]) + tid, reinterpret_cast<const uint4*>(phases + pi + 1) + tid);
    if (tid == 0) sh.trace = (trace && blockIdx.x == 0) ? trace + DS_TRACE_SLOTS * pi : nullptr;
    ds_stamp(sh, 0);      // optional: when block 0 began each phase (nanoseconds)
    if (ph.type == PH_EMBED) {
      for (int r = blockIdx.x; r < ph.M; r += gridDim.x) {
        const int id = ph.tokens[r], pos = ph.wpe ? ph.positions[r] : 0;
        const bool ok = id >= 0 && id < ph.vocab && pos >= 0 && (!ph.wpe || pos < ph.n_positions);
        for (int c = tid; c < ph.width; c += DS_THREADS) {
          float v = 0.f;
          if (ok) {
            v = __bfloat162float(ph.wte[(long long)id * ph.width + c]);
            if (ph.wpe) v += __bfloat162float(ph.wpe[(long long)pos * ph.width + c]);
          }
          ph.resid_out[(long long)r * ph.width + c] = v;
        }
        if (!ok && tid == 0 && status) atomicExch(status, 4);
      }
    } else if (ph.type == PH_LINEAR) {
      ds_linear_phase<PWA, PWB>(ph, ds_smem_raw, sh, wpre, have_pre, params_pre);
    } else if (ph.type == PH_ATTENTION) {
      if (!ds_attention_phase<HDMAX>(ph, phases + pi, ds_smem_raw, sh, page_seq, pages_pre)) failed = true;
    } else if (ph.type == PH_SAMPLE) {
      for (int r = blockIdx.x; r < ph.M; r += gridDim.x) {
        if (!ph.do_sample && ph.partials) {
          // greedy: the readout left every block's (max, sum, argmax) of the row; a warp merges them
          if (warp == 0) {
            const int lane = tid & 31;
            float m = -INFINITY, l = 0.f;
            int idx = 0x7fffffff;
            for (int b = lane; b < ph.n_partials; b += 32) {
              const float4 p = __ldcg(reinterpret_cast<const float4*>(ph.partials + ((long long)r * ph.n_partials + b) * 4));
              ds_track_merge(m, l, idx, p.x, p.y, __float_as_int(p.z));
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
              const float m2 = __shfl_xor_sync(0xffffffffu, m, o);
              const float l2 = __shfl_xor_sync(0xffffffffu, l, o);
              const int i2 = __shfl_xor_sync(0xffffffffu, idx, o);
              ds_track_merge(m, l, idx, m2, l2, i2);
            }
            if (lane == 0) {
              ph.out_ids[r] = idx;
              ph.out_logp[r] = -logf(l);
              ph.adv_tokens[r] = idx;
              ph.adv_positions[r] += 1;
              ph.adv_past[r] += 1;
              ph.adv_ctx[r] += 1;
              ph.counters[r] += 1;
            }
          }
          continue;
        }
        if constexpr (SAMPLES) {      // (the other builds select greedily from the readout's partials only)
          float u = 0.f;
          if (ph.do_sample) u = stream_uniform(ph.seeds[r], (unsigned long long)ph.counters[r]);
          select_row<DS_THREADS>(ph.logits + (long long)r * ph.vocab, ph.vocab, ph.do_sample, ph.temperature, ph.top_k,
                                 ph.top_p, ph.min_p, u, ph.out_ids + r, ph.out_logp + r, sh.sample);
          __syncthreads();
          if (tid == 0) {      // the selected id becomes the next step's token; the sequence moves on by one
            ph.adv_tokens[r] = ph.out_ids[r];
            ph.adv_positions[r] += 1;
            ph.adv_past[r] += 1;
            ph.adv_ctx[r] += 1;
            ph.counters[r] += 1;
          }
        }
      }
    }
    have_pre = false;
    pages_pre = -1;
    params_pre = false;
    ds_stamp(sh, 1);      // ... and when it had finished its share of it
    if (pi + 1 < n_phases) {
      ds_cp_wait();
      ds_grid_arrive(counter);
      // ask for what the next phase needs and nobody writes during the step
      const Phase& nx = sh.phase[(pi + 1) & 1];
      if (nx.type == PH_LINEAR) {
        have_pre = ds_prefetch_weights<PWA, PWB>(nx, wpre);
        if (nx.a_kind == A_LAYERNORM) {
          ds_prefetch_norm_params(nx, ds_smem_raw);
          params_pre = true;
        }
      } else if (nx.type == PH_ATTENTION) {
        // the lengths do not change during the step: the block's items can be listed now; their pages can be asked
        // for only when the phase files the new token itself (then every page it copies was written in earlier steps)
        ds_attn_plan(nx, sh);
        pages_pre = 0;
        if (nx.new_k) {
          pages_pre = min(sh.work.start[sh.work.n], ds_attn_slots(nx.head_dim));
          if (warp == 0 && pages_pre > 0) ds_issue_stream(nx, phases + pi + 1, 0, pages_pre, page_seq, ds_ring_base(ds_smem_raw), sh);
        }
      }
      if (!ds_grid_wait(counter, (unsigned)(pi + 1) * gridDim.x, sh)) failed = true;
    }
  }
  if (failed && tid == 0 && status) atomicExch(status, 3);
}

}  // namespace bt

extern "C" int bt_decode_step_phase_bytes() { return (int)sizeof(bt::Phase); }

// Bytes of dynamic shared memory the step needs for these phases (host copy of the program).
extern "C" long long bt_decode_step_smem_bytes(const void* phases_host, int n_phases) {
  using namespace bt;
  const Phase* ph = reinterpret_cast<const Phase*>(phases_host);
  long long need = 1024;
  for (int i = 0; i < n_phases; ++i) {
    long long bytes = 0;
    if (ph[i].type == PH_LINEAR) {
      bytes = ds_linear_smem(ph[i]);
    } else if (ph[i].type == PH_ATTENTION) {
      bytes = ds_attn_smem(ph[i].head_dim);
    }
    if (bytes > need) need = bytes;
  }
  return need + 128;
}

// Which build of the kernel serves these phases (host copy of the program): 0 the general one, 1 products of 3 and
// 12 blocks per warp (K in 513..768 and 1537..3072) with heads up to 64, 2 products of 4 blocks per warp and long
// ones (K in 769..1024 and over 3072) with heads up to 64; both for greedy selection (or none) only; 3 and 4: the
// same two with the sampler.
extern "C" int bt_decode_step_build(const void* phases_host, int n_phases) {
  using namespace bt;
  const Phase* ph = reinterpret_cast<const Phase*>(phases_host);
  bool fits1 = true, fits2 = true, samples = false;
  for (int i = 0; i < n_phases; ++i) {
    if (ph[i].type == PH_LINEAR) {
      const int pw = (((ph[i].K + 31) / 32) + DS_WARPS - 1) / DS_WARPS;
      const int built = pw <= 1 ? 1 : pw <= 2 ? 2 : pw <= 3 ? 3 : pw <= 4 ? 4 : pw <= 6 ? 6 : pw <= 12 ? 12 : 0;
      if (built != 3 && built != 12) fits1 = false;
      if (built != 4 && built != 0) fits2 = false;
    } else if (ph[i].type == PH_ATTENTION && ph[i].head_dim > 64) {
      fits1 = fits2 = false;
    } else if (ph[i].type == PH_SAMPLE && (ph[i].do_sample || ph[i].partials == nullptr)) {
      samples = true;              // (builds 1 and 2 select greedily from the readout's partials and hold no sampler)
    }
  }
  return fits1 ? (samples ? 3 : 1) : (fits2 ? (samples ? 4 : 2) : 0);
}

// phases_dev: the program in device memory.  `build`: bt_decode_step_build of the program.  counter: one zero-initialised-per-launch unsigned (this call clears
// it).  The launch is cooperative: every block is resident, which the grid barrier relies on.
// trace: optional 8 * n_phases 64-bit slots that receive block 0's timeline of every phase.
extern "C" int bt_decode_step(const void* phases_dev, int n_phases, int build, long long smem_bytes, unsigned* counter,
                              int* status, long long* trace, cudaStream_t stream) {
  using namespace bt;
  BT_CHECK(n_phases >= 1 && smem_bytes <= 200 * 1024, "decode_step: %d phases need %lld bytes of shared memory", n_phases, smem_bytes);
  BT_CHECK(build >= 0 && build <= 4, "decode_step: unknown build %d", build);
  const int n_sms = sm_count();      // (of the current device)
  BT_CHECK(n_sms > 0, "decode_step: cannot read the number of multiprocessors of the current device");
  static long long configured_all[5] = {-1, -1, -1, -1, -1};
  long long& configured = configured_all[build];
  const void* kernels[5] = {(const void*)decode_step_kernel<-1, -1, 128, true>, (const void*)decode_step_kernel<3, 12, 64, false>,
                            (const void*)decode_step_kernel<4, 0, 64, false>, (const void*)decode_step_kernel<3, 12, 64, true>,
                            (const void*)decode_step_kernel<4, 0, 64, true>};
  const void* kernel = kernels[build];
  if (configured < smem_bytes) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes);
    BT_CHECK(e == cudaSuccess, "decode_step: cannot reserve %lld bytes of shared memory: %s", smem_bytes, cudaGetErrorString(e));
    configured = smem_bytes;
  }
  cudaError_t e = cudaMemsetAsync(counter, 0, sizeof(unsigned), stream);
  BT_CHECK(e == cudaSuccess, "decode_step: cannot clear the barrier counter: %s", cudaGetErrorString(e));
  const Phase* program = reinterpret_cast<const Phase*>(phases_dev);
  void* args[] = {(void*)&program, (void*)&n_phases, (void*)&counter, (void*)&status, (void*)&trace};
  e = cudaLaunchCooperativeKernel(kernel, dim3(n_sms), dim3(DS_THREADS), args, (size_t)smem_bytes, stream);
  BT_CHECK(e == cudaSuccess, "decode_step: launch failed: %s", cudaGetErrorString(e));
  count_launch();
  return 0;
}
