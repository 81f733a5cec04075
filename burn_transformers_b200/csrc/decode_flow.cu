// A whole decode step (at most 16 sequences, one token each, bfloat16) as ONE persistent kernel in which data,
// not barriers, tells a block when to go on.
//
// A decode step of a small model is a chain of some sixty short dependent operations (per layer: LayerNorm +
// projection -> attention -> output projection + residual -> LayerNorm + feed-forward up + GELU -> feed-forward
// down + residual).  Every link of the chain needs whole rows that all blocks produced, so every link is a
// hand-over between all multiprocessors; what a link costs is the round trips to the L2 cache that the hand-over
// takes.  A grid barrier costs three (a release fence that waits for the block's stores, the arrival at the
// counter, the poll that sees it) and the load of the rows after it a fourth.  Here a hand-over costs one:
//
//   * Everything that passes from one phase to the next carries a tag that says which launch (and, for the residual
//     stream, which phase) wrote it: a bfloat16 value travels as a 32-bit word (value | tag << 16), a 32-bit value
//     as a 64-bit pair (value, tag).  A word or a pair is written and read by one instruction, so a reader sees
//     either the old tag or the new value with its tag, never a mix.  A consumer simply loads the rows it needs and
//     looks at the tags; a round of loads in which a tag is missing is loaded again (with a limit: see "waits").  No
//     fence, no counter, no second trip.  Buffers are zeroed before first use and tags are never zero.
//   * Weights and cache pages never change during a step.  Two producer warps of every block walk the phase list
//     on their own, ahead of the computing warps: one streams the block's weight tiles through a ring of slots in
//     shared memory (bulk copies, one per row of a tile of 8 output columns and up to 1024 of k; four slots are
//     filled at a time by four groups of lanes), the other the block's pages of keys and values (tensor-map copies
//     with the 128-byte swizzle).  The rings are the only coupling: a slot is handed back when its last reader is done.
//     The weight stream therefore runs through hand-overs and phases without a pause.  The weight producer also sends
//     what the coming phase reads from plain memory (bias values, norm parameters) on its way into the L2 cache.
//   * Matrix products: every block takes the same share of a phase's output columns (N / blocks or one more), in
//     tiles of at most 8.  The six computing warps form groups: G = 6, 3, 2 or 1 warps share a tile and split its k
//     (32 elements at a time, round-robin), so that 6 / G tiles are in work at a time and no block-wide barrier stands
//     between tiles.  A and B come from shared memory with ldmatrix (A: a panel of the step's rows and a row of zeros
//     for the rows it does not have, or 16 rows for more than 8, built once per block and phase from tagged rows: copied, or LayerNorm-ed with all warps on every row, 32-bit statistics in two
//     passes over registers); a group adds its partial sums through shared memory in the order of its warps, and its
//     warps take turns at finishing a tile (bias, activation, residual, tags).
//   * Attention is the tensor-core routine of decode_mma.cuh over the pages in the ring.  With several splits per
//     (sequence, head) every split leaves a tagged partial result and the block of split 0 merges them, in split
//     order, as soon as their tags show up: the projection after it reads plain rows.
//   * Nothing is accumulated with atomics and every sum has a fixed order: results do not depend on timing.
//
// Registers and code.  Eight warps a block, so that a thread may hold 255 registers, and the kernel is built so that
// nothing spills: with most of a multiprocessor's memory taken as shared memory there is little cache for spilled
// registers, and every spilled access would be a trip to the L2 cache.  What runs once a step (token selection) or
// rarely (the merge of splits, full-precision activations) is kept out of line, so that the code of a layer's phases
// stays small enough for the instruction cache.  What a phase needs of its description is read into registers once:
// the description lies in shared memory, and every wait in between would have the compiler read it again.
//
// The one place where the step still meets at a grid barrier is before token selection, which reads the plain
// 32-bit logits (they are also the step's result for the host) or the readout's per-block partials.
//
// Waits.  Every wait (a tag that does not show up, a ring slot that is not filled or not handed back, the grid
// barrier) is bounded.  A block that gives up sets the status word, which every other waiting block looks at now and
// then, so that all blocks leave soon after; a producer warp waits (bounded) for its own copies in flight before it
// returns.  The launch is cooperative (one block per multiprocessor, all resident), which the waiting relies on.
#include "common.cuh"
#include "sampling.cuh"
#include "tma.cuh"
#include "decode_mma.cuh"

namespace bt {

constexpr int DF_CWARPS = 6, DF_CONSUMERS = DF_CWARPS * 32;     // warps that compute
constexpr int DF_THREADS = DF_CONSUMERS + 64;                   // + the weight producer and the page producer
constexpr int DF_MAX_SLOT_K = 1664;              // largest k extent of a weight slot
constexpr int DF_MAX_WSLOTS = 32, DF_MAX_PSLOTS = 16;
constexpr int DF_MAX_ITEMS = 8;                  // (sequence, head, split) items of an attention phase a block takes, at most
constexpr int DF_TABLE_CACHE = 64;               // page-table entries per sequence kept in shared memory
constexpr int DF_SPIN_LIMIT = 1 << 21;           // tries of any wait before a block gives up
constexpr int DF_TRACE_SLOTS = 8;

enum { FP_EMBED = 0, FP_LINEAR = 1, FP_ATTENTION = 2, FP_SAMPLE = 3 };
enum { FA_ROWS = 0, FA_LAYERNORM = 1, FA_RMSNORM = 2 };
enum { FO_WORDS = 0, FO_PAIRS = 1, FO_PLAIN = 2 };

struct FlowPhase {
  int type, M;
  // ---- linear: out[M, N] = act(A @ w^T + bias) (+ residual) ----
  int a_kind;                    // FA_ROWS: tagged bfloat16 words [M][K]; FA_LAYERNORM, FA_RMSNORM: that norm of tagged 32-bit pairs [.][K]
  int N, K, act;
  int out_kind;                  // FO_WORDS: tagged bfloat16 words; FO_PAIRS: tagged 32-bit pairs (the residual stream, added to);
                                 // FO_PLAIN: plain 32-bit (the logits)
  int a_src;                     // FA_LAYERNORM: index of the phase that wrote the pairs this phase reads
  int res_src;                   // FO_PAIRS: index of the phase that last wrote the pairs this phase adds to
  int col_q;                     // set by bt_decode_flow_plan: N / blocks ...
  const void* a;
  const int* rows;               // FA_LAYERNORM: row r of the panel is row rows[r] of `a` (null: r)
  const float* gamma;
  const float* beta;
  float eps;
  int col_r;                     // ... and N % blocks: block b takes col_q columns, one more if b < col_r
  const __nv_bfloat16* w;        // [N, K]
  const float* bias;
  void* out;                     // [M][N] in the layout of out_kind
  float* track;                  // optional [M][blocks][4]: every block's (max, sum of exp(. - max), first argmax) of the rows of `out`
  // ---- attention ----
  const unsigned* q;             // tagged words of the step's projections [M][q_stride]: query head h at h * head_dim
  long long q_stride;
  int k_off, v_off;              // where the new token's key / value channels begin in a row; k_off < 0: the pages hold them already
  __nv_bfloat16* k_pool;         // [page][kv_head][64][head_dim]
  __nv_bfloat16* v_pool;
  const int* table;
  int table_stride, table_len;
  const int* ctx_len;
  int n_heads, n_kv_heads, head_dim, n_splits;
  float scale_log2;
  int window;
  uint2* part;                   // n_splits > 1: tagged pairs [(sequence * heads + head) * splits + split][head_dim + 2]
  unsigned* attn_out;            // tagged words [M][n_heads * head_dim]
  // ---- embed ----
  const int* tokens;
  const int* positions;
  const __nv_bfloat16* wte;
  const __nv_bfloat16* wpe;
  uint2* resid;                  // tagged pairs [M][width]
  int width, vocab, n_positions;
  // ---- sample (and advance) ----
  int do_sample;
  const float* logits;
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
  int n_chunks;                  // set by bt_decode_flow_plan: slots a tile's k takes
  // ---- attention: tensor maps of the layer's key and value pools, seen as [pages * kv_heads * 64 rows][head_dim] ----
  alignas(64) CUtensorMap k_map;
  CUtensorMap v_map;
};
static_assert(sizeof(FlowPhase) % 64 == 0, "tensor maps in an array of phases stay on 64-byte boundaries");

// ---- tagged data ------------------------------------------------------------------------------------------
// Loads and stores of tagged data go to the L2 cache, where all blocks meet (relaxed, gpu scope).  A 32-bit word and a
// 64-bit pair are each one access: never torn.
__device__ __forceinline__ uint4 df_ld_words4(const unsigned* p) {         // four tagged words
  uint4 v;
  asm volatile("ld.relaxed.gpu.global.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void df_ld_pairs2(const uint2* p, uint2& a, uint2& b) {      // two tagged pairs
  unsigned long long x, y;
  asm volatile("ld.relaxed.gpu.global.v2.u64 {%0,%1}, [%2];\n" : "=l"(x), "=l"(y) : "l"(p) : "memory");
  a = make_uint2((unsigned)x, (unsigned)(x >> 32));
  b = make_uint2((unsigned)y, (unsigned)(y >> 32));
}
__device__ __forceinline__ uint2 df_ld_pair(const uint2* p) {
  unsigned long long x;
  asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];\n" : "=l"(x) : "l"(p) : "memory");
  return make_uint2((unsigned)x, (unsigned)(x >> 32));
}
__device__ __forceinline__ void df_st_pair(uint2* p, float v, unsigned tag) {
  const unsigned long long x = (unsigned long long)__float_as_uint(v) | ((unsigned long long)tag << 32);
  asm volatile("st.relaxed.gpu.global.u64 [%0], %1;\n" ::"l"(p), "l"(x) : "memory");
}
__device__ __forceinline__ void df_st_pairs2(uint2* p, float v0, float v1, unsigned tag) {
  const unsigned long long x = (unsigned long long)__float_as_uint(v0) | ((unsigned long long)tag << 32);
  const unsigned long long y = (unsigned long long)__float_as_uint(v1) | ((unsigned long long)tag << 32);
  asm volatile("st.relaxed.gpu.global.v2.u64 [%0], {%1,%2};\n" ::"l"(p), "l"(x), "l"(y) : "memory");
}
__device__ __forceinline__ unsigned df_word(float v, unsigned tag16) {
  return (unsigned)__bfloat16_as_ushort(__float2bfloat16_rn(v)) | (tag16 << 16);
}
__device__ __forceinline__ void df_st_words2(unsigned* p, float v0, float v1, unsigned tag16) {
  asm volatile("st.relaxed.gpu.global.v2.u32 [%0], {%1,%2};\n" ::"l"(p), "r"(df_word(v0, tag16)), "r"(df_word(v1, tag16)) : "memory");
}
__device__ __forceinline__ void df_st_word(unsigned* p, float v, unsigned tag16) {
  asm volatile("st.relaxed.gpu.global.u32 [%0], %1;\n" ::"l"(p), "r"(df_word(v, tag16)) : "memory");
}
__device__ __forceinline__ int df_ld_status(const int* status) {
  int v;
  asm volatile("ld.relaxed.gpu.global.s32 %0, [%1];\n" : "=r"(v) : "l"(status) : "memory");
  return v;
}

// ---- layout of the dynamic shared memory (the host computes the same numbers) --------------------------------
struct FlowLayout {
  int w_slots, p_slots, p_slot_bytes;
  int slot_k, w_row, w_slot_bytes;       // k extent of a weight slot, bytes between its 8 rows (16 apart modulo 128: no bank conflicts), its size
  int panel_rows, panel_stride;          // rows of the panel (the step's rows and one of zeros, or 16) and bytes between them
  long long w_off, p_off, panel_off, rows_off, acc_off, total;
};
__host__ __device__ inline int df_kpad(int K) { return (K + 31) / 32 * 32; }
__host__ __device__ inline int df_col_blocks(int head_dim) { return (head_dim + 63) / 64; }
__host__ __device__ inline int df_page_slot_bytes(int head_dim) { return 2 * df_col_blocks(head_dim) * DS_PAGE * 128; }

// max_k: the longest K of a product; max_ln_k: the longest LayerNorm-ed K; head_dim: 0 without attention.
__host__ __device__ inline FlowLayout df_layout(int rows, int max_k, int max_ln_k, int head_dim, int w_slots, int p_slots, int slot_k) {
  FlowLayout L;
  L.slot_k = slot_k;
  L.w_row = (slot_k * 2 + 127) / 128 * 128 + 16;
  L.w_slot_bytes = 8 * L.w_row;
  L.w_slots = w_slots;
  L.p_slots = p_slots;
  L.p_slot_bytes = head_dim > 0 ? df_page_slot_bytes(head_dim) : 0;
  L.panel_rows = rows > 8 ? 16 : rows + 1;       // (up to 8 rows: a row of zeros behind them stands for all other rows of the tile)
  L.panel_stride = df_kpad(max_k) * 2 + 16;
  long long at = 0;
  L.p_off = at;                                  // page slots first: the swizzle pattern wants 1024-byte boundaries
  at += (long long)p_slots * L.p_slot_bytes;
  L.w_off = at;
  at += (long long)w_slots * L.w_slot_bytes;
  L.panel_off = at;
  at += (long long)L.panel_rows * L.panel_stride;
  L.rows_off = at;                               // attention: query, new key, new value of every item
  at += (long long)DF_MAX_ITEMS * 3 * head_dim * 2;
  at = (at + 15) / 16 * 16;
  L.acc_off = at;                                // attention: the warps' results, two sets
  at += 2ll * DF_CWARPS * head_dim * 4;
  L.total = at + 1024;                           // room to move the base up to a 1024-byte boundary
  return L;
}

struct FlowItem {
  int seq, head, split, L, lo, pg_first, pg_end;   // pages [pg_first, pg_end)
  int kv_head;                                     // the key/value head the query head reads
};
struct FlowWork {
  FlowItem it[DF_MAX_ITEMS];
  int start[DF_MAX_ITEMS + 2];     // where each item's pages begin in the block's stream of pages; [n]: their number
  int n;
};

struct FlowShared {
  volatile int failed;             // a wait of this block ran out (or another block said so): everybody winds down
  volatile unsigned w_issued;      // weight slots the producer has asked for so far
  int ok;
  alignas(16) float red[2][DF_CWARPS][32][4];  // the warps' partial sums of a tile, two sets used in turn (read and written 16 bytes at a time)
  float ml[2][DF_CWARPS][2];
  float trk[DF_CWARPS][16][3];
  alignas(16) float ln[2][DF_CWARPS][8];       // LayerNorm: the warps' sums and squared deviations of (at most 8) rows
  SampleShared sample;
  alignas(64) FlowPhase phase[2];
  FlowWork work;                   // the computing warps' list of attention items
  FlowWork pwork;                  // the page producer's own (it runs ahead)
  const int* ctx_src;
  const int* table_src;
  int ctx_cache[16];
  int table_cache[16][DF_TABLE_CACHE];
  unsigned long long wfull[DF_MAX_WSLOTS], wempty[DF_MAX_WSLOTS];
  unsigned long long pfull[DF_MAX_PSLOTS], pempty[DF_MAX_PSLOTS];
  long long* trace;
  FlowLayout lay;                  // where things lie in the dynamic shared memory (kept here, not in registers)
};

__device__ __forceinline__ void df_stamp(FlowShared& sh, int slot) {
  if (threadIdx.x == 0 && sh.trace) {
    long long t;
    asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t));
    sh.trace[slot] = t;
  }
}
// The same number, but the compiler no longer knows it: what a phase derives from it is computed in that phase (and its
// registers are free again afterwards) instead of once for the whole kernel.
__device__ __forceinline__ int df_opaque(int x) {
  asm volatile("mov.b32 %0, %0;\n" : "+r"(x));
  return x;
}
__device__ __forceinline__ void df_bar_consumers() { asm volatile("bar.sync 1, %0;\n" ::"n"(DF_CONSUMERS) : "memory"); }

// A wait that ran out: remember it here and tell everybody.
__device__ __forceinline__ void df_give_up(FlowShared& sh, int* status, int code) {
  sh.failed = 1;
  if (status) atomicCAS(status, 0, code);
}
// True when the mbarrier's phase with this parity has completed; gives up when the limit runs out or the block has failed.
__device__ __forceinline__ bool df_mbar_wait(unsigned long long* bar, unsigned parity, FlowShared& sh, int* status) {
  for (int i = 0; i < DF_SPIN_LIMIT; ++i) {
    unsigned done;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(done) : "r"(ds_smem(bar)), "r"(parity) : "memory");
    if (done) return true;
    if ((i & 1023) == 1023 && (sh.failed || (status && df_ld_status(status) != 0))) break;
  }
  df_give_up(sh, status, 3);
  return false;
}
__device__ __forceinline__ void df_mbar_arrive(unsigned long long* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(ds_smem(bar)) : "memory");
}

struct FlowArgs {
  const FlowPhase* phases;
  int n_phases;
  unsigned epoch;                  // of this launch, counted per program from 1
  unsigned* counter;               // the grid barrier's (cleared before the launch)
  int* status;
  long long* trace;
  int rows, max_k, max_ln_k, head_dim, w_slots, p_slots, slot_k;
  unsigned tag16;                  // epoch % 65535 + 1: the tag of this launch's bfloat16 words (never zero)
};

__device__ __forceinline__ unsigned df_tag32(unsigned epoch, int phase) { return (epoch << 10) | (unsigned)(phase + 1); }

// ---- how a product's output columns are dealt out -----------------------------------------------------------
// Block b of B takes the columns [b N / B, (b + 1) N / B): every block gets N / B columns or one more, so that all
// multiprocessors pull the same share of the weights.  A block works through its columns in tiles of (at most) 8.
__device__ __forceinline__ void df_columns(const FlowPhase* ph, int& c0, int& c1) {
  const int b = blockIdx.x, q = ph->col_q, r = ph->col_r;
  c0 = b * q + min(b, r);
  c1 = c0 + q + (b < r ? 1 : 0);
}
__device__ __forceinline__ void df_prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];\n" ::"l"(p)); }

// ---- the producers ---------------------------------------------------------------------------------------
// The weight producer: one warp that walks the phases and, for every linear phase, sends the block's tiles through the
// ring: tile after tile, slot_k of k at a time, 8 rows (output columns) per slot.  Four slots are filled at a time: the
// lanes 8 j .. 8 j + 7 wait for the j-th of them to be handed back and copy its 8 rows (one instruction stream would
// not keep up with the readout, which takes a slot every few hundred cycles).  Returns how many slots it filled.
__device__ unsigned df_weight_producer(const FlowArgs& args, int n_phases, const FlowLayout& lay, unsigned char* smem, FlowShared& sh) {
  const int lane = threadIdx.x & 31, grp = lane >> 3, row = lane & 7;
  const unsigned w_slots = (unsigned)lay.w_slots, w_slot_bytes = (unsigned)lay.w_slot_bytes;
  const int slot_k = lay.slot_k;
  const unsigned w_base = ds_smem(smem + lay.w_off) + (unsigned)(row * lay.w_row);
  int* const status = args.status;
  unsigned use = 0, base_slot = 0, base_turn = 0;      // of the next slot to fill (slot = use % slots, turn = use / slots)
  for (int pi = 0; pi < n_phases && !sh.failed; ++pi) {
    const FlowPhase* ph = args.phases + pi;
    if (ph->type != FP_LINEAR) continue;
    const int K = ph->K, n_chunks = ph->n_chunks;
    const __nv_bfloat16* const w = ph->w;
    int c0, c1;
    df_columns(ph, c0, c1);
    // What the phase's computing warps will read from plain memory, on its way into the L2 cache: the block's bias
    // values, and (one block for all) the norm's parameters.
    if (ph->bias && c0 + lane * 32 < c1) df_prefetch_l2(ph->bias + c0 + lane * 32);
    if (ph->a_kind != FA_ROWS && pi % (int)gridDim.x == (int)blockIdx.x)
      for (int k = lane * 32; k < K; k += 32 * 32) {
        df_prefetch_l2(ph->gamma + k);
        if (ph->beta) df_prefetch_l2(ph->beta + k);
      }
    const int total = ((c1 - c0 + 7) >> 3) * n_chunks;      // slots of this phase
    int t = 0, c = grp;                                     // this group's tile and piece of k
    while (c >= n_chunks) {
      c -= n_chunks;
      ++t;
    }
    for (int f0 = 0; f0 < total && !sh.failed; f0 += 4) {
      const bool active = f0 + grp < total;
      unsigned slot = base_slot + (unsigned)grp, turn = base_turn;
      if (slot >= w_slots) {
        slot -= w_slots;
        ++turn;
      }
      // (every group goes on as soon as its own slot is free: the first of the four need not wait for the last)
      bool ok = true;
      if (active && turn > 0) ok = df_mbar_wait(&sh.wempty[slot], (turn - 1) & 1u, sh, status);
      if (active && ok) {
        const int t0 = c0 + 8 * t, rows_here = min(8, c1 - t0), kc = min(slot_k, K - c * slot_k);
        const unsigned bytes = (unsigned)kc * 2u, bar = ds_smem(&sh.wfull[slot]);
        if (row == 0) asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes * (unsigned)rows_here) : "memory");
        if (row < rows_here)
          asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(
                           w_base + slot * w_slot_bytes),
                       "l"(w + ((long long)(t0 + row) * K + (long long)c * slot_k)), "r"(bytes), "r"(bar)
                       : "memory");
      }
      if (!__all_sync(0xffffffffu, ok)) return use;
      const unsigned n_done = (unsigned)min(4, total - f0);
      use += n_done;
      base_slot += n_done;
      if (base_slot >= w_slots) {
        base_slot -= w_slots;
        ++base_turn;
      }
      __syncwarp();
      if (lane == 0) sh.w_issued = use;
      c += 4;
      while (c >= n_chunks) {
        c -= n_chunks;
        ++t;
      }
    }
  }
  return use;
}

// Before a producer warp returns, the copies it asked for last (one ring's worth) have landed: a block must not end
// with copies into its shared memory in flight.  Bounded; there is nothing more to do if they do not land.
__device__ void df_drain(unsigned long long* full, unsigned uses, int slots) {
  const unsigned first = uses > (unsigned)slots ? uses - (unsigned)slots : 0u;
  for (unsigned u = first; u < uses; ++u) {
    const unsigned slot = u % (unsigned)slots, parity = (u / (unsigned)slots) & 1u;
    for (int t = 0; t < (1 << 18); ++t) {
      unsigned done;
      asm volatile(
          "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
          : "=r"(done) : "r"(ds_smem(&full[slot])), "r"(parity) : "memory");
      if (done) break;
    }
  }
}

// ---- attention: the block's items -----------------------------------------------------------------------------
__device__ __forceinline__ int df_ctx_len(const FlowPhase* ph, const FlowShared& sh, int seq) {
  return sh.ctx_src == ph->ctx_len ? sh.ctx_cache[seq] : ph->ctx_len[seq];
}
__device__ __forceinline__ int df_table_entry(const FlowPhase* ph, const FlowShared& sh, int seq, int index) {
  return sh.table_src == ph->table ? sh.table_cache[seq][index] : ph->table[(long long)seq * ph->table_stride + index];
}
__device__ __forceinline__ FlowItem df_item(const FlowPhase* ph, const FlowShared& sh, int item) {
  FlowItem it;
  const int S = ph->n_splits;
  it.split = item % S;
  const int unit = item / S;
  it.head = unit % ph->n_heads;
  it.seq = unit / ph->n_heads;
  it.kv_head = it.head / (ph->n_heads / ph->n_kv_heads);
  it.L = df_ctx_len(ph, sh, it.seq);
  it.lo = ph->window > 0 ? max(0, it.L - ph->window) : 0;
  // (a sequence without keys, L <= 0, owns no page, files nothing and yields zeros)
  const int first = it.lo / DS_PAGE, last = it.L > 0 ? (it.L - 1) / DS_PAGE : first - 1;
  const int per = (last - first + 1 + S - 1) / S;
  it.pg_first = first + it.split * per;
  it.pg_end = min(last + 1, it.pg_first + per);
  return it;
}
// One warp lists the block's items of an attention phase (blockIdx.x, blockIdx.x + grid, ...) into `work`.
__device__ void df_plan(const FlowPhase* ph, const FlowShared& sh, FlowWork& work) {
  const int lane = threadIdx.x & 31;
  const int n_items = ph->M * ph->n_heads * ph->n_splits;
  int pages = -1;
  if (lane < DF_MAX_ITEMS) {
    const int item = blockIdx.x + lane * gridDim.x;
    if (item < n_items) {
      const FlowItem it = df_item(ph, sh, item);
      work.it[lane] = it;
      pages = max(it.pg_end - it.pg_first, 0);
    }
  }
  // an exclusive running sum over the first lanes (items are contiguous from lane 0)
  int incl = max(pages, 0);
#pragma unroll
  for (int o = 1; o < DF_MAX_ITEMS; o <<= 1) {
    const int up = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += up;
  }
  const unsigned have = __ballot_sync(0xffffffffu, pages >= 0);
  const int n = __popc(have);
  if (lane < DF_MAX_ITEMS && pages >= 0) work.start[lane] = incl - pages;
  if (lane == max(n - 1, 0)) {
    work.start[n] = n > 0 ? incl : 0;
    work.n = n;
  }
  __syncwarp();
}

// The page producer: one warp that walks the phases and sends the pages of the block's attention items through the
// ring of page slots, in the order the computing warps take them.
__device__ unsigned df_page_producer(const FlowArgs& args, int n_phases, const FlowLayout& lay, unsigned char* smem, FlowShared& sh) {
  const int lane = threadIdx.x & 31;
  unsigned use = 0;
  for (int pi = 0; pi < n_phases && !sh.failed; ++pi) {
    const FlowPhase* ph = args.phases + pi;
    if (ph->type != FP_ATTENTION) continue;
    df_plan(ph, sh, sh.pwork);
    const int total = sh.pwork.start[sh.pwork.n];
    const int cbs = df_col_blocks(ph->head_dim);
    for (int base = 0; base < total && !sh.failed; base += 32) {
      // every lane looks up one page of the stream
      const int k = base + lane;
      int row = 0;
      if (k < total) {
        int j = 0;
        while (j + 1 < sh.pwork.n && sh.pwork.start[j + 1] <= k) ++j;
        const FlowItem it = sh.pwork.it[j];
        const int pg = it.pg_first + (k - sh.pwork.start[j]);
        const int page = df_table_entry(ph, sh, it.seq, pg % ph->table_len);
        row = (page * ph->n_kv_heads + it.kv_head) * DS_PAGE;
      }
      const int n = min(32, total - base);
      for (int j = 0; j < n; ++j, ++use) {
        const int my_row = __shfl_sync(0xffffffffu, row, j);
        const unsigned slot = use % (unsigned)lay.p_slots, turn = use / (unsigned)lay.p_slots;
        if (turn > 0 && !df_mbar_wait(&sh.pempty[slot], (turn - 1) & 1u, sh, args.status)) return use;
        if (lane == 0) {
          unsigned char* dst = smem + lay.p_off + (size_t)slot * lay.p_slot_bytes;
          const unsigned bar = ds_smem(&sh.pfull[slot]);
          // the slot may just have been written by ordinary stores (the newest key): order them before the copies
          asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
          asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"((unsigned)lay.p_slot_bytes) : "memory");
          for (int cb = 0; cb < cbs; ++cb) {
            asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n" ::"r"(
                             ds_smem(dst + cb * DS_PAGE * 128)),
                         "l"(&ph->k_map), "r"(cb * 64), "r"(my_row), "r"(bar)
                         : "memory");
            asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n" ::"r"(
                             ds_smem(dst + (cbs + cb) * DS_PAGE * 128)),
                         "l"(&ph->v_map), "r"(cb * 64), "r"(my_row), "r"(bar)
                         : "memory");
          }
        }
        __syncwarp();
      }
    }
  }
  return use;
}

// ---- the rows' panel ---------------------------------------------------------------------------------------
__device__ __forceinline__ void df_cp16(const void* smem_dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(ds_smem(smem_dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void df_cp_wait() { asm volatile("cp.async.wait_all;\n" ::: "memory"); }

// True when a tagged wait should stop: the limit ran out, this block has failed or another block said so.
__device__ __forceinline__ bool df_tired(int tries, FlowShared& sh, int* status) {
  return tries >= DF_SPIN_LIMIT || ((tries & 1023) == 1023 && (sh.failed || (status && df_ld_status(status) != 0)));
}

// out[r] = the sum over the warps, in warp order, of what each left for row r (read four rows at a time).
template <int RP>
__device__ __forceinline__ void df_sum_warps(const float (*part)[8], float (&out)[RP]) {
#pragma unroll
  for (int r = 0; r < RP; ++r) out[r] = 0.f;
#pragma unroll
  for (int w2 = 0; w2 < DF_CWARPS; ++w2) {
    if (RP >= 4) {
#pragma unroll
      for (int r4 = 0; r4 < RP / 4; ++r4) {
        const float4 v = *reinterpret_cast<const float4*>(&part[w2][4 * r4]);
        out[4 * r4] += v.x;
        out[4 * r4 + 1] += v.y;
        out[4 * r4 + 2] += v.z;
        out[4 * r4 + 3] += v.w;
      }
    } else {
      const float2 v = *reinterpret_cast<const float2*>(&part[w2][0]);
      out[0] += v.x;
      if (RP > 1) out[RP > 1 ? 1 : 0] += v.y;
    }
  }
}

// LayerNorm of the phase's rows from tagged pairs, all warps on every row: warp w takes the quads (four neighbouring
// channels) [w qpw, (w + 1) qpw) of each row, a lane Q of them (K <= 768 Q).  Rows go in passes of RP (as many as keep
// the loads of a pass in 64 registers): loaded until every tag is the expected one, then each warp's sum per row, the
// mean from the warps' sums in warp order, each warp's squared deviations, the variance, and the normalised rows go
// into the panel as bfloat16, 8 bytes a lane at a time.  An RMS norm (FA_RMSNORM) is the same with the mean left at zero.
template <int Q>
__device__ __forceinline__ void df_layernorm_rows(const FlowPhase& ph, const FlowArgs& args, unsigned char* panel, int stride,
                                                  FlowShared& sh, int tid) {
  constexpr int RP = Q == 1 ? 8 : (Q == 2 ? 4 : 2);
  const int lane = tid & 31, warp = tid >> 5;
  const int K = ph.K, M = ph.M, quads = K >> 2, qpw = (quads + DF_CWARPS - 1) / DF_CWARPS;
  const unsigned tag = df_tag32(args.epoch, ph.a_src);
  const float inv_k = 1.f / (float)K;
  const bool rms = ph.a_kind == FA_RMSNORM;      // no mean is taken off: the rows are scaled by their root mean square
  int qd[Q];
  unsigned has = 0;
  float4 g4[Q], b4[Q];
#pragma unroll
  for (int i = 0; i < Q; ++i) {
    const int k = lane + 32 * i;
    qd[i] = warp * qpw + k;
    g4[i] = b4[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (k < qpw && qd[i] < quads) {
      has |= 1u << i;
      g4[i] = __ldg(reinterpret_cast<const float4*>(ph.gamma) + qd[i]);
      if (ph.beta) b4[i] = __ldg(reinterpret_cast<const float4*>(ph.beta) + qd[i]);
    }
  }
  const uint2* x = reinterpret_cast<const uint2*>(ph.a);
  for (int r0 = 0; r0 < M; r0 += RP) {
    // e[r][i][c]: value and tag of channel 4 qd[i] + c of row r0 + r; the loads' own registers hold the rows
    uint2 e[RP][Q][4];
    unsigned src[RP];          // where each row begins, in pairs
    unsigned mine = 0;
#pragma unroll
    for (int r = 0; r < RP; ++r) {
      const int row = r0 + r;
      src[r] = (unsigned)((row < M ? (ph.rows ? ph.rows[row] : row) : 0) * K);
#pragma unroll
      for (int i = 0; i < Q; ++i) {
#pragma unroll
        for (int c = 0; c < 4; ++c) e[r][i][c] = make_uint2(0u, tag);
        if (row < M && (has & (1u << i))) mine |= 1u << (r * Q + i);
      }
    }
    // All loads of a round in flight together; a round whose tags are not all there is loaded again as a whole
    // (the rows arrive within a fraction of a microsecond of one another: there is little to gain from finer books).
    for (int tries = 0;; ++tries) {
#pragma unroll
      for (int r = 0; r < RP; ++r)
#pragma unroll
        for (int i = 0; i < Q; ++i)
          if (mine & (1u << (r * Q + i))) {
            df_ld_pairs2(x + (src[r] + (unsigned)(qd[i] * 4)), e[r][i][0], e[r][i][1]);
            df_ld_pairs2(x + (src[r] + (unsigned)(qd[i] * 4 + 2)), e[r][i][2], e[r][i][3]);
          }
      unsigned stale = 0;
#pragma unroll
      for (int r = 0; r < RP; ++r)
#pragma unroll
        for (int i = 0; i < Q; ++i) stale |= (e[r][i][0].y ^ tag) | (e[r][i][1].y ^ tag) | (e[r][i][2].y ^ tag) | (e[r][i][3].y ^ tag);
      if (stale == 0u) break;
      if (df_tired(tries, sh, args.status)) {
        df_give_up(sh, args.status, 3);
        break;
      }
    }
    // the warp's sum of every row (what a lane does not hold is zero)
    float part[RP];
#pragma unroll
    for (int r = 0; r < RP; ++r) {
      float t = 0.f;
#pragma unroll
      for (int i = 0; i < Q; ++i)
        t += (__uint_as_float(e[r][i][0].x) + __uint_as_float(e[r][i][1].x)) + (__uint_as_float(e[r][i][2].x) + __uint_as_float(e[r][i][3].x));
      part[r] = t;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
#pragma unroll
      for (int r = 0; r < RP; ++r) part[r] += __shfl_xor_sync(0xffffffffu, part[r], o);
    if (lane < RP) {
      float mine_sum = part[0];
#pragma unroll
      for (int r = 1; r < RP; ++r)
        if (lane == r) mine_sum = part[r];
      sh.ln[0][warp][lane] = mine_sum;
    }
    df_bar_consumers();
    float mean[RP];
    df_sum_warps<RP>(sh.ln[0], mean);
#pragma unroll
    for (int r = 0; r < RP; ++r) mean[r] = rms ? 0.f : mean[r] * inv_k;
#pragma unroll
    for (int r = 0; r < RP; ++r) {
      float t = 0.f;
#pragma unroll
      for (int i = 0; i < Q; ++i)
        if (mine & (1u << (r * Q + i))) {
          const float x0 = __uint_as_float(e[r][i][0].x) - mean[r], x1 = __uint_as_float(e[r][i][1].x) - mean[r];
          const float x2 = __uint_as_float(e[r][i][2].x) - mean[r], x3 = __uint_as_float(e[r][i][3].x) - mean[r];
          t += (x0 * x0 + x1 * x1) + (x2 * x2 + x3 * x3);
        }
      part[r] = t;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
#pragma unroll
      for (int r = 0; r < RP; ++r) part[r] += __shfl_xor_sync(0xffffffffu, part[r], o);
    if (lane < RP) {
      float mine_sum = part[0];
#pragma unroll
      for (int r = 1; r < RP; ++r)
        if (lane == r) mine_sum = part[r];
      sh.ln[1][warp][lane] = mine_sum;
    }
    df_bar_consumers();
    float var[RP];
    df_sum_warps<RP>(sh.ln[1], var);
#pragma unroll
    for (int r = 0; r < RP; ++r) {
      // (the result is rounded to bfloat16: the hardware's reciprocal square root, 2 ulp, is far below that)
      const float rs = rsqrtf(var[r] * inv_k + ph.eps), shift = -mean[r] * rs;
#pragma unroll
      for (int i = 0; i < Q; ++i)
        if (mine & (1u << (r * Q + i))) {
          uint2 packed;
          packed.x = ds_pack(fmaf(fmaf(__uint_as_float(e[r][i][0].x), rs, shift), g4[i].x, b4[i].x),
                             fmaf(fmaf(__uint_as_float(e[r][i][1].x), rs, shift), g4[i].y, b4[i].y));
          packed.y = ds_pack(fmaf(fmaf(__uint_as_float(e[r][i][2].x), rs, shift), g4[i].z, b4[i].z),
                             fmaf(fmaf(__uint_as_float(e[r][i][3].x), rs, shift), g4[i].w, b4[i].w));
          *reinterpret_cast<uint2*>(panel + (unsigned)((r0 + r) * stride + qd[i] * 8)) = packed;
        }
    }
  }
}

// The panel from tagged bfloat16 words [M][K] (what a product or the attention left): loaded until every tag is this
// launch's, packed two to a word.  
__device__ __forceinline__ void df_panel_from_words(const FlowPhase& ph, const FlowArgs& args, unsigned char* panel, int stride,
                                                 FlowShared& sh, int tid) {
  const int K = ph.K, M = ph.M;
  // tagged words [M][K]: four at a time.  A thread takes the quads tid, tid + threads, ... of every row; a batch is
  // B (row, quad) pairs whose loads are in flight together.
  const unsigned tags = args.tag16 << 16;
  const unsigned* a = reinterpret_cast<const unsigned*>(ph.a);
  const int qpr = K / 4, per_row = (qpr + DF_CONSUMERS - 1) / DF_CONSUMERS, items = M * per_row;
  constexpr int B = 16;
  for (int i0 = 0; i0 < items; i0 += B) {
    const int r0 = i0 / per_row, j0 = i0 - r0 * per_row;
    uint4 v[B];
    unsigned mine = 0;
    {
      int r = r0, jq = j0;
#pragma unroll
      for (int j = 0; j < B; ++j) {
        v[j] = make_uint4(tags, tags, tags, tags);
        if (r < M && tid + jq * DF_CONSUMERS < qpr) mine |= 1u << j;
        if (++jq == per_row) {
          jq = 0;
          ++r;
        }
      }
    }
    // (a round whose tags are not all there is loaded again as a whole)
    for (int tries = 0;; ++tries) {
      int r = r0, jq = j0;
#pragma unroll
      for (int j = 0; j < B; ++j) {
        if (mine & (1u << j)) v[j] = df_ld_words4(a + (unsigned)(r * K + (tid + jq * DF_CONSUMERS) * 4));
        if (++jq == per_row) {
          jq = 0;
          ++r;
        }
      }
      unsigned stale = 0;
#pragma unroll
      for (int j = 0; j < B; ++j) stale |= (v[j].x ^ tags) | (v[j].y ^ tags) | (v[j].z ^ tags) | (v[j].w ^ tags);
      if ((stale >> 16) == 0u) break;
      if (df_tired(tries, sh, args.status)) {
        df_give_up(sh, args.status, 3);
        break;
      }
    }
    int r = r0, jq = j0;
#pragma unroll
    for (int j = 0; j < B; ++j) {
      if (mine & (1u << j)) {
        uint2 packed;
        packed.x = __byte_perm(v[j].x, v[j].y, 0x5410);
        packed.y = __byte_perm(v[j].z, v[j].w, 0x5410);
        *reinterpret_cast<uint2*>(panel + (unsigned)(r * stride + (tid + jq * DF_CONSUMERS) * 8)) = packed;
      }
      if (++jq == per_row) {
        jq = 0;
        ++r;
      }
    }
  }
}

// Builds the panel of the phase's rows: row r at panel + r * stride, K bfloat16 and zeros up to the next multiple of 32.
// LNQ: the LayerNorm path takes rows of up to 768 LNQ channels.
template <int LNQ>
__device__ void df_build_panel(const FlowPhase& ph, const FlowArgs& args, const FlowLayout& lay, unsigned char* smem, FlowShared& sh) {
  const int tid = df_opaque(threadIdx.x);
  const int K = ph.K, M = ph.M, KP = df_kpad(K);
  unsigned char* panel = smem + lay.panel_off;
  const int stride = lay.panel_stride;
  // the zeros behind every row's K elements (the products run over whole blocks of 32)
  if (KP > K)
    for (int i = tid; i < M * (KP - K); i += DF_CONSUMERS) {
      const int r = i / (KP - K), c = K + i % (KP - K);
      reinterpret_cast<__nv_bfloat16*>(panel + (size_t)r * stride)[c] = __float2bfloat16_rn(0.f);
    }
  if (ph.a_kind != FA_ROWS) {
    df_layernorm_rows<LNQ>(ph, args, panel, stride, sh, tid);
  } else {
    df_panel_from_words(ph, args, panel, stride, sh, tid);
  }
  df_bar_consumers();
}

// The activation of a product's epilogue.  A result that is rounded to bfloat16 anyway takes the tanh form of GELU with
// the hardware's tanh (relative error about 2^-11, below that rounding), as the prefill's product does; 32-bit results
// get the full-precision functions.
__device__ __noinline__ float df_activation_exact(float x, int act) { return apply_activation(x, act); }
__device__ __forceinline__ float df_activation(float x, int act, bool exact) {
  if (act == kActNone) return x;
  if (act == kActGeluTanh && !exact) {
    float t;
    asm("tanh.approx.f32 %0, %1;\n" : "=f"(t) : "f"(0.7978845608028654f * (x + 0.044715f * x * x * x)));
    return 0.5f * x * (1.f + t);
  }
  return df_activation_exact(x, act);
}

// Running (max, sum of exp(value - max), first index of the max) of the values a thread has finished, for two rows.
struct FlowTrack {
  float m[2], l[2];
  int idx[2];
};
__device__ __forceinline__ void df_track_merge(float& m, float& l, int& idx, float m2, float l2, int idx2) {
  if (m2 > m || (m2 == m && idx2 < idx)) idx = idx2;
  const float mm = fmaxf(m, m2);
  l = mm == -INFINITY ? 0.f : l * expf(m - mm) + l2 * expf(m2 - mm);
  m = mm;
}

__device__ __forceinline__ void df_ldmatrix_x2(unsigned (&r)[2], unsigned smem_addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];\n" : "=r"(r[0]), "=r"(r[1]) : "r"(smem_addr));
}
__device__ __forceinline__ void df_bar_group(int id, int threads) {
  asm volatile("bar.sync %0, %1;\n" ::"r"(id), "r"(threads) : "memory");
}

// How far the computing warps have come in the ring of weight slots: slots consumed so far in the launch, and where the
// next one lies (slot = use % slots, turn = use / slots, carried along instead of divided out).
struct FlowRing {
  unsigned use, slot, turn;
};

// A linear phase for the computing warps.
//
// The block's columns come as T tiles of at most 8.  G warps share a tile (G = 6, 3, 2 or 1: the most that leaves every
// tile a group), splitting its k between them 32 elements at a time; 6 / G tiles are in work together.  Warp 0 of a tile's
// group adds the group's partial sums in warp order and finishes the tile (bias, activation, residual, tags).  A slot of
// the ring belongs to one tile: every warp of the tile's group hands it back with 6 / G of the 6 arrivals that free it.
template <int LNQ>
__device__ void df_linear_phase(const FlowPhase& ph, int pi, const FlowArgs& args, const FlowLayout& lay, unsigned char* smem,
                                FlowShared& sh, FlowRing& ring) {
  const int tid = df_opaque(threadIdx.x), lane = tid & 31, warp = tid >> 5, g = lane >> 2, q = lane & 3;
  // (What the phase needs of its description and of the layout is read once, into registers: both lie in shared
  // memory, and every wait in between would have the compiler read them again.)
  const int N = ph.N, K = ph.K, M = ph.M, out_kind = ph.out_kind, act = ph.act, res_src = ph.res_src;
  const float* const bias_p = ph.bias;
  void* const out_p = ph.out;
  float* const track_p = ph.track;
  int* const status = args.status;
  const unsigned w_slots = (unsigned)lay.w_slots, w_slot_bytes = (unsigned)lay.w_slot_bytes;
  const int slot_k = lay.slot_k, w_row = lay.w_row;
  int c0, c1;
  df_columns(&ph, c0, c1);
  const int T = (c1 - c0 + 7) >> 3, n_chunks = ph.n_chunks;
  if (T == 0) {       // nothing to do in this phase (uniform for the block)
    if (track_p && tid < 16 && tid < M) {
      float* dst = track_p + ((long long)tid * gridDim.x + blockIdx.x) * 4;
      dst[0] = -INFINITY;
      dst[1] = 0.f;
      dst[2] = __int_as_float(0x7fffffff);
    }
    return;
  }
  df_build_panel<LNQ>(ph, args, lay, smem, sh);
  df_stamp(sh, 2);
  // (tiles in work together: as many as there are, and no more than the ring feeds with two slots to spare)
  const int feed = max(1, ((int)w_slots - 2) / n_chunks), want = min(T, feed);
  int G = 1, n_groups = DF_CWARPS, grp = warp, wg = 0;
  if (want == 1) G = 6, n_groups = 1, grp = 0, wg = warp;
  else if (want == 2) G = 3, n_groups = 2, grp = warp / 3, wg = warp - grp * 3;
  else if (want <= 5) G = 2, n_groups = 3, grp = warp >> 1, wg = warp & 1;
  const unsigned panel = ds_smem(smem + lay.panel_off);
  const int stride = lay.panel_stride;
  const bool two_rows = lay.panel_rows == 16;
  const unsigned tag16 = args.tag16, tag_out = df_tag32(args.epoch, pi);
  FlowTrack trk;
  trk.m[0] = trk.m[1] = -INFINITY;
  trk.l[0] = trk.l[1] = 0.f;
  trk.idx[0] = trk.idx[1] = 0x7fffffff;
  // lane's row and k offset inside a 16 x 16 block of A and an 8 x 32 block of W, as ldmatrix wants the addresses
  // (a panel of up to 8 rows: the lanes that address a row of the tile that the step does not have, rows 8 to 15
  // among them, all name the panel's row of zeros, which lies behind the step's rows)
  const int zero_row = lay.panel_rows - 1;
  const unsigned a_lane =
      (unsigned)((((lane >> 3) & 1) ? (two_rows ? 8 + (lane & 7) : zero_row) : (two_rows ? (lane & 7) : min(lane & 7, zero_row))) * stride +
                 (lane >> 4) * 16);
  const unsigned b_lane = (unsigned)((lane & 7) * w_row + (lane >> 3) * 16);
  const unsigned w_base = ds_smem(smem + lay.w_off);
  int round = 0;
  int fin = 0;                  // which warp of a group finishes its tile: they take turns
  for (int t = grp; t < T; t += n_groups, ++round, fin = fin + 1 == G ? 0 : fin + 1) {
    const bool finisher = wg == fin;
    const int tc0 = c0 + t * 8, nc = min(8, c1 - tc0);
    // the finishing warp's bias and residual travel while the products run
    float bias[4] = {0.f, 0.f, 0.f, 0.f};
    uint2 res[4];
    if (finisher) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int r = g + (i >> 1) * 8, cc = 2 * q + (i & 1);
        res[i] = make_uint2(0u, 0u);
        if (r < M && cc < nc) {
          if (bias_p) bias[i] = __ldg(bias_p + tc0 + cc);
          if (out_kind == FO_PAIRS) res[i] = df_ld_pair(reinterpret_cast<const uint2*>(out_p) + (unsigned)(r * N + tc0 + cc));
        }
      }
    }
    float acc[4] = {0.f, 0.f, 0.f, 0.f}, acc2[4] = {0.f, 0.f, 0.f, 0.f};
    // where the tile's first slot lies in the ring
    unsigned use = ring.use + (unsigned)(t * n_chunks), slot = ring.slot + (unsigned)(t * n_chunks), turn = ring.turn;
    while (slot >= w_slots) {
      slot -= w_slots;
      ++turn;
    }
    for (int c = 0; c < n_chunks; ++c, ++use) {
      // Warps run through the ring at their own pace: a warp may come for a slot a whole turn early, when the slot's
      // barrier still counts the turn before (whose parity it would mistake for its own).  So first the producer must
      // have asked for this very use; then the barrier is in this turn, or past it.
      for (int tries = 0; sh.w_issued <= use; ++tries)
        if (df_tired(tries, sh, status)) {
          df_give_up(sh, status, 3);
          break;
        }
      df_mbar_wait(&sh.wfull[slot], turn & 1u, sh, status);
      const unsigned ws = w_base + slot * w_slot_bytes + b_lane;
      const int kc = min(slot_k, K - c * slot_k), units = (kc + 31) >> 5;
      const unsigned pa0 = panel + a_lane + (unsigned)(c * slot_k) * 2u;
      // two units of 32 k at a time: their six loads are under way before the first product needs one
      for (int u = wg; u < units; u += 2 * G) {
        const bool second = u + G < units;
        const unsigned o0 = (unsigned)u * 64u, o1 = (unsigned)(second ? u + G : u) * 64u;
        unsigned b0[4], b1[4];
        ds_ldmatrix_x4(b0, ws + o0);
        ds_ldmatrix_x4(b1, ws + o1);
        unsigned a00[4], a01[4], a10[4], a11[4];
        ds_ldmatrix_x4(a00, pa0 + o0);
        ds_ldmatrix_x4(a01, pa0 + o0 + 32u);
        ds_ldmatrix_x4(a10, pa0 + o1);
        ds_ldmatrix_x4(a11, pa0 + o1 + 32u);
        ds_mma(acc, a00[0], a00[1], a00[2], a00[3], b0[0], b0[1]);
        ds_mma(acc2, a01[0], a01[1], a01[2], a01[3], b0[2], b0[3]);
        if (second) {
          ds_mma(acc, a10[0], a10[1], a10[2], a10[3], b1[0], b1[1]);
          ds_mma(acc2, a11[0], a11[1], a11[2], a11[3], b1[2], b1[3]);
        }
      }
      __syncwarp();
      if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0], %1;\n" ::"r"(ds_smem(&sh.wempty[slot])), "r"(DF_CWARPS / G) : "memory");
      if (++slot == w_slots) {
        slot = 0;
        ++turn;
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[i] += acc2[i];
    if (G > 1) {
      float (*red)[32][4] = sh.red[round & 1];
      *reinterpret_cast<float4*>(red[warp][lane]) = make_float4(acc[0], acc[1], acc[2], acc[3]);
      df_bar_group(2 + grp, G * 32);
      if (finisher) {
        // the group's sums in the order of its warps, whoever finishes
        float4 part[DF_CWARPS];
#pragma unroll
        for (int w2 = 0; w2 < DF_CWARPS; ++w2)
          if (w2 < G) part[w2] = *reinterpret_cast<const float4*>(red[warp - wg + w2][lane]);
        acc[0] = part[0].x, acc[1] = part[0].y, acc[2] = part[0].z, acc[3] = part[0].w;
#pragma unroll
        for (int w2 = 1; w2 < DF_CWARPS; ++w2)
          if (w2 < G) {
            acc[0] += part[w2].x;
            acc[1] += part[w2].y;
            acc[2] += part[w2].z;
            acc[3] += part[w2].w;
          }
      }
    }
    if (!finisher) continue;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = g + (i >> 1) * 8, cc = 2 * q + (i & 1);
      const float v = df_activation(acc[i] + bias[i], act, out_kind != FO_WORDS);
      acc[i] = v;
      if (r < M && cc < nc && track_p) {          // columns come to a thread in rising order: the first maximum stays
        float& m = trk.m[i >> 1];
        if (v > m) {
          trk.l[i >> 1] = trk.l[i >> 1] * __expf(m - v) + 1.f;
          m = v;
          trk.idx[i >> 1] = tc0 + cc;
        } else if (m != -INFINITY) {
          trk.l[i >> 1] += __expf(v - m);
        }
      }
    }
    if (out_kind == FO_PAIRS) {
      // the residual stream: this element was last written by phase res_src (by the thread that holds it in that
      // phase, or by the embedding): wait for its tag, add, write with this phase's tag
      const unsigned want = df_tag32(args.epoch, res_src);
      uint2* out = reinterpret_cast<uint2*>(out_p);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int r = g + (i >> 1) * 8, cc = 2 * q + (i & 1);
        if (r < M && cc < nc) {
          for (int tries = 0; res[i].y != want; ++tries) {
            if (df_tired(tries, sh, status)) {
              df_give_up(sh, status, 3);
              break;
            }
            res[i] = df_ld_pair(out + (unsigned)(r * N + tc0 + cc));
          }
          acc[i] += __uint_as_float(res[i].x);
        }
      }
    }
    const int cc0 = 2 * q;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int r = g + h * 8;
      if (r >= M || cc0 >= nc) continue;
      const bool pair_ok = cc0 + 1 < nc;
      const unsigned o = (unsigned)(r * N + tc0 + cc0);
      if (out_kind == FO_WORDS) {
        unsigned* out = reinterpret_cast<unsigned*>(out_p) + o;
        if (pair_ok && (o & 1) == 0) df_st_words2(out, acc[2 * h], acc[2 * h + 1], tag16);
        else {
          df_st_word(out, acc[2 * h], tag16);
          if (pair_ok) df_st_word(out + 1, acc[2 * h + 1], tag16);
        }
      } else if (out_kind == FO_PAIRS) {
        uint2* out = reinterpret_cast<uint2*>(out_p) + o;
        if (pair_ok && (o & 1) == 0) df_st_pairs2(out, acc[2 * h], acc[2 * h + 1], tag_out);
        else {
          df_st_pair(out, acc[2 * h], tag_out);
          if (pair_ok) df_st_pair(out + 1, acc[2 * h + 1], tag_out);
        }
      } else {
        float* out = reinterpret_cast<float*>(out_p) + o;
        out[0] = acc[2 * h];
        if (pair_ok) out[1] = acc[2 * h + 1];
      }
    }
  }
  ring.use += (unsigned)(T * n_chunks);
  ring.slot += (unsigned)(T * n_chunks);
  while (ring.slot >= w_slots) {
    ring.slot -= w_slots;
    ++ring.turn;
  }
  if (track_p) {
    // the block's (max, sum, argmax) of every row: the four lanes that share a row, then the warps
#pragma unroll
    for (int h = 0; h < 2; ++h) {
#pragma unroll
      for (int o = 1; o <= 2; o <<= 1) {
        const float m2 = __shfl_xor_sync(0xffffffffu, trk.m[h], o);
        const float l2 = __shfl_xor_sync(0xffffffffu, trk.l[h], o);
        const int i2 = __shfl_xor_sync(0xffffffffu, trk.idx[h], o);
        df_track_merge(trk.m[h], trk.l[h], trk.idx[h], m2, l2, i2);
      }
      if (q == 0) {
        sh.trk[warp][g + 8 * h][0] = trk.m[h];
        sh.trk[warp][g + 8 * h][1] = trk.l[h];
        sh.trk[warp][g + 8 * h][2] = __int_as_float(trk.idx[h]);
      }
    }
    df_bar_consumers();
    if (tid < M && tid < 16) {
      const int r = tid;
      float m = sh.trk[0][r][0], l = sh.trk[0][r][1];
      int idx = __float_as_int(sh.trk[0][r][2]);
      for (int w2 = 1; w2 < DF_CWARPS; ++w2) df_track_merge(m, l, idx, sh.trk[w2][r][0], sh.trk[w2][r][1], __float_as_int(sh.trk[w2][r][2]));
      float* dst = track_p + ((long long)r * gridDim.x + blockIdx.x) * 4;
      dst[0] = m;
      dst[1] = l;
      dst[2] = __int_as_float(idx);
    }
    df_bar_consumers();
  }
}


// ---- attention: merging the splits ----
// The block of split 0 merges the splits of its (sequence, head), in split order, as their tags show up: thread d takes
// dim d.  Four splits' worth of loads are in flight together.  (A function of its own, not inlined: what it holds in
// registers is then no burden on the loop over the keys.)
__device__ __noinline__ void df_attention_merge(const FlowPhase& ph, int pi, const FlowArgs& args, FlowShared& sh) {
  const int tid = threadIdx.x, hd = ph.head_dim, S = ph.n_splits, H = ph.n_heads, n_mine = sh.work.n;
  const unsigned tag16 = args.tag16, tag_part = df_tag32(args.epoch, pi);
  for (int mine = 0; mine < n_mine; ++mine) {
    const FlowItem it = sh.work.it[mine];
    if (it.split != 0 || tid >= hd) continue;
    const long long unit = (long long)it.seq * H + it.head;
    const uint2* src = ph.part + unit * S * (hd + 2);
    float Mx = -INFINITY, Lall = 0.f, o = 0.f;
    for (int s0 = 0; s0 < S; s0 += 4) {
      uint2 po[4], pm[4], pl[4];
      unsigned pending = 0;
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (s0 + j < S) pending |= 1u << j;
      const unsigned have = pending;
      for (int tries = 0; pending != 0; ++tries) {
        if (tries >= DF_SPIN_LIMIT || ((tries & 1023) == 1023 && (sh.failed || (args.status && df_ld_status(args.status) != 0)))) {
          df_give_up(sh, args.status, 3);
          break;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (pending & (1u << j)) {
            const uint2* one = src + (long long)(s0 + j) * (hd + 2);
            po[j] = df_ld_pair(one + tid);
            pm[j] = df_ld_pair(one + hd);
            pl[j] = df_ld_pair(one + hd + 1);
          }
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if ((pending & (1u << j)) && po[j].y == tag_part && pm[j].y == tag_part && pl[j].y == tag_part) pending &= ~(1u << j);
      }
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (have & (1u << j)) {
          const float ms = __uint_as_float(pm[j].x);
          if (ms == -INFINITY) continue;
          const float mm = fmaxf(Mx, ms);
          const float a = Mx == -INFINITY ? 0.f : ds_exp2(Mx - mm), b = ds_exp2(ms - mm);
          Lall = Lall * a + __uint_as_float(pl[j].x) * b;
          o = o * a + __uint_as_float(po[j].x) * b;
          Mx = mm;
        }
    }
    df_st_word(ph.attn_out + unit * hd + tid, Lall > 0.f ? o / Lall : 0.f, tag16);
  }
}

// ---- attention ---------------------------------------------------------------------------------------------
// One query per (sequence, head) is the 8-column operand of products whose rows are keys (decode_mma.cuh); the pages
// of the block's items arrive through the ring of page slots in the order of the block's stream of pages.  A warp
// takes chunks of 8 T keys (the c-th chunk of the stream belongs to warp c % 6) and hands every page back when it is
// done with it, whether it had a chunk in it or not.  `puse`: how many page slots the block has consumed so far in the launch.
template <int I, int T>
__device__ void df_attention_items(const FlowPhase& ph, int pi, const FlowArgs& args, const FlowLayout& lay, unsigned char* smem,
                                   FlowShared& sh, unsigned& puse) {
  constexpr int CK = 8 * T, CPP = DS_PAGE / CK;       // keys of a chunk, chunks of a page
  const int tid = df_opaque(threadIdx.x), lane = tid & 31, warp = tid >> 5, g = lane >> 2, q = lane & 3;
  const int hd = ph.head_dim, page_elems = DS_PAGE * hd, cbs = df_col_blocks(hd);
  const int S = ph.n_splits, H = ph.n_heads, group = ph.n_heads / ph.n_kv_heads;
  const float scale_log2 = ph.scale_log2;
  const unsigned tag16 = args.tag16, tag_part = df_tag32(args.epoch, pi);
  __nv_bfloat16* rows = reinterpret_cast<__nv_bfloat16*>(smem + lay.rows_off);      // [items][query, new key, new value][hd]
  float* s_acc = reinterpret_cast<float*>(smem + lay.acc_off);                       // [2][warps][hd]
  if (warp == 0) df_plan(&ph, sh, sh.work);
  df_bar_consumers();
  const int n_mine = sh.work.n, total = sh.work.start[n_mine];
  {
    // Every item's query and new key and value: tagged words of the projections.  A warp takes one of these rows at
    // a time, a lane four of its dims; a row whose tags are not all there is loaded again.
    const int quads = hd >> 2, kinds = ph.k_off >= 0 ? 3 : 1, n_rows = n_mine * kinds;
    const unsigned tags = tag16 << 16;
    const unsigned* const proj = ph.q;
    const int q_stride = (int)ph.q_stride, k_off = ph.k_off, v_off = ph.v_off;
    for (int pair = warp; pair < n_rows; pair += DF_CWARPS) {
      const int j = kinds == 3 ? pair / 3 : pair, r = pair - j * kinds;
      const int seq = sh.work.it[j].seq, head = sh.work.it[j].head;
      const int col = r == 0 ? head * hd : (r == 1 ? k_off : v_off) + sh.work.it[j].kv_head * hd;
      if (lane < quads) {
        const unsigned* src = proj + (unsigned)(seq * q_stride + col + lane * 4);
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        for (int tries = 0;; ++tries) {
          v = df_ld_words4(src);
          if ((((v.x ^ tags) | (v.y ^ tags) | (v.z ^ tags) | (v.w ^ tags)) >> 16) == 0u) break;
          if (df_tired(tries, sh, args.status)) {
            df_give_up(sh, args.status, 3);
            break;
          }
        }
        uint2 packed;
        packed.x = __byte_perm(v.x, v.y, 0x5410);
        packed.y = __byte_perm(v.z, v.w, 0x5410);
        *reinterpret_cast<uint2*>(rows + (j * 3 + r) * hd + lane * 4) = packed;
      }
    }
  }
  df_bar_consumers();
  // where the block's stream of pages stands in the ring (slot = use % slots, turn = use / slots, carried along)
  const unsigned p_slots = (unsigned)lay.p_slots, p_slot_bytes = (unsigned)lay.p_slot_bytes;
  unsigned char* const pages = smem + lay.p_off;
  int* const status = args.status;
  const bool files = ph.k_off >= 0;
  unsigned slot = puse % p_slots, turn = puse / p_slots;
  puse += (unsigned)total;
  unsigned k_lane[2 * I], v_lane[2 * I];
  ds_lane_offsets<I>(lane, k_lane, v_lane);
  for (int mine = 0; mine < n_mine; ++mine) {
    const FlowItem it = sh.work.it[mine];
    const __nv_bfloat16* my_rows = rows + mine * 3 * hd;
    const int k0 = sh.work.start[mine], n_pages = sh.work.start[mine + 1] - k0;
    const int kv_head = it.kv_head;
    const int lo = max(it.lo, it.pg_first * DS_PAGE), hi = min(it.L, it.pg_end * DS_PAGE);
    // the query as the products' 8-column operand (every column the query)
    unsigned qa[I * 4];          // per 16 dims: dims 2q, 2q + 1 and 8 + 2q, 9 + 2q
#pragma unroll
    for (int j = 0; j < I * 4; ++j) {
      const int d = 16 * (j >> 1) + 8 * (j & 1) + 2 * q;
      qa[j] = d < hd ? *reinterpret_cast<const unsigned*>(my_rows + d) : 0u;
    }
    if (ph.k_off >= 0 && it.L > 0 && it.split == 0 && it.head == kv_head * group) {
      // this block also files the new token's key and value in the sequence's page (for the steps to come)
      const int pos = it.L - 1;
      const long long page = df_table_entry(&ph, sh, it.seq, (pos / DS_PAGE) % ph.table_len);
      const long long off = (page * ph.n_kv_heads + kv_head) * (long long)page_elems + (long long)(pos % DS_PAGE) * hd;
      for (int c = tid; c < hd / 8; c += DF_CONSUMERS) {
        *reinterpret_cast<uint4*>(ph.k_pool + off + c * 8) = *reinterpret_cast<const uint4*>(my_rows + hd + c * 8);
        *reinterpret_cast<uint4*>(ph.v_pool + off + c * 8) = *reinterpret_cast<const uint4*>(my_rows + 2 * hd + c * 8);
      }
    }
    float m = -INFINITY, l = 0.f;
    float acc[I * 2][4];
#pragma unroll
    for (int n = 0; n < I * 2; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[n][e] = 0.f;
    for (int p = 0; p < n_pages; ++p) {
      const int k = k0 + p;
      unsigned char* Kt = pages + (size_t)slot * p_slot_bytes;      // the page's key tiles; its value tiles follow
      const unsigned Ks = ds_smem(Kt), Vs = Ks + (unsigned)(cbs * DS_PAGE * 128);
      // Every warp waits for every page, with or without a chunk in it: a warp hands a slot back only in the turn it
      // has seen filled, so that no warp's arrival is counted for the turn before.
      df_mbar_wait(&sh.pfull[slot], turn & 1u, sh, status);
#pragma unroll 1
      for (int h = 0; h < CPP; ++h) {
        if ((k * CPP + h) % DF_CWARPS != warp) continue;
        const int key0 = (it.pg_first + p) * DS_PAGE + h * CK;
        if (key0 >= hi || key0 + CK <= lo) continue;
        if (files && it.L - 1 >= key0 && it.L - 1 < key0 + CK) {
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
        ds_attn_chunk_kt<I, T / 2>(qa, k_lane, v_lane, Ks, Vs, hd, h * CK, key0, lo, hi, scale_log2, m, l, acc, lane);
      }
      __syncwarp();
      if (lane == 0) df_mbar_arrive(&sh.pempty[slot]);      // (every warp, once per page)
      if (++slot == p_slots) {
        slot = 0;
        ++turn;
      }
    }
    df_stamp(sh, 2 + min(mine, 5));
    // a lane summed the weights of its own keys (its quad's: the same in the quad's four lanes)
    l += __shfl_xor_sync(0xffffffffu, l, 4);
    l += __shfl_xor_sync(0xffffffffu, l, 8);
    l += __shfl_xor_sync(0xffffffffu, l, 16);
    // the lanes of quad g hold dims 16 n + g and 16 n + g + 8 of value tile n.  (Two sets of the warps' results, used
    // in turn: the block-wide hand-over of the next item orders this item's reads before the item after that writes.)
    float* my_acc = s_acc + (mine & 1) * DF_CWARPS * hd;
    float (*my_ml)[2] = sh.ml[mine & 1];
    if (q == 0) {
#pragma unroll
      for (int n = 0; n < I * 2; ++n) {
        const int d = 16 * n + g;
        if (d < hd) {
          my_acc[warp * hd + d] = acc[n][0];
          my_acc[warp * hd + d + 8] = acc[n][2];
        }
      }
      if (g == 0) {
        my_ml[warp][0] = m;
        my_ml[warp][1] = l;
      }
    }
    df_bar_consumers();
    if (tid < hd) {
      float Mb = -INFINITY;
#pragma unroll
      for (int w2 = 0; w2 < DF_CWARPS; ++w2) Mb = fmaxf(Mb, my_ml[w2][0]);
      float Lb = 0.f, o = 0.f;
#pragma unroll
      for (int w2 = 0; w2 < DF_CWARPS; ++w2) {
        const float wg = Mb == -INFINITY ? 0.f : ds_exp2(my_ml[w2][0] - Mb);
        Lb += my_ml[w2][1] * wg;
        o += my_acc[w2 * hd + tid] * wg;
      }
      const long long unit = (long long)it.seq * H + it.head;
      if (S == 1) {
        df_st_word(ph.attn_out + unit * hd + tid, Lb > 0.f ? o / Lb : 0.f, tag16);
      } else {
        uint2* dst = ph.part + (unit * S + it.split) * (hd + 2);
        df_st_pair(dst + tid, o, tag_part);
        if (tid == 0) {
          df_st_pair(dst + hd, Mb, tag_part);
          df_st_pair(dst + hd + 1, Lb, tag_part);
        }
      }
    }
  }
  if (S > 1) df_attention_merge(ph, pi, args, sh);
}

// Token selection for the rows this block takes (after the grid barrier): greedy from the readout's per-block
// partials, or the full selection from the logits; the selected id becomes the next step's token.  A function of its
// own: it runs once a step, and its code need not lie among the phases'.
__device__ __noinline__ void df_select(const FlowArgs& args, FlowShared& sh) {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const FlowPhase* ph = args.phases + args.n_phases - 1;
  if (sh.ok) {
    for (int r = blockIdx.x; r < ph->M; r += gridDim.x) {
      if (!ph->do_sample && ph->partials) {
        // greedy: the readout left every block's (max, sum, argmax) of the row; a warp merges them
        if (warp == 0) {
          float m = -INFINITY, l = 0.f;
          int idx = 0x7fffffff;
          for (int b = lane; b < ph->n_partials; b += 32) {
            const float4 p = __ldcg(reinterpret_cast<const float4*>(ph->partials + ((long long)r * ph->n_partials + b) * 4));
            df_track_merge(m, l, idx, p.x, p.y, __float_as_int(p.z));
          }
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) {
            const float m2 = __shfl_xor_sync(0xffffffffu, m, o);
            const float l2 = __shfl_xor_sync(0xffffffffu, l, o);
            const int i2 = __shfl_xor_sync(0xffffffffu, idx, o);
            df_track_merge(m, l, idx, m2, l2, i2);
          }
          if (lane == 0) {
            ph->out_ids[r] = idx;
            ph->out_logp[r] = -logf(l);
            ph->adv_tokens[r] = idx;
            ph->adv_positions[r] += 1;
            ph->adv_past[r] += 1;
            ph->adv_ctx[r] += 1;
            ph->counters[r] += 1;
          }
        }
        continue;
      }
      float u = 0.f;
      if (ph->do_sample) u = stream_uniform(ph->seeds[r], (unsigned long long)ph->counters[r]);
      select_row<DF_THREADS>(ph->logits + (long long)r * ph->vocab, ph->vocab, ph->do_sample, ph->temperature, ph->top_k,
                             ph->top_p, ph->min_p, u, ph->out_ids + r, ph->out_logp + r, sh.sample);
      __syncthreads();
      if (tid == 0) {      // the selected id becomes the next step's token; the sequence moves on by one
        ph->adv_tokens[r] = ph->out_ids[r];
        ph->adv_positions[r] += 1;
        ph->adv_past[r] += 1;
        ph->adv_ctx[r] += 1;
        ph->counters[r] += 1;
      }
    }
  }
}

// ---- the kernel --------------------------------------------------------------------------------------------
// LNQ: rows of up to 768 LNQ channels can be normalised; AI, AT: head sizes up to 32 AI, chunks of 8 AT keys.
template <int LNQ, int AI, int AT>
__global__ void __launch_bounds__(DF_THREADS, 1) decode_flow_kernel(const FlowArgs args) {
  extern __shared__ __align__(128) unsigned char df_smem_raw[];
  __shared__ FlowShared sh;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  unsigned char* smem = df_smem_raw + ((1024u - (ds_smem(df_smem_raw) & 1023u)) & 1023u);
  if (tid == 0) {
    sh.lay = df_layout(args.rows, args.max_k, args.max_ln_k, args.head_dim, args.w_slots, args.p_slots, args.slot_k);
    for (int i = 0; i < args.w_slots; ++i) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(ds_smem(&sh.wfull[i])));
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(ds_smem(&sh.wempty[i])), "r"(DF_CWARPS));
    }
    for (int i = 0; i < args.p_slots; ++i) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(ds_smem(&sh.pfull[i])));
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(ds_smem(&sh.pempty[i])), "r"(DF_CWARPS));
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    sh.failed = 0;
    sh.w_issued = 0;
    sh.ok = 1;
    sh.ctx_src = nullptr;
    sh.table_src = nullptr;
    sh.trace = nullptr;
  }
  __syncthreads();
  const FlowLayout& lay = sh.lay;
  // The weight slots and the panel start as zeros: products run over whole blocks of 32 k, and what lies behind a row's
  // K elements must be a number (zero times it is added), never the bits of a NaN.
  for (long long i = tid; i < (lay.rows_off - lay.w_off) / 16; i += DF_THREADS)
    reinterpret_cast<uint4*>(smem + lay.w_off)[i] = make_uint4(0u, 0u, 0u, 0u);
  // the phase list's first attention phase: its lengths and page tables are read once (they do not change during the step)
  int first_attention = -1;
  for (int pi = 0; pi < args.n_phases && first_attention < 0; ++pi)
    if (args.phases[pi].type == FP_ATTENTION) first_attention = pi;
  __syncthreads();
  if (first_attention >= 0) {
    const FlowPhase* ph = args.phases + first_attention;
    if (ph->M <= 16 && ph->table_len <= DF_TABLE_CACHE) {
      for (int i = tid; i < ph->M * ph->table_len; i += DF_THREADS) {
        const int seq = i / ph->table_len, index = i - seq * ph->table_len;
        sh.table_cache[seq][index] = ph->table[(long long)seq * ph->table_stride + index];
      }
      if (tid < ph->M) sh.ctx_cache[tid] = ph->ctx_len[tid];
      if (tid == 0) {
        sh.ctx_src = ph->ctx_len;
        sh.table_src = ph->table;
      }
    }
  }
  static_assert(sizeof(FlowPhase) % 16 == 0, "phases are copied 16 bytes at a time");
  constexpr int PHASE_VECS = (int)(sizeof(FlowPhase) / 16);
  static_assert(PHASE_VECS <= 64, "two warps copy a phase's description");
  if (tid < PHASE_VECS) reinterpret_cast<uint4*>(&sh.phase[0])[tid] = reinterpret_cast<const uint4*>(args.phases)[tid];
  __syncthreads();
  // token selection comes last (if at all) and is the work of the whole block after the grid barrier
  const bool selects = args.phases[args.n_phases - 1].type == FP_SAMPLE;
  const int n_main = args.n_phases - (selects ? 1 : 0);

  if (warp >= DF_CWARPS) {
    if (warp == DF_CWARPS) {
      // ---- the weight producer ----
      const unsigned uses = df_weight_producer(args, n_main, lay, smem, sh);
      if (lane == 0) df_drain(sh.wfull, uses, lay.w_slots);
    } else if (warp == DF_CWARPS + 1) {
      // ---- the page producer ----
      const unsigned uses = df_page_producer(args, n_main, lay, smem, sh);
      if (lane == 0) df_drain(sh.pfull, uses, lay.p_slots);
    }
  } else {
    // ---- the computing warps ----
    FlowRing ring{0u, 0u, 0u};
    unsigned puse = 0;
    for (int pi = 0; pi < n_main; ++pi) {
      df_bar_consumers();      // everyone is done with the previous phase: its description, the panel, the partial sums
      if (sh.failed) break;    // (uniform: written before the barrier)
      const FlowPhase& ph = sh.phase[pi & 1];
      // the next phase's description travels meanwhile
      // (asked for by the last warps: right after a phase's stores a copy may wait a few hundred nanoseconds for the
      // load/store path, and these warps' share of the next rows is the least likely to be waited for)
      if (pi + 1 < args.n_phases && tid >= DF_CONSUMERS - 64 && tid - (DF_CONSUMERS - 64) < PHASE_VECS)
        df_cp16(reinterpret_cast<uint4*>(&sh.phase[(pi + 1) & 1]) + (tid - (DF_CONSUMERS - 64)),
                reinterpret_cast<const uint4*>(args.phases + pi + 1) + (tid - (DF_CONSUMERS - 64)));
      if (args.trace && tid == 0) sh.trace = blockIdx.x == 0 ? args.trace + DF_TRACE_SLOTS * pi : nullptr;
      df_stamp(sh, 0);
      if (ph.type == FP_EMBED) {
        const unsigned tag = df_tag32(args.epoch, pi);
        for (int r = blockIdx.x; r < ph.M; r += gridDim.x) {
          const int id = ph.tokens[r], pos = ph.wpe ? ph.positions[r] : 0;
          const bool ok = id >= 0 && id < ph.vocab && pos >= 0 && (!ph.wpe || pos < ph.n_positions);
          for (int c = tid * 2; c < ph.width; c += 2 * DF_CONSUMERS) {
            float v0 = 0.f, v1 = 0.f;
            if (ok) {
              const __nv_bfloat162 e = *reinterpret_cast<const __nv_bfloat162*>(ph.wte + (long long)id * ph.width + c);
              v0 = __low2float(e);
              v1 = __high2float(e);
              if (ph.wpe) {
                const __nv_bfloat162 p = *reinterpret_cast<const __nv_bfloat162*>(ph.wpe + (long long)pos * ph.width + c);
                v0 += __low2float(p);
                v1 += __high2float(p);
              }
            }
            df_st_pairs2(ph.resid + (long long)r * ph.width + c, v0, v1, tag);
          }
          if (!ok && tid == 0 && args.status) atomicCAS(args.status, 0, 4);
        }
      } else if (ph.type == FP_LINEAR) {
        df_linear_phase<LNQ>(ph, pi, args, lay, smem, sh, ring);
      } else if (ph.type == FP_ATTENTION) {
        df_attention_items<AI, AT>(ph, pi, args, lay, smem, sh, puse);
      }
      df_stamp(sh, 1);
      df_cp_wait();
    }
  }
  __syncthreads();
  if (selects && !sh.failed) {
    // ---- the grid barrier before token selection: everything the blocks wrote is visible before the arrival is ----
    if (tid == 0) {
      asm volatile("red.release.gpu.global.add.u32 [%0], 1;\n" ::"l"(args.counter) : "memory");
      int ok = 1, spins = 0;
      for (;;) {
        unsigned seen;
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];\n" : "=r"(seen) : "l"(args.counter) : "memory");
        if (seen >= gridDim.x) break;
        if (++spins > DF_SPIN_LIMIT || ((spins & 1023) == 1023 && args.status && df_ld_status(args.status) != 0)) {
          ok = 0;
          break;
        }
      }
      if (!ok) df_give_up(sh, args.status, 3);
      sh.ok = ok;
    }
    __syncthreads();
    df_select(args, sh);
  }
}

}  // namespace bt

namespace bt {

typedef void (*FlowKernel)(const FlowArgs);
// The kernel's variants: rows of up to 768, 1536 or 2304 channels to normalise, head sizes up to 64 or 128.
static FlowKernel df_variant(int max_ln_k, int head_dim, int* index) {
  const int q = max_ln_k <= 768 ? 1 : (max_ln_k <= 1536 ? 2 : 3), big = head_dim > 64 ? 1 : 0;
  *index = (q - 1) * 2 + big;
  switch (*index) {
    case 0: return decode_flow_kernel<1, 2, 4>;
    case 1: return decode_flow_kernel<1, 4, 2>;
    case 2: return decode_flow_kernel<2, 2, 4>;
    case 3: return decode_flow_kernel<2, 4, 2>;
    case 4: return decode_flow_kernel<3, 2, 4>;
    default: return decode_flow_kernel<3, 4, 2>;
  }
}

}  // namespace bt

extern "C" int bt_decode_flow_phase_bytes() { return (int)sizeof(bt::FlowPhase); }

// Sizes the step's shared memory for these phases (host copy of the program, in which it fills col_q, col_r and
// n_chunks of the linear phases: upload the program after this call) and `rows` sequences.
// out[0..7] = max_k, max_ln_k, head_dim, w_slots, p_slots, bytes of dynamic shared memory, slot_k, 0.  Returns 0, or
// non-zero with the library's error text when the step does not fit.
extern "C" int bt_decode_flow_plan(void* phases_host, int n_phases, int rows, long long* out) {
  using namespace bt;
  FlowPhase* ph = reinterpret_cast<FlowPhase*>(phases_host);
  BT_CHECK(n_phases >= 1 && n_phases < 1023, "decode_flow: %d phases are outside 1..1022", n_phases);
  BT_CHECK(rows >= 1 && rows <= 16, "decode_flow: %d rows are outside 1..16", rows);
  int max_k = 32, max_ln_k = 8, head_dim = 0;
  for (int i = 0; i < n_phases; ++i) {
    BT_CHECK(ph[i].type != FP_SAMPLE || i == n_phases - 1, "decode_flow: token selection must be the last phase");
    if (ph[i].type == FP_LINEAR) {
      BT_CHECK(ph[i].K % 8 == 0 && ph[i].K >= 8, "decode_flow: K=%d is no multiple of 8", ph[i].K);
      if (ph[i].K > max_k) max_k = ph[i].K;
      if (ph[i].a_kind != FA_ROWS) {
        BT_CHECK(ph[i].K <= 3 * 768, "decode_flow: a LayerNorm over %d channels exceeds the 2304 the step holds", ph[i].K);
        if (ph[i].K > max_ln_k) max_ln_k = ph[i].K;
      }
    } else if (ph[i].type == FP_ATTENTION) {
      BT_CHECK(ph[i].head_dim % 16 == 0 && ph[i].head_dim >= 16 && ph[i].head_dim <= 128,
               "decode_flow: head_dim %d is outside 16..128 in steps of 16", ph[i].head_dim);
      BT_CHECK(head_dim == 0 || head_dim == ph[i].head_dim, "decode_flow: one head size in all attention phases");
      head_dim = ph[i].head_dim;
    }
  }
  const int n_blocks = sm_count();
  BT_CHECK(n_blocks > 0, "decode_flow: cannot read the number of multiprocessors of the current device");
  int variant = 0;
  FlowKernel kernel = df_variant(max_ln_k, head_dim, &variant);
  cudaFuncAttributes attr;
  cudaError_t e = cudaFuncGetAttributes(&attr, kernel);
  BT_CHECK(e == cudaSuccess, "decode_flow: cannot read the kernel's attributes: %s", cudaGetErrorString(e));
  // (a model whose layers give a block 64 KB of weights and more a phase is the better for every slot: GPT-2 XL at one
  // row 1.75 against 1.85 ms a step with all of shared memory, GPT-2 large at four rows 1.48 against 1.51; GPT-2 small
  // at eight rows is the other way round, 0.404 against 0.400 ms)
  long long widest = 0;
  for (int i = 0; i < n_phases; ++i)
    if (ph[i].type == FP_LINEAR && ph[i].N < 8192 && (long long)ph[i].N * ph[i].K > widest) widest = (long long)ph[i].N * ph[i].K;
  const int kb0 = widest * 2 / n_blocks >= 64 * 1024 ? 227 : 195;
  int slot_k = 32, p_slots = 0, w_slots = 0;
  // The k extent of a weight slot (a multiple of 32; a slot holds one piece of one tile's k): the one that leaves the
  // least of the ring unused; of equals the largest.  Slots of up to 1,664 of k take a wide model's rows of K in one
  // piece (half the hand-overs between the producer and the warps: GPT-2 XL at one row 1.57 against 1.75 ms a step); if
  // such slots leave the ring fewer than 4 of them, slots of at most 1,024 are taken.
  for (int limit : {DF_MAX_SLOT_K, 1024}) {
    long long best = -1;
    for (int c = 32; c <= limit; c += 32) {
      long long cost = 0;
      for (int i = 0; i < n_phases; ++i)
        if (ph[i].type == FP_LINEAR) cost += (long long)ph[i].N * ((ph[i].K + c - 1) / c) * c;
      if (best < 0 || cost <= best) {
        best = cost;
        slot_k = c;
      }
    }
    // Two sizes of shared memory are tried.  195 KB leaves the multiprocessor some 60 KB of first-level cache, where the
    // few registers the compiler spills stay close; if that leaves the weights' ring fewer than 5 slots, everything the
    // block may have (227 KB) is taken, and spilled registers live in the second-level cache.
    // page slots: about 48 KB of them (at least 2, at most 8); weight slots: what is left (at least 4)
    for (int kb = kb0; kb <= 227; kb += 32) {
      const long long budget = (long long)kb * 1024 - (long long)attr.sharedSizeBytes - 1024 - 64;
      p_slots = 0;
      if (head_dim > 0) {
        p_slots = 48 * 1024 / df_page_slot_bytes(head_dim);
        p_slots = p_slots < 2 ? 2 : (p_slots > 8 ? 8 : p_slots);
      }
      for (;;) {
        const FlowLayout fixed = df_layout(rows, max_k, max_ln_k, head_dim, 0, p_slots, slot_k);
        w_slots = (int)((budget - fixed.total) / fixed.w_slot_bytes);
        if (w_slots >= 4 || p_slots <= 2) break;
        --p_slots;
      }
      if (w_slots >= 5) break;
    }
    if (w_slots >= 4 || slot_k <= 1024) break;
  }
  BT_CHECK(w_slots >= 4, "decode_flow: %d rows of K=%d leave no room for the weights' ring in shared memory", rows, max_k);
  if (w_slots > DF_MAX_WSLOTS) w_slots = DF_MAX_WSLOTS;
  // what the kernel would otherwise divide out in every phase
  for (int i = 0; i < n_phases; ++i)
    if (ph[i].type == FP_LINEAR) {
      ph[i].col_q = ph[i].N / n_blocks;
      ph[i].col_r = ph[i].N % n_blocks;
      ph[i].n_chunks = (ph[i].K + slot_k - 1) / slot_k;
    }
  const FlowLayout lay = df_layout(rows, max_k, max_ln_k, head_dim, w_slots, p_slots, slot_k);
  out[0] = max_k;
  out[1] = max_ln_k;
  out[2] = head_dim;
  out[3] = w_slots;
  out[4] = p_slots;
  out[5] = lay.total;
  out[6] = slot_k;
  out[7] = 0;
  return 0;
}

// phases_dev: the program in device memory; plan: what bt_decode_flow_plan gave for it.  epoch: a number that is new
// for every launch of this program (1, 2, 3, ...): it is the tag of everything the launch writes.  counter: one
// unsigned for the grid barrier before token selection (this call clears it).  The launch is cooperative: every block
// is resident, which the waiting relies on.  trace: optional 8 * n_phases 64-bit slots for block 0's timeline.
extern "C" int bt_decode_flow(const void* phases_dev, int n_phases, unsigned epoch, int rows, const long long* plan,
                              unsigned* counter, int* status, long long* trace, cudaStream_t stream) {
  using namespace bt;
  BT_CHECK(n_phases >= 1 && epoch >= 1 && epoch < (1u << 22), "decode_flow: bad phase count %d or epoch %u", n_phases, epoch);
  const int n_sms = sm_count();
  BT_CHECK(n_sms > 0, "decode_flow: cannot read the number of multiprocessors of the current device");
  const long long smem_bytes = plan[5];
  int variant = 0;
  FlowKernel kernel = df_variant((int)plan[1], (int)plan[2], &variant);
  static long long configured[64][6];
  int dev = 0;
  cudaGetDevice(&dev);
  BT_CHECK(dev >= 0 && dev < 64, "decode_flow: device %d is beyond the 64 this library tracks", dev);
  if (configured[dev][variant] < smem_bytes) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes);
    BT_CHECK(e == cudaSuccess, "decode_flow: cannot reserve %lld bytes of shared memory: %s", smem_bytes, cudaGetErrorString(e));
    configured[dev][variant] = smem_bytes;
  }
  cudaError_t e = cudaMemsetAsync(counter, 0, sizeof(unsigned), stream);
  BT_CHECK(e == cudaSuccess, "decode_flow: cannot clear the barrier counter: %s", cudaGetErrorString(e));
  FlowArgs args{reinterpret_cast<const FlowPhase*>(phases_dev), n_phases, epoch, counter, status, trace, rows, (int)plan[0],
                (int)plan[1], (int)plan[2], (int)plan[3], (int)plan[4], (int)plan[6], epoch % 65535u + 1u};
  void* kargs[] = {(void*)&args};
  e = cudaLaunchCooperativeKernel((const void*)kernel, dim3(n_sms), dim3(DF_THREADS), kargs, (size_t)smem_bytes, stream);
  BT_CHECK(e == cudaSuccess, "decode_flow: launch failed: %s", cudaGetErrorString(e));
  count_launch();
  return 0;
}
