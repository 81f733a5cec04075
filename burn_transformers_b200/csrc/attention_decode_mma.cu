// Decode attention on tensor cores (bfloat16): one new token per sequence over that sequence's pages.
//
// grid (n_splits, n_heads, n_seqs), four computing warps and a producer warp a block.  A block owns a run of pages
// of one (sequence, head), which travel through a ring of slots in shared memory: the producer asks the tensor
// memory accelerator for them (a 64 x 64 box per tile, 128-byte swizzle), the first ones before the kernel waits
// for its predecessor (old keys and values do not change during a step), each further one when the warps that read
// the slot have handed it back.  Each computing warp takes 32- or 16-key chunks of the landed pages by itself
// (scores and weighted values with mma.sync, the keys on the tiles' 16 rows and the query as the 8-column operand,
// softmax in 32-bit); no barrier of the whole block stands between pages.  The warps are merged through shared
// memory and the splits of a (sequence, head) through distributed shared memory inside a thread-block cluster (at
// most 8 splits) or through scratch memory, where the block that takes the last ticket merges.  Blocks are small (a
// few pages) so that many are resident on an SM: a block is a chain of latencies, and it is the other blocks that
// hide them.
// The block of split 0 files the new token's key and value in the page (one block per key head does).
// Every wait for a copy is bounded; a wait that runs out sets the status word and makes the result NaN.
#include <cooperative_groups.h>

#include "api.h"
#include "common.cuh"
#include "decode_mma.cuh"
#include "tma.cuh"

namespace cg = cooperative_groups;

namespace bt {

constexpr int DM_WARPS = 4;                     // warps that compute; one more warp asks for the pages
constexpr int DM_THREADS = (DM_WARPS + 1) * 32;
constexpr int DM_WAIT_LIMIT = 1 << 18;
constexpr int DM_SMEM_BUDGET = 64 * 1024;      // for page slots: several blocks share an SM

struct DecodeMmaParams {
  const __nv_bfloat16* q;        // rows of the projections: query head h at q + h * head_dim
  long long q_stride;
  const __nv_bfloat16* new_k;    // the new token's key / value channels in the same rows (null: already filed)
  const __nv_bfloat16* new_v;
  __nv_bfloat16* k_pool;         // [page][kv_head][64][head_dim]
  __nv_bfloat16* v_pool;
  const int* table;
  int table_stride, table_len;
  __nv_bfloat16* out;            // [n_seqs][n_heads * head_dim]
  float* part_acc;               // scratch merge: [unit][split][head_dim]
  float* part_ml;                //                [unit][split][2]
  int* tickets;
  int* status;
  const int* ctx_len;
  int n_heads, n_kv_heads, head_dim;
  float scale_log2;
  int window, slots, use_cluster;
};

template <int I, int T>
__global__ void __launch_bounds__(DM_THREADS)
attention_decode_mma_kernel(const __grid_constant__ CUtensorMap k_map, const __grid_constant__ CUtensorMap v_map, DecodeMmaParams p) {
  constexpr int CK = 8 * T, CPP = DS_PAGE / CK;
  extern __shared__ unsigned char dm_smem_raw[];
  __shared__ __align__(8) unsigned long long full[16], empty[16];
  __shared__ float s_ml[DM_WARPS][2];
  __shared__ float c_ml[2];            // this block's (max, sum), read by its cluster peers
  __shared__ int s_flag;
  pdl_trigger();
  const int split = blockIdx.x, n_splits = gridDim.x;
  const int head = blockIdx.y, seq = blockIdx.z;
  const int kv_head = head / (p.n_heads / p.n_kv_heads);
  const int hd = p.head_dim, cbs = (hd + 63) / 64;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, q = lane & 3;
  const int slot_bytes = 2 * cbs * DS_PAGE * 128;
  unsigned char* ring = dm_smem_raw + ((1024u - (ds_smem(dm_smem_raw) & 1023u)) & 1023u);
  float* s_acc = reinterpret_cast<float*>(ring + (size_t)p.slots * slot_bytes);     // [DM_WARPS][hd]
  float* c_acc = s_acc + DM_WARPS * hd;                                             // [hd], read by the cluster peers

  // lengths and page tables were written before the previous kernel started: safe to read before the wait
  const int* table = p.table + (long long)seq * p.table_stride;
  // (without a window or splits the block's run starts at the sequence's first page whatever its length: the
  // producer's lanes ask for their table entries together with the length, not after it)
  const bool from_first = p.window == 0 && gridDim.x == 1;
  int early_page = 0;
  if (warp == DM_WARPS && from_first) early_page = table[lane % p.table_len];
  const int L = p.ctx_len[seq];                     // keys 0..L-1; the query sits at L-1
  const int lo_all = p.window > 0 ? max(0, L - p.window) : 0;
  // (a sequence without keys, L <= 0, owns no page, files nothing and yields zeros)
  const int first = lo_all / DS_PAGE, last = L > 0 ? (L - 1) / DS_PAGE : first - 1;
  const int per = (last - first + 1 + n_splits - 1) / n_splits;
  const int pg_first = first + split * per, pg_end = min(last + 1, pg_first + per);
  const int n_pages = pg_end > pg_first ? pg_end - pg_first : 0;
  const int lo = max(lo_all, pg_first * DS_PAGE), hi = min(L, pg_end * DS_PAGE);

  if (tid == 0) {
    for (int i = 0; i < p.slots; ++i) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(ds_smem(&full[i])));
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(ds_smem(&empty[i])), "r"(CPP));
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    s_flag = 0;
  }
  __syncthreads();
  // page i of the block's run travels into slot i % slots
  auto ask = [&](int i, int page) {
    const int slot = i % p.slots;
    unsigned char* dst = ring + (size_t)slot * slot_bytes;
    const unsigned bar = ds_smem(&full[slot]);
    const int row = (page * p.n_kv_heads + kv_head) * DS_PAGE;
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"((unsigned)slot_bytes) : "memory");
    for (int cb = 0; cb < cbs; ++cb) {
      asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n" ::"r"(
                       ds_smem(dst + cb * DS_PAGE * 128)),
                   "l"(&k_map), "r"(cb * 64), "r"(row), "r"(bar)
                   : "memory");
      asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n" ::"r"(
                       ds_smem(dst + (cbs + cb) * DS_PAGE * 128)),
                   "l"(&v_map), "r"(cb * 64), "r"(row), "r"(bar)
                   : "memory");
    }
  };
  // the first pages at once, before the wait for the predecessor: old keys and values do not change during a step
  if (warp == DM_WARPS && lane < min(n_pages, p.slots)) ask(lane, from_first ? early_page : table[(pg_first + lane) % p.table_len]);

  pdl_wait();     // the projections of this step are complete from here on
  // The query goes straight into the registers that multiply it, and the new key and value straight to where they are
  // needed (the page in memory; the page's copy in shared memory for the one chunk that holds their position): no
  // staging and no barrier of the block between the wait and the first chunk.
  const __nv_bfloat16* const q_row = p.q + (long long)seq * p.q_stride + head * hd;
  const __nv_bfloat16* const new_k = p.new_k ? p.new_k + (long long)seq * p.q_stride + kv_head * hd : nullptr;
  const __nv_bfloat16* const new_v = p.new_k ? p.new_v + (long long)seq * p.q_stride + kv_head * hd : nullptr;
  unsigned qa[I * 4];          // per 16 dims: dims 2q, 2q + 1 and 8 + 2q, 9 + 2q of the query (every column of the operand)
#pragma unroll
  for (int j = 0; j < I * 4; ++j) {
    const int d = 16 * (j >> 1) + 8 * (j & 1) + 2 * q;
    qa[j] = d < hd ? *reinterpret_cast<const unsigned*>(q_row + d) : 0u;
  }
  if (new_k && L > 0 && split == 0 && head == kv_head * (p.n_heads / p.n_kv_heads)) {
    // this block also files the new token's key and value in the sequence's page
    const int pos = L - 1;
    const long long page = table[(pos / DS_PAGE) % p.table_len];
    const long long off = (page * p.n_kv_heads + kv_head) * (long long)(DS_PAGE * hd) + (long long)(pos % DS_PAGE) * hd;
    for (int c = tid; c < hd / 8; c += DM_THREADS) {
      *reinterpret_cast<uint4*>(p.k_pool + off + c * 8) = *reinterpret_cast<const uint4*>(new_k + c * 8);
      *reinterpret_cast<uint4*>(p.v_pool + off + c * 8) = *reinterpret_cast<const uint4*>(new_v + c * 8);
    }
  }
  unsigned k_lane[2 * I], v_lane[2 * I];
  ds_lane_offsets<I>(lane, k_lane, v_lane);
  float m = -INFINITY, l = 0.f;
  float acc[I * 2][4];
#pragma unroll
  for (int n = 0; n < I * 2; ++n)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[n][e] = 0.f;
  if (warp == DM_WARPS) {
    // ---- the producer warp: each further page as soon as the warps that read its slot's last page have handed
    // the slot back ----
    bool dead = false;
    for (int base = p.slots; base < n_pages; base += 32) {
      const int mine = base + lane < n_pages ? table[(pg_first + base + lane) % p.table_len] : 0;
      const int n = min(32, n_pages - base);
      for (int j = 0; j < n; ++j) {
        const int page = __shfl_sync(0xffffffffu, mine, j), i = base + j;
        if (lane == 0 && !dead) {
          const unsigned parity = (unsigned)(i / p.slots - 1) & 1u;
          bool freed = false;
          for (int t = 0; t < DM_WAIT_LIMIT && !freed; ++t) {
            unsigned done;
            asm volatile(
                "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
                : "=r"(done) : "r"(ds_smem(&empty[i % p.slots])), "r"(parity) : "memory");
            freed = done != 0;
          }
          if (freed) {
            asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
            ask(i, page);
          } else {
            dead = true;      // the warps that wait for this page give up by themselves and report it
          }
        }
      }
    }
  }
  bool ok = true;
  for (int c = warp; c < n_pages * CPP && warp < DM_WARPS; c += DM_WARPS) {
    const int i = c / CPP, h = c % CPP;
    const int key0 = (pg_first + i) * DS_PAGE + h * CK;
    const int slot = i % p.slots;
    unsigned char* Kt = ring + (size_t)slot * slot_bytes;
    const unsigned Ks = ds_smem(Kt), Vs = Ks + (unsigned)(cbs * DS_PAGE * 128);
    const unsigned parity = (unsigned)(i / p.slots) & 1u;
    bool landed = false;      // (a chunk outside the range waits as well: a slot is handed back once per use by each reader)
    for (int t = 0; t < DM_WAIT_LIMIT && !landed; ++t) {
      unsigned done;
      asm volatile(
          "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
          : "=r"(done) : "r"(ds_smem(&full[slot])), "r"(parity) : "memory");
      landed = done != 0;
    }
    if (!landed) ok = false;
    if (key0 < hi && key0 + CK > lo) {
      if (new_k && L - 1 >= key0 && L - 1 < key0 + CK) {
        // the newest key and value are not in their page yet (or only just): they come from the projections.
        // (No other warp touches this chunk's rows; the rows beyond are masked and hold old, finite numbers.)
        const int row = (L - 1) % DS_PAGE;
        for (int ch = lane; ch < hd / 8; ch += 32) {
          const unsigned off = (unsigned)((ch >> 3) * DS_PAGE * 128 + row * 128 + (((ch & 7) ^ (row & 7)) << 4));
          *reinterpret_cast<uint4*>(Kt + off) = *reinterpret_cast<const uint4*>(new_k + ch * 8);
          *reinterpret_cast<uint4*>(Kt + cbs * DS_PAGE * 128 + off) = *reinterpret_cast<const uint4*>(new_v + ch * 8);
        }
        __syncwarp();
      }
      ds_attn_chunk_kt<I, T / 2>(qa, k_lane, v_lane, Ks, Vs, hd, h * CK, key0, lo, hi, p.scale_log2, m, l, acc, lane);
    }
    if (i + p.slots < n_pages) {      // the slot's next page may come
      __syncwarp();
      if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(ds_smem(&empty[slot])) : "memory");
    }
  }
  if (!ok) s_flag = 1;
  // a lane summed the weights of its own keys (the quad g's, the same in its four lanes); the lanes of a quad hold
  // dims 16 n + g and 16 n + g + 8 of the weighted values
  l += __shfl_xor_sync(0xffffffffu, l, 4);
  l += __shfl_xor_sync(0xffffffffu, l, 8);
  l += __shfl_xor_sync(0xffffffffu, l, 16);
  if (q == 0 && warp < DM_WARPS) {
#pragma unroll
    for (int n = 0; n < I * 2; ++n) {
      const int d = 16 * n + g;
      if (d < hd) {
        s_acc[warp * hd + d] = acc[n][0];
        s_acc[warp * hd + d + 8] = acc[n][2];
      }
    }
    if (g == 0) {
      s_ml[warp][0] = m;
      s_ml[warp][1] = l;
    }
  }
  __syncthreads();
  const bool block_failed = s_flag != 0;
  if (block_failed && tid == 0 && p.status) atomicExch(p.status, 1);
  // the block's (max, sum) and its weighted values
  float M = -INFINITY;
#pragma unroll
  for (int w = 0; w < DM_WARPS; ++w) M = fmaxf(M, s_ml[w][0]);
  float wg[DM_WARPS], Lsum = 0.f;
#pragma unroll
  for (int w = 0; w < DM_WARPS; ++w) {
    wg[w] = M == -INFINITY ? 0.f : ds_exp2(s_ml[w][0] - M);
    Lsum += s_ml[w][1] * wg[w];
  }
  if (block_failed) Lsum = NAN;        // a result that cannot be mistaken for a good one
  const long long unit = (long long)seq * p.n_heads + head;
  for (int c = tid; c < hd; c += DM_THREADS) {
    float o = 0.f;
#pragma unroll
    for (int w = 0; w < DM_WARPS; ++w) o += s_acc[w * hd + c] * wg[w];
    if (n_splits == 1)
      p.out[unit * hd + c] = __float2bfloat16_rn(Lsum > 0.f ? o / Lsum : (Lsum == 0.f ? 0.f : NAN));
    else if (p.use_cluster)
      c_acc[c] = o;
    else
      p.part_acc[(unit * n_splits + split) * hd + c] = o;
  }
  if (n_splits == 1) return;

  if (p.use_cluster) {
    // the splits of this (sequence, head) are one cluster: add their partials through distributed shared memory
    if (tid == 0) {
      c_ml[0] = M;
      c_ml[1] = Lsum;
    }
    cg::cluster_group cluster = cg::this_cluster();
    cluster.sync();
    float pm[8], pl[8];
    float Mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      pm[j] = j < n_splits ? cluster.map_shared_rank(c_ml, j)[0] : -INFINITY;
      pl[j] = j < n_splits ? cluster.map_shared_rank(c_ml, j)[1] : 0.f;
      Mx = fmaxf(Mx, pm[j]);
    }
    float Lall = 0.f, wj[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      wj[j] = (j < n_splits && pm[j] != -INFINITY) ? ds_exp2(pm[j] - Mx) : 0.f;
      Lall += wj[j] != 0.f || pl[j] != pl[j] ? pl[j] * wj[j] : 0.f;
    }
    // rank r finishes the channels c with c % n_splits == r
    for (int c = split + tid * n_splits; c < hd; c += DM_THREADS * n_splits) {
      float o = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (j < n_splits) o += cluster.map_shared_rank(c_acc, j)[c] * wj[j];
      p.out[unit * hd + c] = __float2bfloat16_rn(Lall > 0.f ? o / Lall : (Lall == 0.f ? 0.f : NAN));
    }
    cluster.sync();    // nobody leaves while a peer may still read its partials
    return;
  }

  if (tid == 0) {
    p.part_ml[(unit * n_splits + split) * 2] = M;
    p.part_ml[(unit * n_splits + split) * 2 + 1] = Lsum;
  }
  // the block that takes the last ticket merges the splits; nobody waits for anybody
  __threadfence();
  __syncthreads();
  if (tid == 0) s_flag = atomicAdd(&p.tickets[unit], 1);
  __syncthreads();
  if (s_flag != n_splits - 1) return;
  __threadfence();
  float Mx = -INFINITY;
  for (int s2 = 0; s2 < n_splits; ++s2) Mx = fmaxf(Mx, __ldcg(&p.part_ml[(unit * n_splits + s2) * 2]));
  float Lall = 0.f;
  for (int s2 = 0; s2 < n_splits; ++s2) {
    const float ms = __ldcg(&p.part_ml[(unit * n_splits + s2) * 2]);
    if (ms != -INFINITY) Lall += __ldcg(&p.part_ml[(unit * n_splits + s2) * 2 + 1]) * ds_exp2(ms - Mx);
  }
  for (int c = tid; c < hd; c += DM_THREADS) {
    float o = 0.f;
    for (int s2 = 0; s2 < n_splits; ++s2) {
      const float ms = __ldcg(&p.part_ml[(unit * n_splits + s2) * 2]);
      if (ms != -INFINITY) o += __ldcg(&p.part_acc[(unit * n_splits + s2) * hd + c]) * ds_exp2(ms - Mx);
    }
    p.out[unit * hd + c] = __float2bfloat16_rn(Lall > 0.f ? o / Lall : (Lall == 0.f ? 0.f : NAN));
  }
  if (tid == 0) p.tickets[unit] = 0;   // ready for the next call
}

template <int I, int T>
static int launch_decode_mma(const CUtensorMap& km, const CUtensorMap& vm, DecodeMmaParams p, int n_seqs, int n_splits, int max_ctx,
                             cudaStream_t stream) {
  const int cbs = (p.head_dim + 63) / 64;
  const int slot_bytes = 2 * cbs * DS_PAGE * 128;
  const int span = p.window > 0 ? (p.window < max_ctx ? p.window : max_ctx) : max_ctx;
  const int pages_total = (span + DS_PAGE - 1) / DS_PAGE + (p.window > 0 ? 1 : 0);
  const int share = (pages_total + n_splits - 1) / n_splits;
  int fit = DM_SMEM_BUDGET / slot_bytes;
  if (fit > 16) fit = 16;
  // A ring that pages go round more than once has an even number of slots.  With 32-key chunks two warps take the even
  // pages and two the odd ones, so a pair meets a slot again 2 k pages later: with an even count that is the slot's very
  // next use, whose barrier phase the pair cannot mistake; with an odd count the other pair's use would lie in between,
  // and a pair that ran ahead would take the phase before it for its own.
  if (fit > 2) fit &= ~1;
  BT_CHECK(fit >= 1, "attention_decode: one page of head_dim %d does not fit in shared memory", p.head_dim);
  p.slots = share < fit ? (share < 1 ? 1 : share) : fit;
  const size_t smem = 1024 + (size_t)p.slots * slot_bytes + sizeof(float) * (size_t)(DM_WARPS + 1) * p.head_dim + 64;
  auto kern = attention_decode_mma_kernel<I, T>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  BT_CHECK(e == cudaSuccess, "attention_decode: cannot reserve %zu bytes of shared memory", smem);
  const int cluster = p.use_cluster ? n_splits : 1;
  BT_PDL_OK("attention_decode_mma", launch_pdl(kern, dim3(n_splits, p.n_heads, n_seqs), dim3(DM_THREADS), smem, stream, cluster, km, vm, p));
  return 0;
}

}  // namespace bt

// Whether the tensor-core kernel takes this head size (bfloat16 only).
extern "C" int bt_attention_decode_mma_supports(int head_dim) { return head_dim >= 16 && head_dim % 16 == 0 && head_dim <= 128; }

// Arguments as bt_attention_decode (bfloat16), with the size of the pools: `pool_pages` pages of n_kv_heads heads.
extern "C" int bt_attention_decode_mma(const void* q, long long q_row_stride, const void* new_k, const void* new_v, void* k_pool,
                                       void* v_pool, long long pool_pages, const int* kv_table, int table_stride, int table_len,
                                       void* out, float* scratch, int* tickets, int* status, const int* ctx_len, int n_seqs,
                                       int n_heads, int n_kv_heads, int head_dim, float scale, int window, int n_splits,
                                       int max_ctx, int merge, cudaStream_t stream) {
  using namespace bt;
  BT_CHECK(bt_attention_decode_mma_supports(head_dim), "attention_decode: the tensor-core kernel takes head sizes 16..128 in steps of 16, not %d",
           head_dim);
  BT_CHECK(n_heads > 0 && n_kv_heads > 0 && n_heads % n_kv_heads == 0,
           "attention_decode: %d query heads cannot share %d key heads", n_heads, n_kv_heads);
  BT_CHECK(kv_table != nullptr && table_len > 0 && pool_pages > 0, "attention_decode: needs a page table and pools");
  BT_CHECK(n_splits >= 1 && n_splits <= 65535 && n_heads <= 65535 && n_seqs <= 65535, "attention_decode: grid too large");
  BT_CHECK(q_row_stride % 8 == 0, "attention_decode: query rows must be 16-byte aligned");
  BT_CHECK((new_k == nullptr) == (new_v == nullptr), "attention_decode: give both the new key and the new value, or neither");
  BT_CHECK(max_ctx >= 1, "attention_decode: max_ctx must be positive");
  const int use_cluster = n_splits > 1 && n_splits <= 8 && merge == 0;
  BT_CHECK(n_splits == 1 || use_cluster || (scratch != nullptr && tickets != nullptr),
           "attention_decode: %d splits merged through scratch need scratch memory and tickets", n_splits);
  if (n_seqs == 0) return 0;
  CUtensorMap km, vm;
  const unsigned long long rows = (unsigned long long)pool_pages * n_kv_heads * DS_PAGE;
  if (tensor_map_2d_bf16(&km, k_pool, rows, head_dim, head_dim, DS_PAGE) != 0) return 1;
  if (tensor_map_2d_bf16(&vm, v_pool, rows, head_dim, head_dim, DS_PAGE) != 0) return 1;
  DecodeMmaParams p{(const __nv_bfloat16*)q, q_row_stride, (const __nv_bfloat16*)new_k, (const __nv_bfloat16*)new_v,
                    (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, kv_table, table_stride, table_len, (__nv_bfloat16*)out,
                    scratch, scratch ? scratch + (long long)n_seqs * n_heads * n_splits * head_dim : nullptr, tickets, status,
                    ctx_len, n_heads, n_kv_heads, head_dim, scale * 1.4426950408889634f, window, 1, use_cluster};
  if (head_dim <= 64) return launch_decode_mma<2, 4>(km, vm, p, n_seqs, n_splits, max_ctx, stream);
  return launch_decode_mma<4, 2>(km, vm, p, n_seqs, n_splits, max_ctx, stream);
}
