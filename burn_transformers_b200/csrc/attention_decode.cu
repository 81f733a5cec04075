// Attention for steps that bring one token per sequence: one query per (sequence, head) over the keys and
// values of that sequence's pages.  The work is memory traffic, so the kernel is built to put a block's whole
// share of the cache in flight at once:
//   * a page holds, per key head, 64 keys as one contiguous block (and 64 values as another); one thread asks
//     the copy engine for all of the block's pages with bulk asynchronous copies into shared memory
//     (cp.async.bulk, completion counted on an mbarrier) -- before the kernel waits for its predecessor,
//     because pages of earlier tokens do not depend on it;
//   * long contexts are cut by pages into splits that run as separate blocks;
//   * the splits of one (sequence, head) form a thread-block cluster and merge their partial (max, sum,
//     weighted values) through distributed shared memory, in a fixed order: no scratch, no atomics.
//     With more splits than a cluster holds, or when the caller asks for it, the partials go to scratch memory
//     and the block that finishes last (a ticket counter decides, nobody waits) merges them;
//   * the new token's key and value are taken straight from the step's projections, and one block per
//     (sequence, key head) files them in the page, so no separate append kernel runs.
// Scores, softmax and the value mix are 32-bit.
//
// Scratch layout (32-bit): part_acc[seq][head][split][head_dim], part_ml[seq][head][split][2].
// `tickets` holds one int per (sequence, head); it must be zero before the first call and is left zero.
// The only wait in the kernel (for the copies to land) is bounded; if it runs out the block records the
// fact in `status`, writes NaN as its result and still takes part in every barrier.
#include <cooperative_groups.h>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace bt {

constexpr int DEC_MAX_WARPS = 16;   // a block has 4, 8 or 16 warps, chosen by how many keys it owns
constexpr int DEC_WAIT_LIMIT = 1 << 24;   // polls of the copy barrier before giving up (seconds, not microseconds)

template <typename T> struct Chunk;   // 16 bytes of T as floats
template <> struct Chunk<float> {
  static constexpr int N = 4;
  __device__ static void unpack(const uint4& v, float (&f)[4]) {
    f[0] = __uint_as_float(v.x); f[1] = __uint_as_float(v.y); f[2] = __uint_as_float(v.z); f[3] = __uint_as_float(v.w);
  }
  __device__ static void load(const float* p, float (&f)[4]) { unpack(*reinterpret_cast<const uint4*>(p), f); }
};
template <> struct Chunk<__nv_bfloat16> {
  static constexpr int N = 8;
  // a bfloat16 is the upper half of a float: widening is a shift or a mask, exact, and needs no conversion unit
  __device__ static void unpack(const uint4& v, float (&f)[8]) {
    const unsigned w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      f[2 * i] = __uint_as_float(w[i] << 16);
      f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
  __device__ static void load(const __nv_bfloat16* p, float (&f)[8]) { unpack(*reinterpret_cast<const uint4*>(p), f); }
};

struct DecodeParams {
  const void* q;             // rows of the step's projections; query head h at q + h * head_dim
  long long q_row_stride;
  const void* new_k;         // the new token's key/value channels in the same rows, or null when the
  const void* new_v;         // pages already hold them
  void* k_pool;              // pools [page][kv_head][page_size][head_dim]
  void* v_pool;
  const int* table;
  int table_stride, table_len, page_size;
  void* out;
  float* part_acc;
  float* part_ml;
  int* tickets;
  int* status;
  const int* ctx_len;
  int n_heads, n_kv_heads, head_dim;
  float scale;
  int window, G, round_pages, use_cluster;
};

// 2^x by the hardware's approximation (relative error about 2^-22), one instruction
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ unsigned smem_addr(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(unsigned long long* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_addr(bar)), "r"(count));
  asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
}
__device__ __forceinline__ void mbar_expect(unsigned long long* bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_load(void* dst, const void* src, unsigned bytes, unsigned long long* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(smem_addr(dst)),
               "l"(src), "r"(bytes), "r"(smem_addr(bar))
               : "memory");
}
// true when the phase with this parity has completed; gives up after DEC_WAIT_LIMIT polls
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, unsigned parity) {
  for (int i = 0; i < DEC_WAIT_LIMIT; ++i) {
    unsigned done;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(done) : "r"(smem_addr(bar)), "r"(parity) : "memory");
    if (done) return true;
  }
  return false;
}

// CPL: 16-byte chunks per lane (1 or 2).  G (runtime, power of two <= 32): lanes per key row.
// grid (n_splits, n_heads, n_seqs); with use_cluster the n_splits blocks of a (sequence, head) are one cluster.
template <typename T, int CPL>
__global__ void __launch_bounds__(DEC_MAX_WARPS * 32)
attention_decode_kernel(DecodeParams p) {
  constexpr int E = Chunk<T>::N;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __shared__ __align__(8) unsigned long long bar;
  __shared__ float s_ml[DEC_MAX_WARPS][2];
  __shared__ float c_ml[2];            // this block's (max, sum), read by its cluster peers
  __shared__ float s_w[DEC_MAX_WARPS]; // weight of each warp's partial in the block's sum
  __shared__ int s_flag;
  pdl_trigger();
  const int split = blockIdx.x, n_splits = gridDim.x;
  const int head = blockIdx.y, seq = blockIdx.z;
  const int group = p.n_heads / p.n_kv_heads;
  const int kv_head = head / group;
  const int head_dim = p.head_dim, G = p.G, PS = p.page_size;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int n_warps = blockDim.x >> 5;
  const int gl = lane & (G - 1);                    // lane within its key group
  const int sub = lane / G;                         // which key of the warp's batch
  const int keys_per_warp = 32 / G;
  const int n_chunks = head_dim / E;
  const int page_elems = PS * head_dim;             // one page of one key head
  T* Ks = reinterpret_cast<T*>(smem_raw);           // [round_pages][page_size][head_dim]
  T* Vs = Ks + (size_t)p.round_pages * page_elems;
  float* s_acc = reinterpret_cast<float*>(Vs + (size_t)p.round_pages * page_elems);   // [n_warps][head_dim]
  float* c_acc = s_acc + n_warps * head_dim;        // [head_dim], read by the cluster peers

  // lengths and page tables were written before the previous kernel started: safe to read before the wait
  const int L = p.ctx_len[seq];                     // keys 0..L-1; the query sits at L-1
  const int lo = p.window > 0 ? max(0, L - p.window) : 0;
  // a sequence without keys (L <= 0: an empty or finished request that still rides in the batch) owns no page,
  // files nothing and yields zeros; its block still takes part in the cluster and ticket hand-overs
  const int pg_first = lo / PS, pg_last = L > 0 ? (L - 1) / PS : pg_first - 1;
  const int n_pg = pg_last - pg_first + 1;
  const int per = (n_pg + n_splits - 1) / n_splits;
  const int my_first = pg_first + split * per;
  const int my_end = min(pg_last + 1, my_first + per);          // exclusive
  const int n_rounds = my_end > my_first ? (my_end - my_first + p.round_pages - 1) / p.round_pages : 0;
  const T* kbase = reinterpret_cast<const T*>(p.k_pool);
  const T* vbase = reinterpret_cast<const T*>(p.v_pool);
  const int* table = p.table + (long long)seq * p.table_stride;

  if (tid == 0) {
    mbar_init(&bar, 1);
    s_flag = 0;
  }
  __syncthreads();
  // Warp 0 asks for a round's pages: every lane looks up one page of the table and issues that page's two
  // copies, so neither the table reads nor the copy requests queue up behind one another.
  auto issue_round = [&](int r) {
    const int pa = my_first + r * p.round_pages, pb = min(my_end, pa + p.round_pages);
    const unsigned bytes = (unsigned)(page_elems * sizeof(T));
    // shared memory that ordinary instructions have just read is about to be overwritten by the copy engine
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    if (lane == 0) mbar_expect(&bar, 2u * bytes * (unsigned)(pb - pa));
    __syncwarp();
    for (int pg = pa + lane; pg < pb; pg += 32) {
      const long long page = table[pg % p.table_len];
      const long long off = (page * p.n_kv_heads + kv_head) * (long long)page_elems;
      bulk_load(Ks + (size_t)(pg - pa) * page_elems, kbase + off, bytes, &bar);
      bulk_load(Vs + (size_t)(pg - pa) * page_elems, vbase + off, bytes, &bar);
    }
  };
  // Pages of earlier tokens do not depend on the kernels before this one, so their copies start before the
  // wait -- but only when this call files the new token itself (new_k given).  Without that, another kernel
  // of the same step has filed it, and the copies must come after the wait to see it.
  if (warp == 0 && n_rounds > 0 && p.new_k) issue_round(0);

  pdl_wait();   // the projections of this step (and everything before them) are complete from here on

  if (warp == 0 && n_rounds > 0 && !p.new_k) issue_round(0);

  const T* q = reinterpret_cast<const T*>(p.q) + (long long)seq * p.q_row_stride + head * head_dim;
  const T* new_k = p.new_k ? reinterpret_cast<const T*>(p.new_k) + (long long)seq * p.q_row_stride + kv_head * head_dim : nullptr;
  const T* new_v = p.new_v ? reinterpret_cast<const T*>(p.new_v) + (long long)seq * p.q_row_stride + kv_head * head_dim : nullptr;
  if (new_k && L > 0 && split == 0 && head == kv_head * group) {
    // this block also files the new token's key and value in the sequence's page
    const int pos = L - 1;
    const long long page = table[(pos / PS) % p.table_len];
    const long long off = (page * p.n_kv_heads + kv_head) * (long long)page_elems + (long long)(pos % PS) * head_dim;
    T* kd = reinterpret_cast<T*>(p.k_pool) + off;
    T* vd = reinterpret_cast<T*>(p.v_pool) + off;
    for (int c = tid; c < n_chunks; c += blockDim.x) {
      *reinterpret_cast<uint4*>(kd + c * E) = *reinterpret_cast<const uint4*>(new_k + c * E);
      *reinterpret_cast<uint4*>(vd + c * E) = *reinterpret_cast<const uint4*>(new_v + c * E);
    }
  }

  float qr[CPL][E], acc[CPL][E];
#pragma unroll
  for (int c = 0; c < CPL; ++c) {
    const int ch = gl + c * G;
    if (ch < n_chunks) {
      Chunk<T>::load(q + ch * E, qr[c]);
#pragma unroll
      for (int e = 0; e < E; ++e) qr[c][e] *= p.scale * 1.4426950408889634f;   // scores in base 2: exp2 below
    } else {
#pragma unroll
      for (int e = 0; e < E; ++e) qr[c][e] = 0.f;
    }
#pragma unroll
    for (int e = 0; e < E; ++e) acc[c][e] = 0.f;
  }
  float m = -INFINITY, l = 0.f;

  for (int r = 0; r < n_rounds; ++r) {
    if (r > 0) {
      __syncthreads();                       // everyone is done with the previous round's pages
      if (warp == 0) issue_round(r);
    }
    // one thread watches the copies land; the others sleep at the barrier instead of polling
    if (tid == 0 && !mbar_wait(&bar, (unsigned)(r & 1))) s_flag = 1;
    __syncthreads();
    const int pa = my_first + r * p.round_pages, pb = min(my_end, pa + p.round_pages);
    const int key_lo = max(lo, pa * PS), key_hi = min(L, pb * PS);
    if (new_k && key_hi == L && L > 0) {
      // the newest key is not in its page yet (or only just): take it from the projections
      const int row = (L - 1) - pa * PS;
      for (int c = tid; c < n_chunks; c += blockDim.x) {
        *reinterpret_cast<uint4*>(Ks + (size_t)row * head_dim + c * E) = *reinterpret_cast<const uint4*>(new_k + c * E);
        *reinterpret_cast<uint4*>(Vs + (size_t)row * head_dim + c * E) = *reinterpret_cast<const uint4*>(new_v + c * E);
      }
      __syncthreads();
    }
    const int step = n_warps * keys_per_warp;
    // `base` is the same for all lanes of a warp, so the shuffles below always see the whole warp
    for (int base = key_lo + warp * keys_per_warp; base < key_hi; base += 2 * step) {
      float s[2];
      bool valid[2];
      int row[2];
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int key = base + sub + j * step;
        valid[j] = key < key_hi;
        row[j] = valid[j] ? key - pa * PS : 0;
        s[j] = 0.f;
#pragma unroll
        for (int c = 0; c < CPL; ++c) {
          const int ch = gl + c * G;
          if (ch < n_chunks) {
            float kf[E];
            Chunk<T>::load(Ks + (size_t)row[j] * head_dim + ch * E, kf);
#pragma unroll
            for (int e = 0; e < E; ++e) s[j] = fmaf(qr[c][e], kf[e], s[j]);
          }
        }
      }
      for (int o = G >> 1; o > 0; o >>= 1) {
        s[0] += __shfl_xor_sync(0xffffffffu, s[0], o);
        s[1] += __shfl_xor_sync(0xffffffffu, s[1], o);
      }
      float m_new = m;
      if (valid[0]) m_new = fmaxf(m_new, s[0]);
      if (valid[1]) m_new = fmaxf(m_new, s[1]);
      if (m_new == -INFINITY) continue;      // this lane group had no key in the batch (others may have)
      const float corr = fast_exp2(m - m_new);   // m = -inf gives 0
      const float p0 = valid[0] ? fast_exp2(s[0] - m_new) : 0.f;
      const float p1 = valid[1] ? fast_exp2(s[1] - m_new) : 0.f;
      l = l * corr + (p0 + p1);
      m = m_new;
#pragma unroll
      for (int c = 0; c < CPL; ++c) {
        const int ch = gl + c * G;
        if (ch < n_chunks) {
          float v0[E], v1[E];
          Chunk<T>::load(Vs + (size_t)row[0] * head_dim + ch * E, v0);
          Chunk<T>::load(Vs + (size_t)row[1] * head_dim + ch * E, v1);
#pragma unroll
          for (int e = 0; e < E; ++e) acc[c][e] = fmaf(p1, v1[e], fmaf(p0, v0[e], acc[c][e] * corr));
        }
      }
    }
  }
  // merge the key groups of a warp
  for (int o = G; o < 32; o <<= 1) {
    const float m2 = __shfl_xor_sync(0xffffffffu, m, o);
    const float l2 = __shfl_xor_sync(0xffffffffu, l, o);
    const float mm = fmaxf(m, m2);
    const float a = mm == -INFINITY ? 0.f : fast_exp2(m - mm);
    const float b = mm == -INFINITY ? 0.f : fast_exp2(m2 - mm);
    l = l * a + l2 * b;
#pragma unroll
    for (int c = 0; c < CPL; ++c)
#pragma unroll
      for (int e = 0; e < E; ++e) {
        const float other = __shfl_xor_sync(0xffffffffu, acc[c][e], o);
        acc[c][e] = acc[c][e] * a + other * b;
      }
    m = mm;
  }
  // merge the warps through shared memory
  if (sub == 0) {
#pragma unroll
    for (int c = 0; c < CPL; ++c) {
      const int ch = gl + c * G;
      if (ch < n_chunks)
#pragma unroll
        for (int e = 0; e < E; ++e) s_acc[warp * head_dim + ch * E + e] = acc[c][e];
    }
    if (gl == 0) {
      s_ml[warp][0] = m;
      s_ml[warp][1] = l;
    }
  }
  __syncthreads();
  const bool block_failed = s_flag != 0;
  if (block_failed && tid == 0 && p.status) atomicExch(p.status, 1);
  if (warp == 0) {
    // lane w turns warp w's maximum into its weight exp2(m_w - M); lane 0 keeps the block's (M, sum)
    const float mw = lane < n_warps ? s_ml[lane][0] : -INFINITY;
    const float Mb = warp_max(mw);
    const float wg = (lane < n_warps && Mb != -INFINITY) ? fast_exp2(mw - Mb) : 0.f;
    const float Lb = warp_sum(lane < n_warps ? s_ml[lane][1] * wg : 0.f);
    if (lane < n_warps) s_w[lane] = wg;
    if (lane == 0) {
      c_ml[0] = Mb;
      c_ml[1] = block_failed ? NAN : Lb;      // a result that cannot be mistaken for a good one
    }
  }
  __syncthreads();
  const float M = c_ml[0], Lsum = c_ml[1];
  const long long unit = ((long long)seq * p.n_heads + head);
  T* out = reinterpret_cast<T*>(p.out);
  for (int c = tid; c < head_dim; c += blockDim.x) {
    float o = 0.f;
    for (int w = 0; w < n_warps; ++w) o += s_acc[w * head_dim + c] * s_w[w];
    if (n_splits == 1)
      out[unit * head_dim + c] = from_float<T>(Lsum > 0.f ? o / Lsum : (Lsum == 0.f ? 0.f : NAN));
    else if (p.use_cluster)
      c_acc[c] = o;
    else
      p.part_acc[(unit * n_splits + split) * head_dim + c] = o;
  }
  if (n_splits == 1) return;

  if (p.use_cluster) {
    // the splits of this (sequence, head) are one cluster: add their partials through distributed shared memory
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
      wj[j] = (j < n_splits && pm[j] != -INFINITY) ? fast_exp2(pm[j] - Mx) : 0.f;
      Lall += wj[j] != 0.f || pl[j] != pl[j] ? pl[j] * wj[j] : 0.f;
    }
    // rank r finishes the channels c with c % n_splits == r
    for (int c = split + tid * n_splits; c < head_dim; c += blockDim.x * n_splits) {
      float from[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) from[j] = j < n_splits ? cluster.map_shared_rank(c_acc, j)[c] : 0.f;
      float o = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) o += from[j] * wj[j];
      out[unit * head_dim + c] = from_float<T>(Lall > 0.f ? o / Lall : (Lall == 0.f ? 0.f : NAN));
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
    if (ms != -INFINITY) Lall += __ldcg(&p.part_ml[(unit * n_splits + s2) * 2 + 1]) * fast_exp2(ms - Mx);
  }
  for (int c = tid; c < head_dim; c += blockDim.x) {
    float o = 0.f;
    for (int s2 = 0; s2 < n_splits; ++s2) {
      const float ms = __ldcg(&p.part_ml[(unit * n_splits + s2) * 2]);
      if (ms != -INFINITY) o += __ldcg(&p.part_acc[(unit * n_splits + s2) * head_dim + c]) * fast_exp2(ms - Mx);
    }
    out[unit * head_dim + c] = from_float<T>(Lall > 0.f ? o / Lall : (Lall == 0.f ? 0.f : NAN));
  }
  if (tid == 0) p.tickets[unit] = 0;   // ready for the next call
}

template <typename T>
static int launch_decode(DecodeParams p, int n_seqs, int n_splits, int max_ctx, cudaStream_t stream) {
  constexpr int E = Chunk<T>::N;
  const int n_chunks = p.head_dim / E;
  int G = 1;
  while (G < n_chunks && G < 32) G <<= 1;
  const int cpl = (n_chunks + G - 1) / G;
  BT_CHECK(cpl <= 2, "attention_decode: head_dim %d is too large", p.head_dim);
  p.G = G;
  // pages a block holds at a time: its share of the longest context if that fits, else as many as fit
  const size_t page_bytes = (size_t)p.page_size * p.head_dim * sizeof(T);
  const size_t fixed = sizeof(float) * (size_t)(DEC_MAX_WARPS + 1) * p.head_dim;
  const size_t budget = 160 * 1024;
  int span = p.window > 0 ? (p.window < max_ctx ? p.window : max_ctx) : max_ctx;
  int pages_total = (span + p.page_size - 1) / p.page_size + (p.window > 0 ? 1 : 0);
  int share = (pages_total + n_splits - 1) / n_splits;
  int fit = (int)((budget - fixed) / (2 * page_bytes));
  BT_CHECK(fit >= 1, "attention_decode: one page of head_dim %d does not fit in shared memory", p.head_dim);
  p.round_pages = share < fit ? (share < 1 ? 1 : share) : fit;
  const size_t smem = 2 * page_bytes * p.round_pages + fixed;
  dim3 grid(n_splits, p.n_heads, n_seqs);
  // more warps for blocks that own more keys: the per-key work is a dependent chain, so it is spread wide
  const int keys = share * p.page_size;
  const int warps = keys > 256 ? 16 : (keys > 64 ? 8 : 4);
  const int cluster = p.use_cluster ? n_splits : 1;
  cudaError_t e;
  if (cpl == 1) {
    auto kern = attention_decode_kernel<T, 1>;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    BT_CHECK(e == cudaSuccess, "attention_decode: cannot reserve %zu bytes of shared memory", smem);
    BT_PDL_OK("attention_decode", launch_pdl(kern, grid, dim3(warps * 32), smem, stream, cluster, p));
  } else {
    auto kern = attention_decode_kernel<T, 2>;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    BT_CHECK(e == cudaSuccess, "attention_decode: cannot reserve %zu bytes of shared memory", smem);
    BT_PDL_OK("attention_decode", launch_pdl(kern, grid, dim3(warps * 32), smem, stream, cluster, p));
  }
  return 0;
}

}  // namespace bt

// Floats of scratch a call with these sizes needs when its splits merge through scratch memory.
extern "C" long long bt_attention_decode_scratch_floats(int n_seqs, int n_heads, int head_dim, int n_splits) {
  if (n_splits <= 1) return 0;
  return (long long)n_seqs * n_heads * n_splits * (head_dim + 2);
}

// q: one row of the step's projections per sequence (query head h at q + h * head_dim).
// new_k, new_v: the new token's key and value channels in the same rows (q_row_stride apart); when given, the
//   kernel reads the newest key from there and also files it in the page, so no append has to run before it;
//   null when the pages already hold the new token.
// max_ctx: no sequence of the call is longer than this (it sizes the shared memory a block uses).
// merge: 0 = the splits merge inside a thread-block cluster when n_splits <= 8, else through scratch;
//        1 = always through scratch.  scratch: bt_attention_decode_scratch_floats(...) floats, 16-byte aligned;
//   tickets: n_seqs * n_heads ints, zero before the first call, left zero (both only for the scratch merge).
// status: optional int that is set to 1 if a block's wait for its copies ran out.
extern "C" int bt_attention_decode(const void* q, long long q_row_stride, const void* new_k, const void* new_v,
                                   void* k_pool, void* v_pool, const int* kv_table, int table_stride, int table_len,
                                   int page_size, void* out, float* scratch, int* tickets, int* status,
                                   const int* ctx_len, int n_seqs, int n_heads, int n_kv_heads, int head_dim,
                                   float scale, int window, int n_splits, int max_ctx, int merge, int dtype,
                                   cudaStream_t stream) {
  using namespace bt;
  BT_CHECK(head_dim > 0 && head_dim % 8 == 0 && head_dim <= 256,
           "attention_decode: head_dim %d must be a multiple of 8 and at most 256", head_dim);
  BT_CHECK(n_heads > 0 && n_kv_heads > 0 && n_heads % n_kv_heads == 0,
           "attention_decode: %d query heads cannot share %d key heads", n_heads, n_kv_heads);
  BT_CHECK(kv_table != nullptr && table_len > 0 && page_size > 0, "attention_decode: needs a page table");
  BT_CHECK(n_splits >= 1 && n_splits <= 65535 && n_heads <= 65535 && n_seqs <= 65535, "attention_decode: grid too large");
  BT_CHECK(q_row_stride % 8 == 0, "attention_decode: query rows must be 16-byte aligned");
  BT_CHECK((new_k == nullptr) == (new_v == nullptr), "attention_decode: give both the new key and the new value, or neither");
  BT_CHECK(max_ctx >= 1, "attention_decode: max_ctx must be positive");
  const int use_cluster = n_splits > 1 && n_splits <= 8 && merge == 0;
  BT_CHECK(n_splits == 1 || use_cluster || (scratch != nullptr && tickets != nullptr),
           "attention_decode: %d splits merged through scratch need scratch memory and tickets", n_splits);
  if (n_seqs == 0) return 0;
  DecodeParams p{q, q_row_stride, new_k, new_v, k_pool, v_pool, kv_table, table_stride, table_len, page_size, out,
                 scratch, scratch ? scratch + (long long)n_seqs * n_heads * n_splits * head_dim : nullptr, tickets,
                 status, ctx_len, n_heads, n_kv_heads, head_dim, scale, window, 1, 1, use_cluster};
  if (dtype == kF32) return launch_decode<float>(p, n_seqs, n_splits, max_ctx, stream);
  if (dtype == kBF16) return launch_decode<__nv_bfloat16>(p, n_seqs, n_splits, max_ctx, stream);
  return fail("attention_decode: unknown dtype %d", dtype);
}

// ---------------------------------------------------------------------------------------------
// The variant that allocates nothing (see attention_decode_static.h for who it is for and its rules).
// ---------------------------------------------------------------------------------------------
#include "attention_decode_static.h"
#include <mutex>

namespace bt {

// The scratch of bt_attention_decode_static.  In host code this name is only a handle for the runtime:
// the address a kernel may use is looked up per device with cudaGetSymbolAddress below.
static __device__ __align__(256) float g_decode_static_scratch[BT_DECODE_STATIC_SCRATCH_FLOATS];

constexpr int kMaxDevices = 64;
// One ticket per (sequence, head) for the splits' merge: zero when the library is loaded, and every call leaves
// it zero again.
constexpr int kStaticTickets = 1 << 14;
static __device__ int g_decode_static_tickets[kStaticTickets];
// Set to 1 by a block whose bounded wait for its copies ran out (its rows are then NaN); read and cleared by
// bt_attention_decode_static_status.
static __device__ int g_decode_static_status;
static float* g_decode_static_ptr[kMaxDevices] = {nullptr};
static int* g_decode_static_ticket_ptr[kMaxDevices] = {nullptr};
static int* g_decode_static_status_ptr[kMaxDevices] = {nullptr};
static std::mutex g_decode_static_mutex;

// Device address of the scratch array on the current device; looked up once per device.
static int decode_static_scratch(float** ptr, int** tickets, int** status) {
  int device = -1;
  cudaError_t e = cudaGetDevice(&device);
  BT_CHECK(e == cudaSuccess, "attention_decode_static: cudaGetDevice failed: %s", cudaGetErrorString(e));
  BT_CHECK(device >= 0 && device < kMaxDevices, "attention_decode_static: device %d is beyond the %d this library tracks",
           device, kMaxDevices);
  std::lock_guard<std::mutex> lock(g_decode_static_mutex);
  if (g_decode_static_ptr[device] == nullptr) {
    float* found = nullptr;
    e = cudaGetSymbolAddress((void**)&found, g_decode_static_scratch);
    BT_CHECK(e == cudaSuccess && found != nullptr, "attention_decode_static: cudaGetSymbolAddress failed on device %d: %s",
             device, cudaGetErrorString(e));
    int* found_tickets = nullptr;
    e = cudaGetSymbolAddress((void**)&found_tickets, g_decode_static_tickets);
    BT_CHECK(e == cudaSuccess && found_tickets != nullptr,
             "attention_decode_static: cudaGetSymbolAddress failed on device %d: %s", device, cudaGetErrorString(e));
    int* found_status = nullptr;
    e = cudaGetSymbolAddress((void**)&found_status, g_decode_static_status);
    BT_CHECK(e == cudaSuccess && found_status != nullptr,
             "attention_decode_static: cudaGetSymbolAddress failed on device %d: %s", device, cudaGetErrorString(e));
    g_decode_static_ptr[device] = found;
    g_decode_static_ticket_ptr[device] = found_tickets;
    g_decode_static_status_ptr[device] = found_status;
  }
  *ptr = g_decode_static_ptr[device];
  *tickets = g_decode_static_ticket_ptr[device];
  *status = g_decode_static_status_ptr[device];
  return 0;
}

}  // namespace bt

extern "C" int bt_attention_decode_static(const void* q, long long q_row_stride, const void* k_pool,
                                          const void* v_pool, const int* kv_table, int table_stride, int table_len,
                                          int page_size, void* out, const int* ctx_len, int n_seqs, int n_heads,
                                          int n_kv_heads, int head_dim, float scale, int window, int n_splits,
                                          int dtype, cudaStream_t stream) {
  using namespace bt;
  // ranges first, so that the products below cannot wrap
  BT_CHECK(n_seqs >= 0 && n_seqs <= 65535 && n_heads > 0 && n_heads <= 65535 && n_splits >= 1 && n_splits <= 65535 &&
               head_dim > 0 && head_dim <= 256,
           "attention_decode_static: sizes out of range (sequences %d, heads %d, splits %d, head_dim %d)", n_seqs, n_heads,
           n_splits, head_dim);
  BT_CHECK(table_len > 0 && page_size > 0 && page_size <= (1 << 20), "attention_decode_static: bad table_len %d or page_size %d",
           table_len, page_size);
  const long long need = (long long)n_seqs * n_heads * n_splits * (head_dim + 2);
  BT_CHECK(need <= (long long)BT_DECODE_STATIC_SCRATCH_FLOATS,
           "attention_decode_static: %d sequences x %d heads x %d splits x (%d + 2) = %lld floats of scratch exceed the "
           "built-in %d; use fewer splits or bt_attention_decode with scratch of your own",
           n_seqs, n_heads, n_splits, head_dim, need, BT_DECODE_STATIC_SCRATCH_FLOATS);
  BT_CHECK((long long)n_seqs * n_heads <= (long long)kStaticTickets,
           "attention_decode_static: %d sequences x %d heads exceed the built-in %d merge tickets", n_seqs, n_heads,
           kStaticTickets);
  float* scratch = nullptr;
  int* tickets = nullptr;
  int* status = nullptr;
  if (int rc = decode_static_scratch(&scratch, &tickets, &status)) return rc;
  // the longest context the page table can describe sizes the shared memory of a block
  long long span = (long long)table_len * page_size;
  const int max_ctx = span > (1 << 30) ? (1 << 30) : (int)span;
  return bt_attention_decode(q, q_row_stride, nullptr, nullptr, const_cast<void*>(k_pool), const_cast<void*>(v_pool),
                             kv_table, table_stride, table_len, page_size, out, scratch, tickets, status, ctx_len,
                             n_seqs, n_heads, n_kv_heads, head_dim, scale, window, n_splits, max_ctx, /*merge=*/1, dtype,
                             stream);
}

extern "C" int bt_attention_decode_static_status(int* status_out) {
  using namespace bt;
  BT_CHECK(status_out != nullptr, "attention_decode_static_status: needs a place for the answer");
  float* scratch = nullptr;
  int* tickets = nullptr;
  int* status = nullptr;
  if (int rc = decode_static_scratch(&scratch, &tickets, &status)) return rc;
  // a blocking copy of one int out of the library's own word, then the word is cleared: no allocation either way
  cudaError_t e = cudaMemcpy(status_out, status, sizeof(int), cudaMemcpyDeviceToHost);
  BT_CHECK(e == cudaSuccess, "attention_decode_static_status: reading the status failed: %s", cudaGetErrorString(e));
  if (*status_out != 0) {
    e = cudaMemset(status, 0, sizeof(int));
    BT_CHECK(e == cudaSuccess, "attention_decode_static_status: clearing the status failed: %s", cudaGetErrorString(e));
  }
  return 0;
}
