// Attention for steps that bring one token per sequence: one query per (sequence, head) over the
// keys and values of that sequence's pages.  The work is memory traffic, so the kernel is built
// around 16-byte loads: a group of lanes owns one key row, each group has four key rows and four
// value rows in flight, and long contexts are cut into splits that run as separate blocks.  Each
// split leaves a partial (max, sum, weighted values); the block that finishes last (a ticket
// counter decides, nobody waits) merges them.  Scores, softmax and the value mix are 32-bit.
//
// The new token's key and value can be taken straight from the step's projections: every block
// reads that one row from there, and one block per (sequence, key head) copies it into the page, so
// no separate append kernel runs.
//
// Scratch layout (32-bit): part_acc[seq][head][split][head_dim], part_ml[seq][head][split][2].
// `tickets` holds one int per (sequence, head); it must be zero before the first call and is left zero.
#include "common.cuh"

namespace bt {

constexpr int DEC_WARPS = 4;

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
  __device__ static void unpack(const uint4& v, float (&f)[8]) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 x = __bfloat1622float2(h[i]);
      f[2 * i] = x.x;
      f[2 * i + 1] = x.y;
    }
  }
  __device__ static void load(const __nv_bfloat16* p, float (&f)[8]) { unpack(*reinterpret_cast<const uint4*>(p), f); }
};

constexpr int DEC_KB = 4;   // key rows in flight per lane group

struct DecodeParams {
  const void* q;             // rows of the step's projections; query head h at q + h * head_dim
  long long q_row_stride;
  const void* new_k;         // the new token's key/value channels in the same rows, or null when the
  const void* new_v;         // pages already hold them
  void* k_pool_w;            // writable views of the pools, for the append
  void* v_pool_w;
  void* out;
  float* part_acc;
  float* part_ml;
  int* tickets;
  const int* ctx_len;
  int n_heads, n_kv_heads, head_dim;
  float scale;
  int window, G;
};

// CPL: 16-byte chunks per lane (1 or 2).  G (runtime, power of two <= 32): lanes per key row.
template <typename T, int CPL>
__global__ void __launch_bounds__(DEC_WARPS * 32)
attention_decode_kernel(DecodeParams p, KvView kv) {
  constexpr int E = Chunk<T>::N;
  pdl_trigger();
  const int split = blockIdx.x, n_splits = gridDim.x;
  const int head = blockIdx.y, seq = blockIdx.z;
  const int group = p.n_heads / p.n_kv_heads;
  const int kv_head = head / group;
  const int head_dim = p.head_dim, G = p.G;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int gl = lane & (G - 1);                    // lane within its key group
  const int sub = lane / G;                         // which key of the warp's batch
  const int keys_per_warp = 32 / G;
  const int n_chunks = head_dim / E;
  // lengths and page tables were written before the previous kernel started: safe to read before the wait
  const int L = p.ctx_len[seq];                     // keys 0..L-1; the query sits at L-1
  const int lo = p.window > 0 ? max(0, L - p.window) : 0;
  const int per = (L - lo + n_splits - 1) / n_splits;
  const int k_begin = lo + split * per;
  const int k_end = min(L, k_begin + per);
  const T* q = reinterpret_cast<const T*>(p.q) + (long long)seq * p.q_row_stride + head * head_dim;
  const T* new_k = p.new_k ? reinterpret_cast<const T*>(p.new_k) + (long long)seq * p.q_row_stride + kv_head * head_dim : nullptr;
  const T* new_v = p.new_v ? reinterpret_cast<const T*>(p.new_v) + (long long)seq * p.q_row_stride + kv_head * head_dim : nullptr;

  pdl_wait();   // the projections of this step are complete from here on

  if (new_k && split == 0 && head == kv_head * group) {
    // this block also files the new token's key and value in the sequence's page
    const int pos = L - 1;
    T* kd = const_cast<T*>(kv_row<T>(p.k_pool_w, kv, seq, kv_head, p.n_kv_heads, head_dim, pos));
    T* vd = const_cast<T*>(kv_row<T>(p.v_pool_w, kv, seq, kv_head, p.n_kv_heads, head_dim, pos));
    for (int c = threadIdx.x; c < n_chunks; c += blockDim.x) {
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
      for (int e = 0; e < E; ++e) qr[c][e] *= p.scale;
    } else {
#pragma unroll
      for (int e = 0; e < E; ++e) qr[c][e] = 0.f;
    }
#pragma unroll
    for (int e = 0; e < E; ++e) acc[c][e] = 0.f;
  }
  float m = -INFINITY, l = 0.f;

  const int stride = DEC_WARPS * keys_per_warp;     // keys between two rows of one lane group's batch
  // `base` is the same for all lanes of a warp, so the shuffles below always see the whole warp
  for (int base = k_begin + warp * keys_per_warp; base < k_end; base += DEC_KB * stride) {
    uint4 kraw[DEC_KB][CPL], vraw[DEC_KB][CPL];
    bool valid[DEC_KB];
#pragma unroll
    for (int j = 0; j < DEC_KB; ++j) {
      const int key = base + sub + j * stride;
      valid[j] = key < k_end;
      const T* krow = nullptr;
      const T* vrow = nullptr;
      if (valid[j]) {
        if (new_k && key == L - 1) {
          krow = new_k;
          vrow = new_v;
        } else {
          krow = kv_row<T>(kv.k, kv, seq, kv_head, p.n_kv_heads, head_dim, key);
          vrow = kv_row<T>(kv.v, kv, seq, kv_head, p.n_kv_heads, head_dim, key);
        }
      }
#pragma unroll
      for (int c = 0; c < CPL; ++c) {
        const int ch = gl + c * G;
        if (valid[j] && ch < n_chunks) {
          kraw[j][c] = *reinterpret_cast<const uint4*>(krow + ch * E);
          vraw[j][c] = *reinterpret_cast<const uint4*>(vrow + ch * E);
        } else {
          kraw[j][c] = make_uint4(0, 0, 0, 0);
          vraw[j][c] = make_uint4(0, 0, 0, 0);
        }
      }
    }
    float s[DEC_KB];
#pragma unroll
    for (int j = 0; j < DEC_KB; ++j) {
      s[j] = 0.f;
#pragma unroll
      for (int c = 0; c < CPL; ++c) {
        float kf[E];
        Chunk<T>::unpack(kraw[j][c], kf);
#pragma unroll
        for (int e = 0; e < E; ++e) s[j] = fmaf(qr[c][e], kf[e], s[j]);
      }
    }
    for (int o = G >> 1; o > 0; o >>= 1) {
#pragma unroll
      for (int j = 0; j < DEC_KB; ++j) s[j] += __shfl_xor_sync(0xffffffffu, s[j], o);
    }
    float m_new = m;
#pragma unroll
    for (int j = 0; j < DEC_KB; ++j)
      if (valid[j]) m_new = fmaxf(m_new, s[j]);
    if (m_new == -INFINITY) continue;      // this lane group had no key in the batch (others may have)
    const float corr = expf(m - m_new);    // m = -inf gives 0
    float pj[DEC_KB], psum = 0.f;
#pragma unroll
    for (int j = 0; j < DEC_KB; ++j) {
      pj[j] = valid[j] ? expf(s[j] - m_new) : 0.f;
      psum += pj[j];
    }
    l = l * corr + psum;
    m = m_new;
#pragma unroll
    for (int c = 0; c < CPL; ++c) {
#pragma unroll
      for (int e = 0; e < E; ++e) acc[c][e] *= corr;
#pragma unroll
      for (int j = 0; j < DEC_KB; ++j) {
        float vf[E];
        Chunk<T>::unpack(vraw[j][c], vf);
#pragma unroll
        for (int e = 0; e < E; ++e) acc[c][e] = fmaf(pj[j], vf[e], acc[c][e]);
      }
    }
  }
  // merge the key groups of a warp
  for (int o = G; o < 32; o <<= 1) {
    const float m2 = __shfl_xor_sync(0xffffffffu, m, o);
    const float l2 = __shfl_xor_sync(0xffffffffu, l, o);
    const float mm = fmaxf(m, m2);
    const float a = mm == -INFINITY ? 0.f : expf(m - mm);
    const float b = mm == -INFINITY ? 0.f : expf(m2 - mm);
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
  extern __shared__ float sm[];            // [DEC_WARPS][head_dim] + [DEC_WARPS][2] + ticket
  float* s_acc = sm;
  float* s_ml = sm + DEC_WARPS * head_dim;
  int* s_ticket = reinterpret_cast<int*>(s_ml + DEC_WARPS * 2);
  if (sub == 0) {
#pragma unroll
    for (int c = 0; c < CPL; ++c) {
      const int ch = gl + c * G;
      if (ch < n_chunks)
#pragma unroll
        for (int e = 0; e < E; ++e) s_acc[warp * head_dim + ch * E + e] = acc[c][e];
    }
    if (gl == 0) {
      s_ml[warp * 2] = m;
      s_ml[warp * 2 + 1] = l;
    }
  }
  __syncthreads();
  float M = -INFINITY;
#pragma unroll
  for (int w = 0; w < DEC_WARPS; ++w) M = fmaxf(M, s_ml[w * 2]);
  float Lsum = 0.f, wgt[DEC_WARPS];
#pragma unroll
  for (int w = 0; w < DEC_WARPS; ++w) {
    wgt[w] = M == -INFINITY ? 0.f : expf(s_ml[w * 2] - M);
    Lsum += s_ml[w * 2 + 1] * wgt[w];
  }
  const long long unit = ((long long)seq * p.n_heads + head);
  T* out = reinterpret_cast<T*>(p.out);
  for (int c = threadIdx.x; c < head_dim; c += blockDim.x) {
    float o = 0.f;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) o += s_acc[w * head_dim + c] * wgt[w];
    if (n_splits == 1)
      out[unit * head_dim + c] = from_float<T>(Lsum > 0.f ? o / Lsum : 0.f);
    else
      p.part_acc[(unit * n_splits + split) * head_dim + c] = o;
  }
  if (n_splits == 1) return;
  if (threadIdx.x == 0) {
    p.part_ml[(unit * n_splits + split) * 2] = M;
    p.part_ml[(unit * n_splits + split) * 2 + 1] = Lsum;
  }
  // the block that takes the last ticket merges the splits; nobody waits for anybody
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) *s_ticket = atomicAdd(&p.tickets[unit], 1);
  __syncthreads();
  if (*s_ticket != n_splits - 1) return;
  __threadfence();
  float Mx = -INFINITY;
  for (int s2 = 0; s2 < n_splits; ++s2) Mx = fmaxf(Mx, __ldcg(&p.part_ml[(unit * n_splits + s2) * 2]));
  float Lall = 0.f;
  for (int s2 = 0; s2 < n_splits; ++s2) {
    const float ms = __ldcg(&p.part_ml[(unit * n_splits + s2) * 2]);
    if (ms != -INFINITY) Lall += __ldcg(&p.part_ml[(unit * n_splits + s2) * 2 + 1]) * expf(ms - Mx);
  }
  for (int c = threadIdx.x; c < head_dim; c += blockDim.x) {
    float o = 0.f;
    for (int s2 = 0; s2 < n_splits; ++s2) {
      const float ms = __ldcg(&p.part_ml[(unit * n_splits + s2) * 2]);
      if (ms != -INFINITY) o += __ldcg(&p.part_acc[(unit * n_splits + s2) * head_dim + c]) * expf(ms - Mx);
    }
    out[unit * head_dim + c] = from_float<T>(Lall > 0.f ? o / Lall : 0.f);
  }
  if (threadIdx.x == 0) p.tickets[unit] = 0;   // ready for the next call
}

template <typename T>
static int launch_decode(DecodeParams p, const KvView& view, int n_seqs, int n_splits, cudaStream_t stream) {
  constexpr int E = Chunk<T>::N;
  const int n_chunks = p.head_dim / E;
  int G = 1;
  while (G < n_chunks && G < 32) G <<= 1;
  const int cpl = (n_chunks + G - 1) / G;
  BT_CHECK(cpl <= 2, "attention_decode: head_dim %d is too large", p.head_dim);
  p.G = G;
  dim3 grid(n_splits, p.n_heads, n_seqs);
  const size_t smem = sizeof(float) * (size_t)(DEC_WARPS * p.head_dim + DEC_WARPS * 2 + 4);
  if (cpl == 1)
    BT_PDL_OK("attention_decode", launch_pdl(attention_decode_kernel<T, 1>, grid, dim3(DEC_WARPS * 32), smem, stream, 1, p, view));
  else
    BT_PDL_OK("attention_decode", launch_pdl(attention_decode_kernel<T, 2>, grid, dim3(DEC_WARPS * 32), smem, stream, 1, p, view));
  return 0;
}

}  // namespace bt

// Floats of scratch a call with these sizes needs (0 when n_splits == 1).
extern "C" long long bt_attention_decode_scratch_floats(int n_seqs, int n_heads, int head_dim, int n_splits) {
  if (n_splits <= 1) return 0;
  return (long long)n_seqs * n_heads * n_splits * (head_dim + 2);
}

// q: one row of the step's projections per sequence (query head h at q + h * head_dim).
// new_k, new_v: the new token's key and value channels in the same rows (q_row_stride apart); when given, the
//   kernel reads the newest key from there and also files it in the page, so no append has to run before it;
//   null when the pages already hold the new token.
// scratch: bt_attention_decode_scratch_floats(...) floats, 16-byte aligned.
// tickets: n_seqs * n_heads ints, zero before the first call (needed when n_splits > 1); left zero.
extern "C" int bt_attention_decode(const void* q, long long q_row_stride, const void* new_k, const void* new_v,
                                   void* k_pool, void* v_pool, const int* kv_table, int table_stride, int table_len,
                                   int page_size, void* out, float* scratch, int* tickets, const int* ctx_len,
                                   int n_seqs, int n_heads, int n_kv_heads, int head_dim, float scale, int window,
                                   int n_splits, int dtype, cudaStream_t stream) {
  using namespace bt;
  BT_CHECK(head_dim > 0 && head_dim % 8 == 0 && head_dim <= 256,
           "attention_decode: head_dim %d must be a multiple of 8 and at most 256", head_dim);
  BT_CHECK(n_heads > 0 && n_kv_heads > 0 && n_heads % n_kv_heads == 0,
           "attention_decode: %d query heads cannot share %d key heads", n_heads, n_kv_heads);
  BT_CHECK(kv_table != nullptr && table_len > 0 && page_size > 0, "attention_decode: needs a page table");
  BT_CHECK(n_splits >= 1 && n_splits <= 65535 && n_heads <= 65535 && n_seqs <= 65535, "attention_decode: grid too large");
  BT_CHECK(n_splits == 1 || (scratch != nullptr && tickets != nullptr), "attention_decode: %d splits need scratch memory and tickets", n_splits);
  BT_CHECK(q_row_stride % 8 == 0, "attention_decode: query rows must be 16-byte aligned");
  BT_CHECK((new_k == nullptr) == (new_v == nullptr), "attention_decode: give both the new key and the new value, or neither");
  if (n_seqs == 0) return 0;
  KvView view{k_pool, v_pool, kv_table, table_stride, table_len, page_size, 0, nullptr};
  DecodeParams p{q, q_row_stride, new_k, new_v, k_pool, v_pool, out, scratch,
                 scratch ? scratch + (long long)n_seqs * n_heads * n_splits * head_dim : nullptr, tickets, ctx_len,
                 n_heads, n_kv_heads, head_dim, scale, window, 1};
  if (dtype == kF32) return launch_decode<float>(p, view, n_seqs, n_splits, stream);
  if (dtype == kBF16) return launch_decode<__nv_bfloat16>(p, view, n_seqs, n_splits, stream);
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
static float* g_decode_static_ptr[kMaxDevices] = {nullptr};
static int* g_decode_static_ticket_ptr[kMaxDevices] = {nullptr};
static std::mutex g_decode_static_mutex;

// Device address of the scratch array on the current device; looked up once per device.
static int decode_static_scratch(float** ptr, int** tickets) {
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
    g_decode_static_ptr[device] = found;
    g_decode_static_ticket_ptr[device] = found_tickets;
  }
  *ptr = g_decode_static_ptr[device];
  *tickets = g_decode_static_ticket_ptr[device];
  return 0;
}

}  // namespace bt

extern "C" int bt_attention_decode_static(const void* q, long long q_row_stride, const void* k_pool,
                                          const void* v_pool, const int* kv_table, int table_stride, int table_len,
                                          int page_size, void* out, const int* ctx_len, int n_seqs, int n_heads,
                                          int n_kv_heads, int head_dim, float scale, int window, int n_splits,
                                          int dtype, cudaStream_t stream) {
  using namespace bt;
  BT_CHECK(n_seqs >= 0 && n_heads > 0 && head_dim > 0 && n_splits >= 1, "attention_decode_static: bad sizes");
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
  if (int rc = decode_static_scratch(&scratch, &tickets)) return rc;
  return bt_attention_decode(q, q_row_stride, nullptr, nullptr, const_cast<void*>(k_pool), const_cast<void*>(v_pool),
                             kv_table, table_stride, table_len, page_size, out, scratch, tickets, ctx_len, n_seqs,
                             n_heads, n_kv_heads, head_dim, scale, window, n_splits, dtype, stream);
}
