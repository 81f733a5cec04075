// Attention for steps that bring one token per sequence: one query per (sequence, head) over the
// keys and values of that sequence's pages.  The work is memory traffic, so the kernel is built
// around 16-byte loads: a group of lanes owns one key row, several rows are in flight per warp,
// and long contexts are cut into splits that run as separate blocks; a second kernel merges the
// splits' partial (max, sum, weighted values).  Scores, softmax and the value mix are 32-bit.
//
// Scratch layout (32-bit): part_acc[seq][head][split][head_dim], part_ml[seq][head][split][2].
#include "common.cuh"

namespace bt {

constexpr int DEC_WARPS = 4;

template <typename T> struct Chunk;   // 16 bytes of T as floats
template <> struct Chunk<float> {
  static constexpr int N = 4;
  __device__ static void load(const float* p, float (&f)[4]) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
  }
};
template <> struct Chunk<__nv_bfloat16> {
  static constexpr int N = 8;
  __device__ static void load(const __nv_bfloat16* p, float (&f)[8]) {
    const uint4 v = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 x = __bfloat1622float2(h[i]);
      f[2 * i] = x.x;
      f[2 * i + 1] = x.y;
    }
  }
};

// CPL: 16-byte chunks per lane (1 or 2).  G (runtime, power of two <= 32): lanes per key row.
template <typename T, int CPL>
__global__ void __launch_bounds__(DEC_WARPS * 32)
attention_decode_kernel(const T* __restrict__ q, long long q_row_stride, KvView kv, T* __restrict__ out,
                        float* __restrict__ part_acc, float* __restrict__ part_ml, const int* __restrict__ ctx_len,
                        int n_heads, int n_kv_heads, int head_dim, float scale, int window, int G) {
  constexpr int E = Chunk<T>::N;
  const int split = blockIdx.x, n_splits = gridDim.x;
  const int head = blockIdx.y, seq = blockIdx.z;
  const int kv_head = head / (n_heads / n_kv_heads);
  const int L = ctx_len[seq];                       // keys 0..L-1; the query sits at L-1
  const int lo = window > 0 ? max(0, L - window) : 0;
  const int per = (L - lo + n_splits - 1) / n_splits;
  const int k_begin = lo + split * per;
  const int k_end = min(L, k_begin + per);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int gl = lane & (G - 1);                    // lane within its key group
  const int sub = lane / G;                         // which key of the warp's batch
  const int keys_per_warp = 32 / G;
  const int n_chunks = head_dim / E;

  float qr[CPL][E], acc[CPL][E];
#pragma unroll
  for (int c = 0; c < CPL; ++c) {
    const int ch = gl + c * G;
    if (ch < n_chunks) {
      Chunk<T>::load(q + (long long)seq * q_row_stride + head * head_dim + ch * E, qr[c]);
#pragma unroll
      for (int e = 0; e < E; ++e) qr[c][e] *= scale;
    } else {
#pragma unroll
      for (int e = 0; e < E; ++e) qr[c][e] = 0.f;
    }
#pragma unroll
    for (int e = 0; e < E; ++e) acc[c][e] = 0.f;
  }
  float m = -INFINITY, l = 0.f;

  for (int base = k_begin + warp * keys_per_warp; base < k_end; base += DEC_WARPS * keys_per_warp) {
    const int key = base + sub;
    const bool valid = key < k_end;
    float kf[CPL][E];
    const T* krow = nullptr;
    const T* vrow = nullptr;
    if (valid) {
      krow = kv_row<T>(kv.k, kv, seq, kv_head, n_kv_heads, head_dim, key);
      vrow = kv_row<T>(kv.v, kv, seq, kv_head, n_kv_heads, head_dim, key);
    }
    float s = 0.f;
#pragma unroll
    for (int c = 0; c < CPL; ++c) {
      const int ch = gl + c * G;
      if (valid && ch < n_chunks) {
        Chunk<T>::load(krow + ch * E, kf[c]);
#pragma unroll
        for (int e = 0; e < E; ++e) s = fmaf(qr[c][e], kf[c][e], s);
      }
    }
    for (int o = G >> 1; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (valid) {
      const float m_new = fmaxf(m, s);
      const float corr = expf(m - m_new);
      const float p = expf(s - m_new);
      l = l * corr + p;
      m = m_new;
#pragma unroll
      for (int c = 0; c < CPL; ++c) {
        const int ch = gl + c * G;
        if (ch < n_chunks) {
          float vf[E];
          Chunk<T>::load(vrow + ch * E, vf);
#pragma unroll
          for (int e = 0; e < E; ++e) acc[c][e] = fmaf(p, vf[e], acc[c][e] * corr);
        }
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
  extern __shared__ float sm[];            // [DEC_WARPS][head_dim] + [DEC_WARPS][2]
  float* s_acc = sm;
  float* s_ml = sm + DEC_WARPS * head_dim;
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
  const long long unit = ((long long)seq * n_heads + head);
  for (int c = threadIdx.x; c < head_dim; c += blockDim.x) {
    float o = 0.f;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) o += s_acc[w * head_dim + c] * wgt[w];
    if (n_splits == 1)
      out[unit * head_dim + c] = from_float<T>(Lsum > 0.f ? o / Lsum : 0.f);
    else
      part_acc[(unit * n_splits + split) * head_dim + c] = o;
  }
  if (n_splits > 1 && threadIdx.x == 0) {
    part_ml[(unit * n_splits + split) * 2] = M;
    part_ml[(unit * n_splits + split) * 2 + 1] = Lsum;
  }
}

template <typename T>
__global__ void attention_decode_merge_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml,
                                              T* __restrict__ out, int n_splits, int head_dim) {
  const long long unit = blockIdx.x;  // seq * n_heads + head
  float M = -INFINITY;
  for (int s = 0; s < n_splits; ++s) M = fmaxf(M, part_ml[(unit * n_splits + s) * 2]);
  float Lsum = 0.f;
  for (int s = 0; s < n_splits; ++s) {
    const float ms = part_ml[(unit * n_splits + s) * 2];
    if (ms != -INFINITY) Lsum += part_ml[(unit * n_splits + s) * 2 + 1] * expf(ms - M);
  }
  for (int c = threadIdx.x; c < head_dim; c += blockDim.x) {
    float o = 0.f;
    for (int s = 0; s < n_splits; ++s) {
      const float ms = part_ml[(unit * n_splits + s) * 2];
      if (ms != -INFINITY) o += part_acc[(unit * n_splits + s) * head_dim + c] * expf(ms - M);
    }
    out[unit * head_dim + c] = from_float<T>(Lsum > 0.f ? o / Lsum : 0.f);
  }
}

template <typename T>
static int launch_decode(const void* q, long long q_row_stride, const KvView& view, void* out, float* part_acc,
                         float* part_ml, const int* ctx_len, int n_seqs, int n_heads, int n_kv_heads, int head_dim,
                         float scale, int window, int n_splits, cudaStream_t stream) {
  constexpr int E = Chunk<T>::N;
  const int n_chunks = head_dim / E;
  int G = 1;
  while (G < n_chunks && G < 32) G <<= 1;
  const int cpl = (n_chunks + G - 1) / G;
  BT_CHECK(cpl <= 2, "attention_decode: head_dim %d is too large", head_dim);
  dim3 grid(n_splits, n_heads, n_seqs);
  const size_t smem = sizeof(float) * (size_t)(DEC_WARPS * head_dim + DEC_WARPS * 2);
  if (cpl == 1)
    attention_decode_kernel<T, 1><<<grid, DEC_WARPS * 32, smem, stream>>>(
        (const T*)q, q_row_stride, view, (T*)out, part_acc, part_ml, ctx_len, n_heads, n_kv_heads, head_dim, scale, window, G);
  else
    attention_decode_kernel<T, 2><<<grid, DEC_WARPS * 32, smem, stream>>>(
        (const T*)q, q_row_stride, view, (T*)out, part_acc, part_ml, ctx_len, n_heads, n_kv_heads, head_dim, scale, window, G);
  BT_LAUNCH_OK("attention_decode");
  if (n_splits > 1) {
    attention_decode_merge_kernel<T><<<n_seqs * n_heads, 64, 0, stream>>>(part_acc, part_ml, (T*)out, n_splits, head_dim);
    BT_LAUNCH_OK("attention_decode_merge");
  }
  return 0;
}

}  // namespace bt

// Floats of scratch a call with these sizes needs (0 when n_splits == 1).
extern "C" long long bt_attention_decode_scratch_floats(int n_seqs, int n_heads, int head_dim, int n_splits) {
  if (n_splits <= 1) return 0;
  return (long long)n_seqs * n_heads * n_splits * (head_dim + 2);
}

// q: one row per sequence.  scratch: bt_attention_decode_scratch_floats(...) floats, 16-byte aligned.
extern "C" int bt_attention_decode(const void* q, long long q_row_stride, const void* k_pool, const void* v_pool,
                                   const int* kv_table, int table_stride, int table_len, int page_size, void* out,
                                   float* scratch, const int* ctx_len, int n_seqs, int n_heads, int n_kv_heads,
                                   int head_dim, float scale, int window, int n_splits, int dtype,
                                   cudaStream_t stream) {
  using namespace bt;
  BT_CHECK(head_dim > 0 && head_dim % 8 == 0 && head_dim <= 256,
           "attention_decode: head_dim %d must be a multiple of 8 and at most 256", head_dim);
  BT_CHECK(n_heads > 0 && n_kv_heads > 0 && n_heads % n_kv_heads == 0,
           "attention_decode: %d query heads cannot share %d key heads", n_heads, n_kv_heads);
  BT_CHECK(kv_table != nullptr && table_len > 0 && page_size > 0, "attention_decode: needs a page table");
  BT_CHECK(n_splits >= 1 && n_splits <= 65535 && n_heads <= 65535 && n_seqs <= 65535, "attention_decode: grid too large");
  BT_CHECK(n_splits == 1 || scratch != nullptr, "attention_decode: %d splits need scratch memory", n_splits);
  BT_CHECK(q_row_stride % 8 == 0, "attention_decode: query rows must be 16-byte aligned");
  if (n_seqs == 0) return 0;
  KvView view{k_pool, v_pool, kv_table, table_stride, table_len, page_size, 0, nullptr};
  float* part_acc = scratch;
  float* part_ml = scratch ? scratch + (long long)n_seqs * n_heads * n_splits * head_dim : nullptr;
  if (dtype == kF32)
    return launch_decode<float>(q, q_row_stride, view, out, part_acc, part_ml, ctx_len, n_seqs, n_heads, n_kv_heads,
                                head_dim, scale, window, n_splits, stream);
  if (dtype == kBF16)
    return launch_decode<__nv_bfloat16>(q, q_row_stride, view, out, part_acc, part_ml, ctx_len, n_seqs, n_heads,
                                        n_kv_heads, head_dim, scale, window, n_splits, stream);
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
static float* g_decode_static_ptr[kMaxDevices] = {nullptr};
static std::mutex g_decode_static_mutex;

// Device address of the scratch array on the current device; looked up once per device.
static int decode_static_scratch(float** ptr) {
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
    g_decode_static_ptr[device] = found;
  }
  *ptr = g_decode_static_ptr[device];
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
  float* scratch = nullptr;
  if (int rc = decode_static_scratch(&scratch)) return rc;
  return bt_attention_decode(q, q_row_stride, k_pool, v_pool, kv_table, table_stride, table_len, page_size, out, scratch,
                             ctx_len, n_seqs, n_heads, n_kv_heads, head_dim, scale, window, n_splits, dtype, stream);
}
