// Causal attention for steps that bring several tokens per sequence, with plain 32-bit
// arithmetic: scores, online softmax, and the value mix are all fused multiply-adds in 32-bit,
// so this kernel serves the true 32-bit path (and any head size the tensor-core kernel refuses).
// One warp owns a query; lanes own keys for the scores and channels for the value mix.
// The S x S score plane is never stored.
//
// Query t of sequence s sits at position past[s] + (t - seq_start[s]); key j is visible when
// j <= position (causal) and j > position - window (window > 0).  A query that sees no key
// yields zeros.
#include "common.cuh"

namespace bt {

constexpr int PF_BQ = 16;      // queries per block
constexpr int PF_BK = 32;      // keys per tile
constexpr int PF_WARPS = 8;
constexpr int PF_MAXI = 8;     // head_dim <= 256

template <typename T>
__global__ void __launch_bounds__(PF_WARPS * 32)
attention_prefill_simt_kernel(const T* __restrict__ q, long long q_row_stride, KvView kv, T* __restrict__ out,
                              const int* __restrict__ seq_start, const int* __restrict__ past_len, int n_heads,
                              int n_kv_heads, int head_dim, float scale, int causal, int window) {
  extern __shared__ float smem[];
  const int seq = blockIdx.y, head = blockIdx.z;
  const int t0 = seq_start[seq], n_new = seq_start[seq + 1] - t0;
  // longest tiles first: they see the most keys
  const int q_tile = (int)gridDim.x - 1 - (int)blockIdx.x;
  const int q0 = q_tile * PF_BQ;
  if (q0 >= n_new) return;
  const int past = past_len[seq];
  const int kv_len = past + n_new;
  const int kv_head = head / (n_heads / n_kv_heads);
  const int nq = min(PF_BQ, n_new - q0);
  float* Qs = smem;                                // [PF_BQ][head_dim]
  float* Ks = Qs + PF_BQ * head_dim;               // [PF_BK][head_dim + 1]
  float* Vs = Ks + PF_BK * (head_dim + 1);         // [PF_BK][head_dim]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  for (int i = tid; i < PF_BQ * head_dim; i += blockDim.x) {
    const int r = i / head_dim, c = i - r * head_dim;
    Qs[i] = r < nq ? to_float(q[(long long)(t0 + q0 + r) * q_row_stride + head * head_dim + c]) * scale : 0.f;
  }
  // key range this block can see
  const int pos_first = past + q0, pos_last = past + q0 + nq - 1;
  int k_hi = causal ? min(kv_len, pos_last + 1) : kv_len;           // exclusive
  int k_lo = window > 0 ? max(0, pos_first - window + 1) : 0;
  const int tile_lo = k_lo / PF_BK, tile_hi = (k_hi + PF_BK - 1) / PF_BK;

  float m[2], l[2], acc[2][PF_MAXI];
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    m[u] = -INFINITY;
    l[u] = 0.f;
#pragma unroll
    for (int i = 0; i < PF_MAXI; ++i) acc[u][i] = 0.f;
  }

  for (int tile = tile_lo; tile < tile_hi; ++tile) {
    __syncthreads();
    {  // stage the tile: 8 threads per key row
      const int r = tid >> 3, part = tid & 7;
      const int kp = tile * PF_BK + r;
      if (kp < kv_len) {
        const T* kr = kv_row<T>(kv.k, kv, seq, kv_head, n_kv_heads, head_dim, kp);
        const T* vr = kv_row<T>(kv.v, kv, seq, kv_head, n_kv_heads, head_dim, kp);
        for (int c = part; c < head_dim; c += 8) {
          Ks[r * (head_dim + 1) + c] = to_float(kr[c]);
          Vs[r * head_dim + c] = to_float(vr[c]);
        }
      } else {
        for (int c = part; c < head_dim; c += 8) {
          Ks[r * (head_dim + 1) + c] = 0.f;
          Vs[r * head_dim + c] = 0.f;
        }
      }
    }
    __syncthreads();
    const int kp = tile * PF_BK + lane;
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int qi = warp + u * PF_WARPS;
      if (qi >= nq) continue;  // uniform per warp
      const int qpos = past + q0 + qi;
      bool visible = kp < kv_len;
      if (causal) visible = visible && kp <= qpos;
      if (window > 0) visible = visible && kp > qpos - window;
      float s = 0.f;
      const float* qv = Qs + qi * head_dim;
      const float* kvp = Ks + lane * (head_dim + 1);
      for (int c = 0; c < head_dim; ++c) s = fmaf(qv[c], kvp[c], s);
      s = visible ? s : -INFINITY;
      const float m_new = fmaxf(m[u], warp_max(s));
      if (m_new == -INFINITY) continue;  // nothing visible yet (uniform per warp)
      const float p = visible ? expf(s - m_new) : 0.f;
      const float corr = expf(m[u] - m_new);  // m = -inf gives 0
      l[u] = l[u] * corr + warp_sum(p);
      m[u] = m_new;
#pragma unroll
      for (int i = 0; i < PF_MAXI; ++i) acc[u][i] *= corr;
      for (int j = 0; j < PF_BK; ++j) {
        const float pj = __shfl_sync(0xffffffffu, p, j);
        const float* vrow = Vs + j * head_dim;
#pragma unroll
        for (int i = 0; i < PF_MAXI; ++i) {
          const int c = lane + 32 * i;
          if (c < head_dim) acc[u][i] = fmaf(pj, vrow[c], acc[u][i]);
        }
      }
    }
  }
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    const int qi = warp + u * PF_WARPS;
    if (qi >= nq) continue;
    const float inv = l[u] > 0.f ? 1.f / l[u] : 0.f;
    T* dst = out + (long long)(t0 + q0 + qi) * ((long long)n_heads * head_dim) + head * head_dim;
#pragma unroll
    for (int i = 0; i < PF_MAXI; ++i) {
      const int c = lane + 32 * i;
      if (c < head_dim) dst[c] = from_float<T>(acc[u][i] * inv);
    }
  }
}

}  // namespace bt

// kv_table == nullptr selects the packed view: keys and values are read from the step's own
// projections (k, v point at the first key/value channel of row 0, rows kv_row_stride apart).
extern "C" int bt_attention_prefill_simt(const void* q, long long q_row_stride, const void* k, const void* v,
                                         const int* kv_table, int table_stride, int table_len, int page_size,
                                         long long kv_row_stride, void* out, const int* seq_start,
                                         const int* past_len, int n_seqs, int max_new, int n_heads, int n_kv_heads,
                                         int head_dim, float scale, int causal, int window, int dtype,
                                         cudaStream_t stream) {
  using namespace bt;
  BT_CHECK(head_dim > 0 && head_dim <= 32 * PF_MAXI,
           "attention_prefill_simt: head_dim %d must be at least 1 and at most %d", head_dim, 32 * PF_MAXI);
  BT_CHECK(n_heads > 0 && n_kv_heads > 0 && n_heads % n_kv_heads == 0,
           "attention_prefill_simt: %d query heads cannot share %d key heads", n_heads, n_kv_heads);
  BT_CHECK(n_seqs <= 65535 && n_heads <= 65535, "attention_prefill_simt: too many sequences or heads for one launch");
  if (n_seqs == 0 || max_new == 0) return 0;
  KvView view{k, v, kv_table, table_stride, table_len > 0 ? table_len : 1, page_size > 0 ? page_size : 1,
              kv_row_stride, seq_start};
  dim3 grid((max_new + PF_BQ - 1) / PF_BQ, n_seqs, n_heads);
  const size_t smem = sizeof(float) * ((size_t)PF_BQ * head_dim + (size_t)PF_BK * (head_dim + 1) + (size_t)PF_BK * head_dim);
  cudaError_t e;
  if (dtype == kF32) {
    auto kern = attention_prefill_simt_kernel<float>;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    BT_CHECK(e == cudaSuccess, "attention_prefill_simt: cannot reserve %zu bytes of shared memory", smem);
    kern<<<grid, PF_WARPS * 32, smem, stream>>>((const float*)q, q_row_stride, view, (float*)out, seq_start, past_len,
                                                n_heads, n_kv_heads, head_dim, scale, causal, window);
  } else if (dtype == kBF16) {
    auto kern = attention_prefill_simt_kernel<__nv_bfloat16>;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    BT_CHECK(e == cudaSuccess, "attention_prefill_simt: cannot reserve %zu bytes of shared memory", smem);
    kern<<<grid, PF_WARPS * 32, smem, stream>>>((const __nv_bfloat16*)q, q_row_stride, view, (__nv_bfloat16*)out,
                                                seq_start, past_len, n_heads, n_kv_heads, head_dim, scale, causal, window);
  } else {
    return fail("attention_prefill_simt: unknown dtype %d", dtype);
  }
  BT_LAUNCH_OK("attention_prefill_simt");
  return 0;
}
