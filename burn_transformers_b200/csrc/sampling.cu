// Token selection from 32-bit logits, one block per row.
//   greedy:  argmax (lowest index on ties) and its log-probability
//   sample:  z/T, then top-k (ties with the k-th value survive), top-p (an item survives while the
//            mass of strictly larger items is below p), min-p (z >= max + ln(min_p)), then the
//            inverse-CDF rule id = #{k : c_k < u * c_last} on the running sums of the survivors'
//            exp(z - max), u given per row.
// The k-th value and the top-p boundary are found without sorting, by building the boundary's
// order-preserving 32-bit key bit by bit; each bit costs one block-wide count or sum.
// Sparse logit edits (bias, repetition / presence / frequency penalties, bans) are applied by a
// separate small kernel before selection.
#include "common.cuh"

namespace bt {

constexpr int SAMPLE_THREADS = 1024;

__device__ __forceinline__ unsigned ordered_key(float v) {
  const unsigned b = __float_as_uint(v);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

// Draw `index` of the SplitMix64 stream `seed`, mapped to the midpoint of one of 2^23 intervals of (0, 1).
__device__ __forceinline__ float stream_uniform(unsigned long long seed, unsigned long long index) {
  unsigned long long v = seed + 0x9E3779B97F4A7C15ull * (index + 1ull);
  v = (v ^ (v >> 30)) * 0xBF58476D1CE4E5B9ull;
  v = (v ^ (v >> 27)) * 0x94D049BB133111EBull;
  v ^= v >> 31;
  return ((float)(v >> 41) + 0.5f) * (1.0f / 8388608.0f);
}

__device__ __forceinline__ float block_sum_f(float v, float* scratch) { return block_sum(v, scratch); }

__device__ __forceinline__ int block_sum_i(int v, int* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    int w = lane < (int)(blockDim.x >> 5) ? scratch[lane] : 0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) w += __shfl_xor_sync(0xffffffffu, w, o);
    if (lane == 0) scratch[32] = w;
  }
  __syncthreads();
  return scratch[32];
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, long long row_stride, int vocab, int do_sample, float temperature,
              int top_k, float top_p, float min_p, const float* __restrict__ uniforms,
              const unsigned long long* __restrict__ stream_seeds, const int* __restrict__ counters,
              int* __restrict__ out_ids, float* __restrict__ out_logp) {
  __shared__ float fs[33];
  __shared__ int is[33];
  __shared__ float warp_tot[32];
  __shared__ float s_max;
  __shared__ int s_arg;
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.x, tid = threadIdx.x;
  const float* z = logits + (long long)row * row_stride;
  const float inv_t = do_sample ? 1.f / temperature : 1.f;
  const float big = 3.4028234664e38f;
  auto value = [&](int i) -> float {
    float v = z[i];
    if (do_sample) v = fminf(v * inv_t, big);  // z / T, clamped to the largest finite value
    return v;
  };
  // max and first argmax
  float best = -INFINITY;
  int arg = 0x7fffffff;
  for (int i = tid; i < vocab; i += SAMPLE_THREADS) {
    const float v = value(i);
    if (v > best || (v == best && i < arg)) { best = v; arg = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ob = __shfl_xor_sync(0xffffffffu, best, o);
    const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
    if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
  }
  __shared__ float wb[32];
  __shared__ int wa[32];
  if ((tid & 31) == 0) { wb[tid >> 5] = best; wa[tid >> 5] = arg; }
  __syncthreads();
  if (tid < 32) {
    best = wb[tid]; arg = wa[tid];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
      if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
    }
    if (tid == 0) { s_max = best; s_arg = arg; }
  }
  __syncthreads();
  const float zmax = s_max;

  if (!do_sample) {
    float part = 0.f;
    for (int i = tid; i < vocab; i += SAMPLE_THREADS) part += expf(value(i) - zmax);
    const float total = block_sum_f(part, fs);
    if (tid == 0) {
      out_ids[row] = s_arg;
      out_logp[row] = -logf(total);
    }
    return;
  }

  unsigned thr = 0u;  // keep key >= thr
  if (top_k > 0 && top_k < vocab) {
    unsigned t = 0u;
    for (int bit = 31; bit >= 0; --bit) {
      const unsigned cand = t | (1u << bit);
      int cnt = 0;
      for (int i = tid; i < vocab; i += SAMPLE_THREADS) cnt += ordered_key(value(i)) >= cand;
      if (block_sum_i(cnt, is) >= top_k) t = cand;
    }
    thr = t;
  }
  if (top_p > 0.f && top_p < 1.f) {
    float part = 0.f;
    for (int i = tid; i < vocab; i += SAMPLE_THREADS) {
      const float v = value(i);
      if (ordered_key(v) >= thr) part += expf(v - zmax);
    }
    const float need = top_p * block_sum_f(part, fs);
    unsigned t = 0u;
    for (int bit = 31; bit >= 0; --bit) {
      const unsigned cand = t | (1u << bit);
      float mass = 0.f;
      for (int i = tid; i < vocab; i += SAMPLE_THREADS) {
        const float v = value(i);
        const unsigned key = ordered_key(v);
        if (key >= cand && key >= thr) mass += expf(v - zmax);
      }
      if (block_sum_f(mass, fs) >= need) t = cand;
    }
    thr = max(thr, t);
  }
  if (min_p > 0.f) thr = max(thr, ordered_key(zmax + logf(min_p)));

  // running sums in index order: a contiguous chunk per thread, then a block scan
  const int chunk = (vocab + SAMPLE_THREADS - 1) / SAMPLE_THREADS;
  const int lo = min(vocab, tid * chunk), hi = min(vocab, lo + chunk);
  float mine = 0.f;
  for (int i = lo; i < hi; ++i) {
    const float v = value(i);
    if (ordered_key(v) >= thr) mine += expf(v - zmax);
  }
  float incl = mine;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float up = __shfl_up_sync(0xffffffffu, incl, o);
    if ((tid & 31) >= o) incl += up;
  }
  if ((tid & 31) == 31) warp_tot[tid >> 5] = incl;
  __syncthreads();
  if (tid < 32) {
    float w = warp_tot[tid];
    float wi = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float up = __shfl_up_sync(0xffffffffu, wi, o);
      if (tid >= o) wi += up;
    }
    warp_tot[tid] = wi - w;  // exclusive prefix of the warp totals
    if (tid == 31) fs[32] = wi;
  }
  __syncthreads();
  const float total = fs[32];
  const float excl = warp_tot[tid >> 5] + (incl - mine);
  // the row's uniform: given, or draw `counters[row]` of the row's own SplitMix64 stream
  const float u = stream_seeds ? stream_uniform(stream_seeds[row], (unsigned long long)counters[row]) : uniforms[row];
  const float threshold = u * total;
  int below = 0;
  if (excl < threshold) {
    float run = excl;
    for (int i = lo; i < hi; ++i) {
      const float v = value(i);
      if (ordered_key(v) >= thr) run += expf(v - zmax);
      below += run < threshold;
    }
  }
  __syncthreads();
  const int id = min(block_sum_i(below, is), vocab - 1);
  if (tid == 0) {
    out_ids[row] = id;
    out_logp[row] = (value(id) - zmax) - logf(total);
  }
}

// One edit per (row, token): z += add; z = z > 0 ? z / rep : z * rep (rep != 1); z -= sub; ban -> -inf.
__global__ void logit_edit_kernel(float* __restrict__ logits, long long row_stride, const int* __restrict__ rows,
                                  const int* __restrict__ tokens, const float* __restrict__ vals, int n_edits, int vocab) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_edits) return;
  const int tok = tokens[i];
  if (tok < 0 || tok >= vocab) return;
  float* p = logits + (long long)rows[i] * row_stride + tok;
  float z = *p + vals[4 * i];
  const float rep = vals[4 * i + 1];
  if (rep != 1.f) z = z > 0.f ? z / rep : z * rep;
  z -= vals[4 * i + 2];
  z = fminf(z, 3.4028234664e38f);
  if (vals[4 * i + 3] != 0.f) z = -INFINITY;
  *p = z;
}

}  // namespace bt

// Uniforms come from `uniforms` (one per row) or, when `stream_seeds` is given, are drawn on the device:
// row r uses draw counters[r] of the SplitMix64 stream stream_seeds[r].
extern "C" int bt_sample(const float* logits, long long row_stride, int n_rows, int vocab, int do_sample,
                         float temperature, int top_k, float top_p, float min_p, const float* uniforms,
                         const unsigned long long* stream_seeds, const int* counters, int* out_ids,
                         float* out_logp, cudaStream_t stream) {
  using namespace bt;
  BT_CHECK(vocab > 0 && n_rows >= 0, "sample: bad sizes rows=%d vocab=%d", n_rows, vocab);
  BT_CHECK(!do_sample || (temperature > 0.f && (uniforms != nullptr || (stream_seeds != nullptr && counters != nullptr))),
           "sample: sampling needs a positive temperature and uniforms (or stream seeds and counters)");
  if (n_rows == 0) return 0;
  BT_PDL_OK("sample", launch_pdl(sample_kernel, dim3(n_rows), dim3(SAMPLE_THREADS), 0, stream, 1, logits, row_stride, vocab,
                                 do_sample, temperature, top_k, top_p, min_p, uniforms, stream_seeds, counters, out_ids,
                                 out_logp));
  return 0;
}

namespace bt {
// After a decode step whose tokens were selected on the device: the selected ids become the next step's
// tokens, and every sequence moves on by one position.
__global__ void advance_kernel(const int* __restrict__ ids, int* __restrict__ tokens, int* __restrict__ positions,
                               int* __restrict__ past_len, int* __restrict__ ctx_len, int* __restrict__ counters, int n) {
  pdl_trigger();
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  tokens[i] = ids[i];
  positions[i] += 1;
  past_len[i] += 1;
  ctx_len[i] += 1;
  counters[i] += 1;
}
}  // namespace bt

extern "C" int bt_advance(const int* ids, int* tokens, int* positions, int* past_len, int* ctx_len, int* counters,
                          int n, cudaStream_t stream) {
  using namespace bt;
  if (n <= 0) return 0;
  BT_PDL_OK("advance", launch_pdl(advance_kernel, dim3((n + 127) / 128), dim3(128), 0, stream, 1, ids, tokens, positions,
                                  past_len, ctx_len, counters, n));
  return 0;
}

extern "C" int bt_logit_edits(float* logits, long long row_stride, const int* rows, const int* tokens,
                              const float* vals, int n_edits, int vocab, cudaStream_t stream) {
  using namespace bt;
  if (n_edits <= 0) return 0;
  logit_edit_kernel<<<(n_edits + 127) / 128, 128, 0, stream>>>(logits, row_stride, rows, tokens, vals, n_edits, vocab);
  BT_LAUNCH_OK("logit_edits");
  return 0;
}
