// Selection of one token from a row of 32-bit logits by a whole thread block (used by the selection kernel and
// by the fused decode step).
//   greedy:  argmax (lowest index on ties) and its log-probability
//   sample:  z/T, then top-k (ties with the k-th value survive), top-p (an item survives while the
//            mass of strictly larger items is below p), min-p (z >= max + ln(min_p)), then the
//            inverse-CDF rule id = #{k : c_k < u * c_last} on the running sums of the survivors' exp(z - max).
// The k-th value and the top-p boundary are found without sorting, by building the boundary's
// order-preserving 32-bit key bit by bit; each bit costs one block-wide count or sum.
#pragma once
#include "common.cuh"

namespace bt {

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

__device__ __forceinline__ int block_max_i(int v, int* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = max(v, __shfl_xor_sync(0xffffffffu, v, o));
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    int w = lane < (int)(blockDim.x >> 5) ? scratch[lane] : (int)0x80000000;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) w = max(w, __shfl_xor_sync(0xffffffffu, w, o));
    if (lane == 0) scratch[32] = w;
  }
  __syncthreads();
  return scratch[32];
}

struct SampleShared {
  float fs[33];
  int is[33];
  float warp_tot[32];
  float wb[32];
  int wa[32];
  float s_max;
  int s_arg;
};

// Every thread of the block (NT threads, a multiple of 32) calls this with the same arguments; thread 0 writes
// the result.  `u` is the row's uniform in (0, 1) (used when do_sample).
template <int NT>
__device__ void select_row(const float* __restrict__ z, int vocab, int do_sample, float temperature, int top_k,
                           float top_p, float min_p, float u, int* out_id, float* out_logp, SampleShared& sh) {
  const int tid = threadIdx.x;
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
  for (int i = tid; i < vocab; i += NT) {
    const float v = value(i);
    if (v > best || (v == best && i < arg)) { best = v; arg = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ob = __shfl_xor_sync(0xffffffffu, best, o);
    const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
    if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
  }
  if ((tid & 31) == 0) { sh.wb[tid >> 5] = best; sh.wa[tid >> 5] = arg; }
  __syncthreads();
  if (tid < 32) {
    best = tid < NT / 32 ? sh.wb[tid] : -INFINITY;
    arg = tid < NT / 32 ? sh.wa[tid] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
      if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
    }
    if (tid == 0) { sh.s_max = best; sh.s_arg = arg; }
  }
  __syncthreads();
  const float zmax = sh.s_max;

  if (!do_sample) {
    float part = 0.f;
    for (int i = tid; i < vocab; i += NT) part += expf(value(i) - zmax);
    const float total = block_sum_f(part, sh.fs);
    if (tid == 0) {
      *out_id = sh.s_arg;
      *out_logp = -logf(total);
    }
    return;
  }

  unsigned thr = 0u;  // keep key >= thr
  if (top_k > 0 && top_k < vocab) {
    unsigned t = 0u;
    for (int bit = 31; bit >= 0; --bit) {
      const unsigned cand = t | (1u << bit);
      int cnt = 0;
      for (int i = tid; i < vocab; i += NT) cnt += ordered_key(value(i)) >= cand;
      if (block_sum_i(cnt, sh.is) >= top_k) t = cand;
    }
    thr = t;
  }
  if (top_p > 0.f && top_p < 1.f) {
    float part = 0.f;
    for (int i = tid; i < vocab; i += NT) {
      const float v = value(i);
      if (ordered_key(v) >= thr) part += expf(v - zmax);
    }
    const float need = top_p * block_sum_f(part, sh.fs);
    unsigned t = 0u;
    for (int bit = 31; bit >= 0; --bit) {
      const unsigned cand = t | (1u << bit);
      float mass = 0.f;
      for (int i = tid; i < vocab; i += NT) {
        const float v = value(i);
        const unsigned key = ordered_key(v);
        if (key >= cand && key >= thr) mass += expf(v - zmax);
      }
      if (block_sum_f(mass, sh.fs) >= need) t = cand;
    }
    thr = max(thr, t);
  }
  if (min_p > 0.f) thr = max(thr, ordered_key(zmax + logf(min_p)));

  // running sums in index order: a contiguous chunk per thread, then a block scan
  const int chunk = (vocab + NT - 1) / NT;
  const int lo = min(vocab, tid * chunk), hi = min(vocab, lo + chunk);
  float mine = 0.f;
  int last_kept = -1;              // the largest index of this thread's chunk that survived the filters
  for (int i = lo; i < hi; ++i) {
    const float v = value(i);
    if (ordered_key(v) >= thr) {
      mine += expf(v - zmax);
      last_kept = i;
    }
  }
  float incl = mine;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float up = __shfl_up_sync(0xffffffffu, incl, o);
    if ((tid & 31) >= o) incl += up;
  }
  if ((tid & 31) == 31) sh.warp_tot[tid >> 5] = incl;
  __syncthreads();
  if (tid < 32) {
    float w = tid < NT / 32 ? sh.warp_tot[tid] : 0.f;
    float wi = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float up = __shfl_up_sync(0xffffffffu, wi, o);
      if (tid >= o) wi += up;
    }
    sh.warp_tot[tid] = wi - w;  // exclusive prefix of the warp totals
    if (tid == 31) sh.fs[32] = wi;
  }
  __syncthreads();
  const float total = sh.fs[32];
  const float excl = sh.warp_tot[tid >> 5] + (incl - mine);
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
  // The threshold u * total and the running sums are rounded differently (a scan of per-thread sums against serial
  // additions), so with u within a few units in the last place of 1 the last survivor's running sum can stay below
  // the threshold: the count then runs past it, onto indices the filters removed.  The last survivor bounds it.
  const int last_survivor = block_max_i(last_kept, sh.is);
  const int id = min(block_sum_i(below, sh.is), max(last_survivor, 0));
  if (tid == 0) {
    *out_id = id;
    *out_logp = (value(id) - zmax) - logf(total);
  }
}

}  // namespace bt
