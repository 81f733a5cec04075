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
#include "sampling.cuh"

namespace bt {

constexpr int SAMPLE_THREADS = 1024;

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, long long row_stride, int vocab, int do_sample, float temperature,
              int top_k, float top_p, float min_p, const float* __restrict__ uniforms,
              const unsigned long long* __restrict__ stream_seeds, const int* __restrict__ counters,
              int* __restrict__ out_ids, float* __restrict__ out_logp) {
  __shared__ SampleShared sh;
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.x;
  // the row's uniform: given, or draw `counters[row]` of the row's own SplitMix64 stream
  float u = 0.f;
  if (do_sample) u = stream_seeds ? stream_uniform(stream_seeds[row], (unsigned long long)counters[row]) : uniforms[row];
  select_row<SAMPLE_THREADS>(logits + (long long)row * row_stride, vocab, do_sample, temperature, top_k, top_p, min_p, u,
                             out_ids + row, out_logp + row, sh);
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
