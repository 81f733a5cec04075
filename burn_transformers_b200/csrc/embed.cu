// Token embedding with an optional learned position table: x[t] = wte[id[t]] (+ wpe[pos[t]]).
// The sum is formed in 32-bit and written to the 32-bit residual stream.
#include "common.cuh"

namespace bt {

template <typename T>
__global__ void embed_kernel(const int* __restrict__ tokens, const int* __restrict__ positions,
                             const T* __restrict__ wte, const T* __restrict__ wpe, float* __restrict__ out,
                             int width, int vocab, int n_positions, int* __restrict__ status) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const int id = tokens[t];
  const int pos = wpe ? positions[t] : 0;
  if (id < 0 || id >= vocab || pos < 0 || (wpe && pos >= n_positions)) {
    // An id outside the table is a caller's fault; record it and write zeros, never read outside.
    if (threadIdx.x == 0 && status) atomicExch(status, 1 + t);
    for (int c = threadIdx.x; c < width; c += blockDim.x) out[(long long)t * width + c] = 0.f;
    return;
  }
  const T* e = wte + (long long)id * width;
  const T* p = wpe ? wpe + (long long)pos * width : nullptr;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    float v = to_float(e[c]);
    if (p) v += to_float(p[c]);
    out[(long long)t * width + c] = v;
  }
}

}  // namespace bt

extern "C" int bt_embed(const int* tokens, const int* positions, const void* wte, const void* wpe, float* out,
                        int n_tokens, int width, int vocab, int n_positions, int dtype, int* status,
                        cudaStream_t stream) {
  using namespace bt;
  BT_CHECK(n_tokens >= 0 && width > 0 && vocab > 0, "embed: bad sizes n_tokens=%d width=%d vocab=%d", n_tokens, width, vocab);
  if (n_tokens == 0) return 0;
  const int threads = width >= 256 ? 256 : 128;
  if (dtype == kF32)
    BT_PDL_OK("embed", launch_pdl(embed_kernel<float>, dim3(n_tokens), dim3(threads), 0, stream, 1, tokens, positions,
                                  (const float*)wte, (const float*)wpe, out, width, vocab, n_positions, status));
  else if (dtype == kBF16)
    BT_PDL_OK("embed", launch_pdl(embed_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(threads), 0, stream, 1, tokens,
                                  positions, (const __nv_bfloat16*)wte, (const __nv_bfloat16*)wpe, out, width, vocab,
                                  n_positions, status));
  else
    return fail("embed: unknown dtype %d", dtype);
  return 0;
}
