// Writes the new tokens' keys and values from the step's packed projections into the paged pool
// of one layer.  pool[page][kv_head][page_size][head_dim]; a sequence's page for position p is
// table[seq][(p / page_size) % table_len].  In a ring (table_len * page_size shorter than the
// sequence) only the last table_len * page_size positions are written, so no two tokens of the
// same step write the same row.
#include "common.cuh"

namespace bt {

template <typename T>
__global__ void kv_append_kernel(const T* __restrict__ proj, long long row_stride, int k_offset, int v_offset,
                                 const int* __restrict__ positions, const int* __restrict__ token_seq,
                                 const int* __restrict__ ctx_len, const int* __restrict__ table, int table_stride,
                                 int table_len, int page_size, T* __restrict__ k_pool, T* __restrict__ v_pool,
                                 int n_kv_heads, int head_dim) {
  pdl_trigger();
  pdl_wait();      // (every block, also one that has nothing to file: the next kernel's wait rests on this one's)
  const int t = blockIdx.x;
  const int seq = token_seq[t];
  const int pos = positions[t];
  const long long ring = (long long)table_len * page_size;
  if ((long long)pos < (long long)ctx_len[seq] - ring) return;  // older than the ring keeps
  const int lp = pos / page_size;
  const int page = table[(long long)seq * table_stride + (lp % table_len)];
  const int in_page = pos - lp * page_size;
  constexpr int EPC = 16 / sizeof(T);
  const int chunks_per_head = head_dim / EPC;
  const int total = n_kv_heads * chunks_per_head;
  const T* src = proj + (long long)t * row_stride;
  for (int i = threadIdx.x; i < total; i += blockDim.x) {
    const int h = i / chunks_per_head, c = i - h * chunks_per_head;
    const long long dst = (((long long)page * n_kv_heads + h) * page_size + in_page) * head_dim + c * EPC;
    const int so = h * head_dim + c * EPC;
    *reinterpret_cast<uint4*>(k_pool + dst) = *reinterpret_cast<const uint4*>(src + k_offset + so);
    *reinterpret_cast<uint4*>(v_pool + dst) = *reinterpret_cast<const uint4*>(src + v_offset + so);
  }
}

}  // namespace bt

extern "C" int bt_kv_append(const void* proj, long long row_stride, int k_offset, int v_offset, const int* positions,
                            const int* token_seq, const int* ctx_len, const int* table, int table_stride,
                            int table_len, int page_size, void* k_pool, void* v_pool, int n_tokens, int n_kv_heads,
                            int head_dim, int dtype, cudaStream_t stream) {
  using namespace bt;
  BT_CHECK(head_dim > 0 && head_dim % 8 == 0, "kv_append: head_dim %d must be a multiple of 8", head_dim);
  BT_CHECK(row_stride % 8 == 0 && k_offset % 8 == 0 && v_offset % 8 == 0,
           "kv_append: projection rows must be 16-byte aligned (stride %lld, offsets %d %d)", row_stride, k_offset, v_offset);
  BT_CHECK(table_len > 0 && page_size > 0, "kv_append: bad table_len %d or page_size %d", table_len, page_size);
  if (n_tokens == 0) return 0;
  if (dtype == kF32)
    BT_PDL_OK("kv_append", launch_pdl(kv_append_kernel<float>, dim3(n_tokens), dim3(128), 0, stream, 1, (const float*)proj, row_stride,
                                      k_offset, v_offset, positions, token_seq, ctx_len, table, table_stride, table_len,
                                      page_size, (float*)k_pool, (float*)v_pool, n_kv_heads, head_dim));
  else if (dtype == kBF16)
    BT_PDL_OK("kv_append", launch_pdl(kv_append_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(128), 0, stream, 1,
                                      (const __nv_bfloat16*)proj, row_stride, k_offset, v_offset, positions, token_seq, ctx_len,
                                      table, table_stride, table_len, page_size, (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool,
                                      n_kv_heads, head_dim));
  else
    return fail("kv_append: unknown dtype %d", dtype);
  return 0;
}
