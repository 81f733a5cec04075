// Writes the new tokens' keys and values from the step's packed projections into the paged pool
// of one layer.  pool[page][kv_head][page_size][head_dim]; a sequence's page for position p is
// table[seq][(p / page_size) % table_len].  In a ring (table_len * page_size shorter than the
// sequence) only the last table_len * page_size positions are written, so no two tokens of the
// same step write the same row.  Rows move as 16-byte pieces where head size, offsets and stride
// allow it (VEC), else element by element, so that every head size is taken.
#include "common.cuh"

namespace bt {

template <typename T, bool VEC>
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
  constexpr int EPC = VEC ? 16 / sizeof(T) : 1;
  const int chunks_per_head = head_dim / EPC;
  const int total = n_kv_heads * chunks_per_head;
  const T* src = proj + (long long)t * row_stride;
  for (int i = threadIdx.x; i < total; i += blockDim.x) {
    const int h = i / chunks_per_head, c = i - h * chunks_per_head;
    const long long dst = (((long long)page * n_kv_heads + h) * page_size + in_page) * head_dim + c * EPC;
    const int so = h * head_dim + c * EPC;
    if (VEC) {
      *reinterpret_cast<uint4*>(k_pool + dst) = *reinterpret_cast<const uint4*>(src + k_offset + so);
      *reinterpret_cast<uint4*>(v_pool + dst) = *reinterpret_cast<const uint4*>(src + v_offset + so);
    } else {
      k_pool[dst] = src[k_offset + so];
      v_pool[dst] = src[v_offset + so];
    }
  }
}

}  // namespace bt

extern "C" int bt_kv_append(const void* proj, long long row_stride, int k_offset, int v_offset, const int* positions,
                            const int* token_seq, const int* ctx_len, const int* table, int table_stride,
                            int table_len, int page_size, void* k_pool, void* v_pool, int n_tokens, int n_kv_heads,
                            int head_dim, int dtype, cudaStream_t stream) {
  using namespace bt;
  BT_CHECK(head_dim > 0 && n_kv_heads > 0, "kv_append: bad sizes head_dim=%d n_kv_heads=%d", head_dim, n_kv_heads);
  BT_CHECK(table_len > 0 && page_size > 0, "kv_append: bad table_len %d or page_size %d", table_len, page_size);
  if (n_tokens == 0) return 0;
  const int es = dtype == kF32 ? 4 : 2, epc = 16 / es;
  const bool vec = head_dim % epc == 0 && row_stride % epc == 0 && k_offset % epc == 0 && v_offset % epc == 0 &&
                   (unsigned long long)proj % 16 == 0 && (unsigned long long)k_pool % 16 == 0 &&
                   (unsigned long long)v_pool % 16 == 0;
#define BT_KV_APPEND(T, VEC)                                                                                          \
  BT_PDL_OK("kv_append", launch_pdl(kv_append_kernel<T, VEC>, dim3(n_tokens), dim3(128), 0, stream, 1, (const T*)proj, \
                                    row_stride, k_offset, v_offset, positions, token_seq, ctx_len, table, table_stride, \
                                    table_len, page_size, (T*)k_pool, (T*)v_pool, n_kv_heads, head_dim))
  if (dtype == kF32) {
    if (vec) BT_KV_APPEND(float, true); else BT_KV_APPEND(float, false);
  } else if (dtype == kBF16) {
    if (vec) BT_KV_APPEND(__nv_bfloat16, true); else BT_KV_APPEND(__nv_bfloat16, false);
  } else {
    return fail("kv_append: unknown dtype %d", dtype);
  }
#undef BT_KV_APPEND
  return 0;
}
