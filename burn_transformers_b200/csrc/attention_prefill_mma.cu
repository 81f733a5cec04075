// Causal attention for steps that bring several tokens per sequence, bfloat16, on tensor cores
// (mma.sync m16n8k16, 32-bit accumulation, online softmax in 32-bit; the S x S score plane is never stored).
//
// A block owns 64 queries of one (sequence, head): 4 warps x 16 queries.  Keys and values arrive in tiles of
// 64 (one page of the cache, or 64 rows of the step's own projections) by 16-byte asynchronous copies into
// two shared-memory buffers, so tile t+1 loads while tile t is multiplied.  Rows are stored with their
// 16-byte chunks XOR-ed by the row number, which makes the ldmatrix reads of both K (as is) and V
// (transposed) free of bank conflicts.  Tiles that lie wholly in a query tile's future (or before its window)
// are skipped.
//
// Query t of sequence s sits at position past[s] + (t - seq_start[s]); key j is visible when j <= position
// (causal) and j > position - window (window > 0).  A query that sees no key yields zeros.
#include "common.cuh"

namespace bt {

constexpr int FA_BQ = 64, FA_BK = 64, FA_WARPS = 4;

struct FaParams {
  const __nv_bfloat16* q;     // rows of the step's projections; query head h at q + h * HD
  long long q_row_stride;
  KvView kv;
  __nv_bfloat16* out;         // [tokens, n_heads * HD]
  const int* seq_start;
  const int* past_len;
  int n_heads, n_kv_heads;
  float scale_log2;           // scale * log2(e): scores are kept in base 2
  int causal, window;
};

__device__ __forceinline__ unsigned fa_smem(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void fa_cp16(void* dst, const void* src, bool valid) {
  const int bytes = valid ? 16 : 0;   // 0 bytes read: the 16 bytes are filled with zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(fa_smem(dst)), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void fa_ldsm4(unsigned (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(fa_smem(p)));
}
__device__ __forceinline__ void fa_ldsm4_trans(unsigned (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(fa_smem(p)));
}
__device__ __forceinline__ void fa_mma(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float fa_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ unsigned fa_pack(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}

// element (row, col) of a [rows][HD] bfloat16 tile whose 16-byte chunks are XOR-ed with the row number
template <int HD>
__device__ __forceinline__ __nv_bfloat16* fa_at(__nv_bfloat16* tile, int row, int col) {
  constexpr int CH = HD / 8;
  const int chunk = col >> 3;
  return tile + row * HD + (((chunk & ~7) | ((chunk ^ row) & 7)) << 3) + (col & 7);
  static_assert(CH % 8 == 0, "rows must be whole 128-byte lines");
}

template <int HD>
__global__ void __launch_bounds__(FA_WARPS * 32)
attention_prefill_mma_kernel(FaParams p) {
  constexpr int CH = HD / 8;               // 16-byte chunks per row
  constexpr int KS = HD / 16;              // k-steps of the score product
  constexpr int NT = HD / 8;               // 8-wide output tiles
  extern __shared__ __align__(128) unsigned char fa_raw[];
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(fa_raw);        // [64][HD], later the output staging
  __nv_bfloat16* Ks = Qs + FA_BQ * HD;                                  // [2][64][HD]
  __nv_bfloat16* Vs = Ks + 2 * FA_BK * HD;                              // [2][64][HD]
  const int seq = blockIdx.y, head = blockIdx.z;
  const int t0 = p.seq_start[seq], n_new = p.seq_start[seq + 1] - t0;
  const int q_tile = (int)gridDim.x - 1 - (int)blockIdx.x;              // longest tiles first
  const int q0 = q_tile * FA_BQ;
  if (q0 >= n_new) return;
  const int past = p.past_len[seq];
  const int kv_len = past + n_new;
  const int kv_head = head / (p.n_heads / p.n_kv_heads);
  const int nq = min(FA_BQ, n_new - q0);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, qd = lane & 3;

  // key tiles this block can see
  const int pos_first = past + q0, pos_last = past + q0 + nq - 1;
  const int k_hi = p.causal ? min(kv_len, pos_last + 1) : kv_len;
  const int k_lo = p.window > 0 ? max(0, pos_first - p.window + 1) : 0;
  const int tile_lo = k_lo / FA_BK, tile_hi = (k_hi + FA_BK - 1) / FA_BK;

  auto load_kv = [&](int tile, int buf) {
    __nv_bfloat16* kd = Ks + buf * FA_BK * HD;
    __nv_bfloat16* vd = Vs + buf * FA_BK * HD;
    const __nv_bfloat16* kbase;
    const __nv_bfloat16* vbase;
    long long stride;
    if (p.kv.table) {   // a tile is one page of this key head
      const long long page = p.kv.table[(long long)seq * p.kv.table_stride + (tile % p.kv.table_len)];
      const long long off = (page * p.n_kv_heads + kv_head) * (long long)(FA_BK * HD);
      kbase = reinterpret_cast<const __nv_bfloat16*>(p.kv.k) + off;
      vbase = reinterpret_cast<const __nv_bfloat16*>(p.kv.v) + off;
      stride = HD;
    } else {
      const long long off = ((long long)p.kv.seq_start[seq] + (long long)tile * FA_BK) * p.kv.row_stride + (long long)kv_head * HD;
      kbase = reinterpret_cast<const __nv_bfloat16*>(p.kv.k) + off;
      vbase = reinterpret_cast<const __nv_bfloat16*>(p.kv.v) + off;
      stride = p.kv.row_stride;
    }
    for (int i = tid; i < FA_BK * CH; i += FA_WARPS * 32) {
      const int r = i / CH, c = i - r * CH;
      const bool valid = tile * FA_BK + r < kv_len;
      const long long src = valid ? (long long)r * stride + c * 8 : 0;
      const int dc = ((c & ~7) | ((c ^ r) & 7)) << 3;
      fa_cp16(kd + r * HD + dc, kbase + src, valid);
      fa_cp16(vd + r * HD + dc, vbase + src, valid);
    }
  };

  // queries of this block (rows beyond the sequence are zeros)
  for (int i = tid; i < FA_BQ * CH; i += FA_WARPS * 32) {
    const int r = i / CH, c = i - r * CH;
    const bool valid = r < nq;
    const __nv_bfloat16* src = p.q + (long long)(t0 + q0 + (valid ? r : 0)) * p.q_row_stride + head * HD + c * 8;
    fa_cp16(Qs + r * HD + (((c & ~7) | ((c ^ r) & 7)) << 3), src, valid);
  }
  if (tile_lo < tile_hi) load_kv(tile_lo, 0);
  asm volatile("cp.async.commit_group;\n" ::);

  unsigned qf[KS][4];
  float acc_o[NT][4];
#pragma unroll
  for (int j = 0; j < NT; ++j)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc_o[j][i] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const int row0 = warp * 16 + g;                    // this thread's rows in the query tile: row0 and row0 + 8
  const int qpos0 = past + q0 + row0, qpos1 = qpos0 + 8;

  for (int tile = tile_lo; tile < tile_hi; ++tile) {
    const int buf = (tile - tile_lo) & 1;
    if (tile + 1 < tile_hi) load_kv(tile + 1, buf ^ 1);
    asm volatile("cp.async.commit_group;\n" ::);
    asm volatile("cp.async.wait_group 1;\n" ::);     // everything but the newest group has landed
    __syncthreads();
    if (tile == tile_lo) {
#pragma unroll
      for (int ks = 0; ks < KS; ++ks)
        fa_ldsm4(qf[ks], fa_at<HD>(Qs, warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, ks * 16 + (lane >> 4) * 8));
    }
    __nv_bfloat16* kt = Ks + buf * FA_BK * HD;
    __nv_bfloat16* vt = Vs + buf * FA_BK * HD;
    // scores of 16 queries x 64 keys
    float s[FA_BK / 8][4];
#pragma unroll
    for (int j = 0; j < FA_BK / 8; ++j)
#pragma unroll
      for (int i = 0; i < 4; ++i) s[j][i] = 0.f;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
      for (int jp = 0; jp < FA_BK / 16; ++jp) {      // two 8-key tiles per ldmatrix.x4
        unsigned b[4];
        fa_ldsm4(b, fa_at<HD>(kt, jp * 16 + (lane & 7) + (lane >> 4) * 8, ks * 16 + ((lane >> 3) & 1) * 8));
        fa_mma(s[2 * jp], qf[ks], b[0], b[1]);
        fa_mma(s[2 * jp + 1], qf[ks], b[2], b[3]);
      }
    }
    // scale, mask, running maximum
    const int key0 = tile * FA_BK;
    const bool edge = (key0 + FA_BK > kv_len) || (p.causal && key0 + FA_BK - 1 > past + q0 + warp * 16) ||
                      (p.window > 0 && key0 <= past + q0 + warp * 16 + 15 - p.window);
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int j = 0; j < FA_BK / 8; ++j)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float v = s[j][i] * p.scale_log2;
        if (edge) {
          const int key = key0 + j * 8 + 2 * qd + (i & 1);
          const int qpos = (i >> 1) ? qpos1 : qpos0;
          bool hidden = key >= kv_len;
          if (p.causal) hidden = hidden || key > qpos;
          if (p.window > 0) hidden = hidden || key <= qpos - p.window;
          if (hidden) v = -INFINITY;
        }
        s[j][i] = v;
        mx[i >> 1] = fmaxf(mx[i >> 1], v);
      }
    float corr[2], m_use[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
      const float m_new = fmaxf(m_run[h], mx[h]);
      m_use[h] = m_new == -INFINITY ? 0.f : m_new;       // a row that has seen no key yet
      corr[h] = fa_exp2(m_run[h] - m_use[h]);            // m_run = -inf gives 0
      m_run[h] = m_new;
    }
    float ls[2] = {0.f, 0.f};
#pragma unroll
    for (int j = 0; j < FA_BK / 8; ++j)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float e = fa_exp2(s[j][i] - m_use[i >> 1]);
        s[j][i] = e;
        ls[i >> 1] += e;
      }
#pragma unroll
    for (int h = 0; h < 2; ++h) l_run[h] = l_run[h] * corr[h] + ls[h];
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      acc_o[j][0] *= corr[0];
      acc_o[j][1] *= corr[0];
      acc_o[j][2] *= corr[1];
      acc_o[j][3] *= corr[1];
    }
    // value mix: probabilities (rounded to bfloat16) x values
#pragma unroll
    for (int kt16 = 0; kt16 < FA_BK / 16; ++kt16) {
      unsigned a[4];
      a[0] = fa_pack(s[2 * kt16][0], s[2 * kt16][1]);
      a[1] = fa_pack(s[2 * kt16][2], s[2 * kt16][3]);
      a[2] = fa_pack(s[2 * kt16 + 1][0], s[2 * kt16 + 1][1]);
      a[3] = fa_pack(s[2 * kt16 + 1][2], s[2 * kt16 + 1][3]);
#pragma unroll
      for (int jp = 0; jp < NT / 2; ++jp) {            // two 8-dim tiles per ldmatrix.x4.trans
        unsigned b[4];
        fa_ldsm4_trans(b, fa_at<HD>(vt, kt16 * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, jp * 16 + (lane >> 4) * 8));
        fa_mma(acc_o[2 * jp], a, b[0], b[1]);
        fa_mma(acc_o[2 * jp + 1], a, b[2], b[3]);
      }
    }
    __syncthreads();                                   // the buffer may be overwritten by the next load
  }
  asm volatile("cp.async.wait_all;\n" ::);
  // finish: divide by the row sums, stage through shared memory, store 16 bytes at a time
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
  }
  const float inv0 = l_run[0] > 0.f ? 1.f / l_run[0] : 0.f, inv1 = l_run[1] > 0.f ? 1.f / l_run[1] : 0.f;
  __syncthreads();
#pragma unroll
  for (int j = 0; j < NT; ++j) {
    *reinterpret_cast<unsigned*>(fa_at<HD>(Qs, row0, j * 8 + 2 * qd)) = fa_pack(acc_o[j][0] * inv0, acc_o[j][1] * inv0);
    *reinterpret_cast<unsigned*>(fa_at<HD>(Qs, row0 + 8, j * 8 + 2 * qd)) = fa_pack(acc_o[j][2] * inv1, acc_o[j][3] * inv1);
  }
  __syncthreads();
  for (int i = tid; i < FA_BQ * CH; i += FA_WARPS * 32) {
    const int r = i / CH, c = i - r * CH;
    if (r < nq)
      *reinterpret_cast<uint4*>(p.out + (long long)(t0 + q0 + r) * ((long long)p.n_heads * HD) + head * HD + c * 8) =
          *reinterpret_cast<const uint4*>(Qs + r * HD + (((c & ~7) | ((c ^ r) & 7)) << 3));
  }
}

template <int HD>
static int launch_fa(const FaParams& p, int n_seqs, int max_new, cudaStream_t stream) {
  const size_t smem = sizeof(__nv_bfloat16) * (size_t)(FA_BQ * HD + 4 * FA_BK * HD);
  auto kern = attention_prefill_mma_kernel<HD>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  BT_CHECK(e == cudaSuccess, "attention_prefill_mma: cannot reserve %zu bytes of shared memory", smem);
  dim3 grid((max_new + FA_BQ - 1) / FA_BQ, n_seqs, p.n_heads);
  kern<<<grid, FA_WARPS * 32, smem, stream>>>(p);
  BT_LAUNCH_OK("attention_prefill_mma");
  return 0;
}

}  // namespace bt

// Head sizes this kernel is built for; other sizes take the plain 32-bit kernel.
extern "C" int bt_attention_prefill_mma_supports(int head_dim, int page_size) {
  return (head_dim == 64 || head_dim == 128) && page_size == bt::FA_BK;
}

// Arguments as bt_attention_prefill_simt; bfloat16 only.
extern "C" int bt_attention_prefill_mma(const void* q, long long q_row_stride, const void* k, const void* v,
                                        const int* kv_table, int table_stride, int table_len, int page_size,
                                        long long kv_row_stride, void* out, const int* seq_start, const int* past_len,
                                        int n_seqs, int max_new, int n_heads, int n_kv_heads, int head_dim, float scale,
                                        int causal, int window, cudaStream_t stream) {
  using namespace bt;
  BT_CHECK(bt_attention_prefill_mma_supports(head_dim, page_size > 0 ? page_size : FA_BK),
           "attention_prefill_mma: head_dim %d (page size %d) is not supported", head_dim, page_size);
  BT_CHECK(n_heads > 0 && n_kv_heads > 0 && n_heads % n_kv_heads == 0,
           "attention_prefill_mma: %d query heads cannot share %d key heads", n_heads, n_kv_heads);
  BT_CHECK(n_seqs <= 65535 && n_heads <= 65535, "attention_prefill_mma: too many sequences or heads for one launch");
  BT_CHECK(q_row_stride % 8 == 0 && (kv_table != nullptr || kv_row_stride % 8 == 0),
           "attention_prefill_mma: rows must be 16-byte aligned");
  if (n_seqs == 0 || max_new == 0) return 0;
  FaParams p{(const __nv_bfloat16*)q, q_row_stride,
             KvView{k, v, kv_table, table_stride, table_len > 0 ? table_len : 1, FA_BK, kv_row_stride, seq_start},
             (__nv_bfloat16*)out, seq_start, past_len, n_heads, n_kv_heads, scale * 1.4426950408889634f, causal, window};
  if (head_dim == 64) return launch_fa<64>(p, n_seqs, max_new, stream);
  return launch_fa<128>(p, n_seqs, max_new, stream);
}
