// Decode attention on tensor cores: the pieces that the fused decode step and the stand-alone decode attention share.
// The keys of a chunk are the 16 rows of the products' tiles and the one query per (sequence, head) their 8-column
// operand; keys and values lie in shared memory as the tensor memory accelerator leaves them with the 128-byte swizzle
// (tiles of 64 rows x 128 bytes; the 16-byte chunk c of row r lies at chunk c ^ (r & 7)), so that the 8 x 8 blocks
// ldmatrix reads fall into different banks.
#pragma once
#include "common.cuh"

namespace bt {

constexpr int DS_PAGE = 64;          // tokens per page

__device__ __forceinline__ void ds_mma(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned ds_pack(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}
__device__ __forceinline__ float ds_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ unsigned ds_smem(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void ds_ldmatrix_x4(unsigned (&r)[4], unsigned smem_addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr));
}
__device__ __forceinline__ void ds_ldmatrix_x4_trans(unsigned (&r)[4], unsigned smem_addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr));
}
// Shared-memory address of the 16-byte chunk `chunk` (8 dims) of row `row` of a page's keys or values.
__device__ __forceinline__ unsigned ds_swizzled(unsigned tiles, int row, int chunk) {
  return tiles + (unsigned)((chunk >> 3) * DS_PAGE * 128 + row * 128 + (((chunk & 7) ^ (row & 7)) << 4));
}

// One chunk of 16 T2 keys (rows row0.. of the page whose keys lie at Ks and values at Vs, shared-memory addresses):
// scores, the running softmax (32-bit), the weighted values, as S^T = K q^T and O^T = V^T P^T with every column of the
// 8-column operand the query (so the four lanes of a quad hold the same numbers).  A product covers 16 keys x 16 dims,
// and a lane holds the scores of keys g and g + 8 of each 16-key tile.  (With the query as row 0 of a 16-row tile
// instead, a product covers 8 keys x 16 dims and a lane 8 scores of a 32-key chunk: twice the products and the
// softmax arithmetic.)
//   qb: the query for every lane: per 16 dims the dims 2q, 2q + 1 and 8 + 2q, 9 + 2q (two registers);
//   k_lane[j] / v_lane[j]: byte offset, inside a 16-key tile, of what this lane names for ldmatrix at the j-th 16 dims
//   (ds_lane_offsets); T2: 16-key tiles of the chunk; row0: the chunk's first row in the page (a multiple of 8).
// acc[j][0], acc[j][2]: dims 16 j + g and 16 j + g + 8 (the same in the four lanes of a quad); l: the lane's own keys'
// weights, to be summed over g (lanes 4 apart) at the end.
template <int I>
__device__ __forceinline__ void ds_lane_offsets(int lane, unsigned (&k_lane)[2 * I], unsigned (&v_lane)[2 * I]) {
  const int blk = lane >> 3, r = lane & 7;
#pragma unroll
  for (int j = 0; j < 2 * I; ++j) {
    const int kc = 2 * j + (blk >> 1), vc = 2 * j + (blk & 1);      // 16-byte chunks of the row
    k_lane[j] = (unsigned)((kc >> 3) * DS_PAGE * 128 + ((blk & 1) * 8 + r) * 128 + (((kc & 7) ^ r) << 4));
    v_lane[j] = (unsigned)((vc >> 3) * DS_PAGE * 128 + ((blk >> 1) * 8 + r) * 128 + (((vc & 7) ^ r) << 4));
  }
}

template <int I, int T2>
__device__ __forceinline__ void ds_attn_chunk_kt(const unsigned (&qb)[I * 4], const unsigned (&k_lane)[2 * I],
                                                 const unsigned (&v_lane)[2 * I], unsigned Ks, unsigned Vs, int hd, int row0, int key0,
                                                 int lo, int hi, float scale_log2, float& m, float& l, float (&acc)[I * 2][4],
                                                 int lane) {
  const int g = lane >> 2, q = lane & 3;
  const unsigned kb = Ks + (unsigned)row0 * 128u, vb = Vs + (unsigned)row0 * 128u;
  float s[T2][4];
#pragma unroll
  for (int t = 0; t < T2; ++t)
#pragma unroll
    for (int e = 0; e < 4; ++e) s[t][e] = 0.f;
#pragma unroll
  for (int j = 0; j < 2 * I; ++j) {
    if (16 * j < hd) {
#pragma unroll
      for (int t = 0; t < T2; ++t) {
        unsigned kf[4];
        ds_ldmatrix_x4(kf, kb + (unsigned)(t * 16 * 128) + k_lane[j]);
        ds_mma(s[t], kf[0], kf[1], kf[2], kf[3], qb[2 * j], qb[2 * j + 1]);
      }
    }
  }
  // a lane's scores: keys key0 + 16 t + g (s[t][0]) and + 8 (s[t][2])
  float mx = -INFINITY;
#pragma unroll
  for (int t = 0; t < T2; ++t)
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int key = key0 + 16 * t + 8 * e + g;
      const float v = (key >= lo && key < hi) ? s[t][2 * e] * scale_log2 : -INFINITY;
      s[t][2 * e] = v;
      mx = fmaxf(mx, v);
    }
  mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
  mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
  mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
  const float m_new = fmaxf(m, mx);
  const float corr = m_new == -INFINITY ? 1.f : ds_exp2(m - m_new);
  float psum = 0.f;
  unsigned pb[T2][2];
#pragma unroll
  for (int t = 0; t < T2; ++t) {
    const float p0 = s[t][0] == -INFINITY ? 0.f : ds_exp2(s[t][0] - m_new);      // key 16 t + g
    const float p1 = s[t][2] == -INFINITY ? 0.f : ds_exp2(s[t][2] - m_new);      // key 16 t + g + 8
    psum += p0 + p1;
    // the 8-column operand wants keys 2q, 2q + 1 (and + 8) in one lane: they sit in the quads g = 2q and 2q + 1
    const float a0 = __shfl_sync(0xffffffffu, p0, 8 * q), a1 = __shfl_sync(0xffffffffu, p0, 8 * q + 4);
    const float b0 = __shfl_sync(0xffffffffu, p1, 8 * q), b1 = __shfl_sync(0xffffffffu, p1, 8 * q + 4);
    pb[t][0] = ds_pack(a0, a1);
    pb[t][1] = ds_pack(b0, b1);
  }
  l = l * corr + psum;
  m = m_new;
#pragma unroll
  for (int j = 0; j < I * 2; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[j][e] *= corr;
#pragma unroll
  for (int j = 0; j < 2 * I; ++j) {
    if (16 * j < hd) {
#pragma unroll
      for (int t = 0; t < T2; ++t) {
        unsigned vf[4];
        ds_ldmatrix_x4_trans(vf, vb + (unsigned)(t * 16 * 128) + v_lane[j]);
        ds_mma(acc[j], vf[0], vf[1], vf[2], vf[3], pb[t][0], pb[t][1]);
      }
    }
  }
}

}  // namespace bt
