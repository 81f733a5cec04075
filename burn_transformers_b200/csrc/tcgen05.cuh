// Wrappers of the instructions that the tcgen05 matrix products share: mbarriers with bounded waits, tensor-map
// copies, shared-memory operand descriptors, tcgen05.mma / commit / ld, and the epilogue's activation.
#pragma once
#include "common.cuh"
#include "tma.cuh"

namespace bt {

constexpr int TC_BK = 64;                 // bfloat16 per stage row: 128 bytes, the swizzle span
constexpr int TC_WAIT_LIMIT = 1 << 22;    // polls of an mbarrier before giving up

__device__ __forceinline__ unsigned tc_smem(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void tc_bar_init(unsigned long long* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(tc_smem(bar)), "r"(count));
}
__device__ __forceinline__ void tc_bar_expect(unsigned long long* bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(tc_smem(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool tc_bar_wait(unsigned long long* bar, unsigned parity) {
  for (int i = 0; i < TC_WAIT_LIMIT; ++i) {
    unsigned done;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(done) : "r"(tc_smem(bar)), "r"(parity) : "memory");
    if (done) return true;
  }
  return false;
}
__device__ __forceinline__ void tc_tma_load(void* dst, const CUtensorMap* map, int col, int row, unsigned long long* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n" ::"r"(
          tc_smem(dst)),
      "l"(map), "r"(col), "r"(row), "r"(tc_smem(bar))
      : "memory");
}
// Shared-memory operand descriptor: K-major tile of 128-byte rows, 128-byte swizzle, 8-row groups 1024 bytes apart.
__device__ __forceinline__ unsigned long long tc_desc(const void* tile) {
  unsigned long long d = 0;
  d |= (unsigned long long)((tc_smem(tile) & 0x3FFFFu) >> 4);   // start address, 16-byte units
  d |= (unsigned long long)1 << 16;                             // leading byte offset (unused with this swizzle)
  d |= (unsigned long long)(1024 >> 4) << 32;                   // stride byte offset: next group of 8 rows
  d |= (unsigned long long)1 << 46;                             // descriptor version of this architecture
  d |= (unsigned long long)2 << 61;                             // 128-byte swizzle
  return d;
}
__device__ __forceinline__ void tc_mma(unsigned tmem_d, unsigned long long a, unsigned long long b, unsigned idesc, unsigned accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_d),
      "l"(a), "l"(b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tc_commit(unsigned long long* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(tc_smem(bar)) : "memory");
}
__device__ __forceinline__ void tc_ld16(unsigned taddr, float (&v)[16]) {
  unsigned r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

__device__ __forceinline__ void tc_ld32(unsigned taddr, float (&v)[32]) {
  unsigned r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,"
      "%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
// GELU of the epilogue.  When the result is rounded to bfloat16 anyway, the tanh form uses the hardware's tanh
// (relative error about 2^-11, below that rounding); a 32-bit result gets the full-precision functions.
__device__ __forceinline__ unsigned tc_pack(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}
__device__ __forceinline__ float tc_activation(float x, int act, bool exact) {
  if (exact) return apply_activation(x, act);
  if (act == kActGeluTanh) {
    float t;
    asm("tanh.approx.f32 %0, %1;\n" : "=f"(t) : "f"(0.7978845608028654f * (x + 0.044715f * x * x * x)));
    return 0.5f * x * (1.f + t);
  }
  if (act == kActGeluErf) return gelu_erf(x);
  return x;
}
__device__ __forceinline__ void tc_bar_arrive(unsigned long long* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(tc_smem(bar)) : "memory");
}

}  // namespace bt
