// Helpers shared by the int8 paged attention kernels (pool layout constants, MMA and async-copy
// wrappers, the fixed-point scalar steps).
#pragma once

#include "common.cuh"

namespace b200 {

constexpr int kPage = 16;
constexpr int kD = 128;
constexpr int kMetaWords = 40;


// Byte offset of (d, tok) inside a 2 KB V chunk.  The chunk is stored in the operand order of
// the m16n8k32 integer MMA (A = V^T, 16 d x 32 tokens): four 512-byte quarters, each holding one
// 16-byte vector per lane; lane = (d % 8) * 4 + tok / 4 owns, as word (d / 16) * 2 + (d % 16) / 8,
// the four tokens tok & ~3 .. of row d.  A lane's 128-bit load of quarter q therefore yields the
// a0/a1 registers of the d-tiles 2q and 2q+1 for one page.
__host__ __device__ __forceinline__ int v_chunk_offset(int d, int tok) {
  const int wi = ((d >> 4) << 1) | ((d >> 3) & 1);
  const int lane = ((d & 7) << 2) | (tok >> 2);
  return ((wi >> 2) << 9) + (lane << 4) + ((wi & 3) << 2) + (tok & 3);
}



__device__ __forceinline__ void mma_s8s8(int (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                         unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_s8u8(int (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                         unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned word_of(const uint4 (&v)[4], int wi) {
  const uint4& q = v[wi >> 2];
  return (wi & 3) == 0 ? q.x : (wi & 3) == 1 ? q.y : (wi & 3) == 2 ? q.z : q.w;
}


constexpr int kSlotBytes = 4096;           // one slot = a pair of pages (K rows, or V in operand order)
constexpr int kMetaBytes = kMetaWords * 4; // 160

__device__ __forceinline__ void cp_async16(unsigned smem_dst, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_dst), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// sat32((x*m + 2^(s-1)) >> s) for 0 < s < 63 (general form otherwise).  x*m is exact in 64 bits.
__device__ __forceinline__ int mul_shift_sat32(int x, int m, int s) {
  if (s > 0 && s < 63) {
    const long long prod = (long long)x * (long long)m + (1LL << (s - 1));   // |x*m| < 2^62
    return sat32(prod >> s);
  }
  return sat32(mul_shift64((long long)x, (long long)m, s));
}

// The same for a 64-bit accumulator (|x| < 2^31 in practice; exact while x*m fits 64 bits).
__device__ __forceinline__ int mul_shift_sat32_wide(long long x, int m, int s) {
  if (s > 0 && s < 63 && x > -(1LL << 31) && x < (1LL << 31)) {
    const long long prod = x * (long long)m + (1LL << (s - 1));
    return sat32(prod >> s);
  }
  return sat32(mul_shift64(x, (long long)m, s));
}

// min(65535, ((v_mul << 15) / m_ref) >> d): relative V scale in Q0.15.
__device__ __forceinline__ unsigned rel_scale_q15(unsigned v_mul, unsigned m_ref, int d) {
  if (m_ref == 0u || d >= 32) return 0u;
  const unsigned long long num = (unsigned long long)v_mul << 15;
  unsigned long long q;
  if (m_ref >= (1u << 30)) {   // normalised reference: the quotient is below 2^17 and a float
    unsigned est = (unsigned)__fdividef((float)v_mul * 32768.0f, (float)m_ref);   // off by <= 1
    long long r = (long long)(num - (unsigned long long)est * m_ref);
    if (r < 0) { est -= 1; } else if (r >= (long long)m_ref) { est += 1; }
    q = est;
  } else {
    q = num / m_ref;
  }
  q >>= (d < 0 ? 0 : d);
  return q > 65535ull ? 65535u : (unsigned)q;
}


}  // namespace b200
