// SiLU(gate) * up for one element in Q15.16, and the direct sigmoid table, shared by the row kernels and by the
// GEMM epilogue that applies the activation.
#pragma once
#include "common.cuh"

namespace b200 {

// silu_and_mul_int_only_kernel's arithmetic (silu_and_mul_int_only.py:156-226) for one element.
__device__ __forceinline__ int silu_mul_elem(int g, int u, const int32_t* __restrict__ lut) {
  const int a = g > 0 ? -g : g;                                  // -|g|, fits int32 for every g
  const long long prod = (long long)a * 94549LL;                 // -|g| * log2e, Q30.32; y = prod >> 16
  const int yi = (int)(prod >> 32);                              // y >> 16  (<= 0)
  const unsigned idx = ((unsigned)prod) >> 22;                   // (y & 0xFFFF) >> 6
  unsigned E;
  asm("shr.u32 %0, %1, %2;" : "=r"(E) : "r"((unsigned)lut[idx]), "r"((unsigned)(13 - yi)));  // >= 32 gives 0
  E = min(E, 65536u);
  // sneg = floor(E * 2^16 / (2^16 + E)): float estimate (off by at most 1), exact correction
  const unsigned den = 65536u + E;
  const unsigned num = E << 16;                                  // wraps only for E == 2^16 (handled below)
  // E and den are below 2^23, so they convert to float exactly by being placed in the mantissa of 2^23
  // (an OR and an FP add instead of the conversion unit), and the estimate goes back the same way
  // (rounded to nearest instead of truncated: still within one of the quotient).
  const float Ef = __uint_as_float(0x4B000000u | E) - 8388608.0f;
  const float denf = __uint_as_float(0x4B000000u | den) - 8388608.0f;
  unsigned sneg = __float_as_uint(__fdividef(Ef * 65536.0f, denf) + 8388608.0f) - 0x4B000000u;
  const int rem = (int)(num - sneg * den);
  sneg += rem < 0 ? -1 : (rem >= (int)den ? 1 : 0);
  sneg = (E == 65536u) ? 32768u : sneg;
  const int sig = (int)(g > 0 ? 65536u - sneg : sneg);           // <= 2^16: 32 x 32 -> 64 bit products below
  const long long gs = (long long)g * (long long)sig;
  const int t = (int)__funnelshift_r((unsigned)gs, (unsigned)(gs >> 32), 16);   // (g * sig) >> 16, |t| <= |g|
  const long long tu = (long long)t * (long long)u;
  const int hi = (int)(tu >> 32);
  const int res = (int)__funnelshift_r((unsigned)tu, (unsigned)hi, 16);        // low 32 bits of tu >> 16
  // tu >> 16 fits int32 iff bits 47..63 of tu all equal the sign bit of the result
  return (hi >> 15) == (res >> 31) ? res : (hi < 0 ? (int)(-2147483647 - 1) : 2147483647);
}

// The same element with the sigmoid term read from a direct table: E and s = (E << 16) / (65536 + E) depend only
// on key = (-|g| * 94549) >> 22 (the exponent's integer part and the 10 table bits), and s is 0 below key -19456.
#include "silu_sneg.inc"
constexpr int kSnegEntries = 19457;
static __device__ __align__(16) const uint16_t g_silu_sneg[kSnegEntries] = {B200_LUT_kSiluSneg};

__device__ __forceinline__ int silu_mul_elem_table(int g, int u, const uint16_t* __restrict__ sneg_tab) {
  const int a = g > 0 ? -g : g;                                  // -|g|
  const long long prod = (long long)a * 94549LL;
  const int key = (int)(prod >> 22) + (kSnegEntries - 1);        // prod >> 22 >= -2^26: fits
  const unsigned sneg = key < 0 ? 0u : (unsigned)sneg_tab[key];
  const int sig = (int)(g > 0 ? 65536u - sneg : sneg);
  const long long gs = (long long)g * (long long)sig;
  const int t = (int)__funnelshift_r((unsigned)gs, (unsigned)(gs >> 32), 16);
  const long long tu = (long long)t * (long long)u;
  const int hi = (int)(tu >> 32);
  const int res = (int)__funnelshift_r((unsigned)tu, (unsigned)hi, 16);
  return (hi >> 15) == (res >> 31) ? res : (hi < 0 ? (int)(-2147483647 - 1) : 2147483647);
}

// The same element when |g| < 2^23 and |u| < 2^24 (the caller has checked): no product can saturate (|t| <= |g|, so
// |t * u| < 2^47).  With a = -|g| and s the table's sigmoid term of a, (g * sig) >> 16 is (a * s) >> 16 for g <= 0
// and, for g > 0, (g * 2^16 - g * s) >> 16 = g + ((a * s) >> 16) exactly (the first term is a multiple of 2^16):
// one form for both signs.  The table's first entry (key -19456, reached from a = kSnegFirstA) is 0 like everything
// below it, so a is clamped there instead of the key.
constexpr int kSnegFirstA = -863090;     // the smallest a with (a * 94549) >> 22 >= -(kSnegEntries - 1)
static_assert(((long long)kSnegFirstA * 94549LL >> 22) == -(kSnegEntries - 1) &&
              ((long long)(kSnegFirstA - 1) * 94549LL >> 22) == -kSnegEntries, "first key of the sigmoid table");
__device__ __forceinline__ int silu_mul_elem_table_small(int g, int u, const uint16_t* __restrict__ sneg_tab) {
  const int a = max(min(g, -g), kSnegFirstA);
  const long long prod = (long long)a * 94549LL;
  const long long as = (long long)a * (long long)(int)sneg_tab[(int)(prod >> 22) + (kSnegEntries - 1)];
  const int t = (int)__funnelshift_r((unsigned)as, (unsigned)(as >> 32), 16) + max(g, 0);
  const long long tu = (long long)t * (long long)u;
  return (int)__funnelshift_r((unsigned)tu, (unsigned)(tu >> 32), 16);
}

// Stages the direct sigmoid table (kSnegEntries uint16, 38 KB) into shared memory; all threads of the CTA take part.
__device__ __forceinline__ void silu_stage_table(uint16_t* dst) {
  const int4* src = reinterpret_cast<const int4*>(g_silu_sneg);      // 19457 entries: 2432 int4 + one entry
  for (int i = threadIdx.x; i < kSnegEntries / 8; i += blockDim.x) reinterpret_cast<int4*>(dst)[i] = src[i];
  if (threadIdx.x == 0) dst[kSnegEntries - 1] = g_silu_sneg[kSnegEntries - 1];
}
constexpr size_t kSiluTableBytes = ((size_t)kSnegEntries * 2 + 15) / 16 * 16;

}  // namespace b200
