// Shared device/host helpers for the integer-path kernels (sm_100a).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/b200int.h"

namespace b200 {

// ----------------------------------------------------------------------------- host side
void set_error(const char* fmt, ...);
int check_launch(const char* what);

#define B200_REQUIRE(cond, code, ...)   \
  do {                                  \
    if (!(cond)) {                      \
      ::b200::set_error(__VA_ARGS__);   \
      return (code);                    \
    }                                   \
  } while (0)

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Programmatic dependent launch.  Every kernel of the decode step begins with pdl_launch_dependents() (the next
// kernel of the stream may be scheduled, and run whatever it does before its own wait, while this one is still
// running) and executes pdl_wait() before it touches anything an earlier kernel produced or still reads; the wait
// returns when the preceding kernel has completed and its writes are visible.  launch_pdl() launches with the
// attribute that allows this overlap (switched off with the environment variable B200_PDL=0); a kernel launched
// without it, or after a kernel that never triggers, behaves as usual.
bool pdl_enabled();

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// The 1024-entry tables live in luts.cuh; a translation unit that needs them on the device
// includes that header (each gets its own copy, so no relocatable device code is needed).

// ----------------------------------------------------------------------------- device side
#define FULL_MASK 0xffffffffu

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ int sat32(long long v) {
  return v > 2147483647LL ? 2147483647 : (v < -2147483648LL ? (int)(-2147483647 - 1) : (int)v);
}

// |x| with two's-complement wrap (|-2^31| stays -2^31), as the reference's where(x<0,-x,x).
__device__ __forceinline__ int abs_wrap(int x) { return x < 0 ? (int)(0u - (unsigned)x) : x; }

__device__ __forceinline__ int add_sat(int a, int b) {
  int r;
  asm("add.sat.s32 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
__device__ __forceinline__ int sub_sat(int a, int b) {
  int r;
  asm("sub.sat.s32 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}

// Sign-dependent rounding shift by 15 of a 64-bit value: v>=0 ? (v+2^14)>>15 : (v-2^14)>>15.
__device__ __forceinline__ long long rsr15(long long v) {
  return (v >= 0 ? v + 16384 : v - 16384) >> 15;
}

// mul-shift of the attention / requant convention:
//   s >= 0: (x*m + (s>0 ? 2^(s-1) : 0)) >> s ;  s < 0: (x*m) << -s.   64-bit wrap-around.
__device__ __forceinline__ long long mul_shift64(long long x, long long m, int s) {
  unsigned long long prod = (unsigned long long)x * (unsigned long long)m;
  if (s >= 0) {
    if (s == 0) return (long long)prod;
    if (s >= 63) {
      long long t = (long long)(prod + (1ull << 62));
      return t < 0 ? -1 : 0;
    }
    return (long long)(prod + (1ull << (s - 1))) >> s;
  }
  int l = -s;
  return l >= 64 ? 0 : (long long)(prod << l);
}

__device__ __forceinline__ int warp_max(int v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = max(v, __shfl_xor_sync(FULL_MASK, v, o));
  return v;
}
__device__ __forceinline__ long long warp_sum64(long long v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(FULL_MASK, v, o);
  return v;
}

// Block-wide reductions; `scratch` holds >= 33 elements; every thread gets the result.
// Safe to call back to back with the same scratch.
__device__ __forceinline__ int block_max(int v, int* scratch) {
  v = warp_max(v);
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  if (nw == 1) return v;
  __syncthreads();
  if (lane == 0) scratch[wid] = v;
  __syncthreads();
  int r = (lane < nw) ? scratch[lane] : (int)(-2147483647 - 1);
  return warp_max(r);
}
__device__ __forceinline__ long long block_sum64(long long v, long long* scratch) {
  v = warp_sum64(v);
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  if (nw == 1) return v;
  __syncthreads();
  if (lane == 0) scratch[wid] = v;
  __syncthreads();
  long long r = (lane < nw) ? scratch[lane] : 0;
  return warp_sum64(r);
}

// per_token_quant_int8_from_q15's arithmetic for one element: IEEE fp32 multiply, divide,
// round-half-even, clamp.  `mf` = float(absmax).
__device__ __forceinline__ int quant_code(int x, float mf) {
  float q = __fdiv_rn(__fmul_rn(__int2float_rn(x), 127.0f), mf);
  int r = __float2int_rn(q);
  return max(-128, min(127, r));
}
// |estimate - integer| above this sends a value to the exact division: 0.5 - 2^-13.  The estimates below differ from
// the reference's rounded quotient by less than 2^-14.7 (three roundings of 2^-24 on |q| <= 128, and the quotient's own),
// so outside the band both round to the same integer; a band of 2^-10 sent a fifth of the warps there.
constexpr float kQuantTieBand = 0.4998779296875f;
// The same code with the division replaced by a multiply with the row's correctly rounded reciprocal
// (y = __frcp_rn(mf)): a * y is within a few units in the last place of the quotient (|q| <= 128: an absolute error
// below 2^-16), so after rounding to an integer it can only disagree with the division when it lies within a hair
// of a half-integer; in that band (kQuantTieBand, several times any such error) the true division is used.
// Rounding to the nearest-even integer is done by adding 1.5 * 2^23 (-128 <= q <= 127 after the lower clamp).
__device__ __forceinline__ int quant_code_fast(int x, float mf, float y) {
  const float a = __fmul_rn(__int2float_rn(x), 127.0f);
  // x = -2^31 never enters the row's absmax (its |x| wraps to a negative), so its quotient can lie far below
  // -128: the lower clamp of the reference is kept (an upper one is not needed: every other |x| <= absmax)
  const float q = fmaxf(__fmul_rn(a, y), -128.0f);
  float t = __fadd_rn(q, 12582912.0f);                        // integer part now sits in the mantissa
  if (fabsf(__fsub_rn(q, __fsub_rn(t, 12582912.0f))) > kQuantTieBand)    // close to a half-integer
    t = __fadd_rn(fmaxf(__fdiv_rn(a, mf), -128.0f), 12582912.0f);
  return __float_as_int(t) - 0x4B400000;
}
__device__ __forceinline__ float quant_scale(float mf) { return __fdiv_rn(mf, 8323072.0f); }

// quant_code_fast for four values of a row whose absmax is below 2^22: int -> float by placing the value in the
// mantissa of 1.5 * 2^23 (exact for |x| < 2^22) instead of the conversion unit, one multiply with y127 =
// __fmul_rn(127, __frcp_rn(mf)) for the estimate (one more rounding: still below 2^-15), ONE test for "some value
// within the tie band of a half-integer" and then the division for all four.  The codes are the low bytes of the mantissas
// of 1.5 * 2^23 + q.  -2^31 (not counted in the absmax) comes out of the mantissa trick as -25165824, still far below
// -128 * absmax / 127; CLAMP = false leaves out the lower clamp: only for values known not to be -2^31.
template <bool CLAMP>
__device__ __forceinline__ unsigned quant4_bytes_fast_small(int4 v, float mf, float y127) {
  constexpr float kMagic = 12582912.0f;
  const float x0 = __int_as_float(0x4B400000 + v.x) - kMagic, x1 = __int_as_float(0x4B400000 + v.y) - kMagic;
  const float x2 = __int_as_float(0x4B400000 + v.z) - kMagic, x3 = __int_as_float(0x4B400000 + v.w) - kMagic;
  float q0 = __fmul_rn(x0, y127), q1 = __fmul_rn(x1, y127), q2 = __fmul_rn(x2, y127), q3 = __fmul_rn(x3, y127);
  if (CLAMP) {
    q0 = fmaxf(q0, -128.0f); q1 = fmaxf(q1, -128.0f); q2 = fmaxf(q2, -128.0f); q3 = fmaxf(q3, -128.0f);
  }
  float t0 = __fadd_rn(q0, kMagic), t1 = __fadd_rn(q1, kMagic), t2 = __fadd_rn(q2, kMagic), t3 = __fadd_rn(q3, kMagic);
  const float d0 = __fsub_rn(q0, __fsub_rn(t0, kMagic)), d1 = __fsub_rn(q1, __fsub_rn(t1, kMagic));
  const float d2 = __fsub_rn(q2, __fsub_rn(t2, kMagic)), d3 = __fsub_rn(q3, __fsub_rn(t3, kMagic));
  if (fmaxf(fmaxf(fabsf(d0), fabsf(d1)), fmaxf(fabsf(d2), fabsf(d3))) > kQuantTieBand) {
    t0 = __fadd_rn(fmaxf(__fdiv_rn(__fmul_rn(x0, 127.0f), mf), -128.0f), kMagic);
    t1 = __fadd_rn(fmaxf(__fdiv_rn(__fmul_rn(x1, 127.0f), mf), -128.0f), kMagic);
    t2 = __fadd_rn(fmaxf(__fdiv_rn(__fmul_rn(x2, 127.0f), mf), -128.0f), kMagic);
    t3 = __fadd_rn(fmaxf(__fdiv_rn(__fmul_rn(x3, 127.0f), mf), -128.0f), kMagic);
  }
  const unsigned ab = __byte_perm(__float_as_uint(t0), __float_as_uint(t1), 0x0040);
  const unsigned cd = __byte_perm(__float_as_uint(t2), __float_as_uint(t3), 0x0040);
  return __byte_perm(ab, cd, 0x5410);
}

// Packs the LOW BYTES of four words.
__device__ __forceinline__ unsigned pack4(int a, int b, int c, int d) {
  // two byte permutes: (a,b) -> low half, (c,d) -> high half, then merge
  const unsigned ab = __byte_perm((unsigned)a, (unsigned)b, 0x0040);
  const unsigned cd = __byte_perm((unsigned)c, (unsigned)d, 0x0040);
  return __byte_perm(ab, cd, 0x5410);
}

// Fixed-point RMSNorm scalars of one row (rmsnorm_int_only_v2.py:144-218 steps 1, 4).
struct NormRow {
  int p;         // MSB index of the row's absmax (0 for a zero row)
  int zero;      // row is all zeros
};
__device__ __forceinline__ NormRow norm_row_from_absmax(int m) {
  NormRow r;
  r.zero = (m == 0);
  r.p = r.zero ? 0 : (31 - __clz(m));
  return r;
}
__device__ __forceinline__ int norm_normalised_sq(int v, int p) {
  int n = ((int)((unsigned)v << (30 - p))) >> 16;
  return (int)((unsigned)n * (unsigned)n);
}
// inverse_sqrt_q0_31 (rmsnorm_int_only_v2.py:89-117) of ms = ((S / H) >> 1) + 1.
__device__ __forceinline__ int norm_inv_sqrt(long long S, int H, const int32_t* lut) {
  int ms = (int)((S / H) >> 1) + 1;
  if (ms <= 0) return 0;
  int pos = 31 - __clz(ms);
  int even = ((pos + 1) >> 1) << 1;
  int xn = ((int)((unsigned)ms << (30 - even))) >> 21;
  xn = max(0, min(1023, xn));
  return (int)((unsigned)lut[xn] << (16 - (even >> 1)));
}
__device__ __forceinline__ int norm_apply(int v, int inv, int w, int p) {
  long long a = (long long)v * (long long)inv;
  long long b = (long long)((unsigned long long)a * (unsigned long long)(long long)w);
  return sat32(b >> (p + 18));
}

// A per-row integer absmax as a fixed-point scale: value = code * mul / 2^shift with mul in [2^30, 2^31),
// i.e. mul / 2^shift = absmax / (127 * 2^16) rounded up in the last place.
__device__ __forceinline__ void absmax_to_ms_dev(int m, int* mul, int* shift) {
  m = max(m, 1);
  const int p = 31 - __clz(m);
  int k = 37 - p;
  unsigned long long v = (((unsigned long long)m << k) + 63ull) / 127ull;
  if (v >= (1ull << 31)) {
    k -= 1;
    v = (((unsigned long long)m << k) + 63ull) / 127ull;
  }
  *mul = (int)v;
  *shift = k + 16;
}

// The fixed-point epilogue of a W8A8 linear for one exact accumulator: round-half-up shift of acc * cm by s bits,
// saturated, where cm = (x_mul * w_mul) >> 32 and s = x_shift + w_shift - 48.
__device__ __forceinline__ int requant_one(int acc, int cm, int s) {
  if (s > 0 && s < 63) return sat32(((long long)acc * (long long)cm + (1LL << (s - 1))) >> s);
  return sat32(mul_shift64((long long)acc, (long long)cm, s));
}

// A linear's output that has not been requantised yet: the exact int32 accumulators [rows, n] (split-K parts already
// added), the absmax of each token's input row and the weight's per-channel scales.  A row kernel that is handed this
// instead of Q15.16 values applies the epilogue while it loads and leaves zeros behind, so that the buffer can take
// the next GEMM's split-K parts without a clearing launch.  The zeros are stored by a separate call placed AFTER a
// reduction that consumed the loaded values: a store issued right behind the load of the same address waits for
// the load's miss (measured: the requantising kernel took 12 us instead of 4 with the store in front).
struct PendingLinear {
  int32_t* acc;
  const int32_t* x_absmax;
  const int32_t* w_mul;
  const int32_t* w_shift;     // nullable: 31 everywhere
};

__device__ __forceinline__ int2 pending_take2(const PendingLinear& pl, int64_t row, int n, int col, int xm, int xs48) {
  const int2 a = *reinterpret_cast<const int2*>(pl.acc + row * n + col);
  const int2 wm = __ldg(reinterpret_cast<const int2*>(pl.w_mul + col));
  int2 ws = make_int2(31, 31);
  if (pl.w_shift) ws = __ldg(reinterpret_cast<const int2*>(pl.w_shift + col));
  return make_int2(requant_one(a.x, __mulhi(xm, wm.x), xs48 + ws.x), requant_one(a.y, __mulhi(xm, wm.y), xs48 + ws.y));
}

__device__ __forceinline__ void pending_clear2(const PendingLinear& pl, int64_t row, int n, int col) {
  *reinterpret_cast<int2*>(pl.acc + row * n + col) = make_int2(0, 0);
}
__device__ __forceinline__ void pending_clear4(const PendingLinear& pl, int64_t row, int n, int col) {
  *reinterpret_cast<int4*>(pl.acc + row * n + col) = make_int4(0, 0, 0, 0);
}

__device__ __forceinline__ int4 pending_take4(const PendingLinear& pl, int64_t row, int n, int col, int xm, int xs48) {
  const int4 a = *reinterpret_cast<const int4*>(pl.acc + row * n + col);
  const int4 wm = __ldg(reinterpret_cast<const int4*>(pl.w_mul + col));
  int4 ws = make_int4(31, 31, 31, 31);
  if (pl.w_shift) ws = __ldg(reinterpret_cast<const int4*>(pl.w_shift + col));
  int4 r;
  r.x = requant_one(a.x, __mulhi(xm, wm.x), xs48 + ws.x);
  r.y = requant_one(a.y, __mulhi(xm, wm.y), xs48 + ws.y);
  r.z = requant_one(a.z, __mulhi(xm, wm.z), xs48 + ws.z);
  r.w = requant_one(a.w, __mulhi(xm, wm.w), xs48 + ws.w);
  return r;
}

}  // namespace b200
