// q/k-norm + RoPE + Hadamard rotation of one 128-wide head row by one warp (shared by the stand-alone
// RoPE kernel and the fused q/k/v preparation of a decode or prefill step).
#pragma once
#include "common.cuh"
#include "luts.cuh"

namespace b200 {

__device__ __forceinline__ int fwht_scale(int y, int kq15) {
  return sat32(rsr15((long long)y * (long long)kq15));
}

// Lane l ends up with elements 2l, 2l+1 (a0, a1) and 64+2l, 64+2l+1 (b0, b1) of the row, so that the
// rotate-half pairs (j, j+64) sit in one thread.  nw: per-head RMSNorm weight (nullable).
// (lo, hi): the lane's four values of the row as loaded.
__device__ __forceinline__ void rope_row_vals(int2 lo, int2 hi, const int32_t* __restrict__ nw, int pos_in,
                                              const int32_t* __restrict__ cos_sin, int max_pos, int with_fwht, int lane,
                                              int& a0, int& a1, int& b0, int& b1) {
  if (nw != nullptr) {  // per-head fixed-point RMSNorm over the 128 values
    int m = max(max(0, abs_wrap(lo.x)), max(abs_wrap(lo.y), max(abs_wrap(hi.x), abs_wrap(hi.y))));
    m = warp_max(m);
    const NormRow nr = norm_row_from_absmax(m);
    long long S = (long long)norm_normalised_sq(lo.x, nr.p) + (long long)norm_normalised_sq(lo.y, nr.p) +
                  (long long)norm_normalised_sq(hi.x, nr.p) + (long long)norm_normalised_sq(hi.y, nr.p);
    S = warp_sum64(S);
    const int inv = norm_inv_sqrt(S, 128, g_inv_sqrt_lut);
    const int2 wl = *reinterpret_cast<const int2*>(nw + 2 * lane);
    const int2 wh = *reinterpret_cast<const int2*>(nw + 64 + 2 * lane);
    lo.x = nr.zero ? 0 : norm_apply(lo.x, inv, wl.x, nr.p);
    lo.y = nr.zero ? 0 : norm_apply(lo.y, inv, wl.y, nr.p);
    hi.x = nr.zero ? 0 : norm_apply(hi.x, inv, wh.x, nr.p);
    hi.y = nr.zero ? 0 : norm_apply(hi.y, inv, wh.y, nr.p);
  }

  int pos = pos_in;
  pos = max(0, min(max_pos - 1, pos));
  const int2 c = *reinterpret_cast<const int2*>(cos_sin + (int64_t)pos * 128 + 2 * lane);
  const int2 s = *reinterpret_cast<const int2*>(cos_sin + (int64_t)pos * 128 + 64 + 2 * lane);
  a0 = sat32(rsr15((long long)lo.x * c.x - (long long)hi.x * s.x));
  b0 = sat32(rsr15((long long)lo.x * s.x + (long long)hi.x * c.x));
  a1 = sat32(rsr15((long long)lo.y * c.y - (long long)hi.y * s.y));
  b1 = sat32(rsr15((long long)lo.y * s.y + (long long)hi.y * c.y));

  if (with_fwht) {
    // step 1: (2l, 2l+1) pairs
    int t0 = add_sat(a0, a1), t1 = sub_sat(a0, a1), u0 = add_sat(b0, b1), u1 = sub_sat(b0, b1);
    a0 = t0; a1 = t1; b0 = u0; b1 = u1;
#pragma unroll
    for (int bit = 0; bit < 5; ++bit) {  // steps 2..32: lane bits
      const bool lower = ((lane >> bit) & 1) == 0;
      int p;
      p = __shfl_xor_sync(FULL_MASK, a0, 1 << bit); a0 = lower ? add_sat(a0, p) : sub_sat(p, a0);
      p = __shfl_xor_sync(FULL_MASK, a1, 1 << bit); a1 = lower ? add_sat(a1, p) : sub_sat(p, a1);
      p = __shfl_xor_sync(FULL_MASK, b0, 1 << bit); b0 = lower ? add_sat(b0, p) : sub_sat(p, b0);
      p = __shfl_xor_sync(FULL_MASK, b1, 1 << bit); b1 = lower ? add_sat(b1, p) : sub_sat(p, b1);
    }
    // step 64: (j, j+64)
    t0 = add_sat(a0, b0); u0 = sub_sat(a0, b0); t1 = add_sat(a1, b1); u1 = sub_sat(a1, b1);
    a0 = fwht_scale(t0, 2896); b0 = fwht_scale(u0, 2896);
    a1 = fwht_scale(t1, 2896); b1 = fwht_scale(u1, 2896);
  }
}

__device__ __forceinline__ void rope_row(const int32_t* __restrict__ src, const int32_t* __restrict__ nw, int pos_in,
                                         const int32_t* __restrict__ cos_sin, int max_pos, int with_fwht, int lane,
                                         int& a0, int& a1, int& b0, int& b1) {
  const int2 lo = *reinterpret_cast<const int2*>(src + 2 * lane);
  const int2 hi = *reinterpret_cast<const int2*>(src + 64 + 2 * lane);
  rope_row_vals(lo, hi, nw, pos_in, cos_sin, max_pos, with_fwht, lane, a0, a1, b0, b1);
}

}  // namespace b200
