// Memory-bound row kernels of the integer path: Q15.16 conversion, fixed-point RMSNorm
// (+ residual add, + per-token int8 quant), SiLU*up (+ blocked FWHT, + quant), FWHT,
// q/k norm + RoPE + FWHT, per-token quant.  One row stays resident in registers between
// its reductions, so every input element is read from HBM once.
#include <cuda_bf16.h>

#include <cstdlib>

#include "common.cuh"
#include "luts.cuh"
#include "rope.cuh"
#include "silu.cuh"
#include "tp_block.cuh"

namespace b200 {

// ============================================================================ conversions
template <typename SRC>
__device__ __forceinline__ float load_as_f32(const SRC* p, int64_t i);
template <>
__device__ __forceinline__ float load_as_f32<float>(const float* p, int64_t i) { return p[i]; }
template <>
__device__ __forceinline__ float load_as_f32<uint16_t>(const uint16_t* p, int64_t i) {
  return __uint_as_float(((unsigned)p[i]) << 16);
}

// to_fixed (q15_tensor.py:17-22): round-half-even of x*65536 in fp32; the convert saturates.
template <typename SRC>
__global__ void to_fixed_kernel(const SRC* __restrict__ x, int32_t* __restrict__ out, int64_t n) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x) {
    out[i] = __float2int_rn(__fmul_rn(load_as_f32<SRC>(x, i), 65536.0f));
  }
}

// from_fixed (q15_tensor.py:25-27): fp32(x) / 65536, then the output dtype.
template <bool BF16>
__global__ void from_fixed_kernel(const int32_t* __restrict__ x, void* __restrict__ out, int64_t n) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x) {
    float f = __fdiv_rn(__int2float_rn(x[i]), 65536.0f);
    if (BF16) {
      reinterpret_cast<__nv_bfloat16*>(out)[i] = __float2bfloat16_rn(f);
    } else {
      reinterpret_cast<float*>(out)[i] = f;
    }
  }
}

static int elementwise_grid(int64_t n, int threads) {
  int64_t b = (n + threads - 1) / threads;
  const int64_t cap = 148 * 16;
  return (int)(b < cap ? (b < 1 ? 1 : b) : cap);
}

// ============================================================================ RMSNorm rows
// One CTA per row; thread t owns int4 vectors t, t+T, ... (VPT of them).
// FULL: the row is exactly blockDim.x * VPT vectors long (no bounds checks on the vector index).
// PENDING: x is null and the row comes from a linear's exact accumulators, requantised while it is loaded.
template <int VPT, bool FULL, bool PENDING = false>
__global__ void __launch_bounds__(1024)
rmsnorm_rows_kernel(const int32_t* __restrict__ x, const int32_t* __restrict__ res,
                    const int32_t* __restrict__ w, int32_t* __restrict__ res_out,
                    int32_t* __restrict__ norm_out, int8_t* __restrict__ codes,
                    float* __restrict__ scale, int32_t* __restrict__ absmax, int H, const PendingLinear pl) {
  __shared__ long long red64[33];
  __shared__ int red32[33];
  pdl_launch_dependents();
  pdl_wait();
  const int64_t row = blockIdx.x;
  const int nvec = H >> 2;
  const int4* xr = PENDING ? nullptr : reinterpret_cast<const int4*>(x + row * H);
  const int4* rr = res ? reinterpret_cast<const int4*>(res + row * H) : nullptr;
  int4* ro = res ? reinterpret_cast<int4*>(res_out + row * H) : nullptr;
  int pxm = 0, pxs = 0;
  if (PENDING) {
    absmax_to_ms_dev(__ldg(pl.x_absmax + row), &pxm, &pxs);
    pxs -= 48;
  }

  // the norm gains do not depend on the row: with few vectors per thread they are requested up front, so that their
  // latency hides behind the first reduction instead of following the second
  constexpr bool kEarlyGain = VPT <= 2;
  const int4* wr = reinterpret_cast<const int4*>(w);
  int4 gain[kEarlyGain ? VPT : 1];
  if (kEarlyGain) {
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int idx = threadIdx.x + i * blockDim.x;
      gain[i] = (FULL || idx < nvec) ? __ldg(wr + idx) : make_int4(0, 0, 0, 0);
    }
  }

  int4 v[VPT];
  int m = 0;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int idx = threadIdx.x + i * blockDim.x;
    int4 a = make_int4(0, 0, 0, 0);
    if (FULL || idx < nvec) {
      if (PENDING) a = pending_take4(pl, row, H, idx * 4, pxm, pxs);
      else a = __ldcs(xr + idx);
      if (rr) {
        int4 b = __ldcs(rr + idx);
        a.x = (int)((unsigned)a.x + (unsigned)b.x);
        a.y = (int)((unsigned)a.y + (unsigned)b.y);
        a.z = (int)((unsigned)a.z + (unsigned)b.z);
        a.w = (int)((unsigned)a.w + (unsigned)b.w);
        ro[idx] = a;
      }
    }
    v[i] = a;
    m = max(max(m, abs_wrap(a.x)), max(abs_wrap(a.y), max(abs_wrap(a.z), abs_wrap(a.w))));
  }
  m = block_max(m, red32);
  if (PENDING) {   // the accumulators have arrived (the reduction used them): leave zeros behind
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int idx = threadIdx.x + i * blockDim.x;
      if (FULL || idx < nvec) pending_clear4(pl, row, H, idx * 4);
    }
  }
  const NormRow nr = norm_row_from_absmax(m);

  long long S = 0;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    S += (long long)norm_normalised_sq(v[i].x, nr.p) + (long long)norm_normalised_sq(v[i].y, nr.p) +
         (long long)norm_normalised_sq(v[i].z, nr.p) + (long long)norm_normalised_sq(v[i].w, nr.p);
  }
  S = block_sum64(S, red64);
  const int inv = norm_inv_sqrt(S, H, g_inv_sqrt_lut);

  int4* no = norm_out ? reinterpret_cast<int4*>(norm_out + row * H) : nullptr;
  int m2 = 0;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int idx = threadIdx.x + i * blockDim.x;
    if (FULL || idx < nvec) {
      const int4 ww = kEarlyGain ? gain[i] : __ldg(wr + idx);
      int4 o;
      o.x = nr.zero ? 0 : norm_apply(v[i].x, inv, ww.x, nr.p);
      o.y = nr.zero ? 0 : norm_apply(v[i].y, inv, ww.y, nr.p);
      o.z = nr.zero ? 0 : norm_apply(v[i].z, inv, ww.z, nr.p);
      o.w = nr.zero ? 0 : norm_apply(v[i].w, inv, ww.w, nr.p);
      v[i] = o;
      if (no) no[idx] = o;
      m2 = max(max(m2, abs_wrap(o.x)), max(abs_wrap(o.y), max(abs_wrap(o.z), abs_wrap(o.w))));
    }
  }
  if (codes == nullptr) return;
  m2 = max(1, block_max(m2, red32));
  const float mf = __int2float_rn(m2);
  const float my = __frcp_rn(mf);
  unsigned* co = reinterpret_cast<unsigned*>(codes + row * H);
  if (m2 < (1 << 22)) {   // block-uniform: conversions without the conversion unit
    const float my127 = __fmul_rn(my, 127.0f);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int idx = threadIdx.x + i * blockDim.x;
      if (FULL || idx < nvec) {
        co[idx] = quant4_bytes_fast_small<true>(v[i], mf, my127);
      }
    }
  } else {
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int idx = threadIdx.x + i * blockDim.x;
      if (FULL || idx < nvec) {
        co[idx] = pack4(quant_code_fast(v[i].x, mf, my), quant_code_fast(v[i].y, mf, my),
                        quant_code_fast(v[i].z, mf, my), quant_code_fast(v[i].w, mf, my));
      }
    }
  }
  if (threadIdx.x == 0) {
    scale[row] = quant_scale(mf);
    absmax[row] = m2;
  }
}

// Per-row quant only (per_token_quant_int8_from_q15), same row residency.
template <int VPT>
__global__ void __launch_bounds__(1024)
quant_rows_kernel(const int32_t* __restrict__ x, int8_t* __restrict__ codes,
                  float* __restrict__ scale, int32_t* __restrict__ absmax, int K) {
  __shared__ int red32[33];
  pdl_launch_dependents();
  pdl_wait();
  const int64_t row = blockIdx.x;
  const int nvec = K >> 2;
  const int4* xr = reinterpret_cast<const int4*>(x + row * K);
  int4 v[VPT];
  int m = 0;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int idx = threadIdx.x + i * blockDim.x;
    int4 a = make_int4(0, 0, 0, 0);
    if (idx < nvec) a = __ldcs(xr + idx);
    v[i] = a;
    m = max(max(m, abs_wrap(a.x)), max(abs_wrap(a.y), max(abs_wrap(a.z), abs_wrap(a.w))));
  }
  m = max(1, block_max(m, red32));
  const float mf = __int2float_rn(m);
  const float my = __frcp_rn(mf);
  unsigned* co = reinterpret_cast<unsigned*>(codes + row * K);
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int idx = threadIdx.x + i * blockDim.x;
    if (idx < nvec) {
      co[idx] = pack4(quant_code_fast(v[i].x, mf, my), quant_code_fast(v[i].y, mf, my),
                      quant_code_fast(v[i].z, mf, my), quant_code_fast(v[i].w, mf, my));
    }
  }
  if (threadIdx.x == 0) {
    scale[row] = quant_scale(mf);
    absmax[row] = m;
  }
}

// Quantise rows with a GIVEN absmax (tensor-parallel row-split linears: the absmax is the maximum
// over all ranks' shards so that every rank uses the same per-token scale).
__global__ void quant_given_absmax_kernel(const int32_t* __restrict__ x, const int32_t* __restrict__ absmax,
                                          int8_t* __restrict__ codes, int64_t rows, int K) {
  const int nvec = K >> 2;
  const int64_t total = rows * nvec;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / nvec;
    const float mf = __int2float_rn(max(1, absmax[r]));
    const float my = __frcp_rn(mf);
    const int4 v = reinterpret_cast<const int4*>(x)[i];
    // the given absmax need not bound the row (it is the caller's): the reference's upper clamp is kept here
    reinterpret_cast<unsigned*>(codes)[i] = pack4(min(127, quant_code_fast(v.x, mf, my)), min(127, quant_code_fast(v.y, mf, my)),
                                                  min(127, quant_code_fast(v.z, mf, my)), min(127, quant_code_fast(v.w, mf, my)));
  }
}

// Static per-tensor quantisation (per_tensor_quant_int8_static on from_fixed(x), w8a8_int8.py:75-92, :251-254):
// code = clamp(rint((fp32(x) / 65536) / scale)), fp32 arithmetic with IEEE division.
__global__ void static_quant_kernel(const int32_t* __restrict__ x, float scale, int8_t* __restrict__ codes, int64_t n4) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n4; i += (int64_t)gridDim.x * blockDim.x) {
    const int4 v = reinterpret_cast<const int4*>(x)[i];
    int c[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float q = __fdiv_rn(__fdiv_rn(__int2float_rn(c[j]), 65536.0f), scale);
      c[j] = max(-128, min(127, __float2int_rn(q)));
    }
    reinterpret_cast<unsigned*>(codes)[i] = pack4(c[0], c[1], c[2], c[3]);
  }
}

// The GEMM's fixed-point epilogue on its own: out = sat32(mul_shift(acc, (x_mul*w_mul)>>32, x_shift+w_shift-48)).
// acc and out may be the same buffer (each element is read, then written, by one thread).
__global__ void requant_kernel(const int32_t* acc, const int32_t* __restrict__ x_mul,
                               const int32_t* __restrict__ x_shift, const int32_t* __restrict__ w_mul,
                               const int32_t* __restrict__ w_shift, int32_t* out, int64_t m, int n) {
  const int64_t total = m * n;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / n;
    const int c = (int)(i - r * n);
    const int cm = __mulhi(x_mul[r], w_mul[c]);
    const int s = x_shift[r] + (w_shift ? w_shift[c] : 31) - 48;
    out[i] = sat32(mul_shift64((long long)acc[i], (long long)cm, s));
  }
}

struct RowPlan {
  int threads, vpt;
};
static bool plan_rows(int width, RowPlan* p, int64_t rows = 1 << 30) {
  const int nvec = width >> 2;
  // Few rows (a decode batch) leave most SMs with one or two CTAs: spread each row over up to 1024 threads, which
  // shortens the dependent chain load -> reduce -> reduce -> store of a row; many rows keep 256 threads per CTA.
  if (rows <= 1024 && nvec > 256 && std::getenv("B200_ROWS_NARROW") == nullptr) {
    const int threads = nvec >= 1024 ? 1024 : ((nvec + 31) / 32) * 32;
    p->threads = threads;
    p->vpt = (nvec + threads - 1) / threads;
    if (p->vpt <= 8) return true;
  }
  if (nvec <= 256) {
    p->threads = ((nvec + 31) / 32) * 32;
    p->vpt = 1;
    return true;
  }
  int vpt = (nvec + 255) / 256;
  if (vpt <= 8) {
    p->threads = 256;
    p->vpt = vpt;
    return true;
  }
  vpt = (nvec + 1023) / 1024;
  if (vpt <= 8) {
    p->threads = 1024;
    p->vpt = vpt;
    return true;
  }
  return false;
}

#define DISPATCH_VPT(vpt, CALL)   \
  switch (vpt) {                  \
    case 1: { constexpr int V = 1; CALL; } break; \
    case 2: { constexpr int V = 2; CALL; } break; \
    case 3: { constexpr int V = 3; CALL; } break; \
    case 4: { constexpr int V = 4; CALL; } break; \
    case 5: { constexpr int V = 5; CALL; } break; \
    case 6: { constexpr int V = 6; CALL; } break; \
    case 7: { constexpr int V = 7; CALL; } break; \
    default: { constexpr int V = 8; CALL; } break; \
  }

// ============================================================================ SiLU * up (element arithmetic: silu.cuh)
// FWHT-128 of a block spread over an 8-lane group: each lane holds 16 values, index
// i = e + 4*lane8 + 32*k for val[4*k + e] (e = 0..3 inside an int4, k = 0..3).
// Stage order is the reference's (step 1, 2, 4, ... 64), with saturation at every stage.
__device__ __forceinline__ void fwht128_group(int (&val)[16], int lane8) {
#pragma unroll
  for (int k = 0; k < 4; ++k) {  // steps 1 and 2: inside each int4
    int a = val[4 * k], b = val[4 * k + 1], c = val[4 * k + 2], d = val[4 * k + 3];
    int a1 = add_sat(a, b), b1 = sub_sat(a, b), c1 = add_sat(c, d), d1 = sub_sat(c, d);
    val[4 * k] = add_sat(a1, c1);
    val[4 * k + 2] = sub_sat(a1, c1);
    val[4 * k + 1] = add_sat(b1, d1);
    val[4 * k + 3] = sub_sat(b1, d1);
  }
#pragma unroll
  for (int bit = 0; bit < 3; ++bit) {  // steps 4, 8, 16: across the 8 lanes
    const bool lower = ((lane8 >> bit) & 1) == 0;
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const int partner = __shfl_xor_sync(FULL_MASK, val[j], 1 << bit);
      val[j] = lower ? add_sat(val[j], partner) : sub_sat(partner, val[j]);
    }
  }
#pragma unroll
  for (int e = 0; e < 4; ++e) {  // steps 32 and 64: across the four int4 of a lane
    int a = val[e], b = val[4 + e], c = val[8 + e], d = val[12 + e];
    int a1 = add_sat(a, b), b1 = sub_sat(a, b), c1 = add_sat(c, d), d1 = sub_sat(c, d);
    val[e] = add_sat(a1, c1);
    val[8 + e] = sub_sat(a1, c1);
    val[4 + e] = add_sat(b1, d1);
    val[12 + e] = sub_sat(b1, d1);
  }
}

// The n = 128 scale rsr15(y * 2896).  2896 = 16 * 181, so (16a +- 2^14) >> 15 == (a +- 2^10) >> 11 with a = y * 181
// (64 bits), and for y < 0 floor((a - 2^10) / 2^11) == floor((a + 2^10) / 2^11) - 1: one wide multiply-add, one
// funnel shift (the result fits: |result| < |y|) and the sign word.
__device__ __forceinline__ int fwht_scale128(int y) {
  const long long a = (long long)y * 181LL + 1024LL;
  return (int)__funnelshift_r((unsigned)a, (unsigned)(a >> 32), 11) + (y >> 31);
}

// FWHT-128 butterflies without saturation: valid when every input satisfies |v| < 2^24, so that
// no partial sum can leave int32 (seven stages add seven bits).
__device__ __forceinline__ void fwht128_group_nosat(int (&val)[16], int lane8) {
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int a = val[4 * k], b = val[4 * k + 1], c = val[4 * k + 2], d = val[4 * k + 3];
    const int a1 = a + b, b1 = a - b, c1 = c + d, d1 = c - d;
    val[4 * k] = a1 + c1; val[4 * k + 2] = a1 - c1; val[4 * k + 1] = b1 + d1; val[4 * k + 3] = b1 - d1;
  }
#pragma unroll
  for (int bit = 0; bit < 3; ++bit) {
    const bool lower = ((lane8 >> bit) & 1) == 0;
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const int partner = __shfl_xor_sync(FULL_MASK, val[j], 1 << bit);
      val[j] = partner + (lower ? 1 : -1) * val[j];
    }
  }
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const int a = val[e], b = val[4 + e], c = val[8 + e], d = val[12 + e];
    const int a1 = a + b, b1 = a - b, c1 = c + d, d1 = c - d;
    val[e] = a1 + c1; val[8 + e] = a1 - c1; val[4 + e] = b1 + d1; val[12 + e] = b1 - d1;
  }
}

// Threads per CTA: an 8-lane group takes one 128-block per iteration; whole warps, at most kSiluMaxThreads (two
// such CTAs per SM by registers).  Rows with more blocks than groups get the widest CTA: warps that have no block
// left in the last iteration leave it, so an uneven last pass costs nothing, and more warps hide more latency
// (136 blocks: 72 groups beat the even 68; 96 blocks at batch 256: 72 + 24 beat 48 + 48).
constexpr int kSiluMaxThreads = 576;
static int silu_threads(int nblocks) {
  const int max_groups = kSiluMaxThreads / 8;
  return nblocks <= max_groups ? ((nblocks * 8 + 31) / 32) * 32 : max_groups * 8;
}

// One CTA per row at a time (the CTAs walk the rows with the grid as stride, so the tables are staged once per
// CTA).  An 8-lane group takes the 128-blocks group, group + ngroups, ...; the SiLU*up (+ rotation) results of
// the whole row are parked in shared memory until the row's absmax is known, then quantised from there: gate
// and up are read from HBM once.  TABLE: the sigmoid term comes from the 38 KB direct table instead of the exp2
// table, a shift and an exact division (used whenever the row buffer leaves room for it).
// TP: the row is this rank's slice of a token whose absmax spans all ranks' columns (the input of a row-split
// linear): between the two phases the CTA takes part in the absmax agreement over the exchange blocks (one CTA per
// row, all of them resident), quantises with the agreed value and reports it; `scale` is not written.
// ACT = false: `gate_up` already holds SiLU(gate) * up, int32 [rows, I] (the gate_up GEMM applied it in its epilogue);
// the kernel then only rotates and quantises.
template <bool FWHT, bool QUANT, bool TABLE, bool TP = false, bool ACT = true>
__global__ void __launch_bounds__(kSiluMaxThreads, 2)
silu_rows_kernel(const int32_t* __restrict__ gate_up, int32_t* __restrict__ q15_out,
                 int8_t* __restrict__ codes, float* __restrict__ scale,
                 int32_t* __restrict__ absmax, int64_t rows, int I, const TpAgree agree) {
  extern __shared__ __align__(16) int32_t rowbuf[];   // QUANT: [I] results of the row; then the table
  __shared__ int red32[2][32];
  __shared__ int agree_slot;
  int row_no = 0;
  int32_t* lut = rowbuf + (QUANT ? I : 0);
  const uint16_t* sneg_tab = reinterpret_cast<const uint16_t*>(lut);
  pdl_launch_dependents();
  if (!ACT) {
    // no table needed
  } else if (TABLE) {
    silu_stage_table(reinterpret_cast<uint16_t*>(lut));
  } else {
    for (int i = threadIdx.x; i < 1024; i += blockDim.x) lut[i] = g_exp2_silu_lut[i];
  }
  pdl_wait();                          // the tables above do not depend on the preceding kernel; gate_up does
  __syncthreads();

  const int lane8 = threadIdx.x & 7;
  const int group = threadIdx.x >> 3;
  const int ngroups = blockDim.x >> 3;
  const int nblocks = I >> 7;
  const int niter = (nblocks + ngroups - 1) / ngroups;

  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
  const int32_t* gate = gate_up + row * (ACT ? 2 : 1) * (int64_t)I;
  const int32_t* up = gate + I;
  if (row + gridDim.x < rows) {        // this CTA's next row on its way into L2 while this one is worked on
    const char* next = reinterpret_cast<const char*>(gate + (int64_t)gridDim.x * (ACT ? 2 : 1) * I);
    const int chunks = (ACT ? 2 : 1) * I / 128;                         // of 512 bytes: I is a multiple of 128
    for (int c = threadIdx.x; c < chunks; c += blockDim.x)
      asm volatile("cp.async.bulk.prefetch.L2.global [%0], 512;" ::"l"(next + (size_t)c * 512) : "memory");
  }

  int m = 0;
  unsigned small_its = 0;                        // bit `it`: the iteration's values came from the path without saturation
  for (int it = 0; it < niter; ++it) {           // the shuffles need whole warps: a warp leaves when none of its
    const int b = group + it * ngroups;            // four groups has a block left
    const bool live = b < nblocks;
    const unsigned live_mask = __ballot_sync(FULL_MASK, live);
    if (live_mask == 0) break;
    const bool all_live = live_mask == FULL_MASK;  // the usual case: no zero fill in front of the loads
    int val[16];
    auto load = [&](int k, int4& g, int4& u) {
      const int off = b * 128 + k * 32 + lane8 * 4;
      if (all_live) {
        g = __ldcs(reinterpret_cast<const int4*>(gate + off));
        u = ACT ? __ldcs(reinterpret_cast<const int4*>(up + off)) : make_int4(0, 0, 0, 0);
      } else {
        g = make_int4(0, 0, 0, 0);
        u = make_int4(0, 0, 0, 0);
        if (live) {
          g = __ldcs(reinterpret_cast<const int4*>(gate + off));
          if (ACT) u = __ldcs(reinterpret_cast<const int4*>(up + off));
        }
      }
    };
    constexpr bool kCheckFirst = ACT && TABLE;     // all 16 gate / up pairs are needed before the first element
    int4 gq[4], uq[4];
    if (kCheckFirst) {
#pragma unroll
      for (int k = 0; k < 4; ++k) load(k, gq[k], uq[k]);
    }
    // Warp-uniform: every gate and up of the warp's four blocks in [-2^20, 2^20) (16.0), so that neither the
    // products nor the butterflies can saturate (|SiLU * up| < 2^24) and the checks per element are left out.
    // v + 2^20 has a bit above bit 20 exactly when v is outside that range.
    bool small = false;
    if (kCheckFirst) {
      unsigned out = 0;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        constexpr unsigned kOff = 1u << 20;
        out |= ((unsigned)gq[k].x + kOff) | ((unsigned)uq[k].x + kOff);
        out |= ((unsigned)gq[k].y + kOff) | ((unsigned)uq[k].y + kOff);
        out |= ((unsigned)gq[k].z + kOff) | ((unsigned)uq[k].z + kOff);
        out |= ((unsigned)gq[k].w + kOff) | ((unsigned)uq[k].w + kOff);
      }
      small = !__any_sync(FULL_MASK, out >= (1u << 21));
      if (it < 32) small_its |= (small ? 1u : 0u) << it;
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      int4 g, u;
      if (kCheckFirst) {
        g = gq[k];
        u = uq[k];
      } else {
        load(k, g, u);
      }
      if (!ACT) {
        val[4 * k + 0] = g.x; val[4 * k + 1] = g.y; val[4 * k + 2] = g.z; val[4 * k + 3] = g.w;
      } else if (TABLE) {
        if (small) {
          val[4 * k + 0] = silu_mul_elem_table_small(g.x, u.x, sneg_tab);
          val[4 * k + 1] = silu_mul_elem_table_small(g.y, u.y, sneg_tab);
          val[4 * k + 2] = silu_mul_elem_table_small(g.z, u.z, sneg_tab);
          val[4 * k + 3] = silu_mul_elem_table_small(g.w, u.w, sneg_tab);
        } else {
          val[4 * k + 0] = silu_mul_elem_table(g.x, u.x, sneg_tab);
          val[4 * k + 1] = silu_mul_elem_table(g.y, u.y, sneg_tab);
          val[4 * k + 2] = silu_mul_elem_table(g.z, u.z, sneg_tab);
          val[4 * k + 3] = silu_mul_elem_table(g.w, u.w, sneg_tab);
        }
      } else {
        val[4 * k + 0] = silu_mul_elem(g.x, u.x, lut);
        val[4 * k + 1] = silu_mul_elem(g.y, u.y, lut);
        val[4 * k + 2] = silu_mul_elem(g.z, u.z, lut);
        val[4 * k + 3] = silu_mul_elem(g.w, u.w, lut);
      }
    }
    if (FWHT) {
      bool sat = false;
      if (!small) {
        int big = 0;
#pragma unroll
        for (int j = 0; j < 16; ++j) big |= val[j] ^ (val[j] >> 31);   // >= 2^24 iff some |v| >= 2^24 (-2^24 also passes)
        sat = __any_sync(FULL_MASK, big >= (1 << 24));
      }
      if (sat) {
        fwht128_group(val, lane8);                // saturating butterflies, the reference's stage order
      } else {
        fwht128_group_nosat(val, lane8);
      }
#pragma unroll
      for (int j = 0; j < 16; ++j) val[j] = fwht_scale128(val[j]);
    }
    if (live) {
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int off = b * 128 + k * 32 + lane8 * 4;
        const int4 o = make_int4(val[4 * k], val[4 * k + 1], val[4 * k + 2], val[4 * k + 3]);
        if (q15_out != nullptr) *reinterpret_cast<int4*>(q15_out + row * (int64_t)I + off) = o;
        if (QUANT) *reinterpret_cast<int4*>(rowbuf + off) = o;
      }
    }
    if (QUANT) {
      if (small) {                       // no value can be -2^31 here: the largest and the smallest give the absmax
        int hi = val[0], lo = val[0];
#pragma unroll
        for (int j = 1; j < 16; j += 2) {
          hi = __vimax3_s32(hi, val[j], val[(j + 1) & 15]);
          lo = __vimin3_s32(lo, val[j], val[(j + 1) & 15]);
        }
        m = __vimax3_s32(m, hi, -lo);
      } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) m = max(m, abs_wrap(val[j]));
      }
    }
  }
  if (!QUANT) continue;
  // One barrier per row: the reduction scratch alternates between consecutive rows (a slot is written again only
  // after the barrier of the row in between, which every reader of its old value has passed), and every thread
  // quantises exactly the values it parked itself, so warps run on into their next row while others still quantise.
  {
    int* red = red32[(row_no++) & 1];
    m = warp_max(m);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
    __syncthreads();
    m = warp_max((int)(threadIdx.x & 31) < (int)((blockDim.x + 31) >> 5) ? red[threadIdx.x & 31] : 0);
    m = max(1, m);
  }
  if (TP) m = tp_agree_cta(agree, (int)row, m, &agree_slot);
  const float mf = __int2float_rn(m);
  const float my = __frcp_rn(mf);
  unsigned* co = reinterpret_cast<unsigned*>(codes + row * (int64_t)I);
  const bool small_m = m < (1 << 22);    // the usual case (block-uniform): conversions without the conversion unit
  const float my127 = __fmul_rn(my, 127.0f);
  for (int it = 0; it < niter; ++it) {
    const int b = group + it * ngroups;
    if (b >= nblocks) break;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int i = b * 32 + k * 8 + lane8;
      const int4 v = reinterpret_cast<const int4*>(rowbuf)[i];
      if (small_m) {
        co[i] = it < 32 && ((small_its >> it) & 1u) ? quant4_bytes_fast_small<false>(v, mf, my127)
                                       : quant4_bytes_fast_small<true>(v, mf, my127);
      } else {
        co[i] = pack4(quant_code_fast(v.x, mf, my), quant_code_fast(v.y, mf, my), quant_code_fast(v.z, mf, my),
                      quant_code_fast(v.w, mf, my));
      }
    }
  }
  if (threadIdx.x == 0) {
    if (!TP) scale[row] = quant_scale(mf);
    absmax[row] = m;
  }
  if (TP) __syncthreads();             // the agreement's shared word is reused by the next row
  }
}

// SiLU*up only, any inter that is a multiple of 4 (no rotation, no quant).
__global__ void silu_simple_kernel(const int32_t* __restrict__ gate_up, int32_t* __restrict__ out,
                                   int64_t rows, int I) {
  __shared__ int32_t lut[1024];
  for (int i = threadIdx.x; i < 1024; i += blockDim.x) lut[i] = g_exp2_silu_lut[i];
  __syncthreads();
  const int nvec = I >> 2;
  const int64_t total = rows * nvec;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / nvec;
    const int c = (int)(i - r * nvec);
    const int4 g = *reinterpret_cast<const int4*>(gate_up + r * 2 * (int64_t)I + 4 * c);
    const int4 u = *reinterpret_cast<const int4*>(gate_up + r * 2 * (int64_t)I + I + 4 * c);
    *reinterpret_cast<int4*>(out + r * (int64_t)I + 4 * c) =
        make_int4(silu_mul_elem(g.x, u.x, lut), silu_mul_elem(g.y, u.y, lut),
                  silu_mul_elem(g.z, u.z, lut), silu_mul_elem(g.w, u.w, lut));
  }
}

// ============================================================================ FWHT (standalone)
// n == 128: an 8-lane group per row, four rows per warp and iteration.
__global__ void __launch_bounds__(256)
fwht128_rows_kernel(const int32_t* __restrict__ x, int32_t* __restrict__ out, int64_t rows,
                    int normalize) {
  const int lane8 = threadIdx.x & 7;
  const int sub = (threadIdx.x & 31) >> 3;
  const int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t base = warp * 4; base < rows; base += nwarps * 4) {  // warp-uniform trip count
    const int64_t r = base + sub;
    const bool live = r < rows;
    int val[16];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      int4 a = make_int4(0, 0, 0, 0);
      if (live) a = *reinterpret_cast<const int4*>(x + r * 128 + k * 32 + lane8 * 4);
      val[4 * k] = a.x; val[4 * k + 1] = a.y; val[4 * k + 2] = a.z; val[4 * k + 3] = a.w;
    }
    fwht128_group(val, lane8);
    if (normalize) {
#pragma unroll
      for (int j = 0; j < 16; ++j) val[j] = fwht_scale128(val[j]);
    }
    if (live) {
#pragma unroll
      for (int k = 0; k < 4; ++k)
        *reinterpret_cast<int4*>(out + r * 128 + k * 32 + lane8 * 4) =
            make_int4(val[4 * k], val[4 * k + 1], val[4 * k + 2], val[4 * k + 3]);
    }
  }
}

// Any power-of-two n <= 1024: one CTA of n threads per row, ping-pong in shared memory.
__global__ void fwht_generic_kernel(const int32_t* __restrict__ x, int32_t* __restrict__ out,
                                    int n, int normalize, int kq15) {
  extern __shared__ int32_t buf[];  // 2 * n
  const int64_t row = blockIdx.x;
  const int i = threadIdx.x;
  int32_t* src = buf;
  int32_t* dst = buf + n;
  src[i] = x[row * n + i];
  __syncthreads();
  for (int step = 1; step < n; step <<= 1) {
    const int a = src[i], p = src[i ^ step];
    dst[i] = (i & step) == 0 ? add_sat(a, p) : sub_sat(p, a);
    __syncthreads();
    int32_t* t = src; src = dst; dst = t;
  }
  int y = src[i];
  if (normalize) y = fwht_scale(y, kq15);
  out[row * n + i] = y;
}

// ============================================================================ q/k norm + RoPE + FWHT
// One warp per (token, head) row of 128.  Lane l holds elements 2l, 2l+1, 64+2l, 64+2l+1 so
// that the rotate-half pairs (j, j+64) sit in one thread.
__global__ void __launch_bounds__(256)
qk_rope_kernel(const int32_t* __restrict__ positions, const int32_t* __restrict__ q, int64_t q_pitch,
               const int32_t* __restrict__ k, int64_t k_pitch, const int32_t* __restrict__ cos_sin,
               int max_pos, const int32_t* __restrict__ q_norm_w, const int32_t* __restrict__ k_norm_w,
               int32_t* __restrict__ q_out, int32_t* __restrict__ k_out, int64_t tokens, int q_heads,
               int kv_heads, int with_fwht) {
  const int lane = threadIdx.x & 31;
  const int heads = q_heads + kv_heads;
  const int64_t wid = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
  if (wid >= tokens * heads) return;  // whole warps leave together
  const int64_t t = wid / heads;
  const int h = (int)(wid - t * heads);
  const bool is_q = h < q_heads;
  const int32_t* src = is_q ? q + t * q_pitch + (int64_t)h * 128
                            : k + t * k_pitch + (int64_t)(h - q_heads) * 128;
  int32_t* dst = is_q ? q_out + (t * q_heads + h) * 128 : k_out + (t * kv_heads + (h - q_heads)) * 128;
  const int32_t* nw = is_q ? q_norm_w : k_norm_w;

  int a0, a1, b0, b1;
  rope_row(src, nw, positions[t], cos_sin, max_pos, with_fwht, lane, a0, a1, b0, b1);
  *reinterpret_cast<int2*>(dst + 2 * lane) = make_int2(a0, a1);
  *reinterpret_cast<int2*>(dst + 64 + 2 * lane) = make_int2(b0, b1);
}

// ============================================================================ absmax -> (mul, shift)
__device__ __forceinline__ void absmax_to_ms(int m, int* mul, int* shift) {
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

__global__ void absmax_to_ms_kernel(const int32_t* __restrict__ m, int32_t* __restrict__ mul,
                                    int32_t* __restrict__ shift, int64_t n) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x) {
    int a, b;
    absmax_to_ms(m[i], &a, &b);
    mul[i] = a;
    shift[i] = b;
  }
}

}  // namespace b200

// ================================================================================ C ABI
using namespace b200;

extern "C" int b200_to_fixed_f32(const float* x, int32_t* out, int64_t n, b200_stream_t s) {
  B200_REQUIRE(x && out, B200_E_NULL, "to_fixed_f32: null pointer");
  B200_REQUIRE(n >= 0, B200_E_SHAPE, "to_fixed_f32: n=%lld", (long long)n);
  if (n == 0) return B200_OK;
  to_fixed_kernel<float><<<elementwise_grid(n, 256), 256, 0, (cudaStream_t)s>>>(x, out, n);
  return check_launch("to_fixed_f32");
}
extern "C" int b200_to_fixed_bf16(const uint16_t* x, int32_t* out, int64_t n, b200_stream_t s) {
  B200_REQUIRE(x && out, B200_E_NULL, "to_fixed_bf16: null pointer");
  B200_REQUIRE(n >= 0, B200_E_SHAPE, "to_fixed_bf16: n=%lld", (long long)n);
  if (n == 0) return B200_OK;
  to_fixed_kernel<uint16_t><<<elementwise_grid(n, 256), 256, 0, (cudaStream_t)s>>>(x, out, n);
  return check_launch("to_fixed_bf16");
}
extern "C" int b200_from_fixed_f32(const int32_t* x, float* out, int64_t n, b200_stream_t s) {
  B200_REQUIRE(x && out, B200_E_NULL, "from_fixed_f32: null pointer");
  B200_REQUIRE(n >= 0, B200_E_SHAPE, "from_fixed_f32: n=%lld", (long long)n);
  if (n == 0) return B200_OK;
  from_fixed_kernel<false><<<elementwise_grid(n, 256), 256, 0, (cudaStream_t)s>>>(x, out, n);
  return check_launch("from_fixed_f32");
}
extern "C" int b200_from_fixed_bf16(const int32_t* x, uint16_t* out, int64_t n, b200_stream_t s) {
  B200_REQUIRE(x && out, B200_E_NULL, "from_fixed_bf16: null pointer");
  B200_REQUIRE(n >= 0, B200_E_SHAPE, "from_fixed_bf16: n=%lld", (long long)n);
  if (n == 0) return B200_OK;
  from_fixed_kernel<true><<<elementwise_grid(n, 256), 256, 0, (cudaStream_t)s>>>(x, out, n);
  return check_launch("from_fixed_bf16");
}

extern "C" int b200_rmsnorm_q15(const int32_t* x, const int32_t* residual, const int32_t* weight,
                                int32_t* residual_out, int32_t* norm_out, int8_t* codes,
                                float* scale, int32_t* absmax, int64_t rows, int hidden,
                                b200_stream_t s) {
  B200_REQUIRE(x && weight, B200_E_NULL, "rmsnorm_q15: x or weight is null");
  B200_REQUIRE((residual == nullptr) == (residual_out == nullptr), B200_E_NULL,
               "rmsnorm_q15: residual and residual_out must be given together");
  const bool q = codes != nullptr;
  B200_REQUIRE(q == (scale != nullptr) && q == (absmax != nullptr), B200_E_NULL,
               "rmsnorm_q15: codes, scale and absmax must be given together");
  B200_REQUIRE(norm_out || q, B200_E_NULL, "rmsnorm_q15: no output requested");
  B200_REQUIRE(rows >= 0 && rows < (1ll << 31) && hidden > 0, B200_E_SHAPE,
               "rmsnorm_q15: rows=%lld hidden=%d", (long long)rows, hidden);
  B200_REQUIRE(hidden % 4 == 0, B200_E_UNSUPPORTED, "rmsnorm_q15: hidden=%d is not a multiple of 4", hidden);
  RowPlan p;
  B200_REQUIRE(plan_rows(hidden, &p, rows), B200_E_UNSUPPORTED, "rmsnorm_q15: hidden=%d exceeds 32768", hidden);
  if (rows == 0) return B200_OK;
  B200_REQUIRE(aligned16(x) && aligned16(weight) && aligned16(residual) && aligned16(residual_out) &&
                   aligned16(norm_out) && ((uintptr_t)codes & 3u) == 0,
               B200_E_ALIGN, "rmsnorm_q15: int32 buffers must be 16-byte aligned (codes 4-byte)");
  const PendingLinear none = {nullptr, nullptr, nullptr, nullptr};
  if ((hidden >> 2) == p.threads * p.vpt) {
    DISPATCH_VPT(p.vpt, (launch_pdl(rmsnorm_rows_kernel<V, true>, dim3((unsigned)rows), dim3(p.threads), 0, (cudaStream_t)s,
                                    x, residual, weight, residual_out, norm_out, codes, scale, absmax, hidden, none)));
  } else {
    DISPATCH_VPT(p.vpt, (launch_pdl(rmsnorm_rows_kernel<V, false>, dim3((unsigned)rows), dim3(p.threads), 0, (cudaStream_t)s,
                                    x, residual, weight, residual_out, norm_out, codes, scale, absmax, hidden, none)));
  }
  return check_launch("rmsnorm_q15");
}

extern "C" int b200_rmsnorm_q15_pending(int32_t* acc, const int32_t* x_absmax, const int32_t* w_mul, const int32_t* w_shift,
                                        const int32_t* residual, const int32_t* weight, int32_t* residual_out,
                                        int32_t* norm_out, int8_t* codes, float* scale, int32_t* absmax, int64_t rows,
                                        int hidden, b200_stream_t s) {
  B200_REQUIRE(acc && x_absmax && w_mul && weight, B200_E_NULL, "rmsnorm_q15_pending: acc, x_absmax, w_mul or weight is null");
  B200_REQUIRE((residual == nullptr) == (residual_out == nullptr), B200_E_NULL,
               "rmsnorm_q15_pending: residual and residual_out must be given together");
  const bool q = codes != nullptr;
  B200_REQUIRE(q == (scale != nullptr) && q == (absmax != nullptr), B200_E_NULL,
               "rmsnorm_q15_pending: codes, scale and absmax must be given together");
  B200_REQUIRE(norm_out || q, B200_E_NULL, "rmsnorm_q15_pending: no output requested");
  B200_REQUIRE(rows >= 0 && rows < (1ll << 31) && hidden > 0, B200_E_SHAPE,
               "rmsnorm_q15_pending: rows=%lld hidden=%d", (long long)rows, hidden);
  B200_REQUIRE(hidden % 4 == 0, B200_E_UNSUPPORTED, "rmsnorm_q15_pending: hidden=%d is not a multiple of 4", hidden);
  RowPlan p;
  B200_REQUIRE(plan_rows(hidden, &p, rows), B200_E_UNSUPPORTED, "rmsnorm_q15_pending: hidden=%d exceeds 32768", hidden);
  if (rows == 0) return B200_OK;
  B200_REQUIRE(aligned16(acc) && aligned16(w_mul) && aligned16(w_shift) && aligned16(weight) && aligned16(residual) &&
                   aligned16(residual_out) && aligned16(norm_out) && ((uintptr_t)codes & 3u) == 0,
               B200_E_ALIGN, "rmsnorm_q15_pending: int32 buffers must be 16-byte aligned (codes 4-byte)");
  const PendingLinear pl = {acc, x_absmax, w_mul, w_shift};
  if ((hidden >> 2) == p.threads * p.vpt) {
    DISPATCH_VPT(p.vpt, (launch_pdl(rmsnorm_rows_kernel<V, true, true>, dim3((unsigned)rows), dim3(p.threads), 0, (cudaStream_t)s,
                                    (const int32_t*)nullptr, residual, weight, residual_out, norm_out, codes, scale, absmax, hidden, pl)));
  } else {
    DISPATCH_VPT(p.vpt, (launch_pdl(rmsnorm_rows_kernel<V, false, true>, dim3((unsigned)rows), dim3(p.threads), 0, (cudaStream_t)s,
                                    (const int32_t*)nullptr, residual, weight, residual_out, norm_out, codes, scale, absmax, hidden, pl)));
  }
  return check_launch("rmsnorm_q15_pending");
}

extern "C" int b200_per_token_quant_q15(const int32_t* x, int8_t* codes, float* scale,
                                        int32_t* absmax, int64_t rows, int k, b200_stream_t s) {
  B200_REQUIRE(x && codes && scale && absmax, B200_E_NULL, "per_token_quant_q15: null pointer");
  B200_REQUIRE(rows >= 0 && rows < (1ll << 31) && k > 0, B200_E_SHAPE,
               "per_token_quant_q15: rows=%lld k=%d", (long long)rows, k);
  B200_REQUIRE(k % 4 == 0, B200_E_UNSUPPORTED, "per_token_quant_q15: k=%d is not a multiple of 4", k);
  RowPlan p;
  B200_REQUIRE(plan_rows(k, &p, rows), B200_E_UNSUPPORTED, "per_token_quant_q15: k=%d exceeds 32768", k);
  if (rows == 0) return B200_OK;
  B200_REQUIRE(aligned16(x) && ((uintptr_t)codes & 3u) == 0, B200_E_ALIGN,
               "per_token_quant_q15: x must be 16-byte aligned, codes 4-byte");
  DISPATCH_VPT(p.vpt, (launch_pdl(quant_rows_kernel<V>, dim3((unsigned)rows), dim3(p.threads), 0, (cudaStream_t)s,
                                  x, codes, scale, absmax, k)));
  return check_launch("per_token_quant_q15");
}

static int launch_silu(const int32_t* gu, int32_t* q15, int8_t* codes, float* scale, int32_t* absmax,
                       int64_t rows, int inter, bool fwht, cudaStream_t st) {
  const bool quant = codes != nullptr;
  const int nblocks = inter / 128;
  const int threads = silu_threads(nblocks);
  // the direct sigmoid table (38 KB) is used when it fits beside the row buffer with two CTAs per SM
  constexpr size_t kTableBytes = ((size_t)kSnegEntries * 2 + 15) / 16 * 16;
  const size_t row_bytes = (size_t)(quant ? inter : 0) * sizeof(int32_t);
  const bool table = row_bytes + kTableBytes <= 110 * 1024;
  const size_t smem = row_bytes + (table ? kTableBytes : 1024 * sizeof(int32_t));
  int sms = 148, dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
    sms = 148;
  const unsigned grid = (unsigned)(rows < 2 * (int64_t)sms ? rows : 2 * (int64_t)sms);
#define B200_SILU_LAUNCH(F, Q, T)                                                                          \
  do {                                                                                                     \
    cudaError_t e = cudaFuncSetAttribute(silu_rows_kernel<F, Q, T>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                         (int)smem);                                                       \
    if (e != cudaSuccess) {                                                                                \
      set_error("silu_mul_q15: cudaFuncSetAttribute: %s", cudaGetErrorString(e));                          \
      return B200_E_CUDA;                                                                                  \
    }                                                                                                      \
    launch_pdl(silu_rows_kernel<F, Q, T>, dim3(grid), dim3(threads), smem, st, gu, q15, codes, scale, absmax, rows, inter, TpAgree{});    \
  } while (0)
#define B200_SILU_LAUNCH_T(F, Q) do { if (table) B200_SILU_LAUNCH(F, Q, true); else B200_SILU_LAUNCH(F, Q, false); } while (0)
  if (fwht && quant) B200_SILU_LAUNCH_T(true, true);
  else if (fwht) B200_SILU_LAUNCH_T(true, false);
  else if (quant) B200_SILU_LAUNCH_T(false, true);
  else B200_SILU_LAUNCH_T(false, false);
#undef B200_SILU_LAUNCH_T
#undef B200_SILU_LAUNCH
  return check_launch("silu_mul_q15");
}

extern "C" int b200_silu_mul_q15(const int32_t* gate_up, int32_t* q15_out, int8_t* codes, float* scale,
                                 int32_t* absmax, int64_t rows, int inter, int fwht_block,
                                 b200_stream_t s) {
  B200_REQUIRE(gate_up, B200_E_NULL, "silu_mul_q15: gate_up is null");
  const bool q = codes != nullptr;
  B200_REQUIRE(q == (scale != nullptr) && q == (absmax != nullptr), B200_E_NULL,
               "silu_mul_q15: codes, scale and absmax must be given together");
  B200_REQUIRE(q15_out || q, B200_E_NULL, "silu_mul_q15: no output requested");
  B200_REQUIRE(rows >= 0 && rows < (1ll << 31) && inter > 0, B200_E_SHAPE,
               "silu_mul_q15: rows=%lld inter=%d", (long long)rows, inter);
  B200_REQUIRE(fwht_block == 0 || fwht_block == 128, B200_E_UNSUPPORTED,
               "silu_mul_q15: fwht_block=%d (0 or 128 supported)", fwht_block);
  B200_REQUIRE(inter % 4 == 0 && inter <= 49152, B200_E_UNSUPPORTED,
               "silu_mul_q15: inter=%d must be a multiple of 4 and at most 49152", inter);
  if (rows == 0) return B200_OK;
  B200_REQUIRE(aligned16(gate_up) && aligned16(q15_out) && ((uintptr_t)codes & 3u) == 0, B200_E_ALIGN,
               "silu_mul_q15: int32 buffers must be 16-byte aligned (codes 4-byte)");
  cudaStream_t st = (cudaStream_t)s;
  if (inter % 128 != 0) {
    B200_REQUIRE(fwht_block == 0 && !q, B200_E_UNSUPPORTED,
                 "silu_mul_q15: inter=%d must be a multiple of 128 for the rotation or the quant", inter);
    silu_simple_kernel<<<elementwise_grid(rows * (inter / 4), 256), 256, 0, st>>>(gate_up, q15_out, rows, inter);
    return check_launch("silu_mul_q15");
  }
  return launch_silu(gate_up, q15_out, codes, scale, absmax, rows, inter, fwht_block == 128, st);
}

extern "C" int b200_fwht_quant_q15(const int32_t* act, int8_t* codes, float* scale, int32_t* absmax, int64_t rows, int inter,
                                   int fwht_block, b200_stream_t s) {
  B200_REQUIRE(act && codes && scale && absmax, B200_E_NULL, "fwht_quant_q15: null pointer");
  B200_REQUIRE(rows >= 0 && rows < (1ll << 31) && inter > 0, B200_E_SHAPE, "fwht_quant_q15: rows=%lld inter=%d", (long long)rows, inter);
  B200_REQUIRE(fwht_block == 0 || fwht_block == 128, B200_E_UNSUPPORTED, "fwht_quant_q15: fwht_block=%d (0 or 128)", fwht_block);
  B200_REQUIRE(inter % 128 == 0 && inter <= 49152, B200_E_UNSUPPORTED,
               "fwht_quant_q15: inter=%d must be a multiple of 128 and at most 49152", inter);
  if (rows == 0) return B200_OK;
  B200_REQUIRE(aligned16(act) && ((uintptr_t)codes & 3u) == 0, B200_E_ALIGN, "fwht_quant_q15: act must be 16-byte aligned, codes 4-byte");
  const int threads = silu_threads(inter / 128);
  const size_t smem = (size_t)inter * sizeof(int32_t) + 16;
  int sms = 148, dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
    sms = 148;
  const unsigned grid = (unsigned)(rows < 2 * (int64_t)sms ? rows : 2 * (int64_t)sms);
  cudaStream_t st = (cudaStream_t)s;
#define B200_FQ_LAUNCH(F)                                                                                                  \
  do {                                                                                                                     \
    cudaError_t e = cudaFuncSetAttribute(silu_rows_kernel<F, true, true, false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                         (int)smem);                                                                       \
    if (e != cudaSuccess) {                                                                                                \
      set_error("fwht_quant_q15: cudaFuncSetAttribute: %s", cudaGetErrorString(e));                                        \
      return B200_E_CUDA;                                                                                                  \
    }                                                                                                                      \
    launch_pdl(silu_rows_kernel<F, true, true, false, false>, dim3(grid), dim3(threads), smem, st, act, (int32_t*)nullptr, \
               codes, scale, absmax, rows, inter, TpAgree{});                                                              \
  } while (0)
  if (fwht_block == 128) B200_FQ_LAUNCH(true); else B200_FQ_LAUNCH(false);
#undef B200_FQ_LAUNCH
  return check_launch("fwht_quant_q15");
}

extern "C" int b200_tp_silu_absmax_quant(const b200_tp_block* blk, const int32_t* gate_up, int8_t* codes, int32_t* absmax,
                                         int rows, int inter, int fwht_block, b200_stream_t s) {
  TpAgree agree;
  int rc = tp_agree_of(blk, &agree, "tp_silu_absmax_quant");
  if (rc != B200_OK) return rc;
  B200_REQUIRE(gate_up && codes && absmax, B200_E_NULL, "tp_silu_absmax_quant: null pointer");
  // one CTA per row, and every rank's CTA of a row waits for its peers' CTAs of that row: all must be resident
  B200_REQUIRE(rows > 0 && rows <= agree.m_max && rows <= 256, B200_E_SHAPE, "tp_silu_absmax_quant: rows=%d (1..%d, at most 256)",
               rows, agree.m_max);
  B200_REQUIRE(fwht_block == 0 || fwht_block == 128, B200_E_UNSUPPORTED, "tp_silu_absmax_quant: fwht_block=%d (0 or 128)", fwht_block);
  B200_REQUIRE(inter > 0 && inter % 128 == 0 && inter <= 49152, B200_E_UNSUPPORTED,
               "tp_silu_absmax_quant: inter=%d must be a multiple of 128 and at most 49152", inter);
  B200_REQUIRE(aligned16(gate_up) && ((uintptr_t)codes & 3u) == 0, B200_E_ALIGN,
               "tp_silu_absmax_quant: gate_up must be 16-byte aligned, codes 4-byte");
  const int nblocks = inter / 128;
  const int threads = silu_threads(nblocks);
  constexpr size_t kTableBytes = ((size_t)kSnegEntries * 2 + 15) / 16 * 16;
  const size_t row_bytes = (size_t)inter * sizeof(int32_t);
  const bool table = row_bytes + kTableBytes <= 110 * 1024;
  const size_t smem = row_bytes + (table ? kTableBytes : 1024 * sizeof(int32_t));
  cudaStream_t st = (cudaStream_t)s;
#define B200_SILU_TP_LAUNCH(F, T)                                                                                     \
  do {                                                                                                                \
    cudaError_t e = cudaFuncSetAttribute(silu_rows_kernel<F, true, T, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                         (int)smem);                                                                  \
    if (e != cudaSuccess) {                                                                                           \
      set_error("tp_silu_absmax_quant: cudaFuncSetAttribute: %s", cudaGetErrorString(e));                            \
      return B200_E_CUDA;                                                                                             \
    }                                                                                                                 \
    launch_pdl(silu_rows_kernel<F, true, T, true>, dim3((unsigned)rows), dim3(threads), smem, st, gate_up,            \
               (int32_t*)nullptr, codes, (float*)nullptr, absmax, (int64_t)rows, inter, agree);                       \
  } while (0)
  if (fwht_block == 128) { if (table) B200_SILU_TP_LAUNCH(true, true); else B200_SILU_TP_LAUNCH(true, false); }
  else { if (table) B200_SILU_TP_LAUNCH(false, true); else B200_SILU_TP_LAUNCH(false, false); }
#undef B200_SILU_TP_LAUNCH
  return check_launch("tp_silu_absmax_quant");
}

extern "C" int b200_fwht_q15(const int32_t* x, int32_t* out, int64_t rows, int n, int normalize,
                             b200_stream_t s) {
  B200_REQUIRE(x && out, B200_E_NULL, "fwht_q15: null pointer");
  B200_REQUIRE(rows >= 0 && rows < (1ll << 31), B200_E_SHAPE, "fwht_q15: rows=%lld", (long long)rows);
  B200_REQUIRE(n >= 2 && (n & (n - 1)) == 0, B200_E_SHAPE, "fwht_q15: n=%d is not a power of two >= 2", n);
  B200_REQUIRE(n <= 1024, B200_E_UNSUPPORTED, "fwht_q15: n=%d exceeds 1024", n);
  if (rows == 0) return B200_OK;
  cudaStream_t st = (cudaStream_t)s;
  if (n == 128 && aligned16(x) && aligned16(out)) {
    int64_t blocks = (rows + 31) / 32;
    if (blocks > 148 * 8) blocks = 148 * 8;
    fwht128_rows_kernel<<<(unsigned)blocks, 256, 0, st>>>(x, out, rows, normalize);
  } else {
    // round(2^15 / sqrt(n)), as the reference computes it in double precision
    int log2n = 0;
    while ((1 << log2n) < n) ++log2n;
    const int kq15 = (log2n % 2 == 0) ? (32768 >> (log2n / 2))
                                      : (int)(32768.0 / __builtin_sqrt((double)n) + 0.5);
    fwht_generic_kernel<<<(unsigned)rows, n, 2 * n * sizeof(int32_t), st>>>(x, out, n, normalize, kq15);
  }
  return check_launch("fwht_q15");
}

extern "C" int b200_qk_rope_q15(const int32_t* positions, const int32_t* q, int64_t q_pitch,
                                const int32_t* k, int64_t k_pitch, const int32_t* cos_sin, int max_pos,
                                const int32_t* q_norm_w, const int32_t* k_norm_w, int32_t* q_out,
                                int32_t* k_out, int64_t tokens, int q_heads, int kv_heads,
                                int with_fwht, b200_stream_t s) {
  B200_REQUIRE(positions && q && k && cos_sin && q_out && k_out, B200_E_NULL, "qk_rope_q15: null pointer");
  B200_REQUIRE(tokens >= 0 && q_heads > 0 && kv_heads > 0 && max_pos > 0, B200_E_SHAPE,
               "qk_rope_q15: tokens=%lld q_heads=%d kv_heads=%d max_pos=%d", (long long)tokens, q_heads,
               kv_heads, max_pos);
  B200_REQUIRE(q_pitch >= (int64_t)q_heads * 128 && k_pitch >= (int64_t)kv_heads * 128, B200_E_SHAPE,
               "qk_rope_q15: row pitch smaller than heads*128");
  auto a8 = [](const void* p) { return ((uintptr_t)p & 7u) == 0; };
  if (tokens == 0) return B200_OK;
  B200_REQUIRE(a8(q) && a8(k) && a8(cos_sin) && a8(q_out) && a8(k_out) && a8(q_norm_w) && a8(k_norm_w) &&
                   q_pitch % 2 == 0 && k_pitch % 2 == 0,
               B200_E_ALIGN, "qk_rope_q15: buffers must be 8-byte aligned and pitches even");
  const int64_t warps = tokens * (q_heads + kv_heads);
  const int64_t blocks = (warps + 7) / 8;
  B200_REQUIRE(blocks < (1ll << 31), B200_E_SHAPE, "qk_rope_q15: too many rows");
  qk_rope_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)s>>>(positions, q, q_pitch, k, k_pitch, cos_sin,
                                                               max_pos, q_norm_w, k_norm_w, q_out, k_out,
                                                               tokens, q_heads, kv_heads, with_fwht);
  return check_launch("qk_rope_q15");
}

extern "C" int b200_absmax_to_mul_shift(const int32_t* absmax, int32_t* mul, int32_t* shift, int64_t n,
                                        b200_stream_t s) {
  B200_REQUIRE(absmax && mul && shift, B200_E_NULL, "absmax_to_mul_shift: null pointer");
  B200_REQUIRE(n >= 0, B200_E_SHAPE, "absmax_to_mul_shift: n=%lld", (long long)n);
  if (n == 0) return B200_OK;
  absmax_to_ms_kernel<<<elementwise_grid(n, 256), 256, 0, (cudaStream_t)s>>>(absmax, mul, shift, n);
  return check_launch("absmax_to_mul_shift");
}

extern "C" int b200_quant_given_absmax_q15(const int32_t* x, const int32_t* absmax, int8_t* codes, int64_t rows,
                                           int k, b200_stream_t s) {
  B200_REQUIRE(x && absmax && codes, B200_E_NULL, "quant_given_absmax_q15: null pointer");
  B200_REQUIRE(rows >= 0 && k > 0, B200_E_SHAPE, "quant_given_absmax_q15: rows=%lld k=%d", (long long)rows, k);
  B200_REQUIRE(k % 4 == 0, B200_E_UNSUPPORTED, "quant_given_absmax_q15: k=%d is not a multiple of 4", k);
  if (rows == 0) return B200_OK;
  B200_REQUIRE(aligned16(x) && ((uintptr_t)codes & 3u) == 0, B200_E_ALIGN,
               "quant_given_absmax_q15: x must be 16-byte aligned, codes 4-byte");
  quant_given_absmax_kernel<<<elementwise_grid(rows * (k / 4), 256), 256, 0, (cudaStream_t)s>>>(x, absmax, codes, rows, k);
  return check_launch("quant_given_absmax_q15");
}

extern "C" int b200_requant_q15(const int32_t* acc, const int32_t* x_mul, const int32_t* x_shift,
                                const int32_t* w_mul, const int32_t* w_shift, int32_t* out, int64_t m, int64_t n,
                                b200_stream_t s) {
  B200_REQUIRE(acc && x_mul && x_shift && w_mul && out, B200_E_NULL, "requant_q15: null pointer");
  B200_REQUIRE(m >= 0 && n > 0 && n < (1ll << 31), B200_E_SHAPE, "requant_q15: m=%lld n=%lld", (long long)m, (long long)n);
  if (m == 0) return B200_OK;
  requant_kernel<<<elementwise_grid(m * n, 256), 256, 0, (cudaStream_t)s>>>(acc, x_mul, x_shift, w_mul, w_shift, out, m, (int)n);
  return check_launch("requant_q15");
}

extern "C" int b200_static_quant_q15(const int32_t* x, float input_scale, int8_t* codes, int64_t n, b200_stream_t s) {
  B200_REQUIRE(n >= 0 && n % 4 == 0, B200_E_SHAPE, "static_quant_q15: n=%lld must be a multiple of 4", (long long)n);
  B200_REQUIRE(input_scale > 0.0f, B200_E_SHAPE, "static_quant_q15: input_scale must be positive");
  if (n == 0) return B200_OK;
  B200_REQUIRE(x && codes, B200_E_NULL, "static_quant_q15: null pointer");
  B200_REQUIRE(aligned16(x) && ((uintptr_t)codes & 3u) == 0, B200_E_ALIGN, "static_quant_q15: x must be 16-byte and codes 4-byte aligned");
  const float scale = input_scale < 1e-10f ? 1e-10f : input_scale;
  static_quant_kernel<<<elementwise_grid(n / 4, 256), 256, 0, (cudaStream_t)s>>>(x, scale, codes, n / 4);
  return check_launch("static_quant_q15");
}
