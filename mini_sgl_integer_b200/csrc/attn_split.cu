// Decode / extend attention over the int8 paged pool as a chain of small grid-wide kernels that
// meet in a caller-provided workspace instead of inside thread-block clusters.
//
// The softmax is exact (LUT exponential with truncation), so a slice of keys cannot be finished
// before the row maximum and the sum of exponentials over ALL keys are known.  Here every
// 256-key slice of every (row, KV head) is an independent CTA in each pass:
//
//   init     row maxima, sums, reference V scales and output accumulators of the workspace
//   scores   K pages -> integer MMA -> Q15.16 scores to the workspace, atomicMax of the row maxima,
//            atomicMin of the reference V scale
//   expsum   scores -> exponentials -> atomicAdd of the row sums            (reads 4 B per key, head)
//   pv       scores -> probabilities -> byte limbs -> integer MMA with the V pages -> atomicAdd of the
//            int32 partial outputs (integer addition is exact in any order)
//   final    requantise the outputs (and quantise the 128-wide rows for the int8 output)
//
// K and V are read once; the scores cost 4 B written and 8 B read per (key, head) on top, about 18 %
// of the KV bytes for four query heads per KV head.  All CTAs are small and alike, so the grid
// balances itself and many CTAs share an SM.
#include <mutex>

#include "attn_common.cuh"
#include "luts.cuh"

namespace b200 {

constexpr int kSliceKeys = 256;
constexpr int kSlicePages = kSliceKeys / kPage;   // 16
constexpr int kSlicePairs = kSlicePages / 2;      // 8
constexpr int kSplitWarps = 4;
constexpr int kSplitThreads = kSplitWarps * 32;
constexpr int kNegInf = (int)(-2147483647 - 1);

struct SplitParams {
  const int8_t* q;
  const int32_t* q_mul;
  const int32_t* q_shift;
  const int8_t* k_codes;
  const int8_t* v_codes;
  const int32_t* meta;
  const int32_t* page_table;
  int64_t table_pitch;
  const int32_t* kv_lens;
  const int32_t* row_seq;    // nullable
  const int32_t* row_limit;  // nullable
  int32_t* out_q15;
  int8_t* out_codes;
  int32_t* out_absmax;
  int q_heads, kv_heads;
  int64_t num_pages;
  int max_kv_len;
  int rows;
  // workspace
  int32_t* ws_scores;                 // [rows][q_heads][ctx_pad]
  int ctx_pad;
  int32_t* ws_rowmax;                 // [rows][q_heads]
  unsigned long long* ws_rowsum;      // [rows][q_heads]
  unsigned long long* ws_vref;        // [rows][kv_heads]
  int32_t* ws_acc;                    // [rows][q_heads][128]
};

__device__ __forceinline__ void row_lengths(const SplitParams& p, int b, int* seq, int* L, int* L_all) {
  *seq = p.row_seq ? p.row_seq[b] : b;
  *L_all = max(0, min(p.kv_lens[*seq], p.max_kv_len));
  *L = p.row_limit ? max(0, min(p.row_limit[b], *L_all)) : *L_all;
}

__global__ void split_init_kernel(const SplitParams p) {
  const int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  const int64_t nrow = (int64_t)p.rows * p.q_heads;
  if (i < nrow) { p.ws_rowmax[i] = kNegInf; p.ws_rowsum[i] = 0ull; }
  if (i < (int64_t)p.rows * p.kv_heads) p.ws_vref[i] = ~0ull;
  if (i < nrow * (kD / 4)) reinterpret_cast<int4*>(p.ws_acc)[i] = make_int4(0, 0, 0, 0);
}

// ---------------------------------------------------------------------------- scores
template <int G>
__global__ void __launch_bounds__(kSplitThreads, 6)
split_scores_kernel(const SplitParams p) {
  const int sl = blockIdx.x, b = blockIdx.y, kh = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int fr = lane >> 2, fc = lane & 3;
  int seq, L, L_all;
  row_lengths(p, b, &seq, &L, &L_all);
  const int key0 = sl * kSliceKeys;
  if (key0 >= L && !(sl == 0 && L_all > L)) return;
  const int my_keys = max(0, min(L - key0, kSliceKeys));
  const int my_pages = (my_keys + kPage - 1) / kPage;
  const int n_pairs = (my_pages + 1) >> 1;

  __shared__ __align__(128) unsigned char ring[kSplitWarps * 2 * 4096];   // two page pairs per warp
  __shared__ __align__(16) int32_t meta_s[kSlicePages * kMetaWords];
  __shared__ int pages[kSlicePages];

  if (tid < my_pages) {
    int64_t pid = p.page_table[(int64_t)seq * p.table_pitch + (key0 >> 4) + tid];
    pid = pid < 0 ? 0 : (pid >= p.num_pages ? p.num_pages - 1 : pid);
    pages[tid] = (int)pid;
  }
  unsigned qw[8];
  {
    uint4 qa = make_uint4(0, 0, 0, 0), qb = make_uint4(0, 0, 0, 0);
    if (fr < G) {
      const uint4* qp = reinterpret_cast<const uint4*>(p.q + ((int64_t)b * p.q_heads + kh * G + fr) * kD + fc * 32);
      qa = __ldg(qp);
      qb = __ldg(qp + 1);
    }
    qw[0] = qa.x; qw[1] = qa.y; qw[2] = qa.z; qw[3] = qa.w;
    qw[4] = qb.x; qw[5] = qb.y; qw[6] = qb.z; qw[7] = qb.w;
  }
  __syncthreads();
  {
    const unsigned meta_base = (unsigned)__cvta_generic_to_shared(meta_s);
    for (int i = tid; i < my_pages * 10; i += kSplitThreads) {
      const int pg = i / 10, c16 = i - pg * 10;
      cp_async16(meta_base + pg * kMetaBytes + c16 * 16,
                 reinterpret_cast<const unsigned char*>(p.meta + ((int64_t)pages[pg] * p.kv_heads + kh) * kMetaWords) + c16 * 16);
    }
  }
  // both page pairs of this warp (pairs warp and warp + 4) are requested at once
  const unsigned ring_base = (unsigned)__cvta_generic_to_shared(ring) + warp * 8192;
  const int64_t head_off = (int64_t)kh * (kPage * kD) + (lane << 4);
  const int64_t page_stride = (int64_t)p.kv_heads * (kPage * kD);
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const int pp = warp + j * kSplitWarps;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      if (2 * pp + h < my_pages) {
        const unsigned char* src = reinterpret_cast<const unsigned char*>(p.k_codes) + pages[2 * pp + h] * page_stride + head_off;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int ch = lane + 32 * i;
          cp_async16(ring_base + j * 4096 + h * 2048 + (((ch >> 3) << 7) | (((ch & 7) ^ ((ch >> 3) & 1)) << 4)), src + i * 512);
        }
      }
    }
  }
  cp_async_commit();
  cp_async_wait<0>();
  __syncthreads();

  constexpr bool kWide = G > 4;
  const int hp = kWide ? fc : (fc & 1);
  const int krow = kWide ? fr : fr + 8 * (fc >> 1);
  const bool hv0 = 2 * hp < G, hv1 = 2 * hp + 1 < G;
  const int64_t hrow = (int64_t)b * p.q_heads + kh * G;
  const int qm0 = hv0 ? __ldg(p.q_mul + hrow + 2 * hp) : 0, qm1 = hv1 ? __ldg(p.q_mul + hrow + 2 * hp + 1) : 0;
  const int qs0 = hv0 ? __ldg(p.q_shift + hrow + 2 * hp) - 48 : 0, qs1 = hv1 ? __ldg(p.q_shift + hrow + 2 * hp + 1) - 48 : 0;
  int32_t* sc0 = p.ws_scores + (hrow + 2 * hp) * p.ctx_pad + key0;
  int32_t* sc1 = sc0 + p.ctx_pad;
  int lmax0 = kNegInf, lmax1 = kNegInf;
  int best_s = 0x7fffffff;
  unsigned best_m = 0;
  const bool vref_lane = kWide ? (fc == 0) : (hp == 0);
  const int o0 = ((2 * fc) ^ (fr & 1)) << 4, o1 = ((2 * fc + 1) ^ (fr & 1)) << 4;
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const int pp = warp + j * kSplitWarps;
    if (pp >= n_pairs) break;   // warp-uniform
    const unsigned char* slot = ring + warp * 8192 + j * 4096 + fr * 128;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int pg = 2 * pp + h;
      int c[4] = {0, 0, 0, 0};
      if (pg < my_pages) {
        const unsigned char* r0 = slot + h * 2048;
        const uint4 k00 = *reinterpret_cast<const uint4*>(r0 + o0);
        const uint4 k01 = *reinterpret_cast<const uint4*>(r0 + o1);
        const uint4 k10 = *reinterpret_cast<const uint4*>(r0 + 1024 + o0);
        const uint4 k11 = *reinterpret_cast<const uint4*>(r0 + 1024 + o1);
        mma_s8s8(c, k00.x, k10.x, k00.y, k10.y, qw[0], qw[1]);
        mma_s8s8(c, k00.z, k10.z, k00.w, k10.w, qw[2], qw[3]);
        mma_s8s8(c, k01.x, k11.x, k01.y, k11.y, qw[4], qw[5]);
        mma_s8s8(c, k01.z, k11.z, k01.w, k11.w, qw[6], qw[7]);
      }
      // c[0]: (key fr, head 2fc)  [1]: (fr, 2fc+1)  [2]: (fr + 8, 2fc)  [3]: (fr + 8, 2fc+1)
      const int32_t* mt = meta_s + pg * kMetaWords;
#pragma unroll
      for (int kk = 0; kk < (kWide ? 2 : 1); ++kk) {
        int d0, d1, kr;
        if (kWide) {
          d0 = c[2 * kk]; d1 = c[2 * kk + 1]; kr = krow + 8 * kk;
        } else {   // lanes fc >= 2 adopt key row fr + 8 of the lane two to the left (heads 2hp, 2hp+1)
          const int t2 = __shfl_xor_sync(FULL_MASK, c[2], 2);
          const int t3 = __shfl_xor_sync(FULL_MASK, c[3], 2);
          d0 = fc < 2 ? c[0] : t2; d1 = fc < 2 ? c[1] : t3; kr = krow;
        }
        const int kl = pg * 16 + kr;
        if (kl < my_keys) {
          const int km = mt[kr];
          const int ks = reinterpret_cast<const int8_t*>(mt + 32)[kr];
          if (hv0) { const int s0 = mul_shift_sat32(d0, __mulhi(qm0, km), qs0 + ks); sc0[kl] = s0; lmax0 = max(lmax0, s0); }
          if (hv1) { const int s1 = mul_shift_sat32(d1, __mulhi(qm1, km), qs1 + ks); sc1[kl] = s1; lmax1 = max(lmax1, s1); }
          if (vref_lane) {
            const unsigned vm = (unsigned)mt[16 + kr];
            const int vs = reinterpret_cast<const int8_t*>(mt + 36)[kr];
            if (vs < best_s || (vs == best_s && vm > best_m)) { best_s = vs; best_m = vm; }
          }
        }
      }
    }
  }
#pragma unroll
  for (int o = (kWide ? 4 : 2); o < 32; o <<= 1) {
    lmax0 = max(lmax0, __shfl_xor_sync(FULL_MASK, lmax0, o));
    lmax1 = max(lmax1, __shfl_xor_sync(FULL_MASK, lmax1, o));
  }
  if (lane < (kWide ? 4 : 2)) {
    if (hv0 && lmax0 != kNegInf) atomicMax(p.ws_rowmax + hrow + 2 * hp, lmax0);
    if (hv1 && lmax1 != kNegInf) atomicMax(p.ws_rowmax + hrow + 2 * hp + 1, lmax1);
  }
  unsigned long long lvref = best_s == 0x7fffffff
                                 ? ~0ull
                                 : (((unsigned long long)(unsigned)(best_s + 128) << 32) | (unsigned long long)(0xFFFFFFFFu - best_m));
  if (sl == 0 && L_all > L) {   // extend rows: keys behind the causal limit still count for the V reference scale
    for (int key = L + tid; key < L_all; key += kSplitThreads) {
      int64_t pid = p.page_table[(int64_t)seq * p.table_pitch + (key >> 4)];
      pid = pid < 0 ? 0 : (pid >= p.num_pages ? p.num_pages - 1 : pid);
      const int32_t* mt = p.meta + (pid * p.kv_heads + kh) * kMetaWords;
      const unsigned vm = (unsigned)__ldg(mt + 16 + (key & 15));
      const int vs = reinterpret_cast<const int8_t*>(mt + 36)[key & 15];
      const unsigned long long vkey = ((unsigned long long)(unsigned)(vs + 128) << 32) | (unsigned long long)(0xFFFFFFFFu - vm);
      lvref = vkey < lvref ? vkey : lvref;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const unsigned long long other = __shfl_xor_sync(FULL_MASK, lvref, o);
    lvref = other < lvref ? other : lvref;
  }
  if (lane == 0 && lvref != ~0ull) atomicMin(p.ws_vref + (int64_t)b * p.kv_heads + kh, lvref);
}

__device__ __forceinline__ int exp_q16(int score, int row_max) {
  const int x = max(sub_sat(score, row_max), -(1 << 30));                 // <= 0
  const long long prod = (long long)x * 94548LL;                          // y = prod >> 16
  return __ldg(&g_exp2_attn_lut[((unsigned)prod) >> 22]) >> min(31, 13 - (int)(prod >> 32));
}

// ---------------------------------------------------------------------------- sums of exponentials
template <int G>
__global__ void __launch_bounds__(kSplitThreads)
split_expsum_kernel(const SplitParams p) {
  const int sl = blockIdx.x, b = blockIdx.y, kh = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31;
  int seq, L, L_all;
  row_lengths(p, b, &seq, &L, &L_all);
  const int key0 = sl * kSliceKeys;
  if (key0 >= L) return;
  const int my_keys = min(L - key0, kSliceKeys);
  const int64_t hrow = (int64_t)b * p.q_heads + kh * G;
  int lsum[G];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    const int gm = p.ws_rowmax[hrow + g];
    const int32_t* sc = p.ws_scores + (hrow + g) * p.ctx_pad + key0;
    int s = 0;
    for (int kl = tid; kl < my_keys; kl += kSplitThreads) s += exp_q16(sc[kl], gm);   // <= 2 keys x 2^16
    lsum[g] = s;
  }
#pragma unroll
  for (int g = 0; g < G; ++g) {
    const long long s = warp_sum64((long long)lsum[g]);
    if (lane == 0 && s != 0) atomicAdd(p.ws_rowsum + hrow + g, (unsigned long long)s);
  }
}

// ---------------------------------------------------------------------------- PV
template <int G>
__global__ void __launch_bounds__(kSplitThreads, 6)
split_pv_kernel(const SplitParams p) {
  const int sl = blockIdx.x, b = blockIdx.y, kh = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int fr = lane >> 2, fc = lane & 3;
  int seq, L, L_all;
  row_lengths(p, b, &seq, &L, &L_all);
  const int key0 = sl * kSliceKeys;
  if (key0 >= L) return;
  const int my_keys = min(L - key0, kSliceKeys);
  const int my_pages = (my_keys + kPage - 1) / kPage;
  const int n_pairs = (my_pages + 1) >> 1;

  __shared__ __align__(128) unsigned char ring[kSplitWarps * kSlicePairs * 1024];   // warp w: quarter w of every page
  __shared__ __align__(16) uint8_t p_hi[G][kSliceKeys];
  __shared__ __align__(16) uint8_t p_lo[G][kSliceKeys];
  __shared__ int pages[kSlicePages];
  __shared__ unsigned g_inv[G];
  __shared__ int g_max[G];

  if (tid < my_pages) {
    int64_t pid = p.page_table[(int64_t)seq * p.table_pitch + (key0 >> 4) + tid];
    pid = pid < 0 ? 0 : (pid >= p.num_pages ? p.num_pages - 1 : pid);
    pages[tid] = (int)pid;
  }
  const int64_t hrow = (int64_t)b * p.q_heads + kh * G;
  if (tid < G) {
    unsigned long long tot = p.ws_rowsum[hrow + tid];
    if (tot < 1ull) tot = 1ull;
    g_inv[tid] = (unsigned)(2147483647ull / tot);
    g_max[tid] = p.ws_rowmax[hrow + tid];
  }
  __syncthreads();
  // the warp's quarter of every V page of the slice: everything is requested at once
  {
    const unsigned base = (unsigned)__cvta_generic_to_shared(ring) + warp * (kSlicePairs * 1024) + (lane << 4);
    const int64_t head_off = (int64_t)kh * (kPage * kD) + warp * 512 + (lane << 4);
    const int64_t page_stride = (int64_t)p.kv_heads * (kPage * kD);
    for (int pg = 0; pg < my_pages; ++pg)
      cp_async16(base + pg * 512, reinterpret_cast<const unsigned char*>(p.v_codes) + pages[pg] * page_stride + head_off);
    cp_async_commit();
  }
  // probabilities (Q0.15) folded with the relative V scale, as two byte limbs; one key per thread.
  // The key holding the row maximum contributes e = 2^16, so the total is >= 2^16 and inv <= 32767:
  // e * inv < 2^31 and p * rel < 2^31, 32-bit arithmetic is exact here.
  {
    const unsigned long long vref = p.ws_vref[(int64_t)b * p.kv_heads + kh];
    const int v_shift_ref = (int)(vref >> 32) - 128;
    const unsigned v_mul_ref = 0xFFFFFFFFu - (unsigned)(vref & 0xFFFFFFFFull);
    for (int kl = tid; kl < n_pairs * 32; kl += kSplitThreads) {
      unsigned r = 0;
      const bool valid = kl < my_keys;
      if (valid) {
        const int32_t* mt = p.meta + ((int64_t)pages[kl >> 4] * p.kv_heads + kh) * kMetaWords;
        r = rel_scale_q15((unsigned)__ldg(mt + 16 + (kl & 15)), v_mul_ref,
                          (int)reinterpret_cast<const int8_t*>(mt + 36)[kl & 15] - v_shift_ref);
      }
#pragma unroll
      for (int g = 0; g < G; ++g) {
        unsigned w = 0;
        if (valid) {
          const unsigned e = (unsigned)exp_q16(p.ws_scores[(hrow + g) * p.ctx_pad + key0 + kl], g_max[g]);
          w = (((e * g_inv[g]) >> 16) * r + 16384u) >> 15;
        }
        p_hi[g][kl] = (uint8_t)(w >> 8);
        p_lo[g][kl] = (uint8_t)(w & 0xff);
      }
    }
  }
  cp_async_wait<0>();
  __syncthreads();

  int acc_hi[2][4], acc_lo[2][4];
#pragma unroll
  for (int m = 0; m < 2; ++m)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc_hi[m][j] = acc_lo[m][j] = 0;
  const unsigned char* slot = ring + warp * (kSlicePairs * 1024) + lane * 16;
  for (int pp = 0; pp < n_pairs; ++pp) {
    const bool has_b = 2 * pp + 1 < my_pages;
    const uint4 va = *reinterpret_cast<const uint4*>(slot + pp * 1024);
    const uint4 vb = has_b ? *reinterpret_cast<const uint4*>(slot + pp * 1024 + 512) : make_uint4(0, 0, 0, 0);
    unsigned bh0 = 0, bh1 = 0, bl0 = 0, bl1 = 0;   // W^T: head fr, tokens 4 fc .. of page A / B
    if (fr < G) {
      bh0 = *reinterpret_cast<const unsigned*>(&p_hi[fr][pp * 32 + fc * 4]);
      bh1 = *reinterpret_cast<const unsigned*>(&p_hi[fr][pp * 32 + 16 + fc * 4]);
      bl0 = *reinterpret_cast<const unsigned*>(&p_lo[fr][pp * 32 + fc * 4]);
      bl1 = *reinterpret_cast<const unsigned*>(&p_lo[fr][pp * 32 + 16 + fc * 4]);
    }
    mma_s8u8(acc_hi[0], va.x, va.y, vb.x, vb.y, bh0, bh1);
    mma_s8u8(acc_lo[0], va.x, va.y, vb.x, vb.y, bl0, bl1);
    mma_s8u8(acc_hi[1], va.z, va.w, vb.z, vb.w, bh0, bh1);
    mma_s8u8(acc_lo[1], va.z, va.w, vb.z, vb.w, bl0, bl1);
  }
  // C tile m: [0] (d = 32 warp + 16 m + fr, head 2fc)  [1] (.., 2fc+1)  [2] (d + 8, 2fc)  [3] (d + 8, 2fc+1)
#pragma unroll
  for (int m = 0; m < 2; ++m)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int head = 2 * fc + (j & 1);
      const int d = 32 * warp + 16 * m + fr + 8 * (j >> 1);
      const int v = acc_hi[m][j] * 256 + acc_lo[m][j];
      if (head < G && v != 0) atomicAdd(p.ws_acc + (hrow + head) * kD + d, v);
    }
}

// ---------------------------------------------------------------------------- final
__global__ void __launch_bounds__(kD)
split_final_kernel(const SplitParams p) {
  __shared__ int red_s[33];
  const int64_t row = blockIdx.x;             // (b, head)
  const int b = (int)(row / p.q_heads), h = (int)(row - (int64_t)b * p.q_heads);
  const int G = p.q_heads / p.kv_heads;
  const int d = threadIdx.x;
  int seq, L, L_all;
  row_lengths(p, b, &seq, &L, &L_all);
  const unsigned long long vref = p.ws_vref[(int64_t)b * p.kv_heads + h / G];
  const int v_shift_ref = (int)(vref >> 32) - 128;
  const int v_mul_ref = (int)(0xFFFFFFFFu - (unsigned)(vref & 0xFFFFFFFFull));
  const int o = L > 0 ? mul_shift_sat32_wide((long long)p.ws_acc[row * kD + d], v_mul_ref, v_shift_ref - 1) : 0;
  if (p.out_q15) p.out_q15[row * kD + d] = o;
  if (p.out_codes) {
    const int m = max(1, block_max(abs_wrap(o), red_s));
    p.out_codes[row * kD + d] = (int8_t)quant_code(o, __int2float_rn(m));
    if (d == 0) p.out_absmax[row] = m;
  }
}

static size_t split_ws_bytes(int rows, int q_heads, int kv_heads, int max_kv_len, SplitParams* p, void* ws) {
  const int ctx_pad = (int)((((int64_t)max_kv_len + 31) / 32) * 32 > 2147483616 ? 2147483616 : (((int64_t)max_kv_len + 31) / 32) * 32);
  size_t off = 0;
  auto take = [&](size_t bytes) { size_t o = off; off += (bytes + 255) & ~size_t(255); return o; };
  const size_t o_sc = take((size_t)rows * q_heads * ctx_pad * 4);
  const size_t o_max = take((size_t)rows * q_heads * 4);
  const size_t o_sum = take((size_t)rows * q_heads * 8);
  const size_t o_vref = take((size_t)rows * kv_heads * 8);
  const size_t o_acc = take((size_t)rows * q_heads * kD * 4);
  if (p) {
    unsigned char* w = reinterpret_cast<unsigned char*>(ws);
    p->ctx_pad = ctx_pad;
    p->ws_scores = reinterpret_cast<int32_t*>(w + o_sc);
    p->ws_rowmax = reinterpret_cast<int32_t*>(w + o_max);
    p->ws_rowsum = reinterpret_cast<unsigned long long*>(w + o_sum);
    p->ws_vref = reinterpret_cast<unsigned long long*>(w + o_vref);
    p->ws_acc = reinterpret_cast<int32_t*>(w + o_acc);
  }
  return off;
}

template <int G>
static int launch_split(const SplitParams& p, cudaStream_t st) {
  const int slices = (p.max_kv_len + kSliceKeys - 1) / kSliceKeys;
  const int64_t n_init = (int64_t)p.rows * p.q_heads * (kD / 4);
  split_init_kernel<<<(unsigned)((n_init + 255) / 256), 256, 0, st>>>(p);
  dim3 grid(slices, p.rows, p.kv_heads);
  split_scores_kernel<G><<<grid, kSplitThreads, 0, st>>>(p);
  split_expsum_kernel<G><<<grid, kSplitThreads, 0, st>>>(p);
  split_pv_kernel<G><<<grid, kSplitThreads, 0, st>>>(p);
  split_final_kernel<<<(unsigned)(p.rows * p.q_heads), kD, 0, st>>>(p);
  return check_launch("attn_decode_ws");
}

}  // namespace b200

using namespace b200;

extern "C" size_t b200_attn_workspace_bytes(int rows, int q_heads, int kv_heads, int max_kv_len) {
  if (rows <= 0 || q_heads <= 0 || kv_heads <= 0 || max_kv_len <= 0) return 0;
  return split_ws_bytes(rows, q_heads, kv_heads, max_kv_len, nullptr, nullptr);
}

extern "C" int b200_attn_paged_ws(const int8_t* q, const int32_t* q_mul, const int32_t* q_shift,
                                  const int8_t* k_codes, const int8_t* v_codes, const int32_t* meta,
                                  const int32_t* page_table, int64_t table_pitch, const int32_t* kv_lens,
                                  const int32_t* row_seq, const int32_t* row_limit,
                                  int32_t* out_q15, int8_t* out_codes, int32_t* out_absmax, int rows,
                                  int q_heads, int kv_heads, int64_t num_pages, int max_kv_len,
                                  void* workspace, size_t workspace_bytes, b200_stream_t s) {
  B200_REQUIRE(q && q_mul && q_shift && k_codes && v_codes && meta && page_table && kv_lens, B200_E_NULL,
               "attn_paged_ws: null pointer");
  B200_REQUIRE((row_seq == nullptr) == (row_limit == nullptr), B200_E_NULL,
               "attn_paged_ws: row_seq and row_limit must be given together");
  B200_REQUIRE((out_codes == nullptr) == (out_absmax == nullptr), B200_E_NULL,
               "attn_paged_ws: out_codes and out_absmax must be given together");
  B200_REQUIRE(out_q15 || out_codes, B200_E_NULL, "attn_paged_ws: no output requested");
  B200_REQUIRE(rows >= 0 && rows <= 65535 && q_heads > 0 && kv_heads > 0 && kv_heads <= 65535 && num_pages > 0 &&
                   max_kv_len > 0,
               B200_E_SHAPE, "attn_paged_ws: rows=%d q_heads=%d kv_heads=%d num_pages=%lld max_kv_len=%d", rows,
               q_heads, kv_heads, (long long)num_pages, max_kv_len);
  B200_REQUIRE(q_heads % kv_heads == 0, B200_E_SHAPE, "attn_paged_ws: q_heads=%d not a multiple of kv_heads=%d", q_heads, kv_heads);
  const int G = q_heads / kv_heads;
  B200_REQUIRE(G == 1 || G == 2 || G == 4 || G == 8, B200_E_UNSUPPORTED, "attn_paged_ws: group size %d (1, 2, 4 or 8)", G);
  B200_REQUIRE(table_pitch >= (max_kv_len + kPage - 1) / kPage, B200_E_SHAPE,
               "attn_paged_ws: table_pitch=%lld < pages for max_kv_len (%d)", (long long)table_pitch, (max_kv_len + kPage - 1) / kPage);
  if (rows == 0) return B200_OK;
  B200_REQUIRE(aligned16(q) && aligned16(k_codes) && aligned16(v_codes) && aligned16(meta), B200_E_ALIGN,
               "attn_paged_ws: q and pool buffers must be 16-byte aligned");
  const size_t need = split_ws_bytes(rows, q_heads, kv_heads, max_kv_len, nullptr, nullptr);
  B200_REQUIRE(workspace != nullptr, B200_E_NULL, "attn_paged_ws: workspace is null (%zu bytes needed)", need);
  B200_REQUIRE(workspace_bytes >= need && ((uintptr_t)workspace & 255u) == 0, B200_E_SHAPE,
               "attn_paged_ws: workspace of %zu bytes (256-byte aligned) needed, %zu given", need, workspace_bytes);
  SplitParams p;
  p.q = q; p.q_mul = q_mul; p.q_shift = q_shift; p.k_codes = k_codes; p.v_codes = v_codes; p.meta = meta;
  p.page_table = page_table; p.table_pitch = table_pitch; p.kv_lens = kv_lens; p.row_seq = row_seq; p.row_limit = row_limit;
  p.out_q15 = out_q15; p.out_codes = out_codes; p.out_absmax = out_absmax; p.q_heads = q_heads; p.kv_heads = kv_heads;
  p.num_pages = num_pages; p.max_kv_len = max_kv_len; p.rows = rows;
  split_ws_bytes(rows, q_heads, kv_heads, max_kv_len, &p, workspace);
  cudaStream_t st = (cudaStream_t)s;
  switch (G) {
    case 1: return launch_split<1>(p, st);
    case 2: return launch_split<2>(p, st);
    case 4: return launch_split<4>(p, st);
    default: return launch_split<8>(p, st);
  }
}

// ---------------------------------------------------------------------------------------------------
// The workspace passes over a scratch area that lives inside the library.
//
// Some callers cannot hand over a workspace: a binding that only forwards the tensors of the model (a plain
// C host, a tvm-ffi wrapper) has no allocator of its own, and a serving engine that has already given all
// free device memory to the KV pool cannot count on a later allocation to succeed.  For them the scratch is
// a fixed array in device memory that comes with the library image; nothing is allocated or freed, here or
// in any library this file calls.
// ---------------------------------------------------------------------------------------------------
namespace b200 {

constexpr size_t kStaticScratchBytes = size_t(B200_ATTN_STATIC_SCRATCH_BYTES);
static __device__ __align__(256) unsigned char g_attn_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
static void* g_attn_scratch_ptr[kMaxDevices];   // device address of g_attn_scratch, per device ordinal
static std::mutex g_attn_scratch_mutex;

// Device address of the scratch array on the current device; looked up once per device, with that device
// current (each device holds its own copy of the array at its own address).
static int static_scratch_address(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  B200_REQUIRE(e == cudaSuccess, B200_E_CUDA, "attn_paged_static: cudaGetDevice: %s", cudaGetErrorString(e));
  B200_REQUIRE(dev >= 0 && dev < kMaxDevices, B200_E_UNSUPPORTED, "attn_paged_static: device ordinal %d (at most %d devices)", dev, kMaxDevices);
  std::lock_guard<std::mutex> lock(g_attn_scratch_mutex);
  if (g_attn_scratch_ptr[dev] == nullptr) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress((void**)&ptr, g_attn_scratch);
    B200_REQUIRE(e == cudaSuccess && ptr != nullptr, B200_E_CUDA, "attn_paged_static: cudaGetSymbolAddress: %s",
                 cudaGetErrorString(e));
    g_attn_scratch_ptr[dev] = ptr;
  }
  *out = g_attn_scratch_ptr[dev];
  return B200_OK;
}

}  // namespace b200

extern "C" int b200_attn_paged_static(const int8_t* q, const int32_t* q_mul, const int32_t* q_shift,
                                      const int8_t* k_codes, const int8_t* v_codes, const int32_t* meta,
                                      const int32_t* page_table, int64_t table_pitch, const int32_t* kv_lens,
                                      const int32_t* row_seq, const int32_t* row_limit,
                                      int32_t* out_q15, int8_t* out_codes, int32_t* out_absmax, int rows,
                                      int q_heads, int kv_heads, int64_t num_pages, int max_kv_len,
                                      b200_stream_t s) {
  // The size check comes first so that an oversized call is refused before anything else happens.
  if (rows > 0 && q_heads > 0 && kv_heads > 0 && max_kv_len > 0) {
    const size_t need = split_ws_bytes(rows, q_heads, kv_heads, max_kv_len, nullptr, nullptr);
    B200_REQUIRE(need <= kStaticScratchBytes, B200_E_UNSUPPORTED,
                 "attn_paged_static: rows=%d q_heads=%d max_kv_len=%d need %zu bytes of scratch, the built-in "
                 "area holds %zu; use b200_attn_paged_ws with a workspace of your own",
                 rows, q_heads, max_kv_len, need, kStaticScratchBytes);
  }
  void* scratch = nullptr;
  const int rc = static_scratch_address(&scratch);
  if (rc != B200_OK) return rc;
  // Every pass of the chain (re)initialises what it accumulates into (row maxima, sums, reference V scales,
  // output accumulators) in its first kernel, so nothing in the area has to be zero on entry.
  return b200_attn_paged_ws(q, q_mul, q_shift, k_codes, v_codes, meta, page_table, table_pitch, kv_lens, row_seq,
                            row_limit, out_q15, out_codes, out_absmax, rows, q_heads, kv_heads, num_pages,
                            max_kv_len, scratch, kStaticScratchBytes, s);
}
