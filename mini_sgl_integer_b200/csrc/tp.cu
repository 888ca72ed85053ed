// Tensor-parallel exchange steps of the row-split linears over NVLink peer memory (decode sizes).
//
// A row-split linear (o_proj, down_proj) on `size` ranks gives the bits of one GPU when the ranks
//   1. agree on every token's absmax            (one word per rank and token stored into every rank's block),
//   2. quantise their K-slice with it,
//   3. add their exact int32 partial sums       (the owner of a token row fetches them from every rank, channel 1),
//   4. requantise the sum once and hand the finished rows to everybody (channel 3).
// Steps 1 and 4 write straight into the peers' memory, step 3 reads from it; a producer kernel ends with a signal (its last CTA
// stores the channel's new epoch into every rank's flag word), the consumer kernel begins with a bounded
// wait on those flags.  No collective library call, no host synchronisation: a decode step that uses these
// kernels is an ordinary stream of launches and can be captured in a CUDA graph on every rank.
//
// Every wait gives up after a time limit (default 2 s), records the channel in a status word that the host
// can read, and lets the kernel finish on whatever the block holds: a missing peer costs a wrong result and
// an error code, never a hung GPU.
#include "luts.cuh"
#include "tp_block.cuh"

namespace b200 {

static __device__ int g_tp_status = 0;                             // 0 = fine, else channel + 1 of the first expiry
static __device__ unsigned long long g_tp_timeout_ns = 2000000000ull;

// Waits until every rank's signal number `epoch` on channel ch has arrived: threads 0 .. size-1 poll one
// source each; the caller follows with a CTA barrier and reads the peers' data past L1 (__ldcg).
__device__ __forceinline__ void tp_wait_flags(const TpView& v, int ch, int epoch) {
  if ((int)threadIdx.x < v.size) {
    const int32_t* f = v.base[v.rank] + kTpHdrWords + ch * kTpMaxRanks + threadIdx.x;
    if (tp_ld_acquire(f) - epoch < 0) {
      const unsigned long long t0 = tp_now_ns(), limit = g_tp_timeout_ns;
      while (tp_ld_acquire(f) - epoch < 0) {
        if (tp_now_ns() - t0 > limit) {
          atomicCAS(&g_tp_status, 0, ch + 1);
          break;
        }
        __nanosleep(32);
      }
    }
  }
}

// ---------------------------------------------------------------------------- steps 1 + 2: absmax agreement, quantisation
// The absmax of a token row over this rank's K-slice is max(1, max|x|) >= 1, so it doubles as its own arrival
// flag: rank r stores it with one 4-byte store into word [half][row][r] of every rank's block, and a row is
// complete when all `size` words of the row are non-zero - no fence, no separate flag.  The agreed absmax is
// their maximum; the reader clears the words.  The half alternates with a per-rank call counter (header word
// 4) advanced by the last CTA of the reading kernel.
__device__ __forceinline__ int tp_row_absmax(const int4* __restrict__ xr, int nvec, int* red32) {
  int m = 0;
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    const int4 a = xr[i];
    m = max(max(m, abs_wrap(a.x)), max(abs_wrap(a.y), max(abs_wrap(a.z), abs_wrap(a.w))));
  }
  return max(1, block_max(m, red32));
}

// The agreement itself is tp_agree_cta (tp_block.cuh); this builds its argument from a view.
__device__ __forceinline__ TpAgree tp_agree_view(const TpView& v) {
  TpAgree a;
  a.rank = v.rank; a.size = v.size; a.m_max = v.m_max;
  a.amax_off = tp_layout(v.m_max, v.n).amax;
  for (int r = 0; r < kTpMaxRanks; ++r) a.base[r] = v.base[r];
  a.status = &g_tp_status;
  a.timeout_ns = &g_tp_timeout_ns;
  return a;
}

// One CTA per token row of this rank's slice x [rows, k] (row pitch in elements): delivers the row's absmax.
__global__ void __launch_bounds__(256)
tp_absmax_put_kernel(const TpView v, const int32_t* __restrict__ x, int64_t pitch, int k) {
  pdl_launch_dependents();
  pdl_wait();          // what this kernel reads comes from the kernels before it (and from the peers, see below)
  __shared__ int red32[33];
  const TpLayout l = tp_layout(v.m_max, v.n);
  const int half = *reinterpret_cast<volatile int32_t*>(v.base[v.rank] + 4) & 1;
  const int row = blockIdx.x;
  const int m = tp_row_absmax(reinterpret_cast<const int4*>(x + (int64_t)row * pitch), k >> 2, red32);
  if ((int)threadIdx.x < v.size)
    tp_st_relaxed(v.base[threadIdx.x] + l.amax + ((int64_t)half * v.m_max + row) * kTpMaxRanks + v.rank, m);
}

// One CTA per row: waits for every rank's absmax of the row, writes the int8 codes of this rank's slice and the
// agreed absmax (for the requant).
__global__ void __launch_bounds__(256)
tp_quant_wait_kernel(const TpView v, const int32_t* __restrict__ x, int64_t pitch, int k,
                     int8_t* __restrict__ codes, int32_t* __restrict__ absmax_out) {
  pdl_launch_dependents();
  pdl_wait();          // what this kernel reads comes from the kernels before it (and from the peers, see below)
  __shared__ int agreed;
  const TpLayout l = tp_layout(v.m_max, v.n);
  int32_t* hdr = v.base[v.rank];
  const int half = *reinterpret_cast<volatile int32_t*>(hdr + 4) & 1;
  const int row = blockIdx.x;
  const int m = tp_agree_cta(tp_agree_view(v), row, 0, &agreed, false);
  if (threadIdx.x == 0) absmax_out[row] = m;
  const float mf = __int2float_rn(m), my = __frcp_rn(mf);
  const int4* xr = reinterpret_cast<const int4*>(x + (int64_t)row * pitch);
  unsigned* co = reinterpret_cast<unsigned*>(codes + (int64_t)row * k);
  for (int i = threadIdx.x; i < (k >> 2); i += blockDim.x) {
    const int4 a = xr[i];
    co[i] = pack4(quant_code_fast(a.x, mf, my), quant_code_fast(a.y, mf, my), quant_code_fast(a.z, mf, my),
                  quant_code_fast(a.w, mf, my));
  }
}

// Both in one launch: a CTA delivers its row's absmax, waits for the peers' words of the SAME row and quantises.
// A CTA depends only on the peers' CTAs of its row, which never wait before they deliver, so there is no
// grid-wide dependency; all rows' CTAs must be able to run at once (rows <= 512).
__global__ void __launch_bounds__(256)
tp_absmax_quant_kernel(const TpView v, const int32_t* __restrict__ x, int64_t pitch, int k,
                       int8_t* __restrict__ codes, int32_t* __restrict__ absmax_out) {
  pdl_launch_dependents();
  pdl_wait();          // what this kernel reads comes from the kernels before it (and from the peers, see below)
  __shared__ int red32[33];
  __shared__ int agreed;
  const TpLayout l = tp_layout(v.m_max, v.n);
  int32_t* hdr = v.base[v.rank];
  const int half = *reinterpret_cast<volatile int32_t*>(hdr + 4) & 1;
  const int row = blockIdx.x;
  const int4* xr = reinterpret_cast<const int4*>(x + (int64_t)row * pitch);
  // the row stays in registers between the two passes (up to 8 vectors per thread), the rest is read again
  constexpr int kKeep = 8;
  int4 keep[kKeep];
  const int nvec = k >> 2;
  int m = 0;
#pragma unroll
  for (int j = 0; j < kKeep; ++j) {
    const int i = threadIdx.x + j * 256;
    keep[j] = i < nvec ? xr[i] : make_int4(0, 0, 0, 0);
    m = max(max(m, abs_wrap(keep[j].x)), max(abs_wrap(keep[j].y), max(abs_wrap(keep[j].z), abs_wrap(keep[j].w))));
  }
  for (int i = threadIdx.x + kKeep * 256; i < nvec; i += 256) {
    const int4 a = xr[i];
    m = max(max(m, abs_wrap(a.x)), max(abs_wrap(a.y), max(abs_wrap(a.z), abs_wrap(a.w))));
  }
  m = max(1, block_max(m, red32));
  const int a = tp_agree_cta(tp_agree_view(v), row, m, &agreed);
  if (threadIdx.x == 0) absmax_out[row] = a;
  const float mf = __int2float_rn(a), my = __frcp_rn(mf);
  unsigned* co = reinterpret_cast<unsigned*>(codes + (int64_t)row * k);
#pragma unroll
  for (int j = 0; j < kKeep; ++j) {
    const int i = threadIdx.x + j * 256;
    if (i < nvec)
      co[i] = pack4(quant_code_fast(keep[j].x, mf, my), quant_code_fast(keep[j].y, mf, my), quant_code_fast(keep[j].z, mf, my),
                    quant_code_fast(keep[j].w, mf, my));
  }
  for (int i = threadIdx.x + kKeep * 256; i < nvec; i += 256) {
    const int4 b = xr[i];
    co[i] = pack4(quant_code_fast(b.x, mf, my), quant_code_fast(b.y, mf, my), quant_code_fast(b.z, mf, my),
                  quant_code_fast(b.w, mf, my));
  }
}

// ---------------------------------------------------------------------------- step 4: add, requantise, hand out
// The rank owns the token rows [rank * rpr, (rank + 1) * rpr), rpr = ceil(m / size).  After every rank's channel-1
// signal (sent by the GEMM kernels) the accumulators acc[half] of all ranks are complete: fetch every rank's partial
// sums of the own rows, add them, apply the fixed-point epilogue and store the finished Q15.16 row into `out` of
// EVERY rank.  Signals channel 3.
__device__ __forceinline__ int tp_requant_one(int acc, int cm, int s) {
  if (s > 0 && s < 63) return sat32(((long long)acc * (long long)cm + (1LL << (s - 1))) >> s);
  return sat32(mul_shift64((long long)acc, (long long)cm, s));
}

// DIRECT: every rank holds all ranks' partial sums of all rows and writes the finished rows to `dst` (the caller's
// tensor); otherwise the rank finishes the rows it owns, stores them into every rank's `out` and signals channel 3.
template <bool DIRECT>
__global__ void __launch_bounds__(256)
tp_requant_scatter_kernel(const TpView v, const int32_t* __restrict__ absmax, const int32_t* __restrict__ w_mul,
                          const int32_t* __restrict__ w_shift, int32_t* __restrict__ dst, int m, int n) {
  pdl_launch_dependents();
  pdl_wait();          // what this kernel reads comes from the kernels before it (and from the peers, see below)
  const TpLayout l = tp_layout(v.m_max, v.n);
  int32_t* hdr = v.base[v.rank];
  const int epoch = *reinterpret_cast<volatile int32_t*>(hdr + 1);
  const int half = (epoch - 1) & 1;
  tp_wait_flags(v, 1, epoch);
  __syncthreads();
  const int rpr = tp_rows_per_rank(m, v.size);
  const int row0 = DIRECT ? 0 : v.rank * rpr, rows = max(0, min(m, row0 + rpr) - row0);
  const int64_t acc_off = l.acc + (int64_t)half * l.acc_half;
  const int64_t out_off = l.out + (int64_t)half * l.acc_half;
  // every peer has signalled this exchange, so it has finished reading the accumulator half of the PREVIOUS one:
  // clear this rank's copy of it for the exchange after this one (all m_max rows; the grid shares the work)
  {
    int4* old = reinterpret_cast<int4*>(hdr + l.acc + (int64_t)(half ^ 1) * l.acc_half);
    const int64_t vecs = (int64_t)v.m_max * (n >> 2);        // all rows: the previous exchange may have had more than m
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < vecs; i += (int64_t)gridDim.x * blockDim.x)
      old[i] = make_int4(0, 0, 0, 0);
  }
  const int nvec = n >> 2;
  const int64_t total = (int64_t)rows * nvec;
  constexpr int kBatch = 4;                     // independent loads in flight per thread
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i0 = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i0 < total; i0 += stride * kBatch) {
    int4 a[kBatch];
#pragma unroll
    for (int j = 0; j < kBatch; ++j) {
      const int64_t i = i0 + j * stride;
      a[j] = make_int4(0, 0, 0, 0);
      if (i < total) {
        const int tl = (int)(i / nvec);
        const int c = (int)(i - (int64_t)tl * nvec) * 4;
        for (int src = 0; src < v.size; ++src) {      // every rank's partial sums of the row: 16-byte loads, NVLink for peers
          const int4 b = __ldcg(reinterpret_cast<const int4*>(v.base[src] + acc_off + (int64_t)(row0 + tl) * n + c));
          a[j].x += b.x; a[j].y += b.y; a[j].z += b.z; a[j].w += b.w;
        }
      }
    }
#pragma unroll
    for (int j = 0; j < kBatch; ++j) {
      const int64_t i = i0 + j * stride;
      if (i >= total) continue;
      const int tl = (int)(i / nvec);
      const int c = (int)(i - (int64_t)tl * nvec) * 4;
      const int t = row0 + tl;
      int xm, xs;
      absmax_to_ms_dev(__ldg(absmax + t), &xm, &xs);
      xs -= 48;
      const int4 wm = __ldg(reinterpret_cast<const int4*>(w_mul + c));
      int4 ws = make_int4(31, 31, 31, 31);
      if (w_shift) ws = __ldg(reinterpret_cast<const int4*>(w_shift + c));
      int4 r;
      r.x = tp_requant_one(a[j].x, __mulhi(xm, wm.x), xs + ws.x);
      r.y = tp_requant_one(a[j].y, __mulhi(xm, wm.y), xs + ws.y);
      r.z = tp_requant_one(a[j].z, __mulhi(xm, wm.z), xs + ws.z);
      r.w = tp_requant_one(a[j].w, __mulhi(xm, wm.w), xs + ws.w);
      if (DIRECT) {
        *reinterpret_cast<int4*>(dst + (int64_t)t * n + c) = r;
      } else {
        for (int d = 0; d < v.size; ++d) *reinterpret_cast<int4*>(v.base[d] + out_off + (int64_t)t * n + c) = r;
      }
    }
  }
  if (!DIRECT) {
    __syncthreads();
    if (threadIdx.x == 0) tp_signal_if_last(v, 3, gridDim.x, total > 0);
  }
}

// ---------------------------------------------------------------------------- step 5: collect the finished rows
// Waits for every rank's channel-3 signal and copies out[half] (all m rows) to the caller's tensor.
__global__ void __launch_bounds__(256)
tp_collect_kernel(const TpView v, int32_t* __restrict__ dst, int m, int n) {
  pdl_launch_dependents();
  pdl_wait();          // what this kernel reads comes from the kernels before it (and from the peers, see below)
  const TpLayout l = tp_layout(v.m_max, v.n);
  const int32_t* hdr = v.base[v.rank];
  const int half = (*reinterpret_cast<const volatile int32_t*>(hdr + 1) - 1) & 1;
  tp_wait_flags(v, 3, *reinterpret_cast<const volatile int32_t*>(hdr + 3));
  __syncthreads();
  const int4* src = reinterpret_cast<const int4*>(hdr + l.out + (int64_t)half * l.acc_half);
  const int64_t total = (int64_t)m * (n >> 2);
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x)
    reinterpret_cast<int4*>(dst)[i] = __ldcg(src + i);
}

// ---------------------------------------------------------------------------- steps 4 + 5 fused with the following norm
// The row-split linears of a decoder layer are each followed by (residual add +) RMSNorm + per-token quantisation,
// and the next linears only need the int8 codes and the absmax of that.  So the rank that owns a token row does it
// all: fetch the row's partial sums from every rank, requantise, add the residual (kept by the owner only: nobody
// else needs that row's residual again as long as ownership does not move), normalise, quantise, and store the
// CODES (a quarter of the Q15.16 bytes) and the absmax into every rank's `out` half.  Signals channel 3.
// One CTA per owned row; the arithmetic is that of splitk_epilogue_kernel followed by rmsnorm_rows_kernel.
__host__ __device__ inline int tp_owner_rows(int m, int size) { return (m + size - 1) / size; }
__host__ __device__ inline int64_t tp_codes_absmax_off(int m_max, int64_t n) { return tp_align64((int64_t)m_max * n / 4); }

template <int VPT>
__global__ void __launch_bounds__(1024)
tp_owner_norm_kernel(const TpView v, const int32_t* __restrict__ x_absmax, const int32_t* __restrict__ w_mul,
                     const int32_t* __restrict__ w_shift, int32_t* __restrict__ residual, const int32_t* __restrict__ norm_w,
                     int m, int n) {
  pdl_launch_dependents();
  pdl_wait();          // what this kernel reads comes from the kernels before it (and from the peers, see below)
  __shared__ long long red64[33];
  __shared__ int red32[33];
  const TpLayout l = tp_layout(v.m_max, v.n);
  int32_t* hdr = v.base[v.rank];
  const int epoch = *reinterpret_cast<volatile int32_t*>(hdr + 1);
  const int half = (epoch - 1) & 1;
  tp_wait_flags(v, 1, epoch);
  __syncthreads();
  const int rpr = tp_owner_rows(m, v.size);
  const int row0 = v.rank * rpr, rows = max(0, min(m, row0 + rpr) - row0);
  const int64_t acc_off = l.acc + (int64_t)half * l.acc_half;
  const int64_t out_off = l.out + (int64_t)half * l.acc_half;
  {   // every peer has signalled this exchange, so it has finished reading the accumulator half of the previous one
    int4* old = reinterpret_cast<int4*>(hdr + l.acc + (int64_t)(half ^ 1) * l.acc_half);
    const int64_t vecs = (int64_t)v.m_max * (n >> 2);
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < vecs; i += (int64_t)gridDim.x * blockDim.x)
      old[i] = make_int4(0, 0, 0, 0);
  }
  if ((int)blockIdx.x < rows) {
    const int t = row0 + blockIdx.x;
    const int nvec = n >> 2;
    int xm, xs;
    absmax_to_ms_dev(__ldg(x_absmax + t), &xm, &xs);
    xs -= 48;
    int4 val[VPT];
    int mx = 0;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int idx = threadIdx.x + i * blockDim.x;
      int4 a = make_int4(0, 0, 0, 0);
      if (idx < nvec) {
        for (int src = 0; src < v.size; ++src) {
          const int4 b = __ldcg(reinterpret_cast<const int4*>(v.base[src] + acc_off + (int64_t)t * n) + idx);
          a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
        }
        const int4 wm = __ldg(reinterpret_cast<const int4*>(w_mul) + idx);
        int4 ws = make_int4(31, 31, 31, 31);
        if (w_shift) ws = __ldg(reinterpret_cast<const int4*>(w_shift) + idx);
        a.x = tp_requant_one(a.x, __mulhi(xm, wm.x), xs + ws.x);
        a.y = tp_requant_one(a.y, __mulhi(xm, wm.y), xs + ws.y);
        a.z = tp_requant_one(a.z, __mulhi(xm, wm.z), xs + ws.z);
        a.w = tp_requant_one(a.w, __mulhi(xm, wm.w), xs + ws.w);
        if (residual) {
          int4* rr = reinterpret_cast<int4*>(residual + (int64_t)t * n) + idx;
          const int4 b = *rr;
          a.x = (int)((unsigned)a.x + (unsigned)b.x);
          a.y = (int)((unsigned)a.y + (unsigned)b.y);
          a.z = (int)((unsigned)a.z + (unsigned)b.z);
          a.w = (int)((unsigned)a.w + (unsigned)b.w);
          *rr = a;
        }
      }
      val[i] = a;
      mx = max(max(mx, abs_wrap(a.x)), max(abs_wrap(a.y), max(abs_wrap(a.z), abs_wrap(a.w))));
    }
    mx = block_max(mx, red32);
    const NormRow nr = norm_row_from_absmax(mx);
    long long S = 0;
#pragma unroll
    for (int i = 0; i < VPT; ++i)
      S += (long long)norm_normalised_sq(val[i].x, nr.p) + (long long)norm_normalised_sq(val[i].y, nr.p) +
           (long long)norm_normalised_sq(val[i].z, nr.p) + (long long)norm_normalised_sq(val[i].w, nr.p);
    S = block_sum64(S, red64);
    const int inv = norm_inv_sqrt(S, n, g_inv_sqrt_lut);
    int m2 = 0;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int idx = threadIdx.x + i * blockDim.x;
      if (idx < nvec) {
        const int4 ww = __ldg(reinterpret_cast<const int4*>(norm_w) + idx);
        int4 o;
        o.x = nr.zero ? 0 : norm_apply(val[i].x, inv, ww.x, nr.p);
        o.y = nr.zero ? 0 : norm_apply(val[i].y, inv, ww.y, nr.p);
        o.z = nr.zero ? 0 : norm_apply(val[i].z, inv, ww.z, nr.p);
        o.w = nr.zero ? 0 : norm_apply(val[i].w, inv, ww.w, nr.p);
        val[i] = o;
        m2 = max(max(m2, abs_wrap(o.x)), max(abs_wrap(o.y), max(abs_wrap(o.z), abs_wrap(o.w))));
      }
    }
    m2 = max(1, block_max(m2, red32));
    const float mf = __int2float_rn(m2), my = __frcp_rn(mf);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int idx = threadIdx.x + i * blockDim.x;
      if (idx < nvec) {
        const unsigned c4 = pack4(quant_code_fast(val[i].x, mf, my), quant_code_fast(val[i].y, mf, my),
                                  quant_code_fast(val[i].z, mf, my), quant_code_fast(val[i].w, mf, my));
        for (int d = 0; d < v.size; ++d)
          reinterpret_cast<unsigned*>(v.base[d] + out_off)[(int64_t)t * nvec + idx] = c4;
      }
    }
    if (threadIdx.x == 0) {
      const int64_t ao = out_off + tp_codes_absmax_off(v.m_max, v.n) + t;
      for (int d = 0; d < v.size; ++d) v.base[d][ao] = m2;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) tp_signal_if_last(v, 3, gridDim.x, (int)blockIdx.x < rows);
}

// Waits for every rank's channel-3 signal and copies the codes and the absmax of all m rows out of the block.
__global__ void __launch_bounds__(256)
tp_collect_codes_kernel(const TpView v, int8_t* __restrict__ codes, int32_t* __restrict__ absmax, int m, int n) {
  pdl_launch_dependents();
  pdl_wait();          // what this kernel reads comes from the kernels before it (and from the peers, see below)
  const TpLayout l = tp_layout(v.m_max, v.n);
  const int32_t* hdr = v.base[v.rank];
  const int half = (*reinterpret_cast<const volatile int32_t*>(hdr + 1) - 1) & 1;
  tp_wait_flags(v, 3, *reinterpret_cast<const volatile int32_t*>(hdr + 3));
  __syncthreads();
  const int32_t* out = hdr + l.out + (int64_t)half * l.acc_half;
  const int64_t total = (int64_t)m * n / 16;                       // 16-byte vectors of codes
  const int4* src = reinterpret_cast<const int4*>(out);
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x)
    reinterpret_cast<int4*>(codes)[i] = __ldcg(src + i);
  const int32_t* am = out + tp_codes_absmax_off(v.m_max, v.n);
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < m; i += gridDim.x * blockDim.x) absmax[i] = __ldcg(am + i);
}

// ---------------------------------------------------------------------------- small all-gather (channel 2)
// One CTA: stores `words` int32 of src into slot [half][rank] of every rank's block, signals, waits for
// every rank's signal and copies the `size` slots, in rank order, to dst [size][words].
__global__ void __launch_bounds__(256)
tp_gather_kernel(const TpView v, const int32_t* __restrict__ src, int words, int32_t* __restrict__ dst) {
  pdl_launch_dependents();
  pdl_wait();          // what this kernel reads comes from the kernels before it (and from the peers, see below)
  const TpLayout l = tp_layout(v.m_max, v.n);
  int32_t* hdr = v.base[v.rank];
  const int e0 = *reinterpret_cast<volatile int32_t*>(hdr + 2);
  const int half = e0 & 1;
  const int64_t slot = l.gather + ((int64_t)half * kTpMaxRanks + v.rank) * l.gather_slot;
  for (int r = 0; r < v.size; ++r)
    for (int i = threadIdx.x; i < words; i += blockDim.x) v.base[r][slot + i] = src[i];
  __syncthreads();
  if (threadIdx.x == 0) tp_signal_if_last(v, 2, 1);
  __syncthreads();
  tp_wait_flags(v, 2, e0 + 1);
  __syncthreads();
  for (int r = 0; r < v.size; ++r) {
    const int32_t* s = hdr + l.gather + ((int64_t)half * kTpMaxRanks + r) * l.gather_slot;
    for (int i = threadIdx.x; i < words; i += blockDim.x) dst[(int64_t)r * words + i] = __ldcg(s + i);
  }
}

static int view_of(const b200_tp_block* blk, TpView* v, const char* name) {
  B200_REQUIRE(blk, B200_E_NULL, "%s: null block", name);
  B200_REQUIRE(blk->size >= 1 && blk->size <= kTpMaxRanks && blk->rank >= 0 && blk->rank < blk->size, B200_E_SHAPE,
               "%s: rank=%d size=%d", name, blk->rank, blk->size);
  B200_REQUIRE(blk->m_max > 0 && blk->n > 0 && blk->n % 4 == 0, B200_E_SHAPE, "%s: m_max=%d n=%lld", name, blk->m_max,
               (long long)blk->n);
  v->rank = blk->rank; v->size = blk->size; v->m_max = blk->m_max; v->n = blk->n;
  for (int r = 0; r < kTpMaxRanks; ++r) {
    v->base[r] = r < blk->size ? reinterpret_cast<int32_t*>(blk->base[r]) : nullptr;
    B200_REQUIRE(r >= blk->size || (v->base[r] && (reinterpret_cast<uintptr_t>(v->base[r]) & 255u) == 0), B200_E_ALIGN,
                 "%s: base[%d] is null or not 256-byte aligned", name, r);
  }
  return B200_OK;
}

int tp_agree_of(const ::b200_tp_block* blk, TpAgree* out, const char* name) {
  TpView v;
  int rc = view_of(blk, &v, name);
  if (rc != B200_OK) return rc;
  out->rank = v.rank; out->size = v.size; out->m_max = v.m_max;
  out->amax_off = tp_layout(v.m_max, v.n).amax;
  for (int r = 0; r < kTpMaxRanks; ++r) out->base[r] = v.base[r];
  void *st = nullptr, *to = nullptr;
  B200_REQUIRE(cudaGetSymbolAddress(&st, g_tp_status) == cudaSuccess && cudaGetSymbolAddress(&to, g_tp_timeout_ns) == cudaSuccess,
               B200_E_CUDA, "%s: cudaGetSymbolAddress failed", name);
  out->status = reinterpret_cast<int*>(st);
  out->timeout_ns = reinterpret_cast<const unsigned long long*>(to);
  return B200_OK;
}

}  // namespace b200

using namespace b200;

extern "C" size_t b200_tp_block_bytes(int m_max, int64_t n) {
  if (m_max <= 0 || n <= 0) return 0;
  return (size_t)tp_layout(m_max, n).total * sizeof(int32_t);
}

extern "C" int b200_tp_block_clear(const b200_tp_block* blk, b200_stream_t s) {
  TpView v;
  int rc = view_of(blk, &v, "tp_block_clear");
  if (rc != B200_OK) return rc;
  cudaError_t e = cudaMemsetAsync(v.base[v.rank], 0, b200_tp_block_bytes(v.m_max, v.n), (cudaStream_t)s);
  B200_REQUIRE(e == cudaSuccess, B200_E_CUDA, "tp_block_clear: %s", cudaGetErrorString(e));
  return B200_OK;
}

extern "C" int b200_tp_absmax_put(const b200_tp_block* blk, const int32_t* x, int64_t pitch, int rows, int k,
                                  b200_stream_t s) {
  TpView v;
  int rc = view_of(blk, &v, "tp_absmax_put");
  if (rc != B200_OK) return rc;
  B200_REQUIRE(x, B200_E_NULL, "tp_absmax_put: x is null");
  B200_REQUIRE(rows > 0 && rows <= v.m_max && k > 0 && k % 4 == 0 && pitch >= k && pitch % 4 == 0, B200_E_SHAPE,
               "tp_absmax_put: rows=%d (1..%d) k=%d pitch=%lld", rows, v.m_max, k, (long long)pitch);
  B200_REQUIRE(aligned16(x), B200_E_ALIGN, "tp_absmax_put: x must be 16-byte aligned");
  launch_pdl(tp_absmax_put_kernel, dim3(rows), dim3(256), 0, (cudaStream_t)s, v, x, pitch, k);
  return check_launch("tp_absmax_put");
}

extern "C" int b200_tp_quant_wait(const b200_tp_block* blk, const int32_t* x, int64_t pitch, int rows, int k,
                                  int8_t* codes, int32_t* absmax_out, b200_stream_t s) {
  TpView v;
  int rc = view_of(blk, &v, "tp_quant_wait");
  if (rc != B200_OK) return rc;
  B200_REQUIRE(x && codes && absmax_out, B200_E_NULL, "tp_quant_wait: null pointer");
  B200_REQUIRE(rows > 0 && rows <= v.m_max && k > 0 && k % 4 == 0 && pitch >= k && pitch % 4 == 0, B200_E_SHAPE,
               "tp_quant_wait: rows=%d (1..%d) k=%d pitch=%lld", rows, v.m_max, k, (long long)pitch);
  B200_REQUIRE(aligned16(x) && (reinterpret_cast<uintptr_t>(codes) & 3u) == 0, B200_E_ALIGN,
               "tp_quant_wait: x must be 16-byte aligned, codes 4-byte");
  launch_pdl(tp_quant_wait_kernel, dim3(rows), dim3(256), 0, (cudaStream_t)s, v, x, pitch, k, codes, absmax_out);
  return check_launch("tp_quant_wait");
}

extern "C" int b200_tp_absmax_quant(const b200_tp_block* blk, const int32_t* x, int64_t pitch, int rows, int k,
                                    int8_t* codes, int32_t* absmax_out, b200_stream_t s) {
  TpView v;
  int rc = view_of(blk, &v, "tp_absmax_quant");
  if (rc != B200_OK) return rc;
  B200_REQUIRE(x && codes && absmax_out, B200_E_NULL, "tp_absmax_quant: null pointer");
  B200_REQUIRE(rows > 0 && rows <= v.m_max && k > 0 && k % 4 == 0 && pitch >= k && pitch % 4 == 0, B200_E_SHAPE,
               "tp_absmax_quant: rows=%d (1..%d) k=%d pitch=%lld", rows, v.m_max, k, (long long)pitch);
  // every CTA waits for its peers' CTAs of the same row: all rows' CTAs must be able to run at once
  B200_REQUIRE(rows <= 512, B200_E_UNSUPPORTED, "tp_absmax_quant: rows=%d (at most 512; use tp_absmax_put + tp_quant_wait beyond)", rows);
  B200_REQUIRE(aligned16(x) && (reinterpret_cast<uintptr_t>(codes) & 3u) == 0, B200_E_ALIGN,
               "tp_absmax_quant: x must be 16-byte aligned, codes 4-byte");
  launch_pdl(tp_absmax_quant_kernel, dim3(rows), dim3(256), 0, (cudaStream_t)s, v, x, pitch, k, codes, absmax_out);
  return check_launch("tp_absmax_quant");
}

extern "C" int b200_tp_requant_scatter(const b200_tp_block* blk, const int32_t* absmax, const int32_t* w_mul,
                                       const int32_t* w_shift, int m, b200_stream_t s) {
  TpView v;
  int rc = view_of(blk, &v, "tp_requant_scatter");
  if (rc != B200_OK) return rc;
  B200_REQUIRE(absmax && w_mul, B200_E_NULL, "tp_requant_scatter: null pointer");
  B200_REQUIRE(m > 0 && m <= v.m_max, B200_E_SHAPE, "tp_requant_scatter: m=%d (1..%d)", m, v.m_max);
  B200_REQUIRE(aligned16(w_mul) && aligned16(w_shift), B200_E_ALIGN, "tp_requant_scatter: w_mul and w_shift must be 16-byte aligned");
  B200_REQUIRE(!tp_direct(v.size), B200_E_UNSUPPORTED, "tp_requant_scatter: %d ranks exchange directly: use tp_requant_direct", v.size);
  // few CTAs: each ends with a system-scope fence, and many of those at once are slow
  const int64_t vecs = (int64_t)tp_rows_per_rank(m, v.size) * (v.n / 4);
  const int grid = (int)((vecs + 1023) / 1024 < 148 ? (vecs + 1023) / 1024 : 148);
  launch_pdl(tp_requant_scatter_kernel<false>, dim3(grid < 1 ? 1 : grid), dim3(256), 0, (cudaStream_t)s, v, absmax, w_mul, w_shift, (int32_t*)nullptr, m, (int)v.n);
  return check_launch("tp_requant_scatter");
}

extern "C" int b200_tp_requant_direct(const b200_tp_block* blk, const int32_t* absmax, const int32_t* w_mul,
                                      const int32_t* w_shift, int32_t* out_q15, int m, b200_stream_t s) {
  TpView v;
  int rc = view_of(blk, &v, "tp_requant_direct");
  if (rc != B200_OK) return rc;
  B200_REQUIRE(absmax && w_mul && out_q15, B200_E_NULL, "tp_requant_direct: null pointer");
  B200_REQUIRE(m > 0 && m <= v.m_max, B200_E_SHAPE, "tp_requant_direct: m=%d (1..%d)", m, v.m_max);
  B200_REQUIRE(tp_direct(v.size), B200_E_UNSUPPORTED, "tp_requant_direct: %d ranks exchange through row owners: use tp_requant_scatter + tp_collect", v.size);
  B200_REQUIRE(aligned16(w_mul) && aligned16(w_shift) && aligned16(out_q15), B200_E_ALIGN,
               "tp_requant_direct: w_mul, w_shift and out must be 16-byte aligned");
  const int64_t vecs = (int64_t)m * (v.n / 4);
  const int grid = (int)((vecs + 1023) / 1024 < 592 ? (vecs + 1023) / 1024 : 592);
  launch_pdl(tp_requant_scatter_kernel<true>, dim3(grid < 1 ? 1 : grid), dim3(256), 0, (cudaStream_t)s, v, absmax, w_mul, w_shift, out_q15, m, (int)v.n);
  return check_launch("tp_requant_direct");
}

extern "C" int b200_tp_collect(const b200_tp_block* blk, int32_t* out_q15, int m, b200_stream_t s) {
  TpView v;
  int rc = view_of(blk, &v, "tp_collect");
  if (rc != B200_OK) return rc;
  B200_REQUIRE(out_q15, B200_E_NULL, "tp_collect: null pointer");
  B200_REQUIRE(m > 0 && m <= v.m_max, B200_E_SHAPE, "tp_collect: m=%d (1..%d)", m, v.m_max);
  B200_REQUIRE(!tp_direct(v.size), B200_E_UNSUPPORTED, "tp_collect: %d ranks exchange directly: use tp_requant_direct", v.size);
  B200_REQUIRE(aligned16(out_q15), B200_E_ALIGN, "tp_collect: out must be 16-byte aligned");
  const int64_t vecs = (int64_t)m * (v.n / 4);
  const int grid = (int)((vecs + 255) / 256 < 592 ? (vecs + 255) / 256 : 592);
  launch_pdl(tp_collect_kernel, dim3(grid), dim3(256), 0, (cudaStream_t)s, v, out_q15, m, (int)v.n);
  return check_launch("tp_collect");
}

extern "C" int b200_tp_owner_norm(const b200_tp_block* blk, const int32_t* x_absmax, const int32_t* w_mul, const int32_t* w_shift,
                                  int32_t* residual, const int32_t* norm_weight, int m, b200_stream_t s) {
  TpView v;
  int rc = view_of(blk, &v, "tp_owner_norm");
  if (rc != B200_OK) return rc;
  B200_REQUIRE(x_absmax && w_mul && norm_weight, B200_E_NULL, "tp_owner_norm: null pointer");
  B200_REQUIRE(m > 0 && m <= v.m_max, B200_E_SHAPE, "tp_owner_norm: m=%d (1..%d)", m, v.m_max);
  B200_REQUIRE(v.n % 16 == 0 && v.n <= 32768, B200_E_UNSUPPORTED, "tp_owner_norm: n=%lld must be a multiple of 16, at most 32768",
               (long long)v.n);
  B200_REQUIRE(aligned16(w_mul) && aligned16(w_shift) && aligned16(residual) && aligned16(norm_weight), B200_E_ALIGN,
               "tp_owner_norm: w_mul, w_shift, residual and norm_weight must be 16-byte aligned");
  const int nvec = (int)(v.n / 4);
  int threads = ((nvec + 31) / 32) * 32;
  if (threads > 1024) threads = 1024;
  const int vpt = (nvec + threads - 1) / threads;
  const int grid = tp_owner_rows(m, v.size);
  cudaStream_t st = (cudaStream_t)s;
  switch (vpt) {
    case 1: launch_pdl(tp_owner_norm_kernel<1>, dim3(grid), dim3(threads), 0, st, v, x_absmax, w_mul, w_shift, residual, norm_weight, m, (int)v.n); break;
    case 2: launch_pdl(tp_owner_norm_kernel<2>, dim3(grid), dim3(threads), 0, st, v, x_absmax, w_mul, w_shift, residual, norm_weight, m, (int)v.n); break;
    case 3: case 4: launch_pdl(tp_owner_norm_kernel<4>, dim3(grid), dim3(threads), 0, st, v, x_absmax, w_mul, w_shift, residual, norm_weight, m, (int)v.n); break;
    default: launch_pdl(tp_owner_norm_kernel<8>, dim3(grid), dim3(threads), 0, st, v, x_absmax, w_mul, w_shift, residual, norm_weight, m, (int)v.n); break;
  }
  return check_launch("tp_owner_norm");
}

extern "C" int b200_tp_collect_codes(const b200_tp_block* blk, int8_t* codes, int32_t* absmax, int m, b200_stream_t s) {
  TpView v;
  int rc = view_of(blk, &v, "tp_collect_codes");
  if (rc != B200_OK) return rc;
  B200_REQUIRE(codes && absmax, B200_E_NULL, "tp_collect_codes: null pointer");
  B200_REQUIRE(m > 0 && m <= v.m_max, B200_E_SHAPE, "tp_collect_codes: m=%d (1..%d)", m, v.m_max);
  B200_REQUIRE(v.n % 16 == 0, B200_E_UNSUPPORTED, "tp_collect_codes: n=%lld must be a multiple of 16", (long long)v.n);
  B200_REQUIRE(aligned16(codes), B200_E_ALIGN, "tp_collect_codes: codes must be 16-byte aligned");
  const int64_t vecs = (int64_t)m * v.n / 16;
  const int grid = (int)((vecs + 255) / 256 < 296 ? (vecs + 255) / 256 : 296);
  launch_pdl(tp_collect_codes_kernel, dim3(grid < 1 ? 1 : grid), dim3(256), 0, (cudaStream_t)s, v, codes, absmax, m, (int)v.n);
  return check_launch("tp_collect_codes");
}

extern "C" int b200_tp_all_gather(const b200_tp_block* blk, const int32_t* src, int words, int32_t* dst,
                                  b200_stream_t s) {
  TpView v;
  int rc = view_of(blk, &v, "tp_all_gather");
  if (rc != B200_OK) return rc;
  B200_REQUIRE(src && dst, B200_E_NULL, "tp_all_gather: null pointer");
  B200_REQUIRE(words > 0 && words <= 2 * v.m_max, B200_E_SHAPE, "tp_all_gather: words=%d (1..%d)", words, 2 * v.m_max);
  launch_pdl(tp_gather_kernel, dim3(1), dim3(256), 0, (cudaStream_t)s, v, src, words, dst);
  return check_launch("tp_all_gather");
}

extern "C" int b200_tp_status(int* out_host, int reset) {
  B200_REQUIRE(out_host, B200_E_NULL, "tp_status: null pointer");
  cudaError_t e = cudaMemcpyFromSymbol(out_host, g_tp_status, sizeof(int));
  if (e == cudaSuccess && reset) {
    const int zero = 0;
    e = cudaMemcpyToSymbol(g_tp_status, &zero, sizeof(int));
  }
  B200_REQUIRE(e == cudaSuccess, B200_E_CUDA, "tp_status: %s", cudaGetErrorString(e));
  return B200_OK;
}

extern "C" int b200_tp_set_timeout_us(int64_t microseconds) {
  B200_REQUIRE(microseconds > 0 && microseconds <= 60000000, B200_E_SHAPE, "tp_set_timeout_us: %lld (1 .. 60 000 000)",
               (long long)microseconds);
  const unsigned long long ns = (unsigned long long)microseconds * 1000ull;
  cudaError_t e = cudaMemcpyToSymbol(g_tp_timeout_ns, &ns, sizeof(ns));
  B200_REQUIRE(e == cudaSuccess, B200_E_CUDA, "tp_set_timeout_us: %s", cudaGetErrorString(e));
  return B200_OK;
}
