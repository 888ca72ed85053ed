// Tensor-parallel exchange steps of the row-split linears over NVLink peer memory (decode sizes).
//
// A row-split linear (o_proj, down_proj) on `size` ranks gives the bits of one GPU when the ranks
//   1. agree on every token's absmax            (atomicMax into every rank's block, channel 0),
//   2. quantise their K-slice with it,
//   3. add their exact int32 partial sums       (red.global from the GEMM epilogue, channel 1),
//   4. requantise the sum once.
// Steps 1 and 3 write straight into the peers' memory; a producer kernel ends with a signal (its last CTA
// stores the channel's new epoch into every rank's flag word), the consumer kernel begins with a bounded
// wait on those flags.  No collective library call, no host synchronisation: a decode step that uses these
// kernels is an ordinary stream of launches and can be captured in a CUDA graph on every rank.
//
// Every wait gives up after a time limit (default 2 s), records the channel in a status word that the host
// can read, and lets the kernel finish on whatever the block holds: a missing peer costs a wrong result and
// an error code, never a hung GPU.
#include "tp_block.cuh"

namespace b200 {

static __device__ int g_tp_status = 0;                             // 0 = fine, else channel + 1 of the first expiry
static __device__ unsigned long long g_tp_timeout_ns = 2000000000ull;

// Waits until every rank's signal number `epoch` on channel ch has arrived: threads 0 .. size-1 poll one
// source each; the caller follows with a CTA barrier.
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
        __nanosleep(64);
      }
    }
  }
}

// ---------------------------------------------------------------------------- step 1: absmax agreement
// One CTA per token row of this rank's slice x [rows, k] (row pitch in elements): the row's max(1, max|x|)
// is folded into amax[half][row] of every rank.  Signals channel 0.
__global__ void __launch_bounds__(256)
tp_absmax_put_kernel(const TpView v, const int32_t* __restrict__ x, int64_t pitch, int k) {
  __shared__ int red32[33];
  const TpLayout l = tp_layout(v.m_max, v.n);
  const int half = *reinterpret_cast<volatile int32_t*>(v.base[v.rank] + 0) & 1;
  const int row = blockIdx.x;
  const int4* xr = reinterpret_cast<const int4*>(x + (int64_t)row * pitch);
  int m = 0;
  for (int i = threadIdx.x; i < (k >> 2); i += blockDim.x) {
    const int4 a = xr[i];
    m = max(max(m, abs_wrap(a.x)), max(abs_wrap(a.y), max(abs_wrap(a.z), abs_wrap(a.w))));
  }
  m = max(1, block_max(m, red32));
  if ((int)threadIdx.x < v.size) {
    atomicMax(v.base[threadIdx.x] + l.amax + (int64_t)half * v.m_max + row, m);
    __threadfence_system();
  }
  __syncthreads();
  if (threadIdx.x == 0) tp_signal_if_last(v, 0, gridDim.x);
}

// ---------------------------------------------------------------------------- step 2: quantise with the agreed absmax
// One CTA per row: waits for every rank's channel-0 signal, reads the agreed absmax, writes the int8 codes of
// this rank's slice and the absmax (for the requant), and clears the word for its next use.
__global__ void __launch_bounds__(256)
tp_quant_wait_kernel(const TpView v, const int32_t* __restrict__ x, int64_t pitch, int k,
                     int8_t* __restrict__ codes, int32_t* __restrict__ absmax_out) {
  const TpLayout l = tp_layout(v.m_max, v.n);
  int32_t* hdr = v.base[v.rank];
  const int epoch = *reinterpret_cast<volatile int32_t*>(hdr + 0);     // the signal this step's producer sent
  const int half = (epoch - 1) & 1;
  tp_wait_flags(v, 0, epoch);
  __syncthreads();
  const int row = blockIdx.x;
  int32_t* word = hdr + l.amax + (int64_t)half * v.m_max + row;
  const int m = max(1, tp_ld_acquire(word));
  __syncthreads();                                   // everybody has read the word before it is cleared
  if (threadIdx.x == 0) {
    absmax_out[row] = m;
    *word = 0;
  }
  const float mf = __int2float_rn(m), my = __frcp_rn(mf);
  const int4* xr = reinterpret_cast<const int4*>(x + (int64_t)row * pitch);
  unsigned* co = reinterpret_cast<unsigned*>(codes + (int64_t)row * k);
  for (int i = threadIdx.x; i < (k >> 2); i += blockDim.x) {
    const int4 a = xr[i];
    co[i] = pack4(quant_code_fast(a.x, mf, my), quant_code_fast(a.y, mf, my), quant_code_fast(a.z, mf, my),
                  quant_code_fast(a.w, mf, my));
  }
}

// ---------------------------------------------------------------------------- step 4: requantise the summed accumulators
// Waits for every rank's channel-1 signal (sent by the GEMM kernels), applies the fixed-point epilogue to
// acc[half] and clears it.  Four consecutive channels of one token per thread.
__device__ __forceinline__ int tp_requant_one(int acc, int cm, int s) {
  if (s > 0 && s < 63) return sat32(((long long)acc * (long long)cm + (1LL << (s - 1))) >> s);
  return sat32(mul_shift64((long long)acc, (long long)cm, s));
}

__global__ void __launch_bounds__(256)
tp_requant_wait_kernel(const TpView v, const int32_t* __restrict__ absmax, const int32_t* __restrict__ w_mul,
                       const int32_t* __restrict__ w_shift, int32_t* __restrict__ out, int m, int n) {
  const TpLayout l = tp_layout(v.m_max, v.n);
  int32_t* hdr = v.base[v.rank];
  const int epoch = *reinterpret_cast<volatile int32_t*>(hdr + 1);
  const int half = (epoch - 1) & 1;
  tp_wait_flags(v, 1, epoch);
  __syncthreads();
  int32_t* acc = hdr + l.acc + (int64_t)half * l.acc_half;
  const int nvec = n >> 2;
  const int64_t total = (int64_t)m * nvec;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int t = (int)(i / nvec);
    const int c = (int)(i - (int64_t)t * nvec) * 4;
    int xm, xs;
    absmax_to_ms_dev(__ldg(absmax + t), &xm, &xs);
    xs -= 48;
    int4* ap = reinterpret_cast<int4*>(acc + (int64_t)t * n + c);
    const int4 a = __ldcg(ap);                        // written by peers: read from L2, not a stale L1 line
    *ap = make_int4(0, 0, 0, 0);
    const int4 wm = __ldg(reinterpret_cast<const int4*>(w_mul + c));
    int4 ws = make_int4(31, 31, 31, 31);
    if (w_shift) ws = __ldg(reinterpret_cast<const int4*>(w_shift + c));
    int4 r;
    r.x = tp_requant_one(a.x, __mulhi(xm, wm.x), xs + ws.x);
    r.y = tp_requant_one(a.y, __mulhi(xm, wm.y), xs + ws.y);
    r.z = tp_requant_one(a.z, __mulhi(xm, wm.z), xs + ws.z);
    r.w = tp_requant_one(a.w, __mulhi(xm, wm.w), xs + ws.w);
    *reinterpret_cast<int4*>(out + (int64_t)t * n + c) = r;
  }
}

// ---------------------------------------------------------------------------- small all-gather (channel 2)
// One CTA: stores `words` int32 of src into slot [half][rank] of every rank's block, signals, waits for
// every rank's signal and copies the `size` slots, in rank order, to dst [size][words].
__global__ void __launch_bounds__(256)
tp_gather_kernel(const TpView v, const int32_t* __restrict__ src, int words, int32_t* __restrict__ dst) {
  const TpLayout l = tp_layout(v.m_max, v.n);
  int32_t* hdr = v.base[v.rank];
  const int e0 = *reinterpret_cast<volatile int32_t*>(hdr + 2);
  const int half = e0 & 1;
  const int64_t slot = l.gather + ((int64_t)half * kTpMaxRanks + v.rank) * l.gather_slot;
  for (int r = 0; r < v.size; ++r)
    for (int i = threadIdx.x; i < words; i += blockDim.x) v.base[r][slot + i] = src[i];
  __threadfence_system();
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
  tp_absmax_put_kernel<<<rows, 256, 0, (cudaStream_t)s>>>(v, x, pitch, k);
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
  tp_quant_wait_kernel<<<rows, 256, 0, (cudaStream_t)s>>>(v, x, pitch, k, codes, absmax_out);
  return check_launch("tp_quant_wait");
}

extern "C" int b200_tp_requant_wait(const b200_tp_block* blk, const int32_t* absmax, const int32_t* w_mul,
                                    const int32_t* w_shift, int32_t* out_q15, int m, b200_stream_t s) {
  TpView v;
  int rc = view_of(blk, &v, "tp_requant_wait");
  if (rc != B200_OK) return rc;
  B200_REQUIRE(absmax && w_mul && out_q15, B200_E_NULL, "tp_requant_wait: null pointer");
  B200_REQUIRE(m > 0 && m <= v.m_max, B200_E_SHAPE, "tp_requant_wait: m=%d (1..%d)", m, v.m_max);
  B200_REQUIRE(aligned16(w_mul) && aligned16(w_shift) && aligned16(out_q15), B200_E_ALIGN,
               "tp_requant_wait: w_mul, w_shift and out must be 16-byte aligned");
  const int64_t vecs = (int64_t)m * (v.n / 4);
  const int grid = (int)((vecs + 255) / 256 < 1184 ? (vecs + 255) / 256 : 1184);
  tp_requant_wait_kernel<<<grid, 256, 0, (cudaStream_t)s>>>(v, absmax, w_mul, w_shift, out_q15, m, (int)v.n);
  return check_launch("tp_requant_wait");
}

extern "C" int b200_tp_all_gather(const b200_tp_block* blk, const int32_t* src, int words, int32_t* dst,
                                  b200_stream_t s) {
  TpView v;
  int rc = view_of(blk, &v, "tp_all_gather");
  if (rc != B200_OK) return rc;
  B200_REQUIRE(src && dst, B200_E_NULL, "tp_all_gather: null pointer");
  B200_REQUIRE(words > 0 && words <= 2 * v.m_max, B200_E_SHAPE, "tp_all_gather: words=%d (1..%d)", words, 2 * v.m_max);
  tp_gather_kernel<<<1, 256, 0, (cudaStream_t)s>>>(v, src, words, dst);
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
