// The two ends of the integer model and the per-step bookkeeping of a decode batch:
//   * embedding rows (bf16 table) gathered by token id and converted to Q15.16,
//   * arg-max over int32 logits rows (lowest index wins ties),
//   * advancing a decode batch by one token on the device (positions, KV locations, lengths).
// All three are memory-bound row kernels: 16-byte loads and stores, one CTA (or warp) per row.
#include <cuda_bf16.h>

#include "common.cuh"

namespace b200 {

// ---------------------------------------------------------------------------------------------------
// Embedding gather + to_fixed.  One warp per token row; a lane converts 8 bf16 values per trip.
// Ids outside [vocab_start, vocab_start + vocab_rows) give a zero row (a vocabulary shard adds its
// rows to the other shards' zeros).
// ---------------------------------------------------------------------------------------------------
__device__ __forceinline__ int bf16_bits_to_q15(unsigned short b) {
  // same conversion as to_fixed: fp32 product, round half to even, saturating (NaN gives 0)
  return __float2int_rn(__fmul_rn(__uint_as_float((unsigned)b << 16), 65536.0f));
}

__global__ void __launch_bounds__(256)
embedding_q15_kernel(const uint16_t* __restrict__ table, const int32_t* __restrict__ ids, int32_t* __restrict__ out,
                     int64_t rows, int hidden, int64_t vocab_start, int64_t vocab_rows) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int64_t id = (int64_t)ids[row] - vocab_start;
  int4* o = reinterpret_cast<int4*>(out + row * hidden);
  if (id < 0 || id >= vocab_rows) {
    for (int c = lane; c < hidden / 4; c += 32) o[c] = make_int4(0, 0, 0, 0);
    return;
  }
  const uint4* src = reinterpret_cast<const uint4*>(table + id * hidden);
  for (int c = lane; c < hidden / 8; c += 32) {
    const uint4 v = __ldg(src + c);
    int4 a, b;
    a.x = bf16_bits_to_q15((unsigned short)(v.x & 0xffff)); a.y = bf16_bits_to_q15((unsigned short)(v.x >> 16));
    a.z = bf16_bits_to_q15((unsigned short)(v.y & 0xffff)); a.w = bf16_bits_to_q15((unsigned short)(v.y >> 16));
    b.x = bf16_bits_to_q15((unsigned short)(v.z & 0xffff)); b.y = bf16_bits_to_q15((unsigned short)(v.z >> 16));
    b.z = bf16_bits_to_q15((unsigned short)(v.w & 0xffff)); b.w = bf16_bits_to_q15((unsigned short)(v.w >> 16));
    o[2 * c] = a;
    o[2 * c + 1] = b;
  }
}

// ---------------------------------------------------------------------------------------------------
// Arg-max of int32 rows.  (value, index) is packed into one 64-bit key whose unsigned order is
// "larger value first, then smaller index", so the reduction is a plain max.
// ---------------------------------------------------------------------------------------------------
__device__ __forceinline__ unsigned long long argmax_key(int v, unsigned idx) {
  return ((unsigned long long)((unsigned)v ^ 0x80000000u) << 32) | (unsigned long long)(0xFFFFFFFFu - idx);
}

constexpr int kArgmaxThreads = 512;

__global__ void __launch_bounds__(kArgmaxThreads)
argmax_rows_kernel(const int32_t* __restrict__ logits, int64_t pitch, int64_t n, int32_t index_offset,
                   int32_t* __restrict__ out_idx, int32_t* __restrict__ out_val) {
  __shared__ unsigned long long red[kArgmaxThreads / 32];
  pdl_launch_dependents();
  pdl_wait();
  const int32_t* row = logits + (int64_t)blockIdx.x * pitch;
  unsigned long long best = 0ull;      // below every real key: an index < 2^31 makes the low word >= 2^31
  const int64_t n4 = n / 4;
  const int4* row4 = reinterpret_cast<const int4*>(row);
  for (int64_t c = threadIdx.x; c < n4; c += kArgmaxThreads) {
    const int4 v = __ldg(row4 + c);
    const unsigned i0 = (unsigned)(c * 4);
    unsigned long long k0 = argmax_key(v.x, i0), k1 = argmax_key(v.y, i0 + 1), k2 = argmax_key(v.z, i0 + 2), k3 = argmax_key(v.w, i0 + 3);
    k0 = k0 > k1 ? k0 : k1;
    k2 = k2 > k3 ? k2 : k3;
    k0 = k0 > k2 ? k0 : k2;
    best = k0 > best ? k0 : best;
  }
  for (int64_t c = n4 * 4 + threadIdx.x; c < n; c += kArgmaxThreads) {
    const unsigned long long k = argmax_key(__ldg(row + c), (unsigned)c);
    best = k > best ? k : best;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const unsigned long long other = __shfl_xor_sync(FULL_MASK, best, o);
    best = other > best ? other : best;
  }
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = best;
  __syncthreads();
  if (threadIdx.x < 32) {
    unsigned long long b = threadIdx.x < kArgmaxThreads / 32 ? red[threadIdx.x] : 0ull;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const unsigned long long other = __shfl_xor_sync(FULL_MASK, b, o);
      b = other > b ? other : b;
    }
    if (threadIdx.x == 0) {
      const unsigned idx = 0xFFFFFFFFu - (unsigned)(b & 0xFFFFFFFFull);
      out_idx[blockIdx.x] = (int32_t)idx + index_offset;
      if (out_val) out_val[blockIdx.x] = (int32_t)((unsigned)(b >> 32) ^ 0x80000000u);
    }
  }
}

// ---------------------------------------------------------------------------------------------------
// One decode step of bookkeeping for `batch` sequences, all on the device so that the step can be
// replayed from a CUDA graph: the new token of sequence b sits at position seq_lens[b]; its KV slot
// is page_table[b][pos / 16] * 16 + pos % 16; the sequence then has pos + 1 keys.
// ---------------------------------------------------------------------------------------------------
__global__ void decode_prepare_kernel(const int32_t* __restrict__ page_table, int64_t pitch, int32_t* __restrict__ seq_lens,
                                      int32_t* __restrict__ positions, int32_t* __restrict__ out_loc,
                                      int32_t* __restrict__ kv_lens, int batch, int max_len) {
  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= batch) return;
  int pos = seq_lens[b];
  pos = pos < 0 ? 0 : (pos > max_len - 1 ? max_len - 1 : pos);      // a full sequence rewrites its last slot
  const int page = page_table[(int64_t)b * pitch + (pos >> 4)];
  positions[b] = pos;
  out_loc[b] = page * 16 + (pos & 15);
  kv_lens[b] = pos + 1;
  seq_lens[b] = pos + 1;
}

// ---------------------------------------------------------------------------------------------------
// Per-tensor int8 quantisation of a bf16 tensor with a (multiplier, shift) scale: the quantiser the
// reference's prefill path applies to q, k and v (quantize_per_tensor_int8_ms).  Two passes: the
// absolute maximum (bf16 bit patterns of non-negative values order like integers), then the codes.
//   max_abs = max(|x|) clamped below at bf16(1e-8); e = ceil(bf16(log2(max_abs)));
//   multiplier = int32(min(max_abs * 2^(31 - e), 2^31 - 1)); shift = 31 - e + 7;
//   code = clamp(rint((fp32(x) / max_abs) * 127), -128, 127).
// ---------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
ptq_absmax_kernel(const uint16_t* __restrict__ x, int64_t n, unsigned* __restrict__ max_bits) {
  unsigned m = 0;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const unsigned b = x[i] & 0x7fffu;
    if (b <= 0x7f80u) m = max(m, b);            // NaNs do not take part
  }
  m = (unsigned)warp_max((int)m);
  if ((threadIdx.x & 31) == 0 && m) atomicMax(max_bits, m);
}

__device__ __forceinline__ float bf16_round(float v) {   // round to nearest even on the upper 16 bits
  const unsigned u = __float_as_uint(v);
  return __uint_as_float((u + 0x7fffu + ((u >> 16) & 1u)) & 0xffff0000u);
}

__global__ void __launch_bounds__(256)
ptq_codes_kernel(const uint16_t* __restrict__ x, int64_t n, const unsigned* __restrict__ max_bits, int8_t* __restrict__ codes,
                 int32_t* __restrict__ mul_shift) {
  const float floor_v = __uint_as_float(0x322cu << 16);                    // bf16(1e-8)
  const float mx = fmaxf(__uint_as_float(*max_bits << 16), floor_v);
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const float v = __uint_as_float((unsigned)x[i] << 16);
    const float q = __fmul_rn(__fdiv_rn(v, mx), 127.0f);
    codes[i] = (int8_t)max(-128, min(127, __float2int_rn(q)));
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    const float e = ceilf(bf16_round(log2f(mx)));
    const float sh = bf16_round(31.0f - e);                                 // the subtraction happens in bf16
    const float mf = ldexpf(mx, (int)sh);                                   // max_abs * 2^shift, exact
    mul_shift[0] = mf >= 2147483648.0f ? 2147483647 : (int)mf;
    mul_shift[1] = (int)sh + 7;
  }
}

}  // namespace b200

using namespace b200;

extern "C" int b200_embedding_bf16_q15(const uint16_t* table, const int32_t* ids, int32_t* out, int64_t rows,
                                       int hidden, int64_t vocab_start, int64_t vocab_rows, b200_stream_t s) {
  B200_REQUIRE(rows >= 0 && hidden > 0 && vocab_rows > 0, B200_E_SHAPE, "embedding: rows=%lld hidden=%d vocab_rows=%lld",
               (long long)rows, hidden, (long long)vocab_rows);
  B200_REQUIRE(hidden % 8 == 0, B200_E_UNSUPPORTED, "embedding: hidden=%d must be a multiple of 8", hidden);
  if (rows == 0) return B200_OK;
  B200_REQUIRE(table && ids && out, B200_E_NULL, "embedding: null pointer");
  B200_REQUIRE(aligned16(table) && aligned16(out), B200_E_ALIGN, "embedding: table and out must be 16-byte aligned");
  const int64_t blocks = (rows + 7) / 8;
  B200_REQUIRE(blocks < (1ll << 31), B200_E_SHAPE, "embedding: too many rows");
  launch_pdl(embedding_q15_kernel, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)s, table, ids, out, rows, hidden, vocab_start, vocab_rows);
  return check_launch("embedding_bf16_q15");
}

extern "C" int b200_argmax_i32(const int32_t* logits, int64_t rows, int64_t n, int64_t pitch, int32_t index_offset,
                               int32_t* out_idx, int32_t* out_val, b200_stream_t s) {
  B200_REQUIRE(rows >= 0 && n > 0 && pitch >= n && n < (1ll << 31), B200_E_SHAPE, "argmax: rows=%lld n=%lld pitch=%lld",
               (long long)rows, (long long)n, (long long)pitch);
  if (rows == 0) return B200_OK;
  B200_REQUIRE(logits && out_idx, B200_E_NULL, "argmax: null pointer");
  B200_REQUIRE(aligned16(logits) && pitch % 4 == 0, B200_E_ALIGN, "argmax: rows must be 16-byte aligned (pitch a multiple of 4)");
  B200_REQUIRE(rows < (1ll << 31), B200_E_SHAPE, "argmax: too many rows");
  launch_pdl(argmax_rows_kernel, dim3((unsigned)rows), dim3(kArgmaxThreads), 0, (cudaStream_t)s, logits, pitch, n, index_offset, out_idx, out_val);
  return check_launch("argmax_i32");
}

extern "C" int b200_decode_prepare(const int32_t* page_table, int64_t table_pitch, int32_t* seq_lens, int32_t* positions,
                                   int32_t* out_loc, int32_t* kv_lens, int batch, int max_len, b200_stream_t s) {
  B200_REQUIRE(batch >= 0 && max_len > 0 && table_pitch >= (max_len + 15) / 16, B200_E_SHAPE,
               "decode_prepare: batch=%d max_len=%d table_pitch=%lld", batch, max_len, (long long)table_pitch);
  if (batch == 0) return B200_OK;
  B200_REQUIRE(page_table && seq_lens && positions && out_loc && kv_lens, B200_E_NULL, "decode_prepare: null pointer");
  launch_pdl(decode_prepare_kernel, dim3((batch + 127) / 128), dim3(128), 0, (cudaStream_t)s, page_table, table_pitch, seq_lens, positions, out_loc,
             kv_lens, batch, max_len);
  return check_launch("decode_prepare");
}

extern "C" int b200_quantize_per_tensor_int8_ms(const uint16_t* x_bf16, int64_t n, int8_t* codes, int32_t* mul_shift,
                                                uint32_t* scratch_word, b200_stream_t s) {
  B200_REQUIRE(n >= 0 && n < (1ll << 40), B200_E_SHAPE, "quantize_per_tensor_int8_ms: n=%lld", (long long)n);
  if (n == 0) return B200_OK;
  B200_REQUIRE(x_bf16 && codes && mul_shift && scratch_word, B200_E_NULL, "quantize_per_tensor_int8_ms: null pointer");
  cudaError_t e = cudaMemsetAsync(scratch_word, 0, sizeof(uint32_t), (cudaStream_t)s);
  B200_REQUIRE(e == cudaSuccess, B200_E_CUDA, "quantize_per_tensor_int8_ms: cudaMemsetAsync: %s", cudaGetErrorString(e));
  const int grid = (int)((n + 255) / 256 < 1184 ? (n + 255) / 256 : 1184);
  ptq_absmax_kernel<<<grid, 256, 0, (cudaStream_t)s>>>(x_bf16, n, scratch_word);
  ptq_codes_kernel<<<grid, 256, 0, (cudaStream_t)s>>>(x_bf16, n, scratch_word, codes, mul_shift);
  return check_launch("quantize_per_tensor_int8_ms");
}
