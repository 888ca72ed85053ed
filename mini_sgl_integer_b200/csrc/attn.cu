// int8 paged KV pool: store kernels and decode attention with an exact fixed-point softmax.
//
// Pool layout of one layer (page = 16 tokens, head_dim = 128):
//   k_codes [pages][kv_heads][16 tok][128 d]      one (page, head) chunk = 2 KB, token rows
//   v_codes [pages][kv_heads][2048 B]             the same 16 x 128 bytes in the operand order of
//                                                 the integer MMA (see v_chunk_offset): PV
//                                                 contracts over tokens, so 4 tokens of one d
//                                                 share a 32-bit word
//   meta    [pages][kv_heads][40 words]           k_mul[16] v_mul[16] k_shift[16 x i8] v_shift[16 x i8]
//
// Decode: a thread-block cluster owns one (sequence, KV head); each CTA of the cluster takes a
// contiguous run of pages.  The softmax is exact (LUT exp with truncation), so partial results
// cannot be rescaled: the scores of a slice stay in shared memory and the row maximum, the sum of
// exponentials and the partial outputs are exchanged between the CTAs over distributed shared
// memory.  K and V are each read from HBM exactly once.
#include <cooperative_groups.h>

#include "attn_common.cuh"
#include "luts.cuh"
#include "rope.cuh"

namespace cg = cooperative_groups;

namespace b200 {

// ============================================================================ store
// One warp per (token, kv head).  QUANT: rows are Q15.16 int32 and are quantised here;
// otherwise codes and scales are given.
template <bool QUANT>
__global__ void __launch_bounds__(256)
kv_store_kernel(const void* __restrict__ k_in, int64_t k_pitch, const void* __restrict__ v_in,
                int64_t v_pitch, const int32_t* __restrict__ k_mul_in, const int32_t* __restrict__ k_shift_in,
                const int32_t* __restrict__ v_mul_in, const int32_t* __restrict__ v_shift_in,
                const int32_t* __restrict__ out_loc, int8_t* __restrict__ k_codes,
                int8_t* __restrict__ v_codes, int32_t* __restrict__ meta, int64_t tokens, int kv_heads,
                int64_t num_pages) {
  const int lane = threadIdx.x & 31;
  const int64_t wid = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
  if (wid >= tokens * kv_heads) return;
  const int64_t t = wid / kv_heads;
  const int h = (int)(wid - t * kv_heads);
  const int64_t loc = out_loc[t];
  const int64_t pid = loc >> 4;
  const int tok = (int)(loc & 15);
  if (loc < 0 || pid >= num_pages) return;  // out-of-pool locations are dropped, never written

  unsigned kw, vw;
  int kmul, kshift, vmul, vshift;
  if (QUANT) {
    const int32_t* kr = reinterpret_cast<const int32_t*>(k_in) + t * k_pitch + (int64_t)h * kD;
    const int32_t* vr = reinterpret_cast<const int32_t*>(v_in) + t * v_pitch + (int64_t)h * kD;
    const int4 a = *reinterpret_cast<const int4*>(kr + 4 * lane);
    const int4 b = *reinterpret_cast<const int4*>(vr + 4 * lane);
    int mk = max(max(0, abs_wrap(a.x)), max(abs_wrap(a.y), max(abs_wrap(a.z), abs_wrap(a.w))));
    int mv = max(max(0, abs_wrap(b.x)), max(abs_wrap(b.y), max(abs_wrap(b.z), abs_wrap(b.w))));
    mk = max(1, warp_max(mk));
    mv = max(1, warp_max(mv));
    const float fk = __int2float_rn(mk), fv = __int2float_rn(mv);
    const float yk = __frcp_rn(fk), yv = __frcp_rn(fv);
    kw = pack4(quant_code_fast(a.x, fk, yk), quant_code_fast(a.y, fk, yk), quant_code_fast(a.z, fk, yk),
               quant_code_fast(a.w, fk, yk));
    vw = pack4(quant_code_fast(b.x, fv, yv), quant_code_fast(b.y, fv, yv), quant_code_fast(b.z, fv, yv),
               quant_code_fast(b.w, fv, yv));
    absmax_to_ms_dev(mk, &kmul, &kshift);
    absmax_to_ms_dev(mv, &vmul, &vshift);
  } else {
    kw = reinterpret_cast<const unsigned*>(reinterpret_cast<const int8_t*>(k_in) + (t * kv_heads + h) * kD)[lane];
    vw = reinterpret_cast<const unsigned*>(reinterpret_cast<const int8_t*>(v_in) + (t * kv_heads + h) * kD)[lane];
    kmul = k_mul_in[t * kv_heads + h];
    kshift = k_shift_in[t * kv_heads + h];
    vmul = v_mul_in[t * kv_heads + h];
    vshift = v_shift_in[t * kv_heads + h];
  }
  const int64_t chunk = pid * kv_heads + h;
  reinterpret_cast<unsigned*>(k_codes + (chunk * kPage + tok) * kD)[lane] = kw;
  int8_t* vdst = v_codes + chunk * (kD * kPage);
#pragma unroll
  for (int e = 0; e < 4; ++e) vdst[v_chunk_offset(4 * lane + e, tok)] = (int8_t)((vw >> (8 * e)) & 0xff);
  if (lane == 0) {
    int32_t* mt = meta + chunk * kMetaWords;
    mt[tok] = kmul;
    mt[16 + tok] = vmul;
    reinterpret_cast<int8_t*>(mt + 32)[tok] = (int8_t)kshift;
    reinterpret_cast<int8_t*>(mt + 36)[tok] = (int8_t)vshift;
  }
}

// ============================================================================ q/k/v preparation
// Everything between the qkv projection and attention in one launch, one warp per (token, head) of the
// q | k | v heads: q heads get q-norm + RoPE + Hadamard rotation, per-row int8 quantisation and their
// (multiplier, shift); k heads the same and go straight into their page; v heads are quantised and stored
// in operand order.  Same arithmetic, row by row, as qk_rope_kernel, quant_rows_kernel, absmax_to_ms_kernel
// and kv_store_kernel<true> run one after the other.
// PENDING: q, k and v are null and the rows come from the qkv linear's exact accumulators ([tokens, heads * 128],
// q | k | v heads side by side), requantised while they are loaded and zeroed behind.
template <bool PENDING>
__global__ void __launch_bounds__(256)
qkv_prepare_kernel(const int32_t* __restrict__ positions, const int32_t* __restrict__ q, int64_t q_pitch,
                   const int32_t* __restrict__ k, int64_t k_pitch, const int32_t* __restrict__ v, int64_t v_pitch,
                   const int32_t* __restrict__ cos_sin, int max_pos, const int32_t* __restrict__ q_norm_w,
                   const int32_t* __restrict__ k_norm_w, const int32_t* __restrict__ out_loc,
                   int8_t* __restrict__ k_codes, int8_t* __restrict__ v_codes, int32_t* __restrict__ meta,
                   int8_t* __restrict__ q8, int32_t* __restrict__ q_mul, int32_t* __restrict__ q_shift,
                   int64_t tokens, int q_heads, int kv_heads, int64_t num_pages, int with_fwht, const PendingLinear pl) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int heads = q_heads + 2 * kv_heads;
  const int64_t wid = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
  if (wid >= tokens * heads) return;   // whole warps leave together
  const int64_t t = wid / heads;
  const int h = (int)(wid - t * heads);
  const int64_t loc = out_loc[t];
  const int64_t pid = loc >> 4;
  const int tok = (int)(loc & 15);
  const bool in_pool = loc >= 0 && pid < num_pages;     // out-of-pool locations are dropped, never written
  int pxm = 0, pxs = 0;
  int4 pv = make_int4(0, 0, 0, 0);
  int2 plo = make_int2(0, 0), phi = make_int2(0, 0);
  if (PENDING) {     // taken (and zeroed) before any early return: the buffer must be all zero afterwards
    absmax_to_ms_dev(__ldg(pl.x_absmax + t), &pxm, &pxs);
    pxs -= 48;
    if (h < q_heads + kv_heads) {
      plo = pending_take2(pl, t, heads * kD, h * kD + 2 * lane, pxm, pxs);
      phi = pending_take2(pl, t, heads * kD, h * kD + 64 + 2 * lane, pxm, pxs);
    } else {
      pv = pending_take4(pl, t, heads * kD, h * kD + 4 * lane, pxm, pxs);
    }
  }
  if (h < q_heads + kv_heads) {
    const bool is_q = h < q_heads;
    const int hh = is_q ? h : h - q_heads;
    if (!is_q && !in_pool) {
      if (PENDING) {   // dropped, but the buffer must still be all zero afterwards
        pending_clear2(pl, t, heads * kD, h * kD + 2 * lane);
        pending_clear2(pl, t, heads * kD, h * kD + 64 + 2 * lane);
      }
      return;
    }
    int a0, a1, b0, b1;
    if (PENDING) {
      rope_row_vals(plo, phi, is_q ? q_norm_w : k_norm_w, positions[t], cos_sin, max_pos, with_fwht, lane, a0, a1, b0, b1);
    } else {
      const int32_t* src = is_q ? q + t * q_pitch + (int64_t)hh * kD : k + t * k_pitch + (int64_t)hh * kD;
      rope_row(src, is_q ? q_norm_w : k_norm_w, positions[t], cos_sin, max_pos, with_fwht, lane, a0, a1, b0, b1);
    }
    int m = max(max(0, abs_wrap(a0)), max(abs_wrap(a1), max(abs_wrap(b0), abs_wrap(b1))));
    m = max(1, warp_max(m));
    if (PENDING) {   // after a reduction over the loaded values: zeros for the next GEMM's partial sums
      __syncwarp();
      pending_clear2(pl, t, heads * kD, h * kD + 2 * lane);
      pending_clear2(pl, t, heads * kD, h * kD + 64 + 2 * lane);
    }
    const float mf = __int2float_rn(m), my = __frcp_rn(mf);
    const unsigned lo = (unsigned)(quant_code_fast(a0, mf, my) & 0xff) | ((unsigned)(quant_code_fast(a1, mf, my) & 0xff) << 8);
    const unsigned hi = (unsigned)(quant_code_fast(b0, mf, my) & 0xff) | ((unsigned)(quant_code_fast(b1, mf, my) & 0xff) << 8);
    int mul, shift;
    absmax_to_ms_dev(m, &mul, &shift);
    int8_t* row;
    if (is_q) {
      row = q8 + (t * q_heads + hh) * kD;
      if (lane == 0) { q_mul[t * q_heads + hh] = mul; q_shift[t * q_heads + hh] = shift; }
    } else {
      const int64_t chunk = pid * kv_heads + hh;
      row = k_codes + (chunk * kPage + tok) * kD;
      if (lane == 0) {
        int32_t* mt = meta + chunk * kMetaWords;
        mt[tok] = mul;
        reinterpret_cast<int8_t*>(mt + 32)[tok] = (int8_t)shift;
      }
    }
    reinterpret_cast<unsigned short*>(row)[lane] = (unsigned short)lo;            // elements 2l, 2l+1
    reinterpret_cast<unsigned short*>(row + 64)[lane] = (unsigned short)hi;       // elements 64+2l, 64+2l+1
  } else {
    if (!in_pool) {
      if (PENDING) pending_clear4(pl, t, heads * kD, h * kD + 4 * lane);
      return;
    }
    const int hh = h - q_heads - kv_heads;
    const int4 b = PENDING ? pv : *reinterpret_cast<const int4*>(v + t * v_pitch + (int64_t)hh * kD + 4 * lane);
    int mv = max(max(0, abs_wrap(b.x)), max(abs_wrap(b.y), max(abs_wrap(b.z), abs_wrap(b.w))));
    mv = max(1, warp_max(mv));
    if (PENDING) {
      __syncwarp();
      pending_clear4(pl, t, heads * kD, h * kD + 4 * lane);
    }
    const float fv = __int2float_rn(mv), yv = __frcp_rn(fv);
    const unsigned vw = pack4(quant_code_fast(b.x, fv, yv), quant_code_fast(b.y, fv, yv), quant_code_fast(b.z, fv, yv),
                              quant_code_fast(b.w, fv, yv));
    int mul, shift;
    absmax_to_ms_dev(mv, &mul, &shift);
    const int64_t chunk = pid * kv_heads + hh;
    int8_t* vdst = v_codes + chunk * (kD * kPage);
#pragma unroll
    for (int e = 0; e < 4; ++e) vdst[v_chunk_offset(4 * lane + e, tok)] = (int8_t)((vw >> (8 * e)) & 0xff);
    if (lane == 0) {
      int32_t* mt = meta + chunk * kMetaWords;
      mt[16 + tok] = mul;
      reinterpret_cast<int8_t*>(mt + 36)[tok] = (int8_t)shift;
    }
  }
}

// ============================================================================ decode
struct DecodeParams {
  const int8_t* q;
  const int32_t* q_mul;
  const int32_t* q_shift;
  const int8_t* k_codes;
  const int8_t* v_codes;
  const int32_t* meta;
  const int32_t* page_table;
  int64_t table_pitch;
  const int32_t* kv_lens;
  const int32_t* row_seq;    // nullable: query row -> sequence (extend); null = one row per sequence
  const int32_t* row_limit;  // nullable: keys visible to the row (causal limit); null = all of the sequence
  const int32_t* row_order;  // nullable: the rows in the order in which CTAs should take them (longest first)
  int32_t* out_q15;
  int8_t* out_codes;
  int32_t* out_absmax;
  int q_heads, kv_heads;
  int64_t num_pages;
  int max_kv_len;
  int s_max;  // key capacity of one CTA's slice (multiple of 32)
};

constexpr int kDecodeWarps = 8;
constexpr int kDecodeThreads = kDecodeWarps * 32;
static_assert(kDecodeThreads >= kD, "the output stage maps one thread to one d");
constexpr int kVPrefetchPages = 64;         // V pages per CTA requested into L2 during the exponential pass
constexpr int kRingSlot = kSlotBytes + 384; // a pair of pages plus their two scale blocks (2 x 160 B), 128-byte granular
// Both contractions run on the integer tensor-core MMA with the long dimension on M:
//   dots^T [16 keys x 8 heads] = K page [16 x 128] . Q^T [128 x 8]        (4 k-steps of 32 d)
//   out^T  [16 d    x 8 heads] = V^T [16 x 32 tokens] . W^T [32 x 8]      (two pages per k-step)
// so a page is exactly one M tile and the (<= 8) query heads of the group are the N columns.
// Every warp streams its own page pairs (first the K pairs of its share of the slice, then the V
// pairs) through a private ring of shared-memory slots filled by 16-byte asynchronous copies, so
// the loads of the next pair - including the first V pairs - are in flight while the warp
// computes and while the cluster exchanges the softmax statistics.  Each lane reads its MMA
// registers from the slot with 128-bit loads: K rows 32 contiguous bytes per lane (the d axis is
// permuted identically in Q; 16-byte columns are XOR-swizzled by the row parity on the way in),
// V in the operand order of v_chunk_offset.  The per-key fixed-point work (scale, exp, relative V
// scale, probability limbs) runs in flat one-thread-per-key loops between the two MMA phases.
// kStages = ring slots per warp (1 or 2).
template <int G, int kStages>
__global__ void __launch_bounds__(kDecodeThreads, 2)
attn_decode_kernel(const DecodeParams p) {
  pdl_launch_dependents();
  pdl_wait();          // the queries, lengths and the new K/V rows come from the kernels before this one
  cg::cluster_group cluster = cg::this_cluster();
  const int C = (int)cluster.num_blocks();
  const int rank = (int)cluster.block_rank();
  const int kh = blockIdx.y;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // Rows are best taken longest first: the hardware hands out CTAs in grid order (the KV heads of a row
  // together, then the next row), so the long rows start first and the short ones fill the tail of the
  // launch, and CTAs that share an SM are half a wave apart in that order, so their lengths differ and
  // their load and scalar phases interleave.  blockIdx.z is the position in that order: given by the
  // caller (row_order), ranked here for small batches, else as is.
  int b = blockIdx.z;
  if (p.row_order) {
    b = min(max(p.row_order[blockIdx.z], 0), (int)gridDim.z - 1);
  } else {
    const int rows = (int)gridDim.z;
    if (rows > 1 && rows <= 64) {
      __shared__ int len_s[64];
      __shared__ int order_s;
      if (tid < rows) {
        const int sq = p.row_seq ? p.row_seq[tid] : tid;
        int len = min(p.kv_lens[sq], p.max_kv_len);
        if (p.row_limit) len = min(len, p.row_limit[tid]);
        len_s[tid] = len;
      }
      __syncthreads();
      if (tid < rows) {
        const int mine = len_s[tid];
        int before = 0;
        for (int j = 0; j < rows; ++j) {
          const int v = len_s[j];
          before += (v > mine) || (v == mine && j < tid);
        }
        if (before == (int)blockIdx.z) order_s = tid;
      }
      __syncthreads();
      b = order_s;
    }
  }
  const int fr = lane >> 2, fc = lane & 3;   // fragment row / column-group of this lane
  const int S = p.s_max;
  constexpr int kNeg = (int)(-2147483647 - 1);

  extern __shared__ __align__(128) unsigned char smem_raw[];
  unsigned char* ring = smem_raw + warp * (kStages * kRingSlot);       // this warp's slots
  int32_t* sc = reinterpret_cast<int32_t*>(smem_raw + kDecodeWarps * kStages * kRingSlot);  // [G][S]
  uint8_t* w_hi = reinterpret_cast<uint8_t*>(sc + G * S) + warp * (2 * G * 32);  // [G][32]
  uint8_t* w_lo = w_hi + G * 32;                                      // [G][32] (this warp's pair)
  int32_t* pages = reinterpret_cast<int32_t*>(reinterpret_cast<uint8_t*>(sc + G * S) + kDecodeWarps * 2 * G * 32);  // [S / 16]

  __shared__ int q_mul_s[G], q_shift_s[G];
  __shared__ int cta_max[G];
  __shared__ unsigned long long cta_sum[G];
  __shared__ unsigned long long cta_vref;
  __shared__ int cta_acc[G][kD];
  __shared__ int g_max[G];
  __shared__ int g_inv[G];
  __shared__ int red_s[33];

  // b is the query row; its keys come from sequence `seq`.  In an extend batch a row sees only the
  // first `row_limit` keys, but the reference V scale is taken over all L_all keys of the sequence.
  const int seq = p.row_seq ? p.row_seq[b] : b;
  // A lone CTA's slice starts at page 0 whatever the length: its page ids are requested before the length
  // is known (one dependent memory round trip less); ids past the row's last page are never used.
  int64_t pid_early = 0;
  const int cap_pages = (int)min((int64_t)(S / kPage), p.table_pitch);
  if (C == 1 && tid < cap_pages) pid_early = p.page_table[(int64_t)seq * p.table_pitch + tid];
  const int L_all = max(0, min(p.kv_lens[seq], p.max_kv_len));
  const int L = p.row_limit ? max(0, min(p.row_limit[b], L_all)) : L_all;
  const int n_pages = (L + kPage - 1) / kPage;
  const int Ce = C;   // CTAs that work on this row
  // a CTA on its own needs no cluster barrier (and the plain one is cheaper)
  auto row_sync = [&]() { if (Ce > 1) cluster.sync(); else __syncthreads(); };
  const int ppc = (n_pages + Ce - 1) / Ce;               // pages per CTA
  const int pg0 = min(n_pages, rank * ppc);
  const int pg1 = min(n_pages, pg0 + ppc);
  const int my_pages = pg1 - pg0;
  const int key0 = pg0 * kPage;                          // first key of the slice
  const int my_keys = max(0, min(L, pg1 * kPage) - key0);  // valid keys in the slice
  const int n_pairs = (my_pages + 1) >> 1;
  const int n_slots = n_pairs * 32;
  const int n_items = warp < n_pairs ? (n_pairs - warp + kDecodeWarps - 1) / kDecodeWarps : 0;  // pairs of this warp

  // ---- set-up
  if (tid < G) {
    q_mul_s[tid] = p.q_mul[(int64_t)b * p.q_heads + kh * G + tid];
    q_shift_s[tid] = p.q_shift[(int64_t)b * p.q_heads + kh * G + tid];
    cta_max[tid] = kNeg;
    cta_sum[tid] = 0ull;
  }
  if (tid == 0) cta_vref = ~0ull;
  for (int i = tid; i < G * kD; i += kDecodeThreads) (&cta_acc[0][0])[i] = 0;
  for (int i = tid; i < my_pages; i += kDecodeThreads) {
    int64_t pid = (C == 1 && i < kDecodeThreads) ? pid_early : p.page_table[(int64_t)seq * p.table_pitch + pg0 + i];
    pid = pid < 0 ? 0 : (pid >= p.num_pages ? p.num_pages - 1 : pid);
    pages[i] = (int)pid;
  }
  // Q as the MMA's B operand: lane (fr, fc) holds bytes [32 fc, 32 fc + 32) of head fr
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

  // Item j of this warp: j < n_items is the K copy of pair (warp + j * warps), otherwise the V
  // copy of pair (warp + (j - n_items) * warps).  One commit group per item, also when empty.
  // A lane moves the 16-byte columns lane, lane+32, lane+64, lane+96 of each 2 KB chunk; the
  // pages' scale blocks (160 B each) travel behind the codes: whole with K (the K scales for the
  // scores, the V scales for the reference V scale), words 16..39 with V.
  const unsigned ring_base = (unsigned)__cvta_generic_to_shared(ring);
  unsigned k_dst[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int ch = lane + 32 * i;
    k_dst[i] = ((ch >> 3) << 7) | (((ch & 7) ^ ((ch >> 3) & 1)) << 4);
  }
  const int64_t head_off = (int64_t)kh * (kPage * kD) + (lane << 4);
  const int64_t page_stride = (int64_t)p.kv_heads * (kPage * kD);
  auto issue_k = [&](int it) {   // it-th K pair of this warp
    if (it < n_items) {
      const int pp = warp + it * kDecodeWarps;
      const unsigned slot = ring_base + (it % kStages) * kRingSlot;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        if (2 * pp + h < my_pages) {
          const unsigned char* src = reinterpret_cast<const unsigned char*>(p.k_codes) + pages[2 * pp + h] * page_stride + head_off;
#pragma unroll
          for (int i = 0; i < 4; ++i) cp_async16(slot + h * 2048 + k_dst[i], src + i * 512);
        }
      }
      if (lane < 20) {
        const int h = lane >= 10, c16 = lane - 10 * h;
        if (2 * pp + h < my_pages)
          cp_async16(slot + kSlotBytes + h * kMetaBytes + c16 * 16,
                     reinterpret_cast<const unsigned char*>(p.meta + ((int64_t)pages[2 * pp + h] * p.kv_heads + kh) * kMetaWords) + c16 * 16);
      }
    }
    cp_async_commit();
  };
  auto issue_v = [&](int it) {   // it-th V pair of this warp
    if (it < n_items) {
      const int pp = warp + it * kDecodeWarps;
      const unsigned slot0 = ring_base + (it % kStages) * kRingSlot;
      const unsigned slot = slot0 + (lane << 4);
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        if (2 * pp + h < my_pages) {
          const unsigned char* src = reinterpret_cast<const unsigned char*>(p.v_codes) + pages[2 * pp + h] * page_stride + head_off;
#pragma unroll
          for (int i = 0; i < 4; ++i) cp_async16(slot + h * 2048 + i * 512, src + i * 512);
        }
      }
      if (lane < 12) {
        const int h = lane >= 6, c16 = 4 + lane - 6 * h;     // words 16..39: V multipliers and shifts
        if (2 * pp + h < my_pages)
          cp_async16(slot0 + kSlotBytes + h * kMetaBytes + c16 * 16,
                     reinterpret_cast<const unsigned char*>(p.meta + ((int64_t)pages[2 * pp + h] * p.kv_heads + kh) * kMetaWords) + c16 * 16);
      }
    }
    cp_async_commit();
  };
#pragma unroll
  for (int j = 0; j < kStages; ++j) issue_k(j);

  // ---- phase 1: one page (16 keys) per MMA tile gives raw int32 dots; then, one key per lane,
  // the Q15.16 scores of the pair, their running maximum and the reference V scale
  {
    const bool h0 = 2 * fc < G, h1 = 2 * fc + 1 < G;
    int32_t* sc0 = sc + (2 * fc) * S + fr;
    int32_t* sc1 = sc0 + S;
    const int o0 = ((2 * fc) ^ (fr & 1)) << 4, o1 = ((2 * fc + 1) ^ (fr & 1)) << 4;
    int lmax[G], qm[G], qs[G];
#pragma unroll
    for (int g = 0; g < G; ++g) { lmax[g] = kNeg; qm[g] = q_mul_s[g]; qs[g] = q_shift_s[g] - 48; }
    int best_s = 0x7fffffff;
    unsigned best_m = 0;
    for (int it = 0; it < n_items; ++it) {
      const int pp = warp + it * kDecodeWarps;
      cp_async_wait<kStages - 1>();
      __syncwarp();
      const unsigned char* slot0 = ring + (it % kStages) * kRingSlot;
      const unsigned char* slot = slot0 + fr * 128;   // rows fr, fr + 8: same parity
      // everything the pair needs moves to registers first, so that the slot can be refilled while the
      // warp is still busy with this pair
      uint4 kq[2][4];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const unsigned char* r0 = slot + h * 2048;
        kq[h][0] = *reinterpret_cast<const uint4*>(r0 + o0);
        kq[h][1] = *reinterpret_cast<const uint4*>(r0 + o1);
        kq[h][2] = *reinterpret_cast<const uint4*>(r0 + 1024 + o0);
        kq[h][3] = *reinterpret_cast<const uint4*>(r0 + 1024 + o1);
      }
      const int kl = pp * 32 + lane;
      int km = 0, ks = 0, vs = 0;
      unsigned vm = 0;
      if (kl < my_keys) {   // this lane's key: its scales
        const int32_t* mt = reinterpret_cast<const int32_t*>(slot0 + kSlotBytes + (lane >> 4) * kMetaBytes);
        const int tok = lane & 15;
        km = mt[tok];
        ks = reinterpret_cast<const int8_t*>(mt + 32)[tok];
        vm = (unsigned)mt[16 + tok];
        vs = reinterpret_cast<const int8_t*>(mt + 36)[tok];
      }
      __syncwarp();
      issue_k(it + kStages);     // the slot is free again
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        int c[4] = {0, 0, 0, 0};
        if (2 * pp + h < my_pages) {   // (a page that was not copied leaves stale bytes in the registers: unused)
          const uint4 k00 = kq[h][0], k01 = kq[h][1], k10 = kq[h][2], k11 = kq[h][3];
          mma_s8s8(c, k00.x, k10.x, k00.y, k10.y, qw[0], qw[1]);
          mma_s8s8(c, k00.z, k10.z, k00.w, k10.w, qw[2], qw[3]);
          mma_s8s8(c, k01.x, k11.x, k01.y, k11.y, qw[4], qw[5]);
          mma_s8s8(c, k01.z, k11.z, k01.w, k11.w, qw[6], qw[7]);
        }
        // c[0]: (key fr, head 2fc)  c[1]: (fr, 2fc+1)  c[2]: (fr + 8, 2fc)  c[3]: (fr + 8, 2fc+1)
        const int kp = (2 * pp + h) * 16;
        if (h0) { sc0[kp] = c[0]; sc0[kp + 8] = c[2]; }
        if (h1) { sc1[kp] = c[1]; sc1[kp + 8] = c[3]; }
      }
      __syncwarp();              // the pair's raw dots are in place for the lane-per-key pass
      if (kl < my_keys) {
        if (vs < best_s || (vs == best_s && vm > best_m)) { best_s = vs; best_m = vm; }
#pragma unroll
        for (int g = 0; g < G; ++g) {
          const int v = mul_shift_sat32(sc[g * S + kl], __mulhi(qm[g], km), qs[g] + ks);
          sc[g * S + kl] = v;
          lmax[g] = max(lmax[g], v);
        }
      }
    }
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const int m = warp_max(lmax[g]);
      if (lane == 0) atomicMax(&cta_max[g], m);
    }
    unsigned long long lvref = best_s == 0x7fffffff
                                   ? ~0ull
                                   : (((unsigned long long)(unsigned)(best_s + 128) << 32) | (unsigned long long)(0xFFFFFFFFu - best_m));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const unsigned long long other = __shfl_xor_sync(FULL_MASK, lvref, o);
      lvref = other < lvref ? other : lvref;
    }
    if (lane == 0) atomicMin(&cta_vref, lvref);
  }
  if (rank == 0 && L_all > L) {   // extend rows: keys behind the causal limit still count for the V reference scale
    unsigned long long lv = ~0ull;
    for (int key = L + tid; key < L_all; key += kDecodeThreads) {
      int64_t pid = p.page_table[(int64_t)seq * p.table_pitch + (key >> 4)];
      pid = pid < 0 ? 0 : (pid >= p.num_pages ? p.num_pages - 1 : pid);
      const int32_t* mt = p.meta + (pid * p.kv_heads + kh) * kMetaWords;
      const unsigned vm = (unsigned)__ldg(mt + 16 + (key & 15));
      const int vs = reinterpret_cast<const int8_t*>(mt + 36)[key & 15];
      const unsigned long long vkey = ((unsigned long long)(unsigned)(vs + 128) << 32) | (unsigned long long)(0xFFFFFFFFu - vm);
      lv = vkey < lv ? vkey : lv;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const unsigned long long other = __shfl_xor_sync(FULL_MASK, lv, o);
      lv = other < lv ? other : lv;
    }
    if (lane == 0) atomicMin(&cta_vref, lv);
  }
  // The first V pairs are requested between the two halves of the cluster barrier: the release fence
  // of the arrival would otherwise wait for copies that are still in flight.
  if (Ce > 1) cluster.barrier_arrive(); else __syncthreads();
#pragma unroll
  for (int j = 0; j < kStages; ++j) issue_v(j);
  if (Ce > 1) cluster.barrier_wait();

  // ---- exchange 1: row maxima and the V reference scale over the cluster
  if (tid < G) {
    int m = kNeg;
    for (int r = 0; r < Ce; ++r) m = max(m, *cluster.map_shared_rank(&cta_max[tid], r));
    g_max[tid] = m;
  }
  unsigned long long vref = ~0ull;
  for (int r = 0; r < Ce; ++r) {
    const unsigned long long o = *cluster.map_shared_rank(&cta_vref, r);
    vref = o < vref ? o : vref;
  }
  const int v_shift_ref = (int)(vref >> 32) - 128;
  const int v_mul_ref = (int)(0xFFFFFFFFu - (unsigned)(vref & 0xFFFFFFFFull));
  __syncthreads();

  // ---- phase 2: exponentials and their sum
  // HBM idles while the CTAs of a wave, which start together, all sit in this scalar pass: ask L2 for the first
  // V pages of the slice meanwhile (one 2 KB request per thread; 64 pages per CTA keep the resident CTAs'
  // requests well inside L2 - 256 pages per CTA evicted them again and cost 8 %)
  for (int i = tid; i < min(my_pages, kVPrefetchPages); i += kDecodeThreads) {
    const unsigned char* src = reinterpret_cast<const unsigned char*>(p.v_codes) + pages[i] * page_stride + (int64_t)kh * (kPage * kD);
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], 2048;" ::"l"(src) : "memory");
  }
  {
    int lsum[G];   // a thread sees at most S / threads keys, each e <= 2^16: no overflow
    int gm[G];
#pragma unroll
    for (int g = 0; g < G; ++g) { lsum[g] = 0; gm[g] = g_max[g]; }
    // two keys per trip with all loads first: the trips' shared-memory stores would otherwise
    // serialise them (the compiler cannot prove sc[g*S+kl] and sc[g'*S+kl'] distinct)
    for (int kl = tid; kl < n_slots; kl += 2 * kDecodeThreads) {
      const int kl2 = kl + kDecodeThreads;
      const bool in2 = kl2 < n_slots;
      const bool valid1 = kl < my_keys, valid2 = in2 && kl2 < my_keys;
      int s1[G], s2[G];
#pragma unroll
      for (int g = 0; g < G; ++g) {
        s1[g] = valid1 ? sc[g * S + kl] : 0;
        s2[g] = valid2 ? sc[g * S + kl2] : 0;
      }
#pragma unroll
      for (int g = 0; g < G; ++g) {
        int e1 = 0, e2 = 0;
        if (valid1) {
          const int x = max(sub_sat(s1[g], gm[g]), -(1 << 30));                   // <= 0
          const long long prod = (long long)x * 94548LL;                          // y = prod >> 16
          e1 = __ldg(&g_exp2_attn_lut[((unsigned)prod) >> 22]) >> min(31, 13 - (int)(prod >> 32));
        }
        if (valid2) {
          const int x = max(sub_sat(s2[g], gm[g]), -(1 << 30));
          const long long prod = (long long)x * 94548LL;
          e2 = __ldg(&g_exp2_attn_lut[((unsigned)prod) >> 22]) >> min(31, 13 - (int)(prod >> 32));
        }
        s1[g] = e1; s2[g] = e2;
        lsum[g] += e1 + e2;
      }
#pragma unroll
      for (int g = 0; g < G; ++g) {
        sc[g * S + kl] = s1[g];
        if (in2) sc[g * S + kl2] = s2[g];
      }
    }
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const long long s = warp_sum64((long long)lsum[g]);
      if (lane == 0) atomicAdd(&cta_sum[g], (unsigned long long)s);
    }
  }
  row_sync();

  // ---- exchange 2: total of the exponentials -> inv = (2^31 - 1) / max(1, total)
  if (tid < G) {
    unsigned long long tot = 0;
    for (int r = 0; r < Ce; ++r) tot += *cluster.map_shared_rank(&cta_sum[tid], r);
    if (tot < 1ull) tot = 1ull;
    g_inv[tid] = (int)(2147483647ull / tot);
  }
  __syncthreads();

  // ---- phase 3: per pair, one key per lane turns the exponentials into probabilities (Q0.15)
  // folded with the relative V scale, as two byte limbs; then PV, two pages (32 tokens) per
  // k-step, 8 d-tiles of 16.  The key holding the row maximum contributes e = 2^16, so the
  // total is >= 2^16 and inv <= 32767: e * inv < 2^31 and p * rel < 2^31, 32-bit arithmetic is exact.
  {
    unsigned gi[G];
#pragma unroll
    for (int g = 0; g < G; ++g) gi[g] = (unsigned)g_inv[g];
    int acc_hi[8][4], acc_lo[8][4];
#pragma unroll
    for (int m = 0; m < 8; ++m)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc_hi[m][j] = acc_lo[m][j] = 0;
    const uint8_t* ph = w_hi + fr * 32 + fc * 4;
    const uint8_t* pl = w_lo + fr * 32 + fc * 4;
    for (int it = 0; it < n_items; ++it) {
      const int pp = warp + it * kDecodeWarps;
      const int kl = pp * 32 + lane;
      unsigned pr[G];
#pragma unroll
      for (int g = 0; g < G; ++g) pr[g] = ((unsigned)sc[g * S + kl] * gi[g]) >> 16;   // 0 for keys past the end
      cp_async_wait<kStages - 1>();
      __syncwarp();
      const unsigned char* slot0 = ring + (it % kStages) * kRingSlot;
      // V operands and this lane's key scales go to registers, then the slot is refilled at once
      const unsigned char* slot = slot0 + lane * 16;
      const bool has_b = 2 * pp + 1 < my_pages;
      uint4 va[4], vb[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        va[i] = *reinterpret_cast<const uint4*>(slot + i * 512);
        vb[i] = has_b ? *reinterpret_cast<const uint4*>(slot + 2048 + i * 512) : make_uint4(0, 0, 0, 0);
      }
      const int32_t* mt = reinterpret_cast<const int32_t*>(slot0 + kSlotBytes + (lane >> 4) * kMetaBytes);
      const unsigned vm = (unsigned)mt[16 + (lane & 15)];
      const int vs = reinterpret_cast<const int8_t*>(mt + 36)[lane & 15];
      __syncwarp();
      issue_v(it + kStages);
      {
        // this lane's key: relative V scale from the scale block that came with the codes
        // (stale bytes for a key past the end: its probability is 0, so is its weight)
        const unsigned r = kl < my_keys ? rel_scale_q15(vm, (unsigned)v_mul_ref, vs - v_shift_ref) : 0u;
#pragma unroll
        for (int g = 0; g < G; ++g) {
          const unsigned w = (pr[g] * r + 16384u) >> 15;
          w_hi[g * 32 + lane] = (uint8_t)(w >> 8);
          w_lo[g * 32 + lane] = (uint8_t)(w & 0xff);
        }
      }
      __syncwarp();
      unsigned bh0 = 0, bh1 = 0, bl0 = 0, bl1 = 0;   // W^T: head fr, tokens 4 fc .. of page A / B
      if (fr < G) {
        bh0 = *reinterpret_cast<const unsigned*>(ph);
        bh1 = *reinterpret_cast<const unsigned*>(ph + 16);
        bl0 = *reinterpret_cast<const unsigned*>(pl);
        bl1 = *reinterpret_cast<const unsigned*>(pl + 16);
      }
#pragma unroll
      for (int m = 0; m < 8; ++m) {
        const unsigned a0 = word_of(va, 2 * m), a1 = word_of(va, 2 * m + 1);
        const unsigned a2 = word_of(vb, 2 * m), a3 = word_of(vb, 2 * m + 1);
        mma_s8u8(acc_hi[m], a0, a1, a2, a3, bh0, bh1);
        mma_s8u8(acc_lo[m], a0, a1, a2, a3, bl0, bl1);
      }
      __syncwarp();              // the limb bytes are rewritten by the next pair
    }
    cp_async_wait<0>();
    // C tile: [0] (d = 16m + fr, head 2fc)  [1] (.., 2fc+1)  [2] (d + 8, 2fc)  [3] (d + 8, 2fc+1)
#pragma unroll
    for (int m = 0; m < 8; ++m)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int head = 2 * fc + (j & 1);
        const int d = 16 * m + fr + 8 * (j >> 1);
        const int v = acc_hi[m][j] * 256 + acc_lo[m][j];
        if (head < G && v != 0) atomicAdd(&cta_acc[head][d], v);
      }
  }
  row_sync();

  // ---- exchange 3: head g is finished by rank g % C: sum the partial outputs of all CTAs over
  // distributed shared memory, requantise, and (for the int8 output) quantise the 128-wide row
  {
    static_assert(kDecodeThreads == 2 * kD, "two heads are finished at a time, 128 threads each");
    const int d = tid & (kD - 1);
    const int sub = tid >> 7;                          // which of the two heads in flight
    const int my_heads = (G - rank + Ce - 1) / Ce;     // heads rank, rank + Ce, ...: uniform per CTA
    for (int i0 = 0; i0 < my_heads; i0 += 2) {
      const int hi = i0 + sub;
      const bool act = hi < my_heads;
      const int g = rank + hi * Ce;
      const int64_t row = ((int64_t)b * p.q_heads + kh * G + g) * kD;
      int o = 0;
      if (act) {
        long long a = 0;
        for (int r = 0; r < Ce; ++r) a += *cluster.map_shared_rank(&cta_acc[g][d], r);
        o = L > 0 ? mul_shift_sat32_wide(a, v_mul_ref, v_shift_ref - 1) : 0;
        if (p.out_q15) p.out_q15[row + d] = o;
      }
      if (p.out_codes) {   // row quant of the head: its 128 values sit in four warps
        const int wm = warp_max(abs_wrap(o));
        if (lane == 0) red_s[warp] = wm;
        __syncthreads();
        const int m = max(1, max(max(red_s[4 * sub], red_s[4 * sub + 1]), max(red_s[4 * sub + 2], red_s[4 * sub + 3])));
        if (act) {
          p.out_codes[row + d] = (int8_t)quant_code(o, __int2float_rn(m));
          if (d == 0) p.out_absmax[(int64_t)b * p.q_heads + kh * G + g] = m;
        }
        __syncthreads();   // red_s is rewritten by the next pair of heads
      }
    }
  }
  row_sync();  // nobody leaves while a peer still reads its shared memory
}

static size_t decode_smem_bytes(int G, int s_max, int stages) {
  return (size_t)kDecodeWarps * stages * kRingSlot + (size_t)G * s_max * 4 + (size_t)(s_max / 16) * 4 +
         (size_t)kDecodeWarps * 2 * G * 32;
}

template <int G, int kStages>
static int launch_decode(const DecodeParams& p, int batch, int cluster, cudaStream_t st) {
  const size_t smem = decode_smem_bytes(G, p.s_max, kStages);
  if (smem > 200 * 1024) {
    set_error("attn_decode: max_kv_len=%d needs %zu bytes of shared memory per CTA; raise cluster", p.max_kv_len, smem);
    return B200_E_UNSUPPORTED;
  }
  cudaError_t e = cudaFuncSetAttribute(attn_decode_kernel<G, kStages>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) {
    set_error("attn_decode: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    return B200_E_CUDA;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(cluster, p.kv_heads, batch);
  cfg.blockDim = dim3(kDecodeThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cluster;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  e = cudaLaunchKernelEx(&cfg, attn_decode_kernel<G, kStages>, p);
  if (e != cudaSuccess) {
    set_error("attn_decode: launch: %s", cudaGetErrorString(e));
    return B200_E_CUDA;
  }
  return B200_OK;
}

}  // namespace b200

using namespace b200;

static int store_common(bool quant, const void* k, int64_t k_pitch, const void* v, int64_t v_pitch,
                        const int32_t* k_mul, const int32_t* k_shift, const int32_t* v_mul,
                        const int32_t* v_shift, const int32_t* out_loc, int8_t* k_codes, int8_t* v_codes,
                        int32_t* meta, int64_t tokens, int kv_heads, int64_t num_pages, cudaStream_t st,
                        const char* name) {
  B200_REQUIRE(k && v && out_loc && k_codes && v_codes && meta, B200_E_NULL, "%s: null pointer", name);
  B200_REQUIRE(tokens >= 0 && kv_heads > 0 && num_pages > 0, B200_E_SHAPE,
               "%s: tokens=%lld kv_heads=%d num_pages=%lld", name, (long long)tokens, kv_heads, (long long)num_pages);
  B200_REQUIRE(aligned16(k_codes) && aligned16(v_codes) && aligned16(meta), B200_E_ALIGN,
               "%s: pool buffers must be 16-byte aligned", name);
  if (quant) {
    B200_REQUIRE(aligned16(k) && aligned16(v) && k_pitch % 4 == 0 && v_pitch % 4 == 0, B200_E_ALIGN,
                 "%s: k/v rows must be 16-byte aligned", name);
    B200_REQUIRE(k_pitch >= (int64_t)kv_heads * kD && v_pitch >= (int64_t)kv_heads * kD, B200_E_SHAPE,
                 "%s: row pitch smaller than kv_heads*128", name);
  } else {
    B200_REQUIRE(k_mul && k_shift && v_mul && v_shift, B200_E_NULL, "%s: null scale pointer", name);
    B200_REQUIRE(((uintptr_t)k & 3u) == 0 && ((uintptr_t)v & 3u) == 0, B200_E_ALIGN, "%s: codes must be 4-byte aligned", name);
  }
  if (tokens == 0) return B200_OK;
  const int64_t blocks = (tokens * kv_heads + 7) / 8;
  B200_REQUIRE(blocks < (1ll << 31), B200_E_SHAPE, "%s: too many rows", name);
  if (quant)
    kv_store_kernel<true><<<(unsigned)blocks, 256, 0, st>>>(k, k_pitch, v, v_pitch, nullptr, nullptr, nullptr, nullptr,
                                                           out_loc, k_codes, v_codes, meta, tokens, kv_heads, num_pages);
  else
    kv_store_kernel<false><<<(unsigned)blocks, 256, 0, st>>>(k, 0, v, 0, k_mul, k_shift, v_mul, v_shift, out_loc,
                                                            k_codes, v_codes, meta, tokens, kv_heads, num_pages);
  return check_launch(name);
}

extern "C" int b200_qkv_prepare_q15(const int32_t* positions, const int32_t* q, int64_t q_pitch, const int32_t* k,
                                    int64_t k_pitch, const int32_t* v, int64_t v_pitch, const int32_t* cos_sin,
                                    int max_pos, const int32_t* q_norm_w, const int32_t* k_norm_w,
                                    const int32_t* out_loc, int8_t* k_codes, int8_t* v_codes, int32_t* meta,
                                    int8_t* q8, int32_t* q_mul, int32_t* q_shift, int64_t tokens, int q_heads,
                                    int kv_heads, int64_t num_pages, int with_fwht, b200_stream_t s) {
  B200_REQUIRE(tokens >= 0 && q_heads > 0 && kv_heads > 0 && max_pos > 0 && num_pages > 0, B200_E_SHAPE,
               "qkv_prepare_q15: tokens=%lld q_heads=%d kv_heads=%d max_pos=%d num_pages=%lld", (long long)tokens, q_heads,
               kv_heads, max_pos, (long long)num_pages);
  if (tokens == 0) return B200_OK;
  B200_REQUIRE(positions && q && k && v && cos_sin && out_loc && k_codes && v_codes && meta && q8 && q_mul && q_shift,
               B200_E_NULL, "qkv_prepare_q15: null pointer");
  B200_REQUIRE(q_pitch >= (int64_t)q_heads * kD && k_pitch >= (int64_t)kv_heads * kD && v_pitch >= (int64_t)kv_heads * kD,
               B200_E_SHAPE, "qkv_prepare_q15: row pitch smaller than heads*128");
  auto a8 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 7u) == 0; };
  B200_REQUIRE(a8(q) && a8(k) && aligned16(v) && a8(cos_sin) && a8(q_norm_w) && a8(k_norm_w) && q_pitch % 2 == 0 &&
                   k_pitch % 2 == 0 && v_pitch % 4 == 0 && aligned16(k_codes) && aligned16(v_codes) && aligned16(meta) &&
                   (reinterpret_cast<uintptr_t>(q8) & 3u) == 0,
               B200_E_ALIGN, "qkv_prepare_q15: q/k rows 8-byte, v rows and pool buffers 16-byte, q8 4-byte aligned");
  const int64_t warps = tokens * (q_heads + 2 * kv_heads);
  const int64_t blocks = (warps + 7) / 8;
  B200_REQUIRE(blocks < (1ll << 31), B200_E_SHAPE, "qkv_prepare_q15: too many rows");
  const PendingLinear none = {nullptr, nullptr, nullptr, nullptr};
  launch_pdl(qkv_prepare_kernel<false>, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)s, positions, q, q_pitch, k, k_pitch, v, v_pitch, cos_sin,
                                                                    max_pos, q_norm_w, k_norm_w, out_loc, k_codes, v_codes,
                                                                    meta, q8, q_mul, q_shift, tokens, q_heads, kv_heads,
                                                                    num_pages, with_fwht, none);
  return check_launch("qkv_prepare_q15");
}

extern "C" int b200_qkv_prepare_pending(const int32_t* positions, int32_t* acc, const int32_t* x_absmax, const int32_t* w_mul,
                                        const int32_t* w_shift, const int32_t* cos_sin, int max_pos, const int32_t* q_norm_w,
                                        const int32_t* k_norm_w, const int32_t* out_loc, int8_t* k_codes, int8_t* v_codes,
                                        int32_t* meta, int8_t* q8, int32_t* q_mul, int32_t* q_shift, int64_t tokens,
                                        int q_heads, int kv_heads, int64_t num_pages, int with_fwht, b200_stream_t s) {
  B200_REQUIRE(tokens >= 0 && q_heads > 0 && kv_heads > 0 && max_pos > 0 && num_pages > 0, B200_E_SHAPE,
               "qkv_prepare_pending: tokens=%lld q_heads=%d kv_heads=%d max_pos=%d num_pages=%lld", (long long)tokens,
               q_heads, kv_heads, max_pos, (long long)num_pages);
  if (tokens == 0) return B200_OK;
  B200_REQUIRE(positions && acc && x_absmax && w_mul && cos_sin && out_loc && k_codes && v_codes && meta && q8 && q_mul &&
                   q_shift, B200_E_NULL, "qkv_prepare_pending: null pointer");
  auto a8 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 7u) == 0; };
  B200_REQUIRE(aligned16(acc) && aligned16(w_mul) && aligned16(w_shift) && a8(cos_sin) && a8(q_norm_w) && a8(k_norm_w) &&
                   aligned16(k_codes) && aligned16(v_codes) && aligned16(meta) && (reinterpret_cast<uintptr_t>(q8) & 3u) == 0,
               B200_E_ALIGN, "qkv_prepare_pending: acc, scales and pool buffers 16-byte, norm weights 8-byte, q8 4-byte aligned");
  const int64_t warps = tokens * (q_heads + 2 * kv_heads);
  const int64_t blocks = (warps + 7) / 8;
  B200_REQUIRE(blocks < (1ll << 31), B200_E_SHAPE, "qkv_prepare_pending: too many rows");
  const PendingLinear pl = {acc, x_absmax, w_mul, w_shift};
  launch_pdl(qkv_prepare_kernel<true>, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)s, positions, (const int32_t*)nullptr,
             (int64_t)0, (const int32_t*)nullptr, (int64_t)0, (const int32_t*)nullptr, (int64_t)0, cos_sin, max_pos, q_norm_w,
             k_norm_w, out_loc, k_codes, v_codes, meta, q8, q_mul, q_shift, tokens, q_heads, kv_heads, num_pages, with_fwht, pl);
  return check_launch("qkv_prepare_pending");
}

extern "C" int b200_kv_store_q15(const int32_t* k, int64_t k_pitch, const int32_t* v, int64_t v_pitch,
                                 const int32_t* out_loc, int8_t* k_codes, int8_t* v_codes, int32_t* meta,
                                 int64_t tokens, int kv_heads, int64_t num_pages, b200_stream_t s) {
  return store_common(true, k, k_pitch, v, v_pitch, nullptr, nullptr, nullptr, nullptr, out_loc, k_codes, v_codes,
                      meta, tokens, kv_heads, num_pages, (cudaStream_t)s, "kv_store_q15");
}

extern "C" int b200_kv_store_codes(const int8_t* k8, const int8_t* v8, const int32_t* k_mul,
                                   const int32_t* k_shift, const int32_t* v_mul, const int32_t* v_shift,
                                   const int32_t* out_loc, int8_t* k_codes, int8_t* v_codes, int32_t* meta,
                                   int64_t tokens, int kv_heads, int64_t num_pages, b200_stream_t s) {
  return store_common(false, k8, 0, v8, 0, k_mul, k_shift, v_mul, v_shift, out_loc, k_codes, v_codes, meta, tokens,
                      kv_heads, num_pages, (cudaStream_t)s, "kv_store_codes");
}

static int attn_common(const int8_t* q, const int32_t* q_mul, const int32_t* q_shift,
                       const int8_t* k_codes, const int8_t* v_codes, const int32_t* meta,
                       const int32_t* page_table, int64_t table_pitch, const int32_t* kv_lens,
                       const int32_t* row_seq, const int32_t* row_limit, const int32_t* row_order,
                       int32_t* out_q15, int8_t* out_codes, int32_t* out_absmax, int batch,
                       int q_heads, int kv_heads, int64_t num_pages, int max_kv_len, int cluster,
                       b200_stream_t s) {
  B200_REQUIRE(q && q_mul && q_shift && k_codes && v_codes && meta && page_table && kv_lens, B200_E_NULL,
               "attn_decode: null pointer");
  B200_REQUIRE((out_codes == nullptr) == (out_absmax == nullptr), B200_E_NULL,
               "attn_decode: out_codes and out_absmax must be given together");
  B200_REQUIRE(out_q15 || out_codes, B200_E_NULL, "attn_decode: no output requested");
  B200_REQUIRE(batch >= 0 && batch <= 65535 && q_heads > 0 && kv_heads > 0 && kv_heads <= 65535 && num_pages > 0 &&
                   max_kv_len > 0,
               B200_E_SHAPE, "attn_decode: batch=%d q_heads=%d kv_heads=%d num_pages=%lld max_kv_len=%d", batch,
               q_heads, kv_heads, (long long)num_pages, max_kv_len);
  B200_REQUIRE(q_heads % kv_heads == 0, B200_E_SHAPE, "attn_decode: q_heads=%d not a multiple of kv_heads=%d", q_heads, kv_heads);
  const int G = q_heads / kv_heads;
  B200_REQUIRE(G == 1 || G == 2 || G == 4 || G == 8, B200_E_UNSUPPORTED, "attn_decode: group size %d (1, 2, 4 or 8)", G);
  const int max_pages = (max_kv_len + kPage - 1) / kPage;
  B200_REQUIRE(table_pitch >= max_pages, B200_E_SHAPE, "attn_decode: table_pitch=%lld < pages for max_kv_len (%d)",
               (long long)table_pitch, max_pages);
  B200_REQUIRE(aligned16(q) && aligned16(k_codes) && aligned16(v_codes) && aligned16(meta), B200_E_ALIGN,
               "attn_decode: q and pool buffers must be 16-byte aligned");
  // Configuration: the per-CTA fixed work (set-up, exchanges) is paid once per CTA, so the fewest CTAs per
  // (row, KV head) whose slice state still lets two CTAs share an SM win; one CTA with single ring slots
  // is preferred, then the smallest cluster with two slots per warp, then whatever fits at all.
  auto slice_keys = [&](int c) { return ((((max_pages + c - 1) / c) * kPage + 31) / 32) * 32; };
  // Configuration.  Set-up, barriers and the final exchange are paid per CTA and a lone CTA needs no
  // cluster barrier, so one CTA per (row, KV head) wins whenever its slice state lets two CTAs share an
  // SM - with two ring slots per warp if that still fits, else one; longer contexts take the smallest
  // cluster whose slices fit at all (fewer CTAs beat deeper rings in every measurement).
  const int G_static = 1536 + G * kD * 4 + 1024;   // the kernel's static shared arrays plus the per-CTA reserve
  const size_t two_per_sm = (size_t)(233472 / 2 - G_static);
  auto fits2 = [&](int c, int st) { return decode_smem_bytes(G, slice_keys(c), st) <= two_per_sm; };
  int stages;
  if (cluster == 0) {
    cluster = 1;
    while (cluster < 8 && !fits2(cluster, 1)) cluster *= 2;   // fewest CTAs per row first, ring depth second
    stages = fits2(cluster, 2) ? 2 : 1;
  } else {
    B200_REQUIRE(cluster == 1 || cluster == 2 || cluster == 4 || cluster == 8, B200_E_UNSUPPORTED,
                 "attn_decode: cluster=%d (1, 2, 4 or 8)", cluster);
    stages = fits2(cluster, 2) ? 2 : 1;
  }
  const int s_max = slice_keys(cluster);
  if (batch == 0) return B200_OK;
  DecodeParams p;
  p.q = q; p.q_mul = q_mul; p.q_shift = q_shift; p.k_codes = k_codes; p.v_codes = v_codes; p.meta = meta;
  p.page_table = page_table; p.table_pitch = table_pitch; p.kv_lens = kv_lens; p.out_q15 = out_q15;
  p.out_codes = out_codes; p.out_absmax = out_absmax; p.q_heads = q_heads; p.kv_heads = kv_heads;
  p.num_pages = num_pages; p.max_kv_len = max_kv_len; p.row_seq = row_seq; p.row_limit = row_limit; p.row_order = row_order;
  p.s_max = s_max;
  cudaStream_t st = (cudaStream_t)s;
  switch (G) {
    case 1: return stages == 1 ? launch_decode<1, 1>(p, batch, cluster, st) : launch_decode<1, 2>(p, batch, cluster, st);
    case 2: return stages == 1 ? launch_decode<2, 1>(p, batch, cluster, st) : launch_decode<2, 2>(p, batch, cluster, st);
    case 4: return stages == 1 ? launch_decode<4, 1>(p, batch, cluster, st) : launch_decode<4, 2>(p, batch, cluster, st);
    default: return stages == 1 ? launch_decode<8, 1>(p, batch, cluster, st) : launch_decode<8, 2>(p, batch, cluster, st);
  }
}

extern "C" int b200_attn_decode(const int8_t* q, const int32_t* q_mul, const int32_t* q_shift,
                                const int8_t* k_codes, const int8_t* v_codes, const int32_t* meta,
                                const int32_t* page_table, int64_t table_pitch, const int32_t* kv_lens,
                                const int32_t* row_order,
                                int32_t* out_q15, int8_t* out_codes, int32_t* out_absmax, int batch,
                                int q_heads, int kv_heads, int64_t num_pages, int max_kv_len, int cluster,
                                b200_stream_t s) {
  return attn_common(q, q_mul, q_shift, k_codes, v_codes, meta, page_table, table_pitch, kv_lens, nullptr, nullptr, row_order,
                     out_q15, out_codes, out_absmax, batch, q_heads, kv_heads, num_pages, max_kv_len, cluster, s);
}

extern "C" int b200_attn_extend(const int8_t* q, const int32_t* q_mul, const int32_t* q_shift,
                                const int8_t* k_codes, const int8_t* v_codes, const int32_t* meta,
                                const int32_t* page_table, int64_t table_pitch, const int32_t* kv_lens,
                                const int32_t* row_seq, const int32_t* row_limit,
                                int32_t* out_q15, int8_t* out_codes, int32_t* out_absmax, int rows,
                                int q_heads, int kv_heads, int64_t num_pages, int max_kv_len, int cluster,
                                b200_stream_t s) {
  B200_REQUIRE(row_seq && row_limit, B200_E_NULL, "attn_extend: row_seq or row_limit is null");
  return attn_common(q, q_mul, q_shift, k_codes, v_codes, meta, page_table, table_pitch, kv_lens, row_seq, row_limit, nullptr,
                     out_q15, out_codes, out_absmax, rows, q_heads, kv_heads, num_pages, max_kv_len, cluster, s);
}
