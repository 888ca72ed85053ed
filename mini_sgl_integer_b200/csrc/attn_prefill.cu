// Prefill / extend attention over the int8 paged pool: many new tokens per sequence, causal inside the new
// tokens, a cached prefix in front of them.  Same arithmetic as the decode kernel (attn.cu), bit for bit.
//
// A CTA owns one (sequence, KV head, tile of 128 / G consecutive new tokens): 128 query rows = tokens x the G
// query heads of the KV head, 16 rows per warp.  The integer MMA runs with the QUERY rows on M:
//   scores [16 rows x 8 keys]  = Q [16 x 128] . K^T [128 x 8]        (4 k-steps of 32 d; Q stays in registers)
//   out    [16 rows x 8 d]     = W [16 x 32 keys] . V [32 x 8]       (one k-step per pair of pages, 16 d-tiles)
// The 8 columns of a score tile are mapped to the keys {4c, 4c+1} (first tile of a page) and {4c+2, 4c+3} (second
// tile) for column pair c, so a lane ends up with the scores of the keys 4c .. 4c+3 of a page for its two rows:
// exactly the bytes its A operand of the PV product needs (the probability limbs never leave registers), and the
// V page is read as the B operand straight from the pool's operand order (v_chunk_offset).
//
// The softmax is exact (LUT exponential with truncation), so nothing can be rescaled on the fly: the keys are
// walked three times per tile - row maxima, sums of exponentials, then probabilities and PV - and the scores
// are recomputed each time (16 MMAs per 32 keys, negligible beside the per-score fixed-point work).  Keeping
// them instead would take 4 B x 128 rows per key: 2 MB for 4096 keys, beyond shared and tensor memory.  K is
// therefore read three times and V once per tile, from L2 after the first touch (a sequence's K and V for one
// head are 256 B per key); HBM sees every K and V page about once per (sequence, KV head).
// All CTAs of a launch stream the pages through a shared-memory ring filled by 16-byte asynchronous copies.
#include "attn_common.cuh"
#include "luts.cuh"

namespace b200 {

struct PrefillParams {
  const int8_t* q;
  const int32_t* q_mul;
  const int32_t* q_shift;
  const int8_t* k_codes;
  const int8_t* v_codes;
  const int32_t* meta;
  const int32_t* page_table;
  int64_t table_pitch;
  const int32_t* kv_lens;   // [batch] keys per sequence including the new tokens
  const int32_t* q_lens;    // [batch] new tokens per sequence
  const int32_t* q_start;   // [batch] row of the sequence's first new token in q / out
  int32_t* out_q15;
  int8_t* out_codes;
  int32_t* out_absmax;
  int q_heads, kv_heads;
  int64_t num_pages;
  int max_kv_len;
};

constexpr int kPfWarps = 8;
constexpr int kPfThreads = kPfWarps * 32;
constexpr int kPfRows = kPfWarps * 16;             // query rows per CTA
constexpr int kPfStages = 4;
constexpr int kPfStageBytes = 4096 + 4096 + 384;   // K pair (swizzled rows), V pair (operand order), two scale blocks
constexpr int kPfNeg = (int)(-2147483647 - 1);

__device__ __forceinline__ void mma_u8s8(int (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// exp of the decode kernel: LUT[(y & 0xffff) >> 6] >> min(31, 13 - (y >> 16)), y = (x * 94548) >> 16, x <= 0
__device__ __forceinline__ int pf_exp(int score, int row_max) {
  const int x = max(sub_sat(score, row_max), -(1 << 30));
  const long long prod = (long long)x * 94548LL;
  return __ldg(&g_exp2_attn_lut[((unsigned)prod) >> 22]) >> min(31, 13 - (int)(prod >> 32));
}

// kMinBlocks: CTAs per SM the register budget is cut for.
template <int G, int kMinBlocks = 1>
__global__ void __launch_bounds__(kPfThreads, kMinBlocks)
attn_prefill_kernel(const PrefillParams p) {
  constexpr int TQ = kPfRows / G;                    // new tokens per tile
  const int b = blockIdx.z, kh = blockIdx.y;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int fr = lane >> 2, fc = lane & 3;

  const int L_all = max(0, min(p.kv_lens[b], p.max_kv_len));
  const int n_q = max(0, min(p.q_lens[b], L_all));
  const int n_tiles = (n_q + TQ - 1) / TQ;
  if ((int)blockIdx.x >= n_tiles) return;            // whole CTA: this sequence has fewer tiles
  const int tile = n_tiles - 1 - (int)blockIdx.x;    // the tiles with the most keys start first
  const int t0 = tile * TQ;
  const int64_t q_row0 = p.q_start[b];
  const int prefix = L_all - n_q;                    // keys in front of the new tokens
  const int Lt = min(L_all, prefix + min(n_q, t0 + TQ));   // keys the last row of the tile sees
  const int n_pairs = (Lt + 31) >> 5;
  const int n_pages = (Lt + kPage - 1) / kPage;

  extern __shared__ __align__(128) unsigned char smem_raw[];
  unsigned char* ring = smem_raw;                                                    // [stages][kPfStageBytes]
  int32_t* pages = reinterpret_cast<int32_t*>(smem_raw + kPfStages * kPfStageBytes);   // [max pages]
  __shared__ unsigned long long vref_s;

  // ---- page ids of the keys this tile sees; the reference V scale over ALL keys of the sequence
  for (int i = tid; i < n_pages; i += kPfThreads) {
    int64_t pid = p.page_table[(int64_t)b * p.table_pitch + i];
    pages[i] = (int)(pid < 0 ? 0 : (pid >= p.num_pages ? p.num_pages - 1 : pid));
  }
  if (tid == 0) vref_s = ~0ull;
  __syncthreads();
  {
    unsigned long long lv = ~0ull;
    for (int key = tid; key < L_all; key += kPfThreads) {
      int64_t pid = p.page_table[(int64_t)b * p.table_pitch + (key >> 4)];
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
    if (lane == 0) atomicMin(&vref_s, lv);
  }
  __syncthreads();
  const int v_shift_ref = (int)(vref_s >> 32) - 128;
  const int v_mul_ref = (int)(0xFFFFFFFFu - (unsigned)(vref_s & 0xFFFFFFFFull));

  // ---- this lane's two query rows: row r of the CTA is new token t0 + r / G, query head kh * G + r % G
  int lim[2], qm[2], qs[2];
  int64_t orow[2];                                   // element offset of the row in q / out
  unsigned qa[2][8];                                 // Q bytes [32 fc, 32 fc + 32) of the row: A operand words
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = warp * 16 + fr + 8 * h;
    const int tok = t0 + r / G, g = r % G;
    const bool valid = tok < n_q;
    lim[h] = valid ? prefix + tok + 1 : 0;           // keys the row sees (0: a row past the sequence's last token)
    const int64_t hrow = (q_row0 + (valid ? tok : 0)) * p.q_heads + kh * G + g;
    orow[h] = hrow * kD;
    qm[h] = valid ? p.q_mul[hrow] : 0;
    qs[h] = valid ? p.q_shift[hrow] - 48 : 0;
    const uint4* qp = reinterpret_cast<const uint4*>(p.q + hrow * kD + fc * 32);
    const uint4 x0 = valid ? __ldg(qp) : make_uint4(0, 0, 0, 0), x1 = valid ? __ldg(qp + 1) : make_uint4(0, 0, 0, 0);
    qa[h][0] = x0.x; qa[h][1] = x0.y; qa[h][2] = x0.z; qa[h][3] = x0.w;
    qa[h][4] = x1.x; qa[h][5] = x1.y; qa[h][6] = x1.z; qa[h][7] = x1.w;
  }
  // keys this warp needs at all: the largest limit of its 16 rows (uniform over the warp)
  int warp_lim = max(lim[0], lim[1]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) warp_lim = max(warp_lim, __shfl_xor_sync(FULL_MASK, warp_lim, o));

  // ---- the ring: one stage = a pair of pages.  Thread t copies 16-byte chunk t of the pair's K (and V) bytes.
  const unsigned ring_base = (unsigned)__cvta_generic_to_shared(ring);
  const int c_page = tid >> 7, c_chunk = tid & 127;                       // which page of the pair, which 16-byte chunk
  const unsigned k_dst = c_page * 2048 + ((c_chunk >> 3) << 7) + ((((c_chunk & 7) ^ ((c_chunk >> 3) & 1))) << 4);   // row-parity swizzle
  const unsigned v_dst = 4096 + c_page * 2048 + (c_chunk << 4);
  const int64_t chunk_off = (int64_t)kh * (kPage * kD) + (c_chunk << 4);
  const int64_t page_stride = (int64_t)p.kv_heads * (kPage * kD);
  auto issue = [&](int pair, bool with_v) {
    if (pair < n_pairs) {
      const unsigned st = ring_base + (pair % kPfStages) * kPfStageBytes;
      const int pg = 2 * pair + c_page;
      if (pg < n_pages) {
        const int64_t off = pages[pg] * page_stride + chunk_off;
        cp_async16(st + k_dst, reinterpret_cast<const unsigned char*>(p.k_codes) + off);
        if (with_v) cp_async16(st + v_dst, reinterpret_cast<const unsigned char*>(p.v_codes) + off);
      }
      if (tid < 20) {
        const int h = tid >= 10, c16 = tid - 10 * h;
        if (2 * pair + h < n_pages)
          cp_async16(st + 8192 + h * 192 + c16 * 16,
                     reinterpret_cast<const unsigned char*>(p.meta + ((int64_t)pages[2 * pair + h] * p.kv_heads + kh) * kMetaWords) + c16 * 16);
      }
    }
    cp_async_commit();
  };

  // Scores of one pair for this lane: sc[h][pg][e] = row h, key pair * 32 + pg * 16 + 4 fc + e (kPfNeg = not visible)
  auto scores = [&](const unsigned char* st, int pair, int (&sc)[2][2][4]) {
#pragma unroll
    for (int pg = 0; pg < 2; ++pg) {
      const int32_t* mt = reinterpret_cast<const int32_t*>(st + 8192 + pg * 192);
      const int4 km = *reinterpret_cast<const int4*>(mt + 4 * fc);
      const unsigned ksw = reinterpret_cast<const unsigned*>(mt + 32)[fc];
      const int kmv[4] = {km.x, km.y, km.z, km.w};
      const int key0 = pair * 32 + pg * 16 + 4 * fc;
#pragma unroll
      for (int jj = 0; jj < 2; ++jj) {
        const int tok = 4 * (fr >> 1) + 2 * jj + (fr & 1);                   // the key row this lane feeds as column fr
        const unsigned char* kr = st + pg * 2048 + tok * 128;
        const uint4 k0 = *reinterpret_cast<const uint4*>(kr + (((2 * fc) ^ (tok & 1)) << 4));
        const uint4 k1 = *reinterpret_cast<const uint4*>(kr + (((2 * fc + 1) ^ (tok & 1)) << 4));
        int c[4] = {0, 0, 0, 0};
        mma_s8s8(c, qa[0][0], qa[1][0], qa[0][1], qa[1][1], k0.x, k0.y);
        mma_s8s8(c, qa[0][2], qa[1][2], qa[0][3], qa[1][3], k0.z, k0.w);
        mma_s8s8(c, qa[0][4], qa[1][4], qa[0][5], qa[1][5], k1.x, k1.y);
        mma_s8s8(c, qa[0][6], qa[1][6], qa[0][7], qa[1][7], k1.z, k1.w);
        // c[0]: (row fr, key 4 fc + 2 jj)  c[1]: (row fr, + 1)  c[2]: (row fr + 8, key 4 fc + 2 jj)  c[3]: (row fr + 8, + 1)
#pragma unroll
        for (int e2 = 0; e2 < 2; ++e2) {
          const int e = 2 * jj + e2;
          const int ks = (int)(signed char)((ksw >> (8 * e)) & 0xff);
#pragma unroll
          for (int h = 0; h < 2; ++h)
            sc[h][pg][e] = key0 + e < lim[h] ? mul_shift_sat32(c[2 * h + e2], __mulhi(qm[h], kmv[e]), qs[h] + ks) : kPfNeg;
        }
      }
    }
  };

  // ---- pass 1: row maxima
  int row_max[2] = {kPfNeg, kPfNeg};
  for (int j = 0; j < kPfStages - 1; ++j) issue(j, false);
  for (int pair = 0; pair < n_pairs; ++pair) {
    cp_async_wait<kPfStages - 2>();
    __syncthreads();                                   // the pair has landed for everybody; the stage of pair - 1 is free
    issue(pair + kPfStages - 1, false);
    if (pair * 32 >= warp_lim) continue;
    int sc[2][2][4];
    scores(ring + (pair % kPfStages) * kPfStageBytes, pair, sc);
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
      for (int pg = 0; pg < 2; ++pg)
#pragma unroll
        for (int e = 0; e < 4; ++e) row_max[h] = max(row_max[h], sc[h][pg][e]);   // kPfNeg for keys out of sight
  }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    row_max[h] = max(row_max[h], __shfl_xor_sync(FULL_MASK, row_max[h], 1));
    row_max[h] = max(row_max[h], __shfl_xor_sync(FULL_MASK, row_max[h], 2));
    // keys behind the causal limit take part in the reference's maximum as -2^30
    if (lim[h] < L_all) row_max[h] = max(row_max[h], -(1 << 30));
  }
  cp_async_wait<0>();
  __syncthreads();

  // ---- pass 2: sums of exponentials
  unsigned row_sum[2] = {0u, 0u};
  for (int j = 0; j < kPfStages - 1; ++j) issue(j, false);
  for (int pair = 0; pair < n_pairs; ++pair) {
    cp_async_wait<kPfStages - 2>();
    __syncthreads();
    issue(pair + kPfStages - 1, false);
    if (pair * 32 >= warp_lim) continue;
    int sc[2][2][4];
    scores(ring + (pair % kPfStages) * kPfStageBytes, pair, sc);
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
      for (int pg = 0; pg < 2; ++pg)
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (pair * 32 + pg * 16 + 4 * fc + e < lim[h]) row_sum[h] += (unsigned)pf_exp(sc[h][pg][e], row_max[h]);
  }
  unsigned inv[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    unsigned long long tot = row_sum[h];
    tot += __shfl_xor_sync(FULL_MASK, tot, 1);
    tot += __shfl_xor_sync(FULL_MASK, tot, 2);
    if (tot < 1ull) tot = 1ull;
    inv[h] = (unsigned)(2147483647ull / tot);
  }
  cp_async_wait<0>();
  __syncthreads();

  // ---- pass 3: probabilities (Q0.15) folded with the relative V scale, as two byte limbs, times V
  int acc_hi[16][4], acc_lo[16][4];
#pragma unroll
  for (int nt = 0; nt < 16; ++nt)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc_hi[nt][j] = acc_lo[nt][j] = 0;
  for (int j = 0; j < kPfStages - 1; ++j) issue(j, true);
  for (int pair = 0; pair < n_pairs; ++pair) {
    cp_async_wait<kPfStages - 2>();
    __syncthreads();
    issue(pair + kPfStages - 1, true);
    if (pair * 32 >= warp_lim) continue;
    const unsigned char* st = ring + (pair % kPfStages) * kPfStageBytes;
    int sc[2][2][4];
    scores(st, pair, sc);
    unsigned ah[2][2], al[2][2];                        // [row h][page]: four limb bytes = keys 4 fc .. 4 fc + 3
#pragma unroll
    for (int pg = 0; pg < 2; ++pg) {
      const int32_t* mt = reinterpret_cast<const int32_t*>(st + 8192 + pg * 192);
      const int4 vm = *reinterpret_cast<const int4*>(mt + 16 + 4 * fc);
      const unsigned vsw = reinterpret_cast<const unsigned*>(mt + 36)[fc];
      const unsigned vmv[4] = {(unsigned)vm.x, (unsigned)vm.y, (unsigned)vm.z, (unsigned)vm.w};
      unsigned hi[2] = {0u, 0u}, lo[2] = {0u, 0u};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = pair * 32 + pg * 16 + 4 * fc + e;
        const int vs = (int)(signed char)((vsw >> (8 * e)) & 0xff);
        const unsigned r = key < warp_lim ? rel_scale_q15(vmv[e], (unsigned)v_mul_ref, vs - v_shift_ref) : 0u;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          unsigned w = 0u;
          if (key < lim[h]) {
            const unsigned pr = ((unsigned)pf_exp(sc[h][pg][e], row_max[h]) * inv[h]) >> 16;
            w = (pr * r + 16384u) >> 15;
          }
          hi[h] |= (w >> 8) << (8 * e);
          lo[h] |= (w & 0xffu) << (8 * e);
        }
      }
      ah[0][pg] = hi[0]; ah[1][pg] = hi[1]; al[0][pg] = lo[0]; al[1][pg] = lo[1];
    }
    const bool has_b = 2 * pair + 1 < n_pages;
    const unsigned char* vp = st + 4096 + lane * 16;
#pragma unroll
    for (int qd = 0; qd < 4; ++qd) {
      const uint4 va = *reinterpret_cast<const uint4*>(vp + qd * 512);
      const uint4 vb = has_b ? *reinterpret_cast<const uint4*>(vp + 2048 + qd * 512) : make_uint4(0, 0, 0, 0);
      const unsigned wa[4] = {va.x, va.y, va.z, va.w}, wb[4] = {vb.x, vb.y, vb.z, vb.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int nt = 4 * qd + i;
        mma_u8s8(acc_hi[nt], ah[0][0], ah[1][0], ah[0][1], ah[1][1], wa[i], wb[i]);
        mma_u8s8(acc_lo[nt], al[0][0], al[1][0], al[0][1], al[1][1], wa[i], wb[i]);
      }
    }
  }
  cp_async_wait<0>();

  // ---- output: acc -> Q15.16, optionally the per-row int8 codes.  C tile: [0] (row fr, d = 8 nt + 2 fc)  [1] (row fr, d + 1)
  // [2] (row fr + 8, d)  [3] (row fr + 8, d + 1)
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const bool valid = lim[h] > 0;
    int o[32];
    int m = 0;
#pragma unroll
    for (int nt = 0; nt < 16; ++nt)
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int a = acc_hi[nt][2 * h + j] * 256 + acc_lo[nt][2 * h + j];
        const int v = mul_shift_sat32_wide((long long)a, v_mul_ref, v_shift_ref - 1);
        o[2 * nt + j] = v;
        m = max(m, abs_wrap(v));
      }
    if (p.out_q15 && valid) {
#pragma unroll
      for (int nt = 0; nt < 16; ++nt)
        *reinterpret_cast<int2*>(p.out_q15 + orow[h] + 8 * nt + 2 * fc) = make_int2(o[2 * nt], o[2 * nt + 1]);
    }
    if (p.out_codes) {
      m = max(m, __shfl_xor_sync(FULL_MASK, m, 1));
      m = max(1, max(m, __shfl_xor_sync(FULL_MASK, m, 2)));
      if (valid) {
        const float mf = __int2float_rn(m);
#pragma unroll
        for (int nt = 0; nt < 16; ++nt) {
          const unsigned short c2 = (unsigned short)((quant_code(o[2 * nt], mf) & 0xff) | ((quant_code(o[2 * nt + 1], mf) & 0xff) << 8));
          *reinterpret_cast<unsigned short*>(p.out_codes + orow[h] + 8 * nt + 2 * fc) = c2;
        }
        if (fc == 0) p.out_absmax[orow[h] / kD] = m;
      }
    }
  }
}

template <int G>
static int launch_prefill(const PrefillParams& p, int batch, int max_q_len, cudaStream_t st) {
  constexpr int TQ = kPfRows / G;
  const size_t smem = (size_t)kPfStages * kPfStageBytes + (size_t)((p.max_kv_len + kPage - 1) / kPage) * 4;
  if (smem > 200 * 1024) {
    set_error("attn_prefill: max_kv_len=%d needs %zu bytes of shared memory for the page list", p.max_kv_len, smem);
    return B200_E_UNSUPPORTED;
  }
  // Two CTAs per SM (a budget of 128 registers, some spilled) while the page list leaves room: the kernel waits on
  // dependent integer arithmetic, and four warps per scheduler hide more of it than two (1.73 -> 1.58 ms on 16
  // prompts of U[100,1024] tokens).  B200_PREFILL_OCC2=0 keeps one CTA of 250 registers per SM.
  static int occ2 = -1;
  if (occ2 < 0) {
    const char* ev = getenv("B200_PREFILL_OCC2");
    occ2 = (ev && ev[0] == '0') ? 0 : 1;
  }
  const int tiles = (max_q_len + TQ - 1) / TQ;
  if (occ2 == 1 && smem <= 100 * 1024) {
    cudaError_t e2 = cudaFuncSetAttribute(attn_prefill_kernel<G, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e2 != cudaSuccess) {
      set_error("attn_prefill: cudaFuncSetAttribute: %s", cudaGetErrorString(e2));
      return B200_E_CUDA;
    }
    attn_prefill_kernel<G, 2><<<dim3(tiles, p.kv_heads, batch), kPfThreads, smem, st>>>(p);
    return check_launch("attn_prefill");
  }
  cudaError_t e = cudaFuncSetAttribute(attn_prefill_kernel<G>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) {
    set_error("attn_prefill: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    return B200_E_CUDA;
  }
  attn_prefill_kernel<G><<<dim3(tiles, p.kv_heads, batch), kPfThreads, smem, st>>>(p);
  return check_launch("attn_prefill");
}

}  // namespace b200

using namespace b200;

extern "C" int b200_attn_prefill(const int8_t* q, const int32_t* q_mul, const int32_t* q_shift, const int8_t* k_codes,
                                 const int8_t* v_codes, const int32_t* meta, const int32_t* page_table, int64_t table_pitch,
                                 const int32_t* kv_lens, const int32_t* q_lens, const int32_t* q_start, int32_t* out_q15,
                                 int8_t* out_codes, int32_t* out_absmax, int batch, int max_q_len, int q_heads, int kv_heads,
                                 int64_t num_pages, int max_kv_len, b200_stream_t s) {
  B200_REQUIRE(q && q_mul && q_shift && k_codes && v_codes && meta && page_table && kv_lens && q_lens && q_start, B200_E_NULL,
               "attn_prefill: null pointer");
  B200_REQUIRE((out_codes == nullptr) == (out_absmax == nullptr), B200_E_NULL,
               "attn_prefill: out_codes and out_absmax must be given together");
  B200_REQUIRE(out_q15 || out_codes, B200_E_NULL, "attn_prefill: no output requested");
  B200_REQUIRE(batch >= 0 && batch <= 65535 && max_q_len >= 0 && q_heads > 0 && kv_heads > 0 && kv_heads <= 65535 &&
                   num_pages > 0 && max_kv_len > 0,
               B200_E_SHAPE, "attn_prefill: batch=%d max_q_len=%d q_heads=%d kv_heads=%d num_pages=%lld max_kv_len=%d", batch,
               max_q_len, q_heads, kv_heads, (long long)num_pages, max_kv_len);
  B200_REQUIRE(q_heads % kv_heads == 0, B200_E_SHAPE, "attn_prefill: q_heads=%d not a multiple of kv_heads=%d", q_heads, kv_heads);
  const int G = q_heads / kv_heads;
  B200_REQUIRE(G == 1 || G == 2 || G == 4 || G == 8, B200_E_UNSUPPORTED, "attn_prefill: group size %d (1, 2, 4 or 8)", G);
  B200_REQUIRE(table_pitch >= (max_kv_len + kPage - 1) / kPage, B200_E_SHAPE,
               "attn_prefill: table_pitch=%lld < pages for max_kv_len (%d)", (long long)table_pitch, (max_kv_len + kPage - 1) / kPage);
  B200_REQUIRE(aligned16(q) && aligned16(k_codes) && aligned16(v_codes) && aligned16(meta) &&
                   (reinterpret_cast<uintptr_t>(out_q15) & 7u) == 0 && (reinterpret_cast<uintptr_t>(out_codes) & 1u) == 0,
               B200_E_ALIGN, "attn_prefill: q and pool buffers must be 16-byte aligned, out_q15 8-byte");
  if (batch == 0 || max_q_len == 0) return B200_OK;
  B200_REQUIRE((int64_t)((max_q_len + 15) / 16) <= 65535 * 8, B200_E_SHAPE, "attn_prefill: max_q_len=%d", max_q_len);
  PrefillParams p;
  p.q = q; p.q_mul = q_mul; p.q_shift = q_shift; p.k_codes = k_codes; p.v_codes = v_codes; p.meta = meta;
  p.page_table = page_table; p.table_pitch = table_pitch; p.kv_lens = kv_lens; p.q_lens = q_lens; p.q_start = q_start;
  p.out_q15 = out_q15; p.out_codes = out_codes; p.out_absmax = out_absmax; p.q_heads = q_heads; p.kv_heads = kv_heads;
  p.num_pages = num_pages; p.max_kv_len = max_kv_len;
  cudaStream_t st = (cudaStream_t)s;
  switch (G) {
    case 1: return launch_prefill<1>(p, batch, max_q_len, st);
    case 2: return launch_prefill<2>(p, batch, max_q_len, st);
    case 4: return launch_prefill<4>(p, batch, max_q_len, st);
    default: return launch_prefill<8>(p, batch, max_q_len, st);
  }
}
