// W8A8 linear on the 5th-generation tensor cores: int8 x int8 -> int32 accumulators in tensor
// memory (tcgen05.mma kind::i8), operands staged by TMA into 128-byte-swizzled shared memory,
// fixed-point requant epilogue read back with tcgen05.ld.
//
//   acc[t, n]  = sum_k x8[t, k] * w8[n, k]                      exact int32
//   out[t, n]  = sat32(mul_shift(acc, (x_mul[t] * w_mul[n]) >> 32, x_shift[t] + w_shift[n] - 48))
//
// Both operands are K-major (x8 [M, K] and w8 [N, K] row-major), which is what the UMMA wants.
// A tile is 128 x BN outputs (BN = 256 at large M, down to 32 at decode sizes):
//   warp 0        TMA producer (one lane): A tile 128 x 128 B and B tile BN x 128 B per k-block
//   warp 1        allocates tensor memory; one lane issues the MMAs (4 per k-block, K = 32 each)
//   warps 2..9    epilogue: two per 32-lane quarter of the accumulator tile, half the columns each
// The kernel is persistent (one CTA per SM walks a strided list of tiles) and keeps two accumulator
// copies in tensor memory, so the epilogue of one tile overlaps the MMAs of the next.
//
// Decode sizes (M <= 256 tokens) run "weights-stationary" (template flag WS): the operands swap
// roles - 128 weight rows are the UMMA's M side, all the tokens its N side - so every weight byte
// crosses HBM once and a tile's accumulators are out^T.  A thread then holds one weight channel and 32
// tokens, and the store of a token's 32 channels by a warp is one contiguous 128 bytes.  When the
// weight matrix has too few 128-row blocks to occupy the GPU, K is split across CTAs whose int32
// partial sums are added with red.global (integer addition: any order gives the same bits) and a
// second small kernel applies the epilogue.
// Stages are handed over with mbarriers (TMA -> MMA by transaction bytes, MMA -> TMA and
// MMA -> epilogue by tcgen05.commit).  Every wait is bounded: on expiry the waiter raises an
// error flag that the host can read, and the CTA still runs to its end and frees its tensor memory.
#include <cuda.h>

#include "common.cuh"
#include "silu.cuh"
#include "tp_block.cuh"

namespace b200 {

constexpr int kBM = 128;            // rows of x per tile (UMMA M)
constexpr int kBK = 128;            // bytes of K per stage = one 128-byte swizzle row
constexpr int kUmmaK = 32;          // K per tcgen05.mma for 8-bit operands
constexpr int kEpiWarps = 8;         // two per 32-lane quarter of tensor memory, each half of the columns
constexpr int kGemmThreads = 64 + 32 * kEpiWarps;
constexpr unsigned kSpinLimit = 1u << 22;

__device__ int g_gemm_status = 0;   // 0 = fine; otherwise the code of the first wait that gave up

// ----------------------------------------------------------------------------- PTX wrappers
__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(unsigned bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(unsigned bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// Bounded wait for the phase with the given parity; false (and the status flag) on expiry.
__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity, int code) {
  for (unsigned it = 0; it < kSpinLimit; ++it) {
    unsigned ok;
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    if (ok) return true;
  }
  atomicCAS(&g_gemm_status, 0, code);
  return false;
}
__device__ __forceinline__ void tma_load_2d(unsigned dst, const CUtensorMap* map, int c0, int c1, unsigned bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tcgen05_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_commit(unsigned bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void umma_i8(unsigned tmem_d, uint64_t desc_a, uint64_t desc_b, unsigned idesc, unsigned accumulate) {
  asm volatile(
      "{\n.reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_32x32(unsigned taddr, int (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
        "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
        "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory operand descriptor: K-major tile whose rows are 128 bytes, 128-byte swizzle.
// Eight rows form one 1024-byte swizzle atom, so the stride between 8-row groups is 1024 bytes;
// the leading-dimension offset is unused in this mode.  Bits: [0,14) address >> 4,
// [32,46) stride >> 4, [46,48) descriptor version 1, [61,64) layout 2 = SWIZZLE_128B.
__device__ __forceinline__ uint64_t make_smem_desc(unsigned addr) {
  return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor of kind::i8: D = s32 (2 << 4), A = B = signed 8-bit (1 << 7, 1 << 10),
// both K-major (bits 15, 16 clear), N >> 3 at bit 17, M >> 4 at bit 24.
__host__ __device__ constexpr unsigned make_idesc(int m, int n) {
  return (2u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(n >> 3) << 17) | ((unsigned)(m >> 4) << 24);
}

struct GemmParams {
  const int32_t* x_absmax;  // nullable: per-token absmax from which (x_mul, x_shift) are derived on the fly
  const int32_t* x_mul;
  const int32_t* x_shift;
  const int32_t* w_mul;
  const int32_t* w_shift;   // nullable: every channel uses shift 31
  int32_t* out_q15;         // nullable
  int32_t* acc_out;         // nullable
  int M, N, K;
  int splits;               // weights-stationary mode: parts of K per block of weight rows (1 = none)
  int full_blocks;          // weights-stationary mode: the first full_blocks blocks of weight rows are never split
                            // (one tile each, finished in the GEMM kernel); `splits` applies to the blocks after them
  int32_t* partial;         // splits > 1: int32 [M, N] that the parts are added into (zeroed before the launch)
  int split_col0;           // first output channel that belongs to a split block
  int n_peers;              // > 0: tensor-parallel reduction - every part is added into each of these [M, N] buffers
  int32_t* peer[8];         //      (this rank's and its peers', mapped into this process: NVLink peer memory)
  int tp_on;                // the peers' buffers are the accumulator halves of tensor-parallel exchange blocks: the
  TpView tp;                //      half follows the block's channel-1 epoch and the kernel ends with that channel's signal
};

__device__ __forceinline__ void mbar_arrive(unsigned bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void epilogue_bar_sync() {   // the epilogue threads only
  asm volatile("bar.sync 1, %0;" ::"n"(32 * kEpiWarps) : "memory");
}

// Weights-stationary tile list: one whole-K tile per unsplit block, then `splits` parts of K per remaining block.
struct WsTile { int n_blk, kb0, kb1; bool split; };
__device__ __forceinline__ WsTile ws_tile(const GemmParams& p, int tile, int num_kb) {
  WsTile t;
  if (tile < p.full_blocks) {
    t.n_blk = tile; t.kb0 = 0; t.kb1 = num_kb; t.split = false;
    return t;
  }
  const int r = tile - p.full_blocks, blk = r / p.splits, kb_per = (num_kb + p.splits - 1) / p.splits;
  t.n_blk = p.full_blocks + blk;
  t.kb0 = (r - blk * p.splits) * kb_per;
  t.kb1 = min(num_kb, t.kb0 + kb_per);
  t.split = p.splits > 1;
  return t;
}

constexpr int kStagePitch = 20;   // ints per staged row of 16: 16-byte aligned, conflict-free for int4 both ways

// Warp-private 32 x 16 int32 tile, used twice per 32-column chunk: lane = row on the way in, eight
// rows x four int4 (64 contiguous bytes per row) per instruction on the way out (rows r_base..,
// columns col0.. of a row-major [M, N] matrix).
__device__ __forceinline__ void store_chunk(int32_t* stage, int lane, const int (&v)[32], int32_t* out,
                                            int r_base, int col0, int M, int N, bool vec) {
  const int rr = lane >> 2, cc = (lane & 3) * 4;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    __syncwarp();
#pragma unroll
    for (int j = 0; j < 16; j += 4)
      *reinterpret_cast<int4*>(stage + lane * kStagePitch + j) =
          make_int4(v[16 * h + j], v[16 * h + j + 1], v[16 * h + j + 2], v[16 * h + j + 3]);
    __syncwarp();
#pragma unroll
    for (int it = 0; it < 4; ++it) {
      const int r = it * 8 + rr;
      const int row = r_base + r, col = col0 + 16 * h + cc;
      if (row < M && col < N) {
        const int4 o = *reinterpret_cast<const int4*>(stage + r * kStagePitch + cc);
        int32_t* dst = out + (int64_t)row * N + col;
        if (vec) {   // N % 4 == 0 and col % 4 == 0: the whole int4 is inside the row
          *reinterpret_cast<int4*>(dst) = o;
        } else {
          dst[0] = o.x;
          if (col + 1 < N) dst[1] = o.y;
          if (col + 2 < N) dst[2] = o.z;
          if (col + 3 < N) dst[3] = o.w;
        }
      }
    }
  }
}

// Persistent kernel: CTA c computes tiles c, c + gridDim.x, ...  (tile -> n block outer, m block inner,
// so the CTAs running at the same time share one block of weight rows in L2).  The accumulator
// lives in tensor memory twice (2 x BN columns): while the epilogue warps drain one copy, the MMA
// warp already fills the other with the next tile.
template <int BN, int STAGES, bool WS>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_w8a8_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                 const GemmParams p) {
  extern __shared__ __align__(1024) unsigned char smem[];
  constexpr int kABytes = kBM * kBK;
  constexpr int kBBytes = BN * kBK;
  constexpr int kStageBytes = kABytes + kBBytes;
  unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem) + 1023) & ~uintptr_t(1023));
  // barriers: full[S], empty[S], tmem_full[2], tmem_empty[2]
  uint64_t* bars = reinterpret_cast<uint64_t*>(tiles + STAGES * kStageBytes);
  unsigned* tmem_slot = reinterpret_cast<unsigned*>(bars + 2 * STAGES + 4);
  int32_t* col_scale = reinterpret_cast<int32_t*>(tmem_slot + 4);   // [2 slots][mul BN | shift BN]
  int32_t* stage_all = col_scale + 4 * BN;                          // [epilogue warps][32][kStagePitch]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_kb = (p.K + kBK - 1) / kBK;
  // WS: a tile is (block of 128 weight rows, part of K); otherwise (block of BN weight rows, block of 128 tokens)
  const int m_tiles = WS ? 1 : (p.M + kBM - 1) / kBM;
  const int n_tiles = WS ? (p.N + kBM - 1) / kBM : (p.N + BN - 1) / BN;
  const int num_tiles = WS ? p.full_blocks + (n_tiles - p.full_blocks) * p.splits : m_tiles * n_tiles;
  const unsigned full0 = smem_u32(bars), empty0 = smem_u32(bars + STAGES);
  const unsigned tfull0 = smem_u32(bars + 2 * STAGES), tempty0 = smem_u32(bars + 2 * STAGES + 2);

  if (warp == 0 && lane == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(tfull0 + 8 * s, 1);
      mbar_init(tempty0 + 8 * s, kEpiWarps);   // one arrival per epilogue warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {   // the whole warp allocates 2 x BN columns (a power of two >= 32) of tensor memory
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(2 * BN) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  pdl_launch_dependents();
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const unsigned tmem_base = *tmem_slot;
  pdl_wait();               // barriers, tensor memory and descriptors are set up; the operands come from earlier kernels
  // exchange-block mode: word offset, inside this rank's block, of the accumulator half in use
  int64_t tp_acc_off = 0;
  if (WS && p.tp_on) {
    const TpLayout l = tp_layout(p.tp.m_max, p.tp.n);
    const int half = *reinterpret_cast<volatile int32_t*>(p.tp.base[p.tp.rank] + 1) & 1;
    tp_acc_off = l.acc + (int64_t)half * l.acc_half;
  }

  if (warp == 0) {
    if (lane == 0) {
      unsigned it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int n_blk = tile / m_tiles, m_blk = tile - n_blk * m_tiles, kb0 = 0, kb1 = num_kb;
        if (WS) {
          const WsTile t = ws_tile(p, tile, num_kb);
          n_blk = t.n_blk; kb0 = t.kb0; kb1 = t.kb1;
        }
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const unsigned s = it % STAGES, ph = (it / STAGES) & 1;
          ok = mbar_wait(empty0 + 8 * s, ph ^ 1, 1);
          if (!ok) break;
          mbar_expect_tx(full0 + 8 * s, kStageBytes);
          const unsigned a_dst = smem_u32(tiles + s * kStageBytes);
          // map_a always feeds the 128-row operand: token rows, or weight rows in WS mode (map_b: all tokens)
          tma_load_2d(a_dst, &map_a, kb * kBK, (WS ? n_blk : m_blk) * kBM, full0 + 8 * s);
          tma_load_2d(a_dst + kABytes, &map_b, kb * kBK, WS ? 0 : n_blk * BN, full0 + 8 * s);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr unsigned idesc = make_idesc(kBM, BN);
      unsigned it = 0, lt = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++lt) {
        const unsigned slot = lt & 1, aph = (lt >> 1) & 1;
        ok = mbar_wait(tempty0 + 8 * slot, aph ^ 1, 4);   // the epilogue has drained this accumulator copy
        if (!ok) break;
        tcgen05_fence_after();
        const unsigned tmem_d = tmem_base + slot * BN;
        int kb0 = 0, kb1 = num_kb;
        if (WS) {
          const WsTile t = ws_tile(p, tile, num_kb);
          kb0 = t.kb0; kb1 = t.kb1;
        }
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const unsigned s = it % STAGES, ph = (it / STAGES) & 1;
          ok = mbar_wait(full0 + 8 * s, ph, 2);
          if (!ok) break;
          tcgen05_fence_after();
          const unsigned a_addr = smem_u32(tiles + s * kStageBytes);
          const uint64_t da = make_smem_desc(a_addr), db = make_smem_desc(a_addr + kABytes);
#pragma unroll
          for (int k = 0; k < kBK / kUmmaK; ++k) {
            // the next 32 bytes of K inside the swizzle row: start address + 32 (encoded >> 4)
            umma_i8(tmem_d, da + (uint64_t)(k * kUmmaK >> 4), db + (uint64_t)(k * kUmmaK >> 4), idesc,
                    (kb > kb0 || k > 0) ? 1u : 0u);
          }
          tcgen05_commit(empty0 + 8 * s);   // frees the stage once these MMAs have read it
        }
        // accumulators complete: release the epilogue.  After an expired wait nothing is committed, so the
        // epilogue's own wait runs out too and no partial sums are stored or added anywhere.
        if (ok) tcgen05_commit(tfull0 + 8 * slot);
      }
    }
  } else {
    // epilogue warps 2..9: TMEM lane quarter = warp % 4 (one accumulator row per thread); the two
    // warps of a quarter take alternate 32-column chunks of the tile
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;
    const int et = threadIdx.x - 64;   // 0 .. 32 * kEpiWarps - 1
    int32_t* stage = stage_all + (warp - 2) * (32 * kStagePitch);
    unsigned lt = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++lt) {
      const int n_blk = tile / m_tiles, m_blk = tile - n_blk * m_tiles;
      const unsigned slot = lt & 1, aph = (lt >> 1) & 1;
      int32_t* cs = col_scale + slot * 2 * BN;
      if (WS) {
        // rows of the accumulator tile are weight channels, columns are tokens
        const WsTile wt = ws_tile(p, tile, num_kb);
        const int ch = wt.n_blk * kBM + q * 32 + lane;
        const bool direct = !wt.split && p.n_peers == 0;
        const bool empty_part = wt.kb0 >= wt.kb1;      // a part of K with no k-blocks: nothing was accumulated
        if (direct && p.out_q15) {
          for (int c = et; c < BN; c += 32 * kEpiWarps) {
            const int t = min(c, p.M - 1);
            int tm, ts;
            if (p.x_absmax) absmax_to_ms_dev(__ldg(p.x_absmax + t), &tm, &ts);
            else { tm = __ldg(p.x_mul + t); ts = __ldg(p.x_shift + t); }
            cs[c] = tm;
            cs[BN + c] = ts - 48;
          }
        }
        int wm = 0, ws = 0;
        if (ch < p.N && direct && p.out_q15) { wm = __ldg(p.w_mul + ch); ws = p.w_shift ? __ldg(p.w_shift + ch) : 31; }
        epilogue_bar_sync();
        if (ok) ok = mbar_wait(tfull0 + 8 * slot, aph, 3);
        tcgen05_fence_after();
#pragma unroll 1
        for (int c0 = half * 32; c0 < BN; c0 += 64) {
          int v[32];
          tmem_ld_32x32(tmem_base + ((unsigned)(q * 32) << 16) + slot * BN + (unsigned)c0, v);
          if (!ok || c0 >= p.M || ch >= p.N || empty_part) continue;
          if (p.tp_on) {
            // exchange-block mode: the parts are added into the rank's OWN accumulators (L2 atomics); the peers fetch
            // them from there once this kernel has signalled
            int32_t* dst = p.tp.base[p.tp.rank] + tp_acc_off;
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (c0 + j < p.M) atomicAdd(dst + (int64_t)(c0 + j) * p.N + ch, v[j]);
          } else if (p.n_peers > 0) {
            // tensor-parallel sum: the tile's partial sums go straight into every rank's accumulator (a warp's
            // 32 channels of one token are one 128-byte reduction over NVLink); integer adds commute, so every
            // rank ends up with the same bits whatever the arrival order
            for (int r = 0; r < p.n_peers; ++r) {
              int32_t* dst = p.peer[r];
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (c0 + j < p.M) atomicAdd(dst + (int64_t)(c0 + j) * p.N + ch, v[j]);
            }
          } else if (!direct) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (c0 + j < p.M) atomicAdd(p.partial + (int64_t)(c0 + j) * p.N + ch, v[j]);   // result unused: a reduction
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              if (c0 + j < p.M) {
                const int64_t o = (int64_t)(c0 + j) * p.N + ch;
                if (p.acc_out) p.acc_out[o] = v[j];
                if (p.out_q15) p.out_q15[o] = requant_one(v[j], __mulhi(cs[c0 + j], wm), cs[BN + c0 + j] + ws);
              }
            }
          }
        }
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(tempty0 + 8 * slot);
        continue;
      }
      const int row = m_blk * kBM + q * 32 + lane;
      // the tile's per-column scales go to shared memory once (double-buffered by accumulator slot)
      if (p.out_q15) {
        for (int c = et; c < BN; c += 32 * kEpiWarps) {
          const int col = min(n_blk * BN + c, p.N - 1);
          cs[c] = __ldg(p.w_mul + col);
          cs[BN + c] = (p.w_shift ? __ldg(p.w_shift + col) : 31) - 48;   // x_shift + w_shift - 48 later
        }
      }
      int xm = 0, xs = 0;
      if (row < p.M && p.out_q15) {
        if (p.x_absmax) absmax_to_ms_dev(__ldg(p.x_absmax + row), &xm, &xs);
        else { xm = __ldg(p.x_mul + row); xs = __ldg(p.x_shift + row); }
      }
      epilogue_bar_sync();
      if (ok) ok = mbar_wait(tfull0 + 8 * slot, aph, 3);
      tcgen05_fence_after();
#pragma unroll 1
      for (int c0 = half * 32; c0 < BN; c0 += 64) {   // the quarter's two warps take alternate 32-column chunks
        int v[32];
        tmem_ld_32x32(tmem_base + ((unsigned)(q * 32) << 16) + slot * BN + (unsigned)c0, v);
        const int col0 = n_blk * BN + c0;
        if (!ok || col0 >= p.N) continue;   // warp-uniform
        // A thread holds 32 columns of ONE row; storing that directly would touch 32 rows per
        // instruction.  The chunk goes through a padded shared-memory tile so that each store
        // instruction writes four rows of 128 contiguous bytes.
        const int r_base = m_blk * kBM + q * 32;
        const bool vec = (p.N & 3) == 0;
        if (p.acc_out) {
          store_chunk(stage, lane, v, p.acc_out, r_base, col0, p.M, p.N, vec);
        }
        if (p.out_q15) {
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            const int4 wm = *reinterpret_cast<const int4*>(cs + c0 + j);
            const int4 ws = *reinterpret_cast<const int4*>(cs + BN + c0 + j);
            v[j + 0] = requant_one(v[j + 0], __mulhi(xm, wm.x), xs + ws.x);
            v[j + 1] = requant_one(v[j + 1], __mulhi(xm, wm.y), xs + ws.y);
            v[j + 2] = requant_one(v[j + 2], __mulhi(xm, wm.z), xs + ws.z);
            v[j + 3] = requant_one(v[j + 3], __mulhi(xm, wm.w), xs + ws.w);
          }
          store_chunk(stage, lane, v, p.out_q15, r_base, col0, p.M, p.N, vec);
        }
      }
      // this warp has read its quarter of the accumulator copy: hand it back to the MMA warp
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty0 + 8 * slot);
    }
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(2 * BN) : "memory");
  }
  // exchange-block mode: nothing was written into a peer's memory, so only the CTA that arrives last pays a
  // system-scope fence before the flag stores (each CTA orders its own additions with a device-scope fence)
  if (WS && p.tp_on && threadIdx.x == 0) {
    __threadfence();
    tp_signal_if_last(p.tp, 1, gridDim.x, false);
  }
}

// ----------------------------------------------------------------------------- two-CTA tiles
// Large M: a pair of CTAs (a cluster of two, on neighbouring SMs) computes one 256 x 256 tile with
// tcgen05.mma.cta_group::2.  Each CTA stages its own 128 token rows of x and only HALF of the tile's weight
// rows (128 of 256), so the shared-memory traffic per MMA drops by a third against two independent
// 128 x 256 tiles - on one CTA the operand reads of an N = 256 MMA alone take three quarters of the
// shared-memory bandwidth.  Protocol (one elected thread each):
//   both CTAs    TMA warp: waits for its own "empty" barrier, loads its A and B halves; the bytes of both
//                CTAs are counted on the LEADER's "full" barrier (barrier address with the peer bit cleared)
//   leader CTA   MMA warp: waits for "full", issues four MMAs per k-block, commits to the "empty" barriers
//                of both CTAs (multicast commit), and after the last k-block to both "accumulator full" barriers
//   both CTAs    sixteen epilogue warps drain their own 128 rows of the accumulator from their own tensor memory
//                and arrive on the leader's "accumulator empty" barrier (the requant is about a dozen integer
//                instructions per output: with eight warps the epilogue of a tile outlasted its MMAs)
// Every wait is bounded as in the one-CTA kernel; both CTAs meet at a cluster barrier before tensor memory is freed.
constexpr unsigned kPeerBitMask = 0xFEFFFFFFu;   // shared::cluster address of the same offset in the pair's even CTA

__device__ __forceinline__ void tma_load_2d_2sm(unsigned dst, const CUtensorMap* map, int c0, int c1, unsigned leader_bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(leader_bar)
      : "memory");
}
__device__ __forceinline__ void umma_i8_2sm(unsigned tmem_d, uint64_t desc_a, uint64_t desc_b, unsigned idesc, unsigned accumulate) {
  asm volatile(
      "{\n.reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tcgen05_commit_pair(unsigned bar) {   // arrives on `bar` in both CTAs of the pair
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(bar), "h"((unsigned short)3) : "memory");
}
__device__ __forceinline__ void mbar_arrive_leader(unsigned bar) {    // arrive on the leader CTA's barrier at this offset
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(bar & kPeerBitMask) : "memory");
}
__device__ __forceinline__ void cluster_barrier() {
  asm volatile("barrier.cluster.arrive.aligned;\nbarrier.cluster.wait.aligned;" ::: "memory");
}

constexpr int kEpiWarps2 = 16;        // the two-CTA kernel: four per 32-lane quarter, a quarter of the columns each
constexpr int kGemmThreads2 = 64 + 32 * kEpiWarps2;

template <int STAGES>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads2, 1)
gemm_w8a8_2sm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                     const GemmParams p) {
  constexpr int BN = 256;                      // tile columns of the pair; each CTA stages BN / 2 weight rows
  constexpr int kABytes = kBM * kBK;           // 128 token rows
  constexpr int kBBytes = (BN / 2) * kBK;      // 128 weight rows
  constexpr int kStageBytes = kABytes + kBBytes;
  extern __shared__ __align__(1024) unsigned char smem[];
  unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(tiles + STAGES * kStageBytes);   // full[S], empty[S], tfull[2], tempty[2]
  unsigned* tmem_slot = reinterpret_cast<unsigned*>(bars + 2 * STAGES + 4);
  int32_t* col_scale = reinterpret_cast<int32_t*>(tmem_slot + 4);               // [2 slots][mul BN | shift BN]
  int32_t* stage_all = col_scale + 4 * BN;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  unsigned rank;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const int num_kb = (p.K + kBK - 1) / kBK;
  const int m_tiles = (p.M + 2 * kBM - 1) / (2 * kBM), n_tiles = (p.N + BN - 1) / BN;
  const int num_tiles = m_tiles * n_tiles;
  const unsigned full0 = smem_u32(bars), empty0 = smem_u32(bars + STAGES);
  const unsigned tfull0 = smem_u32(bars + 2 * STAGES), tempty0 = smem_u32(bars + 2 * STAGES + 2);

  if (warp == 0 && lane == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full0 + 8 * s, 1);             // the leader's expect-tx arrival (bytes of both CTAs)
      mbar_init(empty0 + 8 * s, 1);            // one multicast commit
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(tfull0 + 8 * s, 1);
      mbar_init(tempty0 + 8 * s, 2 * kEpiWarps2);  // the epilogue warps of both CTAs (used on the leader only)
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {   // one warp of each CTA, same warp index: the pair's allocation (all 512 columns: 2 x BN)
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(2 * BN) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  pdl_launch_dependents();
  tcgen05_fence_before();
  __syncthreads();
  cluster_barrier();       // the peer's barriers exist before anything is signalled across the pair
  tcgen05_fence_after();
  const unsigned tmem_base = *tmem_slot;
  pdl_wait();              // everything above is independent of the kernels before this one; the operands are not

  if (warp == 0) {
    if (lane == 0) {
      unsigned it = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        const int n_blk = tile / m_tiles, m_blk = tile - n_blk * m_tiles;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const unsigned s = it % STAGES, ph = (it / STAGES) & 1;
          ok = mbar_wait(empty0 + 8 * s, ph ^ 1, 1);
          if (!ok) break;
          if (leader) mbar_expect_tx(full0 + 8 * s, 2 * kStageBytes);
          const unsigned a_dst = smem_u32(tiles + s * kStageBytes);
          const unsigned lbar = (full0 + 8 * s) & kPeerBitMask;
          tma_load_2d_2sm(a_dst, &map_a, kb * kBK, m_blk * 2 * kBM + (int)rank * kBM, lbar);
          tma_load_2d_2sm(a_dst + kABytes, &map_b, kb * kBK, n_blk * BN + (int)rank * (BN / 2), lbar);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && leader) {
      constexpr unsigned idesc = make_idesc(2 * kBM, BN);
      unsigned it = 0, lt = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, ++lt) {
        const unsigned slot = lt & 1, aph = (lt >> 1) & 1;
        ok = mbar_wait(tempty0 + 8 * slot, aph ^ 1, 4);
        if (!ok) break;
        tcgen05_fence_after();
        const unsigned tmem_d = tmem_base + slot * BN;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const unsigned s = it % STAGES, ph = (it / STAGES) & 1;
          ok = mbar_wait(full0 + 8 * s, ph, 2);
          if (!ok) break;
          tcgen05_fence_after();
          const unsigned a_addr = smem_u32(tiles + s * kStageBytes);
          const uint64_t da = make_smem_desc(a_addr), db = make_smem_desc(a_addr + kABytes);
#pragma unroll
          for (int k = 0; k < kBK / kUmmaK; ++k)
            umma_i8_2sm(tmem_d, da + (uint64_t)(k * kUmmaK >> 4), db + (uint64_t)(k * kUmmaK >> 4), idesc,
                        (kb > 0 || k > 0) ? 1u : 0u);
          tcgen05_commit_pair(empty0 + 8 * s);
        }
        if (ok) tcgen05_commit_pair(tfull0 + 8 * slot);   // nothing is released after an expired wait
      }
    }
  } else {
    const int q = warp & 3;
    const int part = (warp - 2) >> 2;          // which of the interleaved 32-column chunks this warp takes
    const int et = threadIdx.x - 64;
    int32_t* stage = stage_all + (warp - 2) * (32 * kStagePitch);
    unsigned lt = 0;
    bool ok = true;
    for (int tile = pair; tile < num_tiles; tile += num_pairs, ++lt) {
      const int n_blk = tile / m_tiles, m_blk = tile - n_blk * m_tiles;
      const unsigned slot = lt & 1, aph = (lt >> 1) & 1;
      const int r_base = m_blk * 2 * kBM + (int)rank * kBM + q * 32;
      const int row = r_base + lane;
      int32_t* cs = col_scale + slot * 2 * BN;
      if (p.out_q15) {
        for (int c = et; c < BN; c += 32 * kEpiWarps2) {
          const int col = min(n_blk * BN + c, p.N - 1);
          cs[c] = __ldg(p.w_mul + col);
          cs[BN + c] = (p.w_shift ? __ldg(p.w_shift + col) : 31) - 48;
        }
      }
      int xm = 0, xs = 0;
      if (row < p.M && p.out_q15) {
        if (p.x_absmax) absmax_to_ms_dev(__ldg(p.x_absmax + row), &xm, &xs);
        else { xm = __ldg(p.x_mul + row); xs = __ldg(p.x_shift + row); }
      }
      asm volatile("bar.sync 1, %0;" ::"n"(32 * kEpiWarps2) : "memory");
      if (ok) ok = mbar_wait(tfull0 + 8 * slot, aph, 3);
      tcgen05_fence_after();
#pragma unroll 1
      for (int c0 = part * 32; c0 < BN; c0 += 32 * (kEpiWarps2 / 4)) {
        int v[32];
        tmem_ld_32x32(tmem_base + ((unsigned)(q * 32) << 16) + slot * BN + (unsigned)c0, v);
        const int col0 = n_blk * BN + c0;
        if (!ok || col0 >= p.N) continue;
        const bool vec = (p.N & 3) == 0;
        if (p.acc_out) store_chunk(stage, lane, v, p.acc_out, r_base, col0, p.M, p.N, vec);
        if (p.out_q15) {
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            const int4 wm = *reinterpret_cast<const int4*>(cs + c0 + j);
            const int4 ws = *reinterpret_cast<const int4*>(cs + BN + c0 + j);
            v[j + 0] = requant_one(v[j + 0], __mulhi(xm, wm.x), xs + ws.x);
            v[j + 1] = requant_one(v[j + 1], __mulhi(xm, wm.y), xs + ws.y);
            v[j + 2] = requant_one(v[j + 2], __mulhi(xm, wm.z), xs + ws.z);
            v[j + 3] = requant_one(v[j + 3], __mulhi(xm, wm.w), xs + ws.w);
          }
          store_chunk(stage, lane, v, p.out_q15, r_base, col0, p.M, p.N, vec);
        }
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_leader(tempty0 + 8 * slot);
    }
  }
  tcgen05_fence_before();
  __syncthreads();
  cluster_barrier();       // the leader's MMAs read the peer's shared memory and write its tensor memory until here
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(2 * BN) : "memory");
  }
}

// The two-CTA kernel with the operands swapped, for 65..256 tokens (decode batches): the pair's 256 accumulator rows
// are WEIGHT rows, the 256 columns are tokens.  Each CTA stages its own 128 weight rows and HALF of the token tile per
// k-block (32 KB instead of the 48 KB of the one-CTA weights-stationary tile, whose CTAs each re-read all tokens):
// at these sizes the time goes into moving operands from L2 into shared memory, not into MMAs.  Tiles follow the
// weights-stationary list in blocks of 256 weight rows: whole-K tiles for the first full_blocks, `splits` parts of K
// for the rest, whose partial sums are added into `partial` with reductions (a warp's 32 lanes are 32 consecutive
// channels of one token: one 128-byte reduction per instruction).
template <int STAGES>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads2, 1)
gemm_w8a8_2sm_ws_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                        const GemmParams p) {
  constexpr int BN = 256;                      // token columns of the pair's tile; each CTA stages BN / 2 token rows
  constexpr int kABytes = kBM * kBK;           // 128 weight rows
  constexpr int kBBytes = (BN / 2) * kBK;      // 128 token rows
  constexpr int kStageBytes = kABytes + kBBytes;
  extern __shared__ __align__(1024) unsigned char smem[];
  unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(tiles + STAGES * kStageBytes);   // full[S], empty[S], tfull[2], tempty[2]
  unsigned* tmem_slot = reinterpret_cast<unsigned*>(bars + 2 * STAGES + 4);
  int32_t* tok_scale = reinterpret_cast<int32_t*>(tmem_slot + 4);               // [2 slots][mul BN | shift BN] per token

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  unsigned rank;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const int num_kb = (p.K + kBK - 1) / kBK;
  const int w_blocks = (p.N + 2 * kBM - 1) / (2 * kBM);
  const int num_tiles = p.full_blocks + (w_blocks - p.full_blocks) * p.splits;
  const unsigned full0 = smem_u32(bars), empty0 = smem_u32(bars + STAGES);
  const unsigned tfull0 = smem_u32(bars + 2 * STAGES), tempty0 = smem_u32(bars + 2 * STAGES + 2);

  if (warp == 0 && lane == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(tfull0 + 8 * s, 1);
      mbar_init(tempty0 + 8 * s, 2 * kEpiWarps2);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(2 * BN) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  pdl_launch_dependents();
  tcgen05_fence_before();
  __syncthreads();
  cluster_barrier();
  tcgen05_fence_after();
  const unsigned tmem_base = *tmem_slot;
  pdl_wait();

  if (warp == 0) {
    if (lane == 0) {
      unsigned it = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        const WsTile t = ws_tile(p, tile, num_kb);
        for (int kb = t.kb0; kb < t.kb1; ++kb, ++it) {
          const unsigned s = it % STAGES, ph = (it / STAGES) & 1;
          ok = mbar_wait(empty0 + 8 * s, ph ^ 1, 1);
          if (!ok) break;
          if (leader) mbar_expect_tx(full0 + 8 * s, 2 * kStageBytes);
          const unsigned a_dst = smem_u32(tiles + s * kStageBytes);
          const unsigned lbar = (full0 + 8 * s) & kPeerBitMask;
          tma_load_2d_2sm(a_dst, &map_w, kb * kBK, t.n_blk * 2 * kBM + (int)rank * kBM, lbar);
          tma_load_2d_2sm(a_dst + kABytes, &map_x, kb * kBK, (int)rank * (BN / 2), lbar);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && leader) {
      constexpr unsigned idesc = make_idesc(2 * kBM, BN);
      unsigned it = 0, lt = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, ++lt) {
        const unsigned slot = lt & 1, aph = (lt >> 1) & 1;
        ok = mbar_wait(tempty0 + 8 * slot, aph ^ 1, 4);
        if (!ok) break;
        tcgen05_fence_after();
        const unsigned tmem_d = tmem_base + slot * BN;
        const WsTile t = ws_tile(p, tile, num_kb);
        for (int kb = t.kb0; kb < t.kb1; ++kb, ++it) {
          const unsigned s = it % STAGES, ph = (it / STAGES) & 1;
          ok = mbar_wait(full0 + 8 * s, ph, 2);
          if (!ok) break;
          tcgen05_fence_after();
          const unsigned a_addr = smem_u32(tiles + s * kStageBytes);
          const uint64_t da = make_smem_desc(a_addr), db = make_smem_desc(a_addr + kABytes);
#pragma unroll
          for (int k = 0; k < kBK / kUmmaK; ++k)
            umma_i8_2sm(tmem_d, da + (uint64_t)(k * kUmmaK >> 4), db + (uint64_t)(k * kUmmaK >> 4), idesc,
                        (kb > t.kb0 || k > 0) ? 1u : 0u);
          tcgen05_commit_pair(empty0 + 8 * s);
        }
        if (ok) tcgen05_commit_pair(tfull0 + 8 * slot);   // nothing is released after an expired wait
      }
    }
  } else {
    const int q = warp & 3;
    const int part = (warp - 2) >> 2;          // which of the interleaved 32-token chunks this warp takes
    const int et = threadIdx.x - 64;
    unsigned lt = 0;
    bool ok = true;
    for (int tile = pair; tile < num_tiles; tile += num_pairs, ++lt) {
      const WsTile t = ws_tile(p, tile, num_kb);
      const unsigned slot = lt & 1, aph = (lt >> 1) & 1;
      const int ch = t.n_blk * 2 * kBM + (int)rank * kBM + q * 32 + lane;
      const bool direct = !t.split;
      const bool empty_part = t.kb0 >= t.kb1;      // a part of K with no k-blocks: nothing was accumulated
      int32_t* cs = tok_scale + slot * 2 * BN;
      if (direct && p.out_q15) {
        for (int c = et; c < BN; c += 32 * kEpiWarps2) {
          const int tk = min(c, p.M - 1);
          int tm, ts;
          if (p.x_absmax) absmax_to_ms_dev(__ldg(p.x_absmax + tk), &tm, &ts);
          else { tm = __ldg(p.x_mul + tk); ts = __ldg(p.x_shift + tk); }
          cs[c] = tm;
          cs[BN + c] = ts - 48;
        }
      }
      int wm = 0, ws = 0;
      if (ch < p.N && direct && p.out_q15) { wm = __ldg(p.w_mul + ch); ws = p.w_shift ? __ldg(p.w_shift + ch) : 31; }
      asm volatile("bar.sync 1, %0;" ::"n"(32 * kEpiWarps2) : "memory");
      if (ok) ok = mbar_wait(tfull0 + 8 * slot, aph, 3);
      tcgen05_fence_after();
#pragma unroll 1
      for (int c0 = part * 32; c0 < BN; c0 += 32 * (kEpiWarps2 / 4)) {
        if (!ok || c0 >= p.M || empty_part) continue;   // warp-uniform
        int v[32];
        tmem_ld_32x32(tmem_base + ((unsigned)(q * 32) << 16) + slot * BN + (unsigned)c0, v);
        if (ch >= p.N) continue;
        if (!direct) {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (c0 + j < p.M) atomicAdd(p.partial + (int64_t)(c0 + j) * p.N + ch, v[j]);   // result unused: a reduction
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            if (c0 + j < p.M) {
              const int64_t o = (int64_t)(c0 + j) * p.N + ch;
              if (p.acc_out) p.acc_out[o] = v[j];
              if (p.out_q15) p.out_q15[o] = requant_one(v[j], __mulhi(cs[c0 + j], wm), cs[BN + c0 + j] + ws);
            }
          }
        }
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_leader(tempty0 + 8 * slot);
    }
  }
  tcgen05_fence_before();
  __syncthreads();
  cluster_barrier();
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(2 * BN) : "memory");
  }
}

// The gate_up projection with SiLU(gate) * up applied in the epilogue (decode batches, up to 256 tokens).  The weight
// keeps the checkpoint's layout [gate rows | up rows] (N = 2 I rows); a CTA pair takes 128 activation channels: each
// CTA stages 64 gate rows AND the 64 up rows of the same channels per k-block (two TMA boxes into one 128-row
// operand tile), so that after the MMAs its tensor-memory lanes 0..63 hold the gate and lanes 64..127 the up
// accumulators of the same (channel, token) pairs.  Epilogue warps of lane quarters 2 and 3 requantise their up
// values and hand them through shared memory to the warps of quarters 0 and 1, which requantise the gate values,
// apply the fixed-point SiLU * up (direct sigmoid table in shared memory) and store act[token][channel]: half the
// bytes of the Q15.16 gate_up tensor, and the row kernel that follows only rotates and quantises.  Blocks of the
// split tail add their parts into `partial` ([M, 2 I], standard columns) and are finished by silu_tail_kernel.
constexpr int kActStages = 4;

template <int STAGES>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads2, 1)
gemm_gate_up_silu_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                         const GemmParams p) {
  constexpr int BN = 256;
  constexpr int kABytes = kBM * kBK;           // 64 gate rows + 64 up rows
  constexpr int kBBytes = (BN / 2) * kBK;      // 128 token rows
  constexpr int kStageBytes = kABytes + kBBytes;
  extern __shared__ __align__(1024) unsigned char smem[];
  unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(tiles + STAGES * kStageBytes);
  unsigned* tmem_slot = reinterpret_cast<unsigned*>(bars + 2 * STAGES + 4);
  int32_t* tok_scale = reinterpret_cast<int32_t*>(tmem_slot + 4);               // [2 slots][mul BN | shift BN] per token
  uint16_t* sneg_tab = reinterpret_cast<uint16_t*>(tok_scale + 4 * BN);
  int32_t* hand = reinterpret_cast<int32_t*>(reinterpret_cast<unsigned char*>(sneg_tab) + kSiluTableBytes);   // [8 warp pairs][32 tokens][32 lanes]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  unsigned rank;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const int num_kb = (p.K + kBK - 1) / kBK;
  const int I = p.N >> 1;                       // activation channels; a multiple of 128
  const int w_blocks = I / kBM;
  const int num_tiles = p.full_blocks + (w_blocks - p.full_blocks) * p.splits;
  const unsigned full0 = smem_u32(bars), empty0 = smem_u32(bars + STAGES);
  const unsigned tfull0 = smem_u32(bars + 2 * STAGES), tempty0 = smem_u32(bars + 2 * STAGES + 2);

  if (warp == 0 && lane == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(tfull0 + 8 * s, 1);
      mbar_init(tempty0 + 8 * s, 2 * kEpiWarps2);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(2 * BN) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  pdl_launch_dependents();
  silu_stage_table(sneg_tab);                   // constant data: staged before the wait on the preceding kernel
  tcgen05_fence_before();
  __syncthreads();
  cluster_barrier();
  tcgen05_fence_after();
  const unsigned tmem_base = *tmem_slot;
  pdl_wait();

  if (warp == 0) {
    if (lane == 0) {
      unsigned it = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        const WsTile t = ws_tile(p, tile, num_kb);
        const int ch0 = t.n_blk * kBM + (int)rank * (kBM / 2);          // first of this CTA's 64 channels
        for (int kb = t.kb0; kb < t.kb1; ++kb, ++it) {
          const unsigned s = it % STAGES, ph = (it / STAGES) & 1;
          ok = mbar_wait(empty0 + 8 * s, ph ^ 1, 1);
          if (!ok) break;
          if (leader) mbar_expect_tx(full0 + 8 * s, 2 * kStageBytes);
          const unsigned a_dst = smem_u32(tiles + s * kStageBytes);
          const unsigned lbar = (full0 + 8 * s) & kPeerBitMask;
          tma_load_2d_2sm(a_dst, &map_w, kb * kBK, ch0, lbar);                       // 64 gate rows
          tma_load_2d_2sm(a_dst + kABytes / 2, &map_w, kb * kBK, I + ch0, lbar);     // the 64 up rows of the same channels
          tma_load_2d_2sm(a_dst + kABytes, &map_x, kb * kBK, (int)rank * (BN / 2), lbar);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && leader) {
      constexpr unsigned idesc = make_idesc(2 * kBM, BN);
      unsigned it = 0, lt = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, ++lt) {
        const unsigned slot = lt & 1, aph = (lt >> 1) & 1;
        ok = mbar_wait(tempty0 + 8 * slot, aph ^ 1, 4);
        if (!ok) break;
        tcgen05_fence_after();
        const unsigned tmem_d = tmem_base + slot * BN;
        const WsTile t = ws_tile(p, tile, num_kb);
        for (int kb = t.kb0; kb < t.kb1; ++kb, ++it) {
          const unsigned s = it % STAGES, ph = (it / STAGES) & 1;
          ok = mbar_wait(full0 + 8 * s, ph, 2);
          if (!ok) break;
          tcgen05_fence_after();
          const unsigned a_addr = smem_u32(tiles + s * kStageBytes);
          const uint64_t da = make_smem_desc(a_addr), db = make_smem_desc(a_addr + kABytes);
#pragma unroll
          for (int k = 0; k < kBK / kUmmaK; ++k)
            umma_i8_2sm(tmem_d, da + (uint64_t)(k * kUmmaK >> 4), db + (uint64_t)(k * kUmmaK >> 4), idesc,
                        (kb > t.kb0 || k > 0) ? 1u : 0u);
          tcgen05_commit_pair(empty0 + 8 * s);
        }
        if (ok) tcgen05_commit_pair(tfull0 + 8 * slot);
      }
    }
  } else {
    const int q = warp & 3;
    const int part = (warp - 2) >> 2;
    const int et = threadIdx.x - 64;
    const bool is_up = q >= 2;
    const int cl = (q & 1) * 32 + lane;                                  // channel inside the CTA's 64
    const int pair_id = (q & 1) * 4 + part;                              // the gate warp and the up warp of the same lanes
    int32_t* my_hand = hand + pair_id * 1024;
    unsigned lt = 0;
    unsigned okw = 1;                                                    // agreed by all epilogue threads, see below
    for (int tile = pair; tile < num_tiles; tile += num_pairs, ++lt) {
      const WsTile t = ws_tile(p, tile, num_kb);
      const unsigned slot = lt & 1, aph = (lt >> 1) & 1;
      const int chan = t.n_blk * kBM + (int)rank * (kBM / 2) + cl;       // < I by construction (I % 128 == 0)
      const int wrow = is_up ? I + chan : chan;                          // weight row = column of the standard layout
      const bool direct = !t.split;
      const bool empty_part = t.kb0 >= t.kb1;
      int32_t* cs = tok_scale + slot * 2 * BN;
      if (direct) {
        for (int c = et; c < BN; c += 32 * kEpiWarps2) {
          const int tk = min(c, p.M - 1);
          int tm, ts;
          absmax_to_ms_dev(__ldg(p.x_absmax + tk), &tm, &ts);
          cs[c] = tm;
          cs[BN + c] = ts - 48;
        }
      }
      int wm = 0, ws = 0;
      if (direct) { wm = __ldg(p.w_mul + wrow); ws = p.w_shift ? __ldg(p.w_shift + wrow) : 31; }
      asm volatile("bar.sync 1, %0;" ::"n"(32 * kEpiWarps2) : "memory");
      unsigned mine = okw ? (mbar_wait(tfull0 + 8 * slot, aph, 3) ? 1u : 0u) : 0u;
      // the two warps of a pair meet at barriers below, so whether the accumulator arrived must be ONE decision for
      // all epilogue threads (a wait that ran out in one warp only would leave its partner at a barrier)
      asm volatile("{\n.reg .pred pi, po;\nsetp.ne.u32 pi, %1, 0;\nbar.red.and.pred po, 1, %2, pi;\nselp.u32 %0, 1, 0, po;\n}"
                   : "=r"(okw) : "r"(mine), "n"(32 * kEpiWarps2) : "memory");
      tcgen05_fence_after();
#pragma unroll 1
      for (int c0 = part * 32; c0 < BN; c0 += 32 * (kEpiWarps2 / 4)) {
        if (!okw || c0 >= p.M || empty_part) continue;                   // uniform over both warps of a pair
        int v[32];
        tmem_ld_32x32(tmem_base + ((unsigned)(q * 32) << 16) + slot * BN + (unsigned)c0, v);
        if (!direct) {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (c0 + j < p.M) atomicAdd(p.partial + (int64_t)(c0 + j) * p.N + wrow, v[j]);
          continue;
        }
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = requant_one(v[j], __mulhi(cs[c0 + j], wm), cs[BN + c0 + j] + ws);
        if (is_up) {
#pragma unroll
          for (int j = 0; j < 32; ++j) my_hand[j * 32 + lane] = v[j];
          asm volatile("bar.sync %0, 64;" ::"r"(2 + pair_id) : "memory");       // handed over
          asm volatile("bar.sync %0, 64;" ::"r"(2 + pair_id) : "memory");       // taken: the buffer may be written again
        } else {
          asm volatile("bar.sync %0, 64;" ::"r"(2 + pair_id) : "memory");
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int u = my_hand[j * 32 + lane];
            if (c0 + j < p.M) p.out_q15[(int64_t)(c0 + j) * I + chan] = silu_mul_elem_table(v[j], u, sneg_tab);
          }
          asm volatile("bar.sync %0, 64;" ::"r"(2 + pair_id) : "memory");
        }
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_leader(tempty0 + 8 * slot);
    }
  }
  tcgen05_fence_before();
  __syncthreads();
  cluster_barrier();
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(2 * BN) : "memory");
  }
}

// Finishes the split tail of gemm_gate_up_silu_kernel: channels [col0, I) of every token from the summed parts in
// `partial` ([M, 2 I]: gate at column c, up at column I + c), zeroing what it read; four channels per thread.
__global__ void __launch_bounds__(256)
silu_tail_kernel(int32_t* partial, const GemmParams p) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.y;
  const int I = p.N >> 1;
  const int c = p.split_col0 + (blockIdx.x * 256 + threadIdx.x) * 4;
  if (c >= I) return;
  int xm, xs;
  absmax_to_ms_dev(__ldg(p.x_absmax + t), &xm, &xs);
  xs -= 48;
  int32_t* gp = partial + (int64_t)t * p.N + c;
  const int4 g = *reinterpret_cast<const int4*>(gp);
  const int4 u = *reinterpret_cast<const int4*>(gp + I);
  const int4 gm = __ldg(reinterpret_cast<const int4*>(p.w_mul + c)), um = __ldg(reinterpret_cast<const int4*>(p.w_mul + I + c));
  int4 gs = make_int4(31, 31, 31, 31), us = gs;
  if (p.w_shift) { gs = __ldg(reinterpret_cast<const int4*>(p.w_shift + c)); us = __ldg(reinterpret_cast<const int4*>(p.w_shift + I + c)); }
  int4 r;
  r.x = silu_mul_elem_table(requant_one(g.x, __mulhi(xm, gm.x), xs + gs.x), requant_one(u.x, __mulhi(xm, um.x), xs + us.x), g_silu_sneg);
  r.y = silu_mul_elem_table(requant_one(g.y, __mulhi(xm, gm.y), xs + gs.y), requant_one(u.y, __mulhi(xm, um.y), xs + us.y), g_silu_sneg);
  r.z = silu_mul_elem_table(requant_one(g.z, __mulhi(xm, gm.z), xs + gs.z), requant_one(u.z, __mulhi(xm, um.z), xs + us.z), g_silu_sneg);
  r.w = silu_mul_elem_table(requant_one(g.w, __mulhi(xm, gm.w), xs + gs.w), requant_one(u.w, __mulhi(xm, um.w), xs + us.w), g_silu_sneg);
  *reinterpret_cast<int4*>(p.out_q15 + (int64_t)t * I + c) = r;
  // behind the result's store (a store right behind the load of the same address waits for the load's miss)
  *reinterpret_cast<int4*>(gp) = make_int4(0, 0, 0, 0);
  *reinterpret_cast<int4*>(gp + I) = make_int4(0, 0, 0, 0);
}

// Clears columns [0, 4 * vec_cols) of m rows (row pitch in elements) before the split-K parts are added into them.
__global__ void __launch_bounds__(256)
zero_cols_kernel(int32_t* __restrict__ base, int m, int vec_cols, int64_t pitch) {
  pdl_launch_dependents();
  pdl_wait();               // the buffer may still be read by the kernel before this one
  const int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (i >= (int64_t)m * vec_cols) return;
  const int64_t r = i / vec_cols;
  *reinterpret_cast<int4*>(base + r * pitch + (i - r * vec_cols) * 4) = make_int4(0, 0, 0, 0);
}

// The epilogue on its own, for the split-K parts gathered in `partial` ([M, N] int32; may be `out` itself):
// four consecutive channels of one token per thread.  With `clear` the sums are zeroed once read: `partial` is then a
// workspace that stays zero between calls, and no clearing launch is needed in front of the next GEMM.
__global__ void __launch_bounds__(256)
splitk_epilogue_kernel(int32_t* partial, const GemmParams p, int clear) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.y;
  const int c = p.split_col0 + (blockIdx.x * 256 + threadIdx.x) * 4;   // only the split blocks' columns
  if (c >= p.N) return;
  int xm, xs;
  if (p.x_absmax) absmax_to_ms_dev(__ldg(p.x_absmax + t), &xm, &xs);
  else { xm = __ldg(p.x_mul + t); xs = __ldg(p.x_shift + t); }
  xs -= 48;
  const int64_t o = (int64_t)t * p.N + c;
  if (c + 3 < p.N && (p.N & 3) == 0) {
    const int4 a = *reinterpret_cast<const int4*>(partial + o);
    const int4 wm = __ldg(reinterpret_cast<const int4*>(p.w_mul + c));
    int4 ws = make_int4(31, 31, 31, 31);
    if (p.w_shift) ws = __ldg(reinterpret_cast<const int4*>(p.w_shift + c));
    int4 r;
    r.x = requant_one(a.x, __mulhi(xm, wm.x), xs + ws.x);
    r.y = requant_one(a.y, __mulhi(xm, wm.y), xs + ws.y);
    r.z = requant_one(a.z, __mulhi(xm, wm.z), xs + ws.z);
    r.w = requant_one(a.w, __mulhi(xm, wm.w), xs + ws.w);
    *reinterpret_cast<int4*>(p.out_q15 + o) = r;
    // behind the result's store: a store issued right behind the load of the same address waits for the load's miss
    if (clear) *reinterpret_cast<int4*>(partial + o) = make_int4(0, 0, 0, 0);
  } else {
    for (int j = 0; j < 4 && c + j < p.N; ++j) {
      const int a = partial[o + j];
      if (clear) partial[o + j] = 0;
      p.out_q15[o + j] = requant_one(a, __mulhi(xm, __ldg(p.w_mul + c + j)), xs + (p.w_shift ? __ldg(p.w_shift + c + j) : 31));
    }
  }
}

// ----------------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  }
  return fn;
}

// int8 matrix [rows, K] row-major; box = 128 bytes of K x box_rows rows, 128-byte swizzle, zero fill.
static bool make_map(CUtensorMap* map, const void* base, int64_t rows, int64_t K, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)K};
  const cuuint32_t box[2] = {(cuuint32_t)kBK, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

static int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
  }
  return n;
}

template <int BN, int STAGES, bool WS = false>
static int launch_gemm(const CUtensorMap& ma, const CUtensorMap& mb, const GemmParams& p, cudaStream_t st) {
  constexpr size_t smem = (size_t)STAGES * (kBM * kBK + BN * kBK) + 1024 + (2 * STAGES + 4) * 8 + 16 + 4 * BN * 4 + kEpiWarps * 32 * kStagePitch * 4;
  static_assert(smem <= 227 * 1024, "shared memory budget");
  cudaError_t e = cudaFuncSetAttribute(gemm_w8a8_kernel<BN, STAGES, WS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) {
    set_error("gemm_w8a8: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    return B200_E_CUDA;
  }
  const int tiles = WS ? p.full_blocks + ((p.N + kBM - 1) / kBM - p.full_blocks) * p.splits
                       : ((p.N + BN - 1) / BN) * ((p.M + kBM - 1) / kBM);
  const int grid = tiles < sm_count() ? tiles : sm_count();
  launch_pdl(gemm_w8a8_kernel<BN, STAGES, WS>, dim3(grid), dim3(kGemmThreads), smem, st, ma, mb, p);
  return check_launch("gemm_w8a8");
}

template <int STAGES>
static int launch_gemm_2sm(const CUtensorMap& ma, const CUtensorMap& mb, const GemmParams& p, cudaStream_t st) {
  constexpr int BN = 256;
  constexpr size_t smem = (size_t)STAGES * (kBM * kBK + (BN / 2) * kBK) + 1024 + (2 * STAGES + 4) * 8 + 16 + 4 * BN * 4 + kEpiWarps2 * 32 * kStagePitch * 4;
  static_assert(smem <= 227 * 1024, "shared memory budget");
  cudaError_t e = cudaFuncSetAttribute(gemm_w8a8_2sm_kernel<STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) {
    set_error("gemm_w8a8: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    return B200_E_CUDA;
  }
  const int tiles = ((p.N + BN - 1) / BN) * ((p.M + 2 * kBM - 1) / (2 * kBM));
  const int pairs = tiles < sm_count() / 2 ? tiles : sm_count() / 2;
  launch_pdl(gemm_w8a8_2sm_kernel<STAGES>, dim3(2 * pairs), dim3(kGemmThreads2), smem, st, ma, mb, p);
  return check_launch("gemm_w8a8 (two-CTA tiles)");
}

template <int STAGES>
static int launch_gemm_2sm_ws(const CUtensorMap& mw, const CUtensorMap& mx, const GemmParams& p, cudaStream_t st) {
  constexpr int BN = 256;
  constexpr size_t smem = (size_t)STAGES * (kBM * kBK + (BN / 2) * kBK) + 1024 + (2 * STAGES + 4) * 8 + 16 + 4 * BN * 4;
  static_assert(smem <= 227 * 1024, "shared memory budget");
  cudaError_t e = cudaFuncSetAttribute(gemm_w8a8_2sm_ws_kernel<STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) {
    set_error("gemm_w8a8: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    return B200_E_CUDA;
  }
  const int tiles = p.full_blocks + ((p.N + 2 * kBM - 1) / (2 * kBM) - p.full_blocks) * p.splits;
  const int pairs = tiles < sm_count() / 2 ? tiles : sm_count() / 2;
  launch_pdl(gemm_w8a8_2sm_ws_kernel<STAGES>, dim3(2 * pairs), dim3(kGemmThreads2), smem, st, mw, mx, p);
  return check_launch("gemm_w8a8 (two-CTA weights-stationary tiles)");
}

static bool pair_ws_enabled() {
  static int on = -1;
  if (on < 0) {
    const char* e = getenv("B200_GEMM_PAIR_WS");
    on = (e && e[0] == '0') ? 0 : 1;
  }
  return on == 1;
}

}  // namespace b200

using namespace b200;

static int gemm_impl(const int8_t* x8, const int8_t* w8, const int32_t* x_absmax, const int32_t* x_mul,
                     const int32_t* x_shift, const int32_t* w_mul, const int32_t* w_shift, int32_t* out_q15,
                     int32_t* acc_out, int64_t m, int64_t n, int64_t k, b200_stream_t s, int32_t* zero_ws = nullptr) {
  // zero_ws: a caller-kept [m, n] int32 workspace that is all zero on entry; split-K parts are added into it without
  // a clearing launch.  With a Q15.16 output the requantising kernel zeroes it again; with acc_out == zero_ws (no
  // Q15.16 output) it holds the exact accumulators on return and whoever consumes them clears it.
  B200_REQUIRE(x8 && w8, B200_E_NULL, "gemm_w8a8: x8 or w8 is null");
  B200_REQUIRE(out_q15 || acc_out, B200_E_NULL, "gemm_w8a8: no output requested");
  B200_REQUIRE(!out_q15 || (((x_mul && x_shift) || x_absmax) && w_mul), B200_E_NULL,
               "gemm_w8a8: the Q15.16 output needs the token scales (x_mul and x_shift, or x_absmax) and w_mul");
  B200_REQUIRE(m >= 0 && n > 0 && k > 0 && m < (1ll << 31) && n < (1ll << 31) && k < (1ll << 31), B200_E_SHAPE,
               "gemm_w8a8: m=%lld n=%lld k=%lld", (long long)m, (long long)n, (long long)k);
  B200_REQUIRE(k % 16 == 0, B200_E_UNSUPPORTED, "gemm_w8a8: k=%lld must be a multiple of 16 (TMA row pitch)", (long long)k);
  if (m == 0) return B200_OK;
  B200_REQUIRE(aligned16(x8) && aligned16(w8) && aligned16(out_q15) && aligned16(acc_out), B200_E_ALIGN,
               "gemm_w8a8: buffers must be 16-byte aligned");
  CUtensorMap ma, mb;
  GemmParams p;
  p.x_absmax = x_absmax; p.x_mul = x_mul; p.x_shift = x_shift; p.w_mul = w_mul; p.w_shift = w_shift;
  p.out_q15 = out_q15; p.acc_out = acc_out; p.M = (int)m; p.N = (int)n; p.K = (int)k;
  p.splits = 1; p.full_blocks = 0; p.partial = nullptr; p.n_peers = 0; p.tp_on = 0; p.split_col0 = 0;
  cudaStream_t st = (cudaStream_t)s;
  const int num_kb = (int)((k + kBK - 1) / kBK);
  // 65..256 tokens: CTA pairs on blocks of 256 weight rows (each CTA stages half of the 256-token tile; rows beyond
  // the batch are zero fill that costs no traffic); fewer tokens: single CTAs on blocks of 128 weight rows with a
  // token tile as narrow as the batch.  (Measured on four layers + lm_head of the 8B shape: the pair form wins by
  // 4 % at 96 and 128 tokens, 1 % at 64, nothing at 48.  B200_GEMM_PAIR_MIN moves the boundary.)
  static int pair_min = -1;
  if (pair_min < 0) { const char* e = getenv("B200_GEMM_PAIR_MIN"); pair_min = e ? atoi(e) : 65; }
  const bool pair_ws = m >= pair_min && m <= 256 && pair_ws_enabled();
  const int block_rows = pair_ws ? 2 * kBM : kBM, units = pair_ws ? sm_count() / 2 : sm_count();
  const int w_blocks = (int)((n + block_rows - 1) / block_rows);
  if (pair_ws || m <= 128 || (m <= 256 && w_blocks < sm_count())) {
    // decode sizes: weights-stationary, K split so that about one CTA (pair) per SM (pair) streams the weights
    // With more blocks than units the whole waves run unsplit and only the blocks of the last, partial wave are
    // split, so that it costs a fraction of a wave instead of a whole one.
    const int tail = w_blocks % units;
    const int split_blocks = w_blocks < units ? w_blocks : tail;
    int splits = split_blocks > 0 ? units / split_blocks : 1;
    splits = splits < 1 ? 1 : (splits > 8 ? 8 : splits);
    while (splits > 1 && num_kb / splits < 4) --splits;
    while (splits > 1 && (splits - 1) * ((num_kb + splits - 1) / splits) >= num_kb) --splits;   // no empty part
    p.splits = splits;
    p.full_blocks = splits > 1 ? w_blocks - split_blocks : 0;
    const int64_t col0 = (int64_t)p.full_blocks * block_rows;     // first column that parts are added into
    p.split_col0 = (int)col0;
    if (splits > 1) {
      // the parts are added into the exact-accumulator output if the caller wants it, else into the
      // Q15.16 output buffer itself, which the epilogue kernel then rewrites in place
      p.partial = zero_ws ? zero_ws : (acc_out ? acc_out : out_q15);
      // (a kernel rather than a memset node: it takes part in the programmatic launch chain of the step)
      if (zero_ws) {
        // already zero
      } else if ((n - col0) % 4 == 0 && col0 % 4 == 0 && n % 4 == 0) {
        const int64_t vecs = (int64_t)m * ((n - col0) / 4);
        launch_pdl(zero_cols_kernel, dim3((unsigned)((vecs + 255) / 256)), dim3(256), 0, st, p.partial + col0, (int)m, (int)((n - col0) / 4), (int64_t)n);
        int rcz = check_launch("gemm_w8a8 (clearing the partial sums)");
        if (rcz != B200_OK) return rcz;
      } else {
        cudaError_t e = cudaMemset2DAsync(p.partial + col0, (size_t)n * sizeof(int32_t), 0, (size_t)(n - col0) * sizeof(int32_t),
                                          (size_t)m, st);
        B200_REQUIRE(e == cudaSuccess, B200_E_CUDA, "gemm_w8a8: cudaMemset2DAsync: %s", cudaGetErrorString(e));
      }
    }
    const int bn = m <= 32 ? 32 : (m <= 64 ? 64 : (m <= 128 ? 128 : 256));
    B200_REQUIRE(make_map(&ma, w8, n, k, kBM), B200_E_CUDA, "gemm_w8a8: cuTensorMapEncodeTiled failed for w8");
    B200_REQUIRE(make_map(&mb, x8, m, k, pair_ws ? kBM : bn), B200_E_CUDA, "gemm_w8a8: cuTensorMapEncodeTiled failed for x8");
    int rc;
    if (pair_ws) {
      rc = launch_gemm_2sm_ws<6>(ma, mb, p, st);
    } else switch (bn) {
      case 256: rc = launch_gemm<256, 4, true>(ma, mb, p, st); break;
      case 128: rc = launch_gemm<128, 6, true>(ma, mb, p, st); break;
      case 64: rc = launch_gemm<64, 8, true>(ma, mb, p, st); break;
      default: rc = launch_gemm<32, 10, true>(ma, mb, p, st); break;
    }
    if (rc != B200_OK || splits == 1 || !out_q15) return rc;
    launch_pdl(splitk_epilogue_kernel, dim3((unsigned)((n - col0 + 1023) / 1024), (unsigned)m), dim3(256), 0, st, p.partial, p, zero_ws ? 1 : 0);
    return check_launch("gemm_w8a8 (split-K epilogue)");
  }
  B200_REQUIRE(make_map(&ma, x8, m, k, kBM), B200_E_CUDA, "gemm_w8a8: cuTensorMapEncodeTiled failed for x8");
  // large problems: 256 x 256 tiles on CTA pairs, when there are enough of them to occupy every pair
  if (((m + 2 * kBM - 1) / (2 * kBM)) * ((n + 255) / 256) >= sm_count() / 2) {
    B200_REQUIRE(make_map(&mb, w8, n, k, kBM), B200_E_CUDA, "gemm_w8a8: cuTensorMapEncodeTiled failed for w8");
    return launch_gemm_2sm<5>(ma, mb, p, st);
  }
  // tile width: wide tiles for throughput at large M; narrow ones at decode sizes so that enough CTAs
  // stream the weights (one m block there, so the tile count is n / BN)
  const int64_t m_tiles = (m + kBM - 1) / kBM;
  int bn = 256;
  while (bn > 32 && m_tiles * ((n + bn - 1) / bn) < sm_count()) bn >>= 1;
  B200_REQUIRE(make_map(&mb, w8, n, k, bn), B200_E_CUDA, "gemm_w8a8: cuTensorMapEncodeTiled failed for w8");
  switch (bn) {
    case 256: return launch_gemm<256, 4>(ma, mb, p, st);
    case 128: return launch_gemm<128, 6>(ma, mb, p, st);
    case 64: return launch_gemm<64, 8>(ma, mb, p, st);
    default: return launch_gemm<32, 10>(ma, mb, p, st);
  }
}

extern "C" int b200_gemm_w8a8(const int8_t* x8, const int8_t* w8, const int32_t* x_mul, const int32_t* x_shift,
                              const int32_t* w_mul, const int32_t* w_shift, int32_t* out_q15, int32_t* acc_out,
                              int64_t m, int64_t n, int64_t k, b200_stream_t s) {
  return gemm_impl(x8, w8, nullptr, x_mul, x_shift, w_mul, w_shift, out_q15, acc_out, m, n, k, s);
}

extern "C" int b200_gemm_w8a8_absmax(const int8_t* x8, const int8_t* w8, const int32_t* x_absmax, const int32_t* w_mul,
                                     const int32_t* w_shift, int32_t* out_q15, int32_t* acc_out, int64_t m, int64_t n,
                                     int64_t k, b200_stream_t s) {
  B200_REQUIRE(x_absmax || !out_q15, B200_E_NULL, "gemm_w8a8_absmax: x_absmax is null");
  return gemm_impl(x8, w8, x_absmax, nullptr, nullptr, w_mul, w_shift, out_q15, acc_out, m, n, k, s);
}

extern "C" int b200_gemm_w8a8_absmax_ws(const int8_t* x8, const int8_t* w8, const int32_t* x_absmax, const int32_t* w_mul,
                                        const int32_t* w_shift, int32_t* out_q15, int32_t* zero_ws, int64_t m, int64_t n,
                                        int64_t k, b200_stream_t s) {
  B200_REQUIRE(x_absmax && out_q15 && zero_ws, B200_E_NULL, "gemm_w8a8_absmax_ws: null pointer");
  B200_REQUIRE(aligned16(zero_ws) && zero_ws != out_q15, B200_E_ALIGN,
               "gemm_w8a8_absmax_ws: the workspace must be 16-byte aligned and distinct from the output");
  return gemm_impl(x8, w8, x_absmax, nullptr, nullptr, w_mul, w_shift, out_q15, nullptr, m, n, k, s, zero_ws);
}

extern "C" int b200_gemm_w8a8_acc_ws(const int8_t* x8, const int8_t* w8, int32_t* zero_ws, int64_t m, int64_t n, int64_t k,
                                     b200_stream_t s) {
  B200_REQUIRE(zero_ws, B200_E_NULL, "gemm_w8a8_acc_ws: the workspace is null");
  return gemm_impl(x8, w8, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, zero_ws, m, n, k, s, zero_ws);
}

extern "C" int b200_gemm_gate_up_silu(const int8_t* x8, const int8_t* w8, const int32_t* x_absmax, const int32_t* w_mul,
                                      const int32_t* w_shift, int32_t* act_out, int32_t* zero_ws, int64_t m, int64_t n2,
                                      int64_t k, b200_stream_t s) {
  B200_REQUIRE(x8 && w8 && x_absmax && w_mul && act_out && zero_ws, B200_E_NULL, "gemm_gate_up_silu: null pointer");
  B200_REQUIRE(m >= 0 && m <= 256 && n2 > 0 && k > 0 && n2 < (1ll << 31) && k < (1ll << 31), B200_E_SHAPE,
               "gemm_gate_up_silu: m=%lld (at most 256) n2=%lld k=%lld", (long long)m, (long long)n2, (long long)k);
  B200_REQUIRE(n2 % 256 == 0 && k % 16 == 0, B200_E_UNSUPPORTED,
               "gemm_gate_up_silu: n2=%lld must be a multiple of 256 (128 activation channels per CTA pair), k=%lld of 16",
               (long long)n2, (long long)k);
  if (m == 0) return B200_OK;
  B200_REQUIRE(aligned16(x8) && aligned16(w8) && aligned16(act_out) && aligned16(zero_ws) && aligned16(w_mul) && aligned16(w_shift),
               B200_E_ALIGN, "gemm_gate_up_silu: buffers must be 16-byte aligned");
  GemmParams p;
  p.x_absmax = x_absmax; p.x_mul = nullptr; p.x_shift = nullptr; p.w_mul = w_mul; p.w_shift = w_shift;
  p.out_q15 = act_out; p.acc_out = nullptr; p.M = (int)m; p.N = (int)n2; p.K = (int)k;
  p.n_peers = 0; p.tp_on = 0;
  const int inter = (int)(n2 / 2), w_blocks = inter / kBM, num_kb = (int)((k + kBK - 1) / kBK), units = sm_count() / 2;
  const int tail = w_blocks % units;
  const int split_blocks = w_blocks < units ? w_blocks : tail;
  int splits = split_blocks > 0 ? units / split_blocks : 1;
  splits = splits < 1 ? 1 : (splits > 8 ? 8 : splits);
  while (splits > 1 && num_kb / splits < 4) --splits;
  while (splits > 1 && (splits - 1) * ((num_kb + splits - 1) / splits) >= num_kb) --splits;
  p.splits = splits;
  p.full_blocks = splits > 1 ? w_blocks - split_blocks : 0;
  p.split_col0 = p.full_blocks * kBM;
  p.partial = zero_ws;
  CUtensorMap mw, mx;
  B200_REQUIRE(make_map(&mw, w8, n2, k, kBM / 2), B200_E_CUDA, "gemm_gate_up_silu: cuTensorMapEncodeTiled failed for w8");
  B200_REQUIRE(make_map(&mx, x8, m, k, kBM), B200_E_CUDA, "gemm_gate_up_silu: cuTensorMapEncodeTiled failed for x8");
  constexpr size_t smem = (size_t)kActStages * (kBM * kBK + 128 * kBK) + 1024 + (2 * kActStages + 4) * 8 + 16 + 4 * 256 * 4 +
                          kSiluTableBytes + 8 * 1024 * 4;
  static_assert(smem <= 227 * 1024, "shared memory budget");
  cudaError_t e = cudaFuncSetAttribute(gemm_gate_up_silu_kernel<kActStages>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  B200_REQUIRE(e == cudaSuccess, B200_E_CUDA, "gemm_gate_up_silu: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
  cudaStream_t st = (cudaStream_t)s;
  const int tiles = p.full_blocks + (w_blocks - p.full_blocks) * p.splits;
  const int pairs = tiles < units ? tiles : units;
  launch_pdl(gemm_gate_up_silu_kernel<kActStages>, dim3(2 * pairs), dim3(kGemmThreads2), smem, st, mw, mx, p);
  int rc = check_launch("gemm_gate_up_silu");
  if (rc != B200_OK || splits == 1) return rc;
  launch_pdl(silu_tail_kernel, dim3((unsigned)((inter - p.split_col0 + 1023) / 1024), (unsigned)m), dim3(256), 0, st, zero_ws, p);
  return check_launch("gemm_gate_up_silu (split tail)");
}

extern "C" int b200_gemm_w8a8_reduce_peers(const int8_t* x8, const int8_t* w8, int32_t* const* peer_acc, int n_peers,
                                           int64_t m, int64_t n, int64_t k, b200_stream_t s) {
  B200_REQUIRE(x8 && w8 && peer_acc, B200_E_NULL, "gemm_w8a8_reduce_peers: null pointer");
  B200_REQUIRE(n_peers >= 1 && n_peers <= 8, B200_E_SHAPE, "gemm_w8a8_reduce_peers: n_peers=%d (1..8)", n_peers);
  B200_REQUIRE(m >= 0 && m <= 256 && n > 0 && k > 0 && n < (1ll << 31) && k < (1ll << 31), B200_E_UNSUPPORTED,
               "gemm_w8a8_reduce_peers: m=%lld n=%lld k=%lld (decode sizes: m <= 256)", (long long)m, (long long)n, (long long)k);
  B200_REQUIRE(k % 16 == 0, B200_E_UNSUPPORTED, "gemm_w8a8_reduce_peers: k=%lld must be a multiple of 16", (long long)k);
  if (m == 0) return B200_OK;
  B200_REQUIRE(aligned16(x8) && aligned16(w8), B200_E_ALIGN, "gemm_w8a8_reduce_peers: operands must be 16-byte aligned");
  GemmParams p;
  p.x_absmax = nullptr; p.x_mul = nullptr; p.x_shift = nullptr; p.w_mul = nullptr; p.w_shift = nullptr;
  p.out_q15 = nullptr; p.acc_out = nullptr; p.M = (int)m; p.N = (int)n; p.K = (int)k; p.partial = nullptr; p.split_col0 = 0;
  p.n_peers = n_peers;
  p.tp_on = 0;
  for (int r = 0; r < 8; ++r) {
    p.peer[r] = r < n_peers ? peer_acc[r] : nullptr;
    B200_REQUIRE(r >= n_peers || p.peer[r] != nullptr, B200_E_NULL, "gemm_w8a8_reduce_peers: peer_acc[%d] is null", r);
  }
  const int w_blocks = (int)((n + kBM - 1) / kBM), num_kb = (int)((k + kBK - 1) / kBK);
  int splits = sm_count() / w_blocks;
  splits = splits < 1 ? 1 : (splits > 8 ? 8 : splits);
  while (splits > 1 && num_kb / splits < 4) --splits;
  while (splits > 1 && (splits - 1) * ((num_kb + splits - 1) / splits) >= num_kb) --splits;
  p.splits = splits;
  p.full_blocks = 0;
  CUtensorMap ma, mb;
  const int bn = m <= 32 ? 32 : (m <= 64 ? 64 : (m <= 128 ? 128 : 256));
  B200_REQUIRE(make_map(&ma, w8, n, k, kBM), B200_E_CUDA, "gemm_w8a8_reduce_peers: cuTensorMapEncodeTiled failed for w8");
  B200_REQUIRE(make_map(&mb, x8, m, k, bn), B200_E_CUDA, "gemm_w8a8_reduce_peers: cuTensorMapEncodeTiled failed for x8");
  cudaStream_t st = (cudaStream_t)s;
  switch (bn) {
    case 256: return launch_gemm<256, 4, true>(ma, mb, p, st);
    case 128: return launch_gemm<128, 6, true>(ma, mb, p, st);
    case 64: return launch_gemm<64, 8, true>(ma, mb, p, st);
    default: return launch_gemm<32, 10, true>(ma, mb, p, st);
  }
}

extern "C" int b200_gemm_w8a8_tp(const b200_tp_block* blk, const int8_t* x8, const int8_t* w8, int64_t m, int64_t n,
                                 int64_t k, b200_stream_t s) {
  B200_REQUIRE(blk && x8 && w8, B200_E_NULL, "gemm_w8a8_tp: null pointer");
  B200_REQUIRE(blk->size >= 1 && blk->size <= kTpMaxRanks && blk->rank >= 0 && blk->rank < blk->size, B200_E_SHAPE,
               "gemm_w8a8_tp: rank=%d size=%d", blk->rank, blk->size);
  B200_REQUIRE(m >= 1 && m <= 256 && m <= blk->m_max && n == blk->n && k > 0 && k < (1ll << 31), B200_E_UNSUPPORTED,
               "gemm_w8a8_tp: m=%lld (1..min(256, %d)) n=%lld (the block's %lld) k=%lld", (long long)m, blk->m_max,
               (long long)n, (long long)blk->n, (long long)k);
  B200_REQUIRE(k % 16 == 0 && n % 4 == 0, B200_E_UNSUPPORTED, "gemm_w8a8_tp: k=%lld must be a multiple of 16, n=%lld of 4",
               (long long)k, (long long)n);
  B200_REQUIRE(aligned16(x8) && aligned16(w8), B200_E_ALIGN, "gemm_w8a8_tp: operands must be 16-byte aligned");
  GemmParams p;
  p.x_absmax = nullptr; p.x_mul = nullptr; p.x_shift = nullptr; p.w_mul = nullptr; p.w_shift = nullptr;
  p.out_q15 = nullptr; p.acc_out = nullptr; p.M = (int)m; p.N = (int)n; p.K = (int)k; p.partial = nullptr; p.split_col0 = 0;
  p.n_peers = 0;
  p.tp_on = 1;
  p.tp.rank = blk->rank; p.tp.size = blk->size; p.tp.m_max = blk->m_max; p.tp.n = blk->n;
  for (int r = 0; r < 8; ++r) {
    p.peer[r] = nullptr;
    p.tp.base[r] = r < blk->size ? reinterpret_cast<int32_t*>(blk->base[r]) : nullptr;
    B200_REQUIRE(r >= blk->size || p.tp.base[r] != nullptr, B200_E_NULL, "gemm_w8a8_tp: base[%d] is null", r);
  }
  const int w_blocks = (int)((n + kBM - 1) / kBM), num_kb = (int)((k + kBK - 1) / kBK);
  int splits = sm_count() / w_blocks;
  splits = splits < 1 ? 1 : (splits > 8 ? 8 : splits);
  while (splits > 1 && num_kb / splits < 4) --splits;
  while (splits > 1 && (splits - 1) * ((num_kb + splits - 1) / splits) >= num_kb) --splits;
  p.splits = splits;
  p.full_blocks = 0;
  CUtensorMap ma, mb;
  const int bn = m <= 32 ? 32 : (m <= 64 ? 64 : (m <= 128 ? 128 : 256));
  B200_REQUIRE(make_map(&ma, w8, n, k, kBM), B200_E_CUDA, "gemm_w8a8_tp: cuTensorMapEncodeTiled failed for w8");
  B200_REQUIRE(make_map(&mb, x8, m, k, bn), B200_E_CUDA, "gemm_w8a8_tp: cuTensorMapEncodeTiled failed for x8");
  cudaStream_t st = (cudaStream_t)s;
  switch (bn) {
    case 256: return launch_gemm<256, 4, true>(ma, mb, p, st);
    case 128: return launch_gemm<128, 6, true>(ma, mb, p, st);
    case 64: return launch_gemm<64, 8, true>(ma, mb, p, st);
    default: return launch_gemm<32, 10, true>(ma, mb, p, st);
  }
}

extern "C" int b200_gemm_status(int* out_host, int reset) {
  B200_REQUIRE(out_host, B200_E_NULL, "gemm_status: null pointer");
  cudaError_t e = cudaMemcpyFromSymbol(out_host, g_gemm_status, sizeof(int));
  if (e == cudaSuccess && reset) {
    const int zero = 0;
    e = cudaMemcpyToSymbol(g_gemm_status, &zero, sizeof(int));
  }
  if (e != cudaSuccess) {
    set_error("gemm_status: %s", cudaGetErrorString(e));
    return B200_E_CUDA;
  }
  return B200_OK;
}
