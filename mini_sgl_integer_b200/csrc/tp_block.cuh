// Layout of a tensor-parallel exchange block and the signal / wait steps on it.
//
// Every rank owns one block of device memory with this layout; all blocks are mapped into every
// process (NVLink peer / symmetric memory), so a kernel on rank r can add into, or store to, the
// block of rank p with plain global-memory instructions.  No multicast, no multimem.
//
//   header   64 words, touched by the owner only:
//              [0..3]  epoch[ch]    number of signals this rank has sent on channel ch
//              [4]     absmax exchanges this rank has completed; [12] CTAs of the running one that are done
//              [8..11] arrive[ch]   CTAs of the running producer kernel that have finished
//   flags    [4 channels][8 sources]: flags[ch][src] = the epoch of rank src's last signal on ch
//            (written by rank src, read by the owner)
//   amax     [2][m_max][8]        per-token absmax of every rank's K-slice: word [.][t][src] is written by rank src
//                                 with ONE 4-byte store (always >= 1, so the value is its own arrival flag)
//   gather   [2][8][2 * m_max]    small all-gather slots, one per source rank
//   acc      [2][m_max * n]       the rank's own int32 partial sums (its GEMM adds its split-K parts here with L2
//                                 atomics); READ by the peers with 16-byte loads over NVLink
//   out      [2][m_max * n]       the finished Q15.16 rows, every rank's rows written by their owner
//
// A row-split linear moves its partial sums by PULL: a GEMM only accumulates locally and signals; the rank that
// owns a token row (rank t / ceil(m / size)) then fetches the row's partial sums from every rank's `acc`, adds
// them, requantises and stores the finished row into every rank's `out`.  That is (size - 1) / size of the
// [m, n] matrix in and out of each rank, instead of (size - 1) whole copies as remote atomics (which ran at about
// 14 G additions/s over NVLink here).  With one or two ranks every rank fetches all rows and finishes them itself:
// the same bytes, one exchange step instead of two.  A rank clears an accumulator half one exchange after it was
// used, when the peers' next signal shows that they have finished reading it.
//
// The two halves of amax / gather / acc / out alternate between consecutive exchanges (the half is the parity
// of a counter in the header: word 4 for the absmax exchange, the channel's epoch for the others); the arrival
// of the NEXT exchange (other half) orders the clearing of amax / acc and the reads of out before the half is
// written again.
//
// Channels: 1 = partial sums complete, 2 = small all-gather, 3 = finished rows delivered (0 is unused: the
// absmax exchange needs no flag).
#pragma once

#include "common.cuh"

namespace b200 {

constexpr int kTpMaxRanks = 8;
constexpr int kTpChannels = 4;
constexpr int kTpHdrWords = 64;
constexpr int kTpFlagWords = kTpChannels * kTpMaxRanks;

__host__ __device__ inline int64_t tp_align64(int64_t words) { return (words + 63) & ~int64_t(63); }   // 256 bytes

struct TpLayout {
  int64_t flags, amax, gather, acc, out, total;   // offsets in int32 words from the block's base
  int64_t gather_slot;                       // words per (half, source) slot
  int64_t acc_half;                          // words per accumulator half (and per `out` half)
};

__host__ __device__ inline TpLayout tp_layout(int m_max, int64_t n) {
  TpLayout l;
  l.flags = kTpHdrWords;
  l.amax = l.flags + tp_align64(kTpFlagWords);
  l.gather = l.amax + tp_align64(2 * (int64_t)m_max * kTpMaxRanks);
  l.gather_slot = tp_align64(2 * (int64_t)m_max);
  l.acc = l.gather + 2 * kTpMaxRanks * l.gather_slot;
  l.acc_half = tp_align64((int64_t)m_max * n);
  l.out = l.acc + 2 * l.acc_half;
  l.total = l.out + 2 * l.acc_half;
  return l;
}

// Up to kTpDirectRanks ranks every rank fetches every rank's partial sums of ALL rows and finishes all rows itself
// ("direct": one exchange step); beyond, each row is finished by one owner rank, which hands it out
// (reduce-scatter + all-gather: two steps, 1 / size of the bytes each).
constexpr int kTpDirectRanks = 2;
__host__ __device__ inline bool tp_direct(int size) { return size <= kTpDirectRanks; }
// Token rows per owner for a matrix of m rows (all of them in direct mode).
__host__ __device__ inline int tp_rows_per_rank(int m, int size) { return tp_direct(size) ? m : (m + size - 1) / size; }

// What a kernel needs of the exchange: plain pointers and sizes, passed by value.
struct TpView {
  int rank, size, m_max;
  int64_t n;
  int32_t* base[kTpMaxRanks];
};

__device__ __forceinline__ unsigned long long tp_now_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// System-scope acquire load: about 0.2 us on this part, where a system-scope FENCE costs 1.4 - 3.5 us; the
// waits below therefore poll with it and need no fence of their own.
__device__ __forceinline__ int tp_ld_acquire(const int32_t* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void tp_st_relaxed(int32_t* p, int v) {
  asm volatile("st.relaxed.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Called by ONE thread of a CTA after a CTA barrier that follows the CTA's remote writes.  One system-scope fence
// per CTA orders all of them (the barrier makes them this thread's predecessors; fences are cumulative) before
// the arrival count; the CTA that arrives last raises the channel's epoch and stores it into flags[ch][rank] of
// every rank.
__device__ __forceinline__ void tp_signal_if_last(const TpView& v, int ch, unsigned ctas, bool wrote_remote = true) {
  int32_t* hdr = v.base[v.rank];
  if (wrote_remote) __threadfence_system();   // (a CTA without remote writes has nothing to publish: the fence is slow)
  const unsigned old = atomicAdd(reinterpret_cast<unsigned*>(hdr + 8 + ch), 1u);
  if (old + 1 == ctas) {
    hdr[8 + ch] = 0;
    const int e = hdr[ch] + 1;
    hdr[ch] = e;
    __threadfence_system();          // the other CTAs' arrivals (and what they fenced) before the flag stores
    for (int r = 0; r < v.size; ++r) tp_st_relaxed(v.base[r] + kTpHdrWords + ch * kTpMaxRanks + v.rank, e);
  }
}

// What a kernel of another translation unit needs to take part in the absmax agreement (steps 1 + 2 of the exchange)
// for the row it has just produced: the blocks, and where the status word and the time limit live.
struct TpAgree {
  int rank, size, m_max;
  int64_t amax_off;                   // word offset of amax[0][0][0] inside a block
  int32_t* base[kTpMaxRanks];
  int* status;
  const unsigned long long* timeout_ns;
};

// Called by ALL threads of the CTA that owns token row `row` (one CTA per row, gridDim.x rows): delivers the row's
// local absmax (>= 1) to every rank (`deliver`), waits (bounded) for every rank's word of the row - thread t polls
// rank t's word, so eight peers cost one poll latency, not eight -, clears them and returns the maximum.  `slot` is
// one int of shared memory.
__device__ __forceinline__ int tp_agree_cta(const TpAgree& a, int row, int local, int* slot, bool deliver = true) {
  int32_t* hdr = a.base[a.rank];
  const int half = *reinterpret_cast<volatile int32_t*>(hdr + 4) & 1;
  const int64_t words = a.amax_off + ((int64_t)half * a.m_max + row) * kTpMaxRanks;
  if (threadIdx.x == 0) *slot = 1;
  if (deliver && (int)threadIdx.x < a.size) tp_st_relaxed(a.base[threadIdx.x] + words + a.rank, local);
  __syncthreads();                               // the slot is initialised; this rank's own word is out
  if ((int)threadIdx.x < a.size) {
    int32_t* word = hdr + words + threadIdx.x;
    int w = tp_ld_acquire(word);
    if (w == 0) {
      const unsigned long long t0 = tp_now_ns(), limit = *a.timeout_ns;
      while ((w = tp_ld_acquire(word)) == 0) {
        if (tp_now_ns() - t0 > limit) {
          atomicCAS(a.status, 0, 1);
          break;
        }
        __nanosleep(32);
      }
    }
    *word = 0;
    atomicMax(slot, w);
  }
  __syncthreads();
  if (threadIdx.x == 0 && atomicAdd(reinterpret_cast<unsigned*>(hdr + 12), 1u) + 1 == gridDim.x) {
    hdr[12] = 0;
    hdr[4] += 1;                      // read by the next launch, after this one has ended
  }
  return *slot;
}

// Host side (tp.cu): fills `out` from a block descriptor; returns a status code and sets the error string.
int tp_agree_of(const ::b200_tp_block* blk, TpAgree* out, const char* name);

}  // namespace b200
