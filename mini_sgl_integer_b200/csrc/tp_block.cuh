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
//   nblk     [1024]               owner only: parts of K that have arrived per block of 128 output channels
//   amax     [2][m_max][8]        per-token absmax of every rank's K-slice: word [.][t][src] is written by rank src
//                                 with ONE 4-byte store (always >= 1, so the value is its own arrival flag)
//   gather   [2][8][2 * m_max]    small all-gather slots, one per source rank
//   acc      [2][m_max * n]       owner only: the rank's own partial sums (its split-K parts are added here)
//   rs       [2][8][rows_cap * n] reduce-scatter slots: rs[.][src] holds rank src's partial sums of the token
//                                 rows THIS rank owns (rows_cap = ceil(m_max / size)), written by rank src
//   out      [2][m_max * n]       the finished Q15.16 rows, every rank's rows written by their owner
//
// A row-split linear moves its int32 partial sums with plain 16-byte stores: every rank sends each token row
// only to the row's owner (rank t / ceil(m / size)), the owner adds the `size` slots, requantises and stores the
// finished row into every rank's `out`.  That is (size - 1) / size of the [m, n] matrix out of each rank twice,
// instead of (size - 1) whole copies as remote atomics.  With two ranks the bytes are the same either way, so
// every rank receives all rows and finishes them itself: one exchange step instead of two.
//
// The two halves of amax / gather / acc / rs / out alternate between consecutive exchanges (the half is the
// parity of a counter in the header: word 4 for the absmax exchange, the channel's epoch for the others);
// whoever consumes amax or acc clears it afterwards, and the arrival of the NEXT exchange (other half) orders
// that clearing, and the reads of rs / out, before any peer writes the half again.
//
// Channels: 1 = partial sums delivered, 2 = small all-gather, 3 = finished rows delivered (0 is unused: the
// absmax exchange needs no flag).
#pragma once

#include "common.cuh"

namespace b200 {

constexpr int kTpMaxRanks = 8;
constexpr int kTpChannels = 4;
constexpr int kTpHdrWords = 64;
constexpr int kTpFlagWords = kTpChannels * kTpMaxRanks;

__host__ __device__ inline int64_t tp_align64(int64_t words) { return (words + 63) & ~int64_t(63); }   // 256 bytes

constexpr int kTpNblkWords = 1024;

struct TpLayout {
  int64_t flags, nblk, amax, gather, acc, rs, out, total;   // offsets in int32 words from the block's base
  int64_t gather_slot;                       // words per (half, source) slot
  int64_t acc_half;                          // words per accumulator half (and per `out` half)
  int64_t rs_half;                           // words per reduce-scatter half
};

__host__ __device__ inline TpLayout tp_layout(int m_max, int64_t n) {
  TpLayout l;
  l.flags = kTpHdrWords;
  l.nblk = l.flags + tp_align64(kTpFlagWords);
  l.amax = l.nblk + kTpNblkWords;
  l.gather = l.amax + tp_align64(2 * (int64_t)m_max * kTpMaxRanks);
  l.gather_slot = tp_align64(2 * (int64_t)m_max);
  l.acc = l.gather + 2 * kTpMaxRanks * l.gather_slot;
  l.acc_half = tp_align64((int64_t)m_max * n);
  l.rs = l.acc + 2 * l.acc_half;
  l.rs_half = tp_align64(2 * (int64_t)m_max * n);   // size * ceil(m_max / size) rows; two full matrices in direct mode
  l.out = l.rs + 2 * l.rs_half;
  l.total = l.out + 2 * l.acc_half;
  return l;
}

// Up to kTpDirectRanks ranks every rank receives every rank's partial sums of ALL rows and finishes all rows itself
// ("direct": one exchange step); beyond, each row goes to one owner rank, which finishes it and hands it out
// (reduce-scatter + all-gather: two steps, 1 / size of the bytes each).
constexpr int kTpDirectRanks = 2;
__host__ __device__ inline bool tp_direct(int size) { return size <= kTpDirectRanks; }
// Token rows per owner for a matrix of m rows (all of them in direct mode), and the slot pitch in rows.
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

}  // namespace b200
