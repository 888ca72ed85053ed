// Layout of a tensor-parallel exchange block and the signal / wait steps on it.
//
// Every rank owns one block of device memory with this layout; all blocks are mapped into every
// process (NVLink peer / symmetric memory), so a kernel on rank r can add into, or store to, the
// block of rank p with plain global-memory instructions.  No multicast, no multimem.
//
//   header   64 words, touched by the owner only:
//              [0..3]  epoch[ch]    number of signals this rank has sent on channel ch
//              [8..11] arrive[ch]   CTAs of the running producer kernel that have finished
//   flags    [4 channels][8 sources]: flags[ch][src] = the epoch of rank src's last signal on ch
//            (written by rank src, read by the owner)
//   amax     [2][m_max]           per-token absmax agreed between the ranks (atomicMax by everybody)
//   gather   [2][8][2 * m_max]    small all-gather slots, one per source rank
//   acc      [2][m_max * n]       int32 accumulators that every rank adds its partial sums into
//
// The two halves of amax / gather / acc alternate between consecutive exchanges on a channel (the
// half is the parity of the channel's epoch), and whoever consumes a half clears it afterwards; the
// signal of the NEXT exchange (other half) orders that clearing before any peer writes the half again.
//
// Channels: 0 = absmax agreement, 1 = accumulator sums, 2 = small all-gather.
#pragma once

#include "common.cuh"

namespace b200 {

constexpr int kTpMaxRanks = 8;
constexpr int kTpChannels = 4;
constexpr int kTpHdrWords = 64;
constexpr int kTpFlagWords = kTpChannels * kTpMaxRanks;

__host__ __device__ inline int64_t tp_align64(int64_t words) { return (words + 63) & ~int64_t(63); }   // 256 bytes

struct TpLayout {
  int64_t flags, amax, gather, acc, total;   // offsets in int32 words from the block's base
  int64_t gather_slot;                       // words per (half, source) slot
  int64_t acc_half;                          // words per accumulator half
};

__host__ __device__ inline TpLayout tp_layout(int m_max, int64_t n) {
  TpLayout l;
  l.flags = kTpHdrWords;
  l.amax = l.flags + tp_align64(kTpFlagWords);
  l.gather = l.amax + tp_align64(2 * (int64_t)m_max);
  l.gather_slot = tp_align64(2 * (int64_t)m_max);
  l.acc = l.gather + 2 * kTpMaxRanks * l.gather_slot;
  l.acc_half = tp_align64((int64_t)m_max * n);
  l.total = l.acc + 2 * l.acc_half;
  return l;
}

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
__device__ __forceinline__ int tp_ld_acquire(const int32_t* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void tp_st_release(int32_t* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Called by ONE thread of a CTA once every thread of the CTA has issued its remote writes and executed
// __threadfence_system() (a CTA barrier in between).  The CTA that arrives last raises the channel's epoch
// and stores it into flags[ch][rank] of every rank.
__device__ __forceinline__ void tp_signal_if_last(const TpView& v, int ch, unsigned ctas) {
  int32_t* hdr = v.base[v.rank];
  const unsigned old = atomicAdd(reinterpret_cast<unsigned*>(hdr + 8 + ch), 1u);
  if (old + 1 == ctas) {
    hdr[8 + ch] = 0;
    const int e = hdr[ch] + 1;
    hdr[ch] = e;
    __threadfence_system();
    for (int r = 0; r < v.size; ++r) tp_st_release(v.base[r] + kTpHdrWords + ch * kTpMaxRanks + v.rank, e);
  }
}

}  // namespace b200
