// ks_join.cuh -- K3: interval-overlap join over the start-ordered timeline of all tenants.
//
// With the launches ordered by start_ns, launch i overlaps exactly those later launches j (j > i in the order) with
// start_j < end_i -- a contiguous run behind i -- that belong to another tenant, are not solo launches and satisfy
// start_i < end_j (only false for a zero-length j that starts with i).  Every unordered pair is found once, from its
// earlier member.
//
// A CTA stages a tile of the timeline plus a look-ahead window in shared memory as separate start / duration / info
// arrays; start times are stored relative to the window's first entry in 32 bits whenever the window spans less than
// 2^31 ns (always, for a busy trace), so the searches and comparisons are 32-bit.  Consecutive lanes take consecutive launches and
// find where their run of candidates ends by a galloping search (most runs are empty or a few entries long).  An
// exclusive scan of the run lengths numbers the CANDIDATES of the tile; they are then examined ONCE, in rounds of
// kJoinChunk consecutive candidates (merge-path style: one binary search for the owner of a thread's first candidate,
// then a walk), so a 150 us kernel that overlaps forty short ones is spread over many lanes.  The pairs that pass go to a
// shared-memory queue in candidate order (one block-wide scan of the threads' counts) and the queue leaves as one
// contiguous, coalesced run of the sample stream behind a single update of the global sample counter.  One sample per pair:
//     sort key = n_keys + kid_a * n_keys + kid_b       (a = the launch of the lower tenant)
//     lane 0 = duration of a, lane 1 = duration of b, lane 2 = max(end) - min(start)
// Runs that leave the staged window (a launch longer than the look-ahead) are finished by their owner from global
// memory.
#pragma once

#include "ks_common.cuh"

namespace ks {

constexpr int kJoinThreads = 256;
constexpr int kJoinPerThread = 4;
constexpr int kJoinTile = kJoinThreads * kJoinPerThread;  // 1024 launches per CTA
constexpr int kJoinAhead = 512;                           // look-ahead window
constexpr int kJoinWindow = kJoinTile + kJoinAhead;

struct JoinArgs {
  const unsigned long long* tl_start;
  const unsigned long long* tl_dm;
  const uint32_t* kid_of_slot;
  uint64_t n;       // timeline entries that may be read
  uint64_t n_own;   // 0, or: only the first n_own entries look for partners (the others are only found); a slice of a longer
                    // timeline is joined this way, window after window
  uint4* samples;   // {sort key, duration of a, duration of b, span}
  uint32_t* idx_a;  // stage API: positions instead of samples (may be null)
  uint32_t* idx_b;
  uint64_t capacity;  // entries the sample stream (or idx arrays) can hold
  uint64_t n_halo;    // the first n_halo timeline entries belong to the previous time window: a pair is emitted only if
                      // its later member is at or behind this position (single owner across windows)
  Control* ctl;
};

// A window entry.  TimeT = uint32_t when the window's start times fit 31 bits relative to its first entry (then every
// comparison and the staging traffic are 32-bit), unsigned long long otherwise.
template <typename TimeT>
struct JoinEntryT {
  TimeT start;
  uint32_t dur;
  uint32_t info;  // dictionary slot | solo << 23 | tenant << 24
};
using JoinEntry = JoinEntryT<unsigned long long>;

// window entries keep the timeline's meta word; slots are translated to dense key ids only for the pairs that are
// emitted (about one lookup per two launches instead of three per two)
__device__ __forceinline__ bool info_solo(uint32_t info) { return (info & kMetaSoloBit) != 0; }
__device__ __forceinline__ uint32_t info_tenant(uint32_t info) { return info >> 24; }

__device__ __forceinline__ JoinEntry join_entry(const JoinArgs& a, uint64_t j) {
  JoinEntry e;
  e.start = a.tl_start[j];
  const unsigned long long dm = a.tl_dm[j];
  e.dur = (uint32_t)dm;
  e.info = (uint32_t)(dm >> 32);
  return e;
}

template <typename TimeT>
__device__ __forceinline__ bool join_pair_ok(const JoinEntryT<TimeT>& ei, const JoinEntryT<TimeT>& ej) {
  return !info_solo(ej.info) && ((ei.info ^ ej.info) >> 24) != 0 && ei.start < ej.start + ej.dur;
}

constexpr int kJoinChunk = kJoinThreads * 4;  // candidates examined per round: four consecutive ones per thread

struct JoinShared {
  unsigned long long start_raw[kJoinWindow];  // TimeT view: the first sizeof(TimeT) * kJoinWindow bytes
  uint32_t dur[kJoinWindow];
  uint32_t info[kJoinWindow];
  __align__(16) uint32_t run_off[kJoinTile + 4];  // run lengths, then their exclusive scan
  __align__(16) uint4 queue[kJoinChunk];          // the samples of one round, in the order they leave for global memory
  uint32_t warp_tot[kJoinThreads / 32];
  unsigned long long base_out;
  uint32_t spill;
  uint32_t wide;
};

// One sample (or one index pair, as a uint4 {a, b, 0, 0}) of the pair (i, j); gi / gj are the global positions.
template <bool kIndexOutput, typename TimeT>
__device__ __forceinline__ uint4 join_sample(const JoinArgs& a, const JoinEntryT<TimeT>& ei, const JoinEntryT<TimeT>& ej, uint64_t gi, uint64_t gj, uint32_t nk) {
  const bool i_is_a = info_tenant(ei.info) < info_tenant(ej.info);
  if constexpr (kIndexOutput) {
    return make_uint4((uint32_t)(i_is_a ? gi : gj), (uint32_t)(i_is_a ? gj : gi), 0u, 0u);
  } else {
    const uint32_t kid_i = __ldg(a.kid_of_slot + (ei.info & kMetaSlotMask)), kid_j = __ldg(a.kid_of_slot + (ej.info & kMetaSlotMask));
    const uint32_t ka = i_is_a ? kid_i : kid_j, kb = i_is_a ? kid_j : kid_i;
    return make_uint4(nk + ka * nk + kb, i_is_a ? ei.dur : ej.dur, i_is_a ? ej.dur : ei.dur, (uint32_t)(max(ei.start + ei.dur, ej.start + ej.dur) - ei.start));
  }
}
template <bool kIndexOutput>
__device__ __forceinline__ void join_store(const JoinArgs& a, unsigned long long out, const uint4& v) {
  if (out >= a.capacity) return;
  if constexpr (kIndexOutput) { a.idx_a[out] = v.x; a.idx_b[out] = v.y; }
  else a.samples[out] = v;
}

// The tile's work once the window is staged.  base = start_ns the TimeT values are relative to (0 for 64-bit).
// Candidates are examined ONCE: in rounds of kJoinChunk consecutive candidates, four per thread, the pairs that pass go to
// a shared-memory queue in candidate order (one block-wide scan of the threads' counts), and the queue leaves for global
// memory as one contiguous, coalesced run behind a single update of the global sample counter.
template <bool kIndexOutput, typename TimeT>
__device__ __forceinline__ void join_tile(const JoinArgs& a, JoinShared& sh, uint64_t t0, uint32_t tn, uint32_t wn, unsigned long long base) {
  using Entry = JoinEntryT<TimeT>;
  const TimeT* s_start = reinterpret_cast<const TimeT*>(sh.start_raw);
  const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
  const uint32_t nk = a.ctl->n_keys;
  auto entry = [&](uint32_t i) -> Entry { Entry e; e.start = s_start[i]; e.dur = sh.dur[i]; e.info = sh.info[i]; return e; };

  // ---- run length of every launch of the tile inside the window (consecutive lanes, consecutive launches)
  bool spills = false;
#pragma unroll
  for (int k = 0; k < kJoinPerThread; ++k) {
    const uint32_t li = k * kJoinThreads + tid;
    uint32_t len = 0;
    if (li < tn && !info_solo(sh.info[li]) && sh.dur[li]) {
      const TimeT end_i = s_start[li] + sh.dur[li];
      // gallop: [lo, hi) brackets the first staged entry with start >= end_i
      uint32_t lo = li + 1, step = 1, hi = lo;
      while (hi < wn && s_start[hi] < end_i) { lo = hi + 1; hi += step; step <<= 1; }
      hi = min(hi, wn);
      while (lo < hi) {
        const uint32_t mid = (lo + hi) >> 1;
        if (s_start[mid] < end_i) lo = mid + 1; else hi = mid;
      }
      len = lo - (li + 1);
      if (lo == wn && t0 + wn < a.n) spills = true;  // the run may go on behind the window
    }
    sh.run_off[li] = len;
  }
  if (spills) atomicOr(&sh.spill, 1u);
  __syncthreads();
  // ---- exclusive scan of the run lengths (thread t scans launches 4t .. 4t+3)
  uint32_t len4[kJoinPerThread], mine = 0;
  {
    const uint4 v = *reinterpret_cast<const uint4*>(sh.run_off + tid * kJoinPerThread);
    len4[0] = v.x; len4[1] = v.y; len4[2] = v.z; len4[3] = v.w;
    mine = v.x + v.y + v.z + v.w;
  }
  const uint32_t inc = warp_incl_scan(mine);
  if (lane == 31) sh.warp_tot[warp] = inc;
  __syncthreads();
  uint32_t off = inc - mine, total = 0;
  for (uint32_t w = 0; w < kJoinThreads / 32; ++w) {
    if (w < warp) off += sh.warp_tot[w];
    total += sh.warp_tot[w];
  }
  {
    uint4 o;
    o.x = off; o.y = off + len4[0]; o.z = o.y + len4[1]; o.w = o.z + len4[2];
    *reinterpret_cast<uint4*>(sh.run_off + tid * kJoinPerThread) = o;
  }
  if (tid == 0) sh.run_off[kJoinTile] = total;
  __syncthreads();
  const bool any_spill = sh.spill != 0;

  // ---- rounds over the candidates
  for (uint32_t cb = 0; cb < total; cb += kJoinChunk) {
    const uint32_t c0 = min(total, cb + tid * 4u), c1 = min(total, c0 + 4u);
    uint32_t pair[4], n_valid = 0;  // li | lj << 16 of the candidates that pass
    if (c0 < c1) {
      uint32_t lo = 0, hi = kJoinTile;  // last launch whose run starts at or before candidate c0
      while (lo + 1 < hi) {
        const uint32_t mid = (lo + hi) >> 1;
        if (sh.run_off[mid] <= c0) lo = mid; else hi = mid;
      }
      uint32_t li = lo;
      Entry ei = entry(li);
      for (uint32_t q = c0; q < c1; ++q) {
        while (sh.run_off[li + 1] <= q) { ++li; ei = entry(li); }
        const uint32_t lj = li + 1 + (q - sh.run_off[li]);
        const Entry ej = entry(lj);
        if (join_pair_ok(ei, ej) && t0 + lj >= a.n_halo) pair[n_valid++] = li | (lj << 16);
      }
    }
    const uint32_t vinc = warp_incl_scan(n_valid);
    __syncthreads();  // the previous round's queue has left; warp_tot is free
    if (lane == 31) sh.warp_tot[warp] = vinc;
    __syncthreads();
    uint32_t pos = vinc - n_valid, qn = 0;
    for (uint32_t w = 0; w < kJoinThreads / 32; ++w) {
      if (w < warp) pos += sh.warp_tot[w];
      qn += sh.warp_tot[w];
    }
    if (qn == 0) continue;  // uniform
    if (tid == 0) sh.base_out = atomicAdd(&a.ctl->n_pairs, (unsigned long long)qn);
#pragma unroll
    for (uint32_t v = 0; v < 4; ++v) {
      if (v < n_valid) {
        const uint32_t li = pair[v] & 0xFFFFu, lj = pair[v] >> 16;
        sh.queue[pos + v] = join_sample<kIndexOutput>(a, entry(li), entry(lj), t0 + li, t0 + lj, nk);
      }
    }
    __syncthreads();
    const unsigned long long out0 = sh.base_out;
    for (uint32_t i = tid; i < qn; i += kJoinThreads) join_store<kIndexOutput>(a, out0 + i, sh.queue[i]);
  }

  // ---- runs that continue behind the window (a launch longer than the look-ahead): their owner walks the rest from global
  // memory (64-bit times), counts, reserves its own range of the sample stream and walks again to write
  if (any_spill) {
#pragma unroll 1
    for (int k = 0; k < kJoinPerThread; ++k) {
      const uint32_t sl = tid * kJoinPerThread + k;
      if (!(sl < tn && sl + 1 + len4[k] == wn)) continue;  // only runs that reached the end of the window
      JoinEntry es;
      es.start = base + s_start[sl];
      es.dur = sh.dur[sl];
      es.info = sh.info[sl];
      if (info_solo(es.info) || !es.dur) continue;
      const unsigned long long end_s = es.start + es.dur;
      unsigned long long out = 0;
      for (int pass = 0; pass < 2; ++pass) {
        uint32_t cnt = 0;
        for (uint64_t j = t0 + wn; j < a.n; ++j) {
          const JoinEntry ej = join_entry(a, j);
          if (ej.start >= end_s) break;
          if (!join_pair_ok(es, ej) || j < a.n_halo) continue;
          if (pass == 1) join_store<kIndexOutput>(a, out + cnt, join_sample<kIndexOutput>(a, es, ej, t0 + sl, j, nk));
          ++cnt;
        }
        if (pass == 0) {
          if (!cnt) break;
          out = atomicAdd(&a.ctl->n_pairs, (unsigned long long)cnt);
        }
      }
    }
  }
}

template <bool kIndexOutput>
__global__ void __launch_bounds__(kJoinThreads) k_join(const JoinArgs a) {
  __shared__ JoinShared sh;
  const uint32_t tid = threadIdx.x;
  const uint64_t t0 = (uint64_t)blockIdx.x * kJoinTile;
  const uint64_t n_own = a.n_own ? min(a.n_own, a.n) : a.n;
  if (t0 >= n_own) return;
  const uint32_t tn = (uint32_t)min((uint64_t)kJoinTile, n_own - t0);  // launches of this tile
  const uint32_t wn = (uint32_t)min((uint64_t)kJoinWindow, a.n - t0);  // staged entries
  // the window is in start order: it fits 31 bits relative to its first entry iff its last entry does
  const unsigned long long base = a.tl_start[t0];
  const bool wide = a.tl_start[t0 + wn - 1] - base >= 0x80000000ull;
  if (tid == 0) sh.spill = 0;
  if (!wide) {
    uint32_t* s32 = reinterpret_cast<uint32_t*>(sh.start_raw);
    for (uint32_t i = tid; i < wn; i += kJoinThreads) {
      s32[i] = (uint32_t)(a.tl_start[t0 + i] - base);
      const unsigned long long dm = a.tl_dm[t0 + i];
      sh.dur[i] = (uint32_t)dm;
      sh.info[i] = (uint32_t)(dm >> 32);
    }
    __syncthreads();
    join_tile<kIndexOutput, uint32_t>(a, sh, t0, tn, wn, base);
  } else {
    for (uint32_t i = tid; i < wn; i += kJoinThreads) {
      sh.start_raw[i] = a.tl_start[t0 + i];
      const unsigned long long dm = a.tl_dm[t0 + i];
      sh.dur[i] = (uint32_t)dm;
      sh.info[i] = (uint32_t)(dm >> 32);
    }
    __syncthreads();
    join_tile<kIndexOutput, unsigned long long>(a, sh, t0, tn, wn, 0ull);
  }
}

constexpr size_t join_smem_bytes() { return 0; }

}  // namespace ks
