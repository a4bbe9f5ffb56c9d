// ks_join.cuh -- K3: interval-overlap join over the start-ordered timeline of all tenants.
//
// With the launches ordered by start_ns, launch i overlaps exactly those later launches j (j > i in the order) with
// start_j < end_i -- a contiguous run behind i -- that belong to another tenant, are not solo launches and satisfy
// start_i < end_j (only false for a zero-length j that starts with i).  Every unordered pair is found once, from its
// earlier member.
//
// A CTA stages a tile of the timeline plus a look-ahead window in shared memory (dictionary slots already translated
// to dense key ids).  Each thread finds, by binary search over the staged start times, where its launches' runs of
// candidates end; an exclusive scan of the run lengths then lets the CTA walk the CANDIDATES, not the launches, in
// strides of the block size (a load-balanced search: the owner of candidate q is found by binary search over the
// scanned run offsets), so a 150 us kernel that overlaps forty short ones costs forty lanes one step instead of one
// lane forty steps.  Valid candidates are compacted with ballots, the CTA reserves a contiguous range of the sample
// stream with one counter update, and consecutive lanes write consecutive samples:
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

struct JoinArgs {
  const unsigned long long* tl_start;
  const unsigned long long* tl_dm;
  const uint32_t* kid_of_slot;
  uint64_t n;
  uint32_t* skey;
  uint32_t* lane0;
  uint32_t* lane1;
  uint32_t* lane2;
  uint32_t* idx_a;  // stage API: positions instead of samples (may be null)
  uint32_t* idx_b;
  uint64_t capacity;  // entries the sample stream (or idx arrays) can hold
  Control* ctl;
};

struct JoinEntry {
  unsigned long long start;
  uint32_t dur;
  uint32_t info;  // kid | tenant << 16 | solo << 24
};

__device__ __forceinline__ JoinEntry join_entry(const JoinArgs& a, uint64_t j) {
  JoinEntry e;
  e.start = a.tl_start[j];
  const unsigned long long dm = a.tl_dm[j];
  e.dur = (uint32_t)dm;
  const uint32_t meta = (uint32_t)(dm >> 32);
  e.info = __ldg(a.kid_of_slot + (meta & kMetaSlotMask)) | ((meta >> 24) << 16) | (((meta >> 23) & 1u) << 24);
  return e;
}

__device__ __forceinline__ bool join_pair_ok(const JoinEntry& ei, const JoinEntry& ej) {
  return !(ej.info >> 24) && (((ei.info ^ ej.info) >> 16) & 0xFFu) != 0 && ei.start < ej.start + ej.dur;
}

template <bool kIndexOutput>
__device__ __forceinline__ void join_emit(const JoinArgs& a, unsigned long long out, const JoinEntry& ei, const JoinEntry& ej, uint64_t gi, uint64_t gj,
                                          uint32_t nk) {
  if (out >= a.capacity) return;
  const bool i_is_a = ((ei.info >> 16) & 0xFFu) < ((ej.info >> 16) & 0xFFu);
  if constexpr (kIndexOutput) {
    a.idx_a[out] = (uint32_t)(i_is_a ? gi : gj);
    a.idx_b[out] = (uint32_t)(i_is_a ? gj : gi);
  } else {
    const uint32_t kid_i = ei.info & 0xFFFFu, kid_j = ej.info & 0xFFFFu;
    const uint32_t ka = i_is_a ? kid_i : kid_j, kb = i_is_a ? kid_j : kid_i;
    a.skey[out] = nk + ka * nk + kb;
    a.lane0[out] = i_is_a ? ei.dur : ej.dur;
    a.lane1[out] = i_is_a ? ej.dur : ei.dur;
    a.lane2[out] = (uint32_t)(max(ei.start + ei.dur, ej.start + ej.dur) - ei.start);
  }
}

template <bool kIndexOutput>
__global__ void __launch_bounds__(kJoinThreads) k_join(const JoinArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  JoinEntry* win = reinterpret_cast<JoinEntry*>(smem_raw);                    // [kJoinTile + kJoinAhead]
  uint32_t* run_off = reinterpret_cast<uint32_t*>(win + kJoinTile + kJoinAhead);  // [kJoinTile + 1] exclusive run offsets
  __shared__ uint32_t warp_tot[kJoinThreads / 32];
  __shared__ unsigned long long s_base;
  __shared__ uint32_t s_spill;

  const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
  const uint64_t t0 = (uint64_t)blockIdx.x * kJoinTile;
  if (t0 >= a.n) return;
  const uint32_t tn = (uint32_t)min((uint64_t)kJoinTile, a.n - t0);                 // launches of this tile
  const uint32_t wn = (uint32_t)min((uint64_t)(kJoinTile + kJoinAhead), a.n - t0);  // staged entries
  for (uint32_t i = tid; i < wn; i += kJoinThreads) win[i] = join_entry(a, t0 + i);
  if (tid == 0) s_spill = 0;
  __syncthreads();
  const uint32_t nk = a.ctl->n_keys;

  // ---- run length of every launch of the tile inside the window: candidates (li, li + 1 .. hi - 1)
  // thread t owns launches 4t .. 4t+3 so that the scan below is a plain blocked scan
  uint32_t len[kJoinPerThread], mine = 0;
  bool spills = false;
#pragma unroll
  for (int k = 0; k < kJoinPerThread; ++k) {
    const uint32_t li = tid * kJoinPerThread + k;
    len[k] = 0;
    if (li < tn) {
      const JoinEntry ei = win[li];
      if (!(ei.info >> 24) && ei.dur) {
        const unsigned long long end_i = ei.start + ei.dur;
        uint32_t lo = li + 1, hi = wn;  // first staged entry with start >= end_i
        while (lo < hi) {
          const uint32_t mid = (lo + hi) >> 1;
          if (win[mid].start < end_i) lo = mid + 1; else hi = mid;
        }
        len[k] = lo - (li + 1);
        if (lo == wn && t0 + wn < a.n) spills = true;  // the run may go on behind the window
      }
    }
    mine += len[k];
  }
  if (spills) atomicOr(&s_spill, 1u);
  const uint32_t inc = warp_incl_scan(mine);
  if (lane == 31) warp_tot[warp] = inc;
  __syncthreads();
  uint32_t off = inc - mine, total = 0;
  for (uint32_t w = 0; w < kJoinThreads / 32; ++w) {
    if (w < warp) off += warp_tot[w];
    total += warp_tot[w];
  }
#pragma unroll
  for (int k = 0; k < kJoinPerThread; ++k) {
    run_off[tid * kJoinPerThread + k] = off;
    off += len[k];
  }
  if (tid == kJoinThreads - 1) run_off[kJoinTile] = total;
  __syncthreads();
  const bool any_spill = s_spill != 0;

  auto owner_of = [&](uint32_t q) -> uint32_t {  // last launch whose run starts at or before candidate q
    uint32_t lo = 0, hi = kJoinTile;
    while (lo + 1 < hi) {
      const uint32_t mid = (lo + hi) >> 1;
      if (run_off[mid] <= q) lo = mid; else hi = mid;
    }
    return lo;
  };

  // ---- pass 0 counts the valid candidates, pass 1 writes them (block-ordered compaction)
  uint32_t n_valid = 0, spill_valid = 0;
  unsigned long long out_base = 0;
  for (int pass = 0; pass < 2; ++pass) {
    uint32_t running = 0;  // valid candidates of earlier rounds (pass 1)
    for (uint32_t q0 = 0; q0 < total; q0 += kJoinThreads) {
      const uint32_t q = q0 + tid;
      bool ok = false;
      uint32_t li = 0, lj = 0;
      if (q < total) {
        li = owner_of(q);
        lj = li + 1 + (q - run_off[li]);
        ok = join_pair_ok(win[li], win[lj]);
      }
      const uint32_t ballot = __ballot_sync(0xFFFFFFFFu, ok);
      if (pass == 0) {
        if (lane == 0) n_valid += __popc(ballot);
      } else {
        __syncthreads();
        if (lane == 0) warp_tot[warp] = __popc(ballot);
        __syncthreads();
        uint32_t before = running, round_total = 0;
        for (uint32_t w = 0; w < kJoinThreads / 32; ++w) {
          if (w < warp) before += warp_tot[w];
          round_total += warp_tot[w];
        }
        if (ok) join_emit<kIndexOutput>(a, out_base + before + __popc(ballot & lanemask_lt()), win[li], win[lj], t0 + li, t0 + lj, nk);
        running += round_total;
      }
    }
    // runs that continue behind the window: their owner walks the rest from global memory
    uint32_t spill_cnt = 0;
    if (any_spill) {
#pragma unroll 1
      for (int k = 0; k < kJoinPerThread; ++k) {
        const uint32_t li = tid * kJoinPerThread + k;
        if (!(li < tn && li + 1 + len[k] == wn)) continue;  // only runs that reached the end of the window
        const JoinEntry ei = win[li];
        if ((ei.info >> 24) || !ei.dur) continue;
        const unsigned long long end_i = ei.start + ei.dur;
        for (uint64_t j = t0 + wn; j < a.n; ++j) {
          const JoinEntry ej = join_entry(a, j);
          if (ej.start >= end_i) break;
          if (!join_pair_ok(ei, ej)) continue;
          if (pass == 1) join_emit<kIndexOutput>(a, out_base + n_valid + spill_valid + spill_cnt, ei, ej, t0 + li, j, nk);
          ++spill_cnt;
        }
      }
    }
    if (pass == 0) {
      // totals: window candidates (lane 0 of each warp holds its warp's count) and spilled ones (every thread)
      n_valid = __shfl_sync(0xFFFFFFFFu, n_valid, 0);
      __syncthreads();
      if (lane == 0) warp_tot[warp] = n_valid;
      __syncthreads();
      uint32_t cta_valid = 0;
      for (uint32_t w = 0; w < kJoinThreads / 32; ++w) cta_valid += warp_tot[w];
      n_valid = cta_valid;
      uint32_t cta_spill = 0;
      if (any_spill) {
        const uint32_t sinc = warp_incl_scan(spill_cnt);
        __syncthreads();
        if (lane == 31) warp_tot[warp] = sinc;
        __syncthreads();
        spill_valid = sinc - spill_cnt;
        for (uint32_t w = 0; w < kJoinThreads / 32; ++w) {
          if (w < warp) spill_valid += warp_tot[w];
          cta_spill += warp_tot[w];
        }
      }
      __syncthreads();
      if (tid == 0) s_base = (cta_valid + cta_spill) ? atomicAdd(&a.ctl->n_pairs, (unsigned long long)(cta_valid + cta_spill)) : 0ull;
      __syncthreads();
      if (cta_valid + cta_spill == 0) return;
      out_base = s_base;
    }
  }
}

constexpr size_t join_smem_bytes() { return (size_t)(kJoinTile + kJoinAhead) * sizeof(JoinEntry) + (kJoinTile + 1) * sizeof(uint32_t); }

}  // namespace ks
