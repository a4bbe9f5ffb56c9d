// ks_join.cuh -- K3: interval-overlap join over the start-ordered timeline of all tenants.
//
// With the launches ordered by start_ns, launch i overlaps exactly those later launches j (j > i in the order) with
// start_j < end_i -- a contiguous run behind i -- that belong to another tenant, are not solo launches and satisfy
// start_i < end_j (only false for a zero-length j that starts with i).  Every unordered pair is found once, from its
// earlier member.  A CTA stages a tile of the timeline plus a look-ahead window in shared memory (dictionary slots
// already translated to dense key ids), counts its pairs, reserves a contiguous range of the sample stream with one
// counter update, and writes one sample per pair:
//     sort key = n_keys + kid_a * n_keys + kid_b       (a = the launch of the lower tenant)
//     lane 0 = duration of a, lane 1 = duration of b, lane 2 = max(end) - min(start)
// Runs that leave the staged window continue from global memory.
#pragma once

#include "ks_common.cuh"

namespace ks {

constexpr int kJoinThreads = 256;
constexpr int kJoinPerThread = 4;
constexpr int kJoinTile = kJoinThreads * kJoinPerThread;  // 1024 launches per CTA
constexpr int kJoinAhead = 1024;                          // look-ahead window

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
  e.info = a.kid_of_slot[meta & kMetaSlotMask] | ((meta >> 24) << 16) | (((meta >> 23) & 1u) << 24);
  return e;
}

template <bool kIndexOutput>
__global__ void __launch_bounds__(kJoinThreads) k_join(const JoinArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  JoinEntry* win = reinterpret_cast<JoinEntry*>(smem_raw);  // [kJoinTile + kJoinAhead]
  __shared__ uint32_t warp_tot[kJoinThreads / 32];
  __shared__ unsigned long long s_base;

  const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
  const uint64_t t0 = (uint64_t)blockIdx.x * kJoinTile;
  if (t0 >= a.n) return;
  const uint32_t wn = (uint32_t)min((uint64_t)(kJoinTile + kJoinAhead), a.n - t0);
  for (uint32_t i = tid; i < wn; i += kJoinThreads) win[i] = join_entry(a, t0 + i);
  __syncthreads();
  const uint32_t nk = a.ctl->n_keys;

  auto fetch = [&](uint64_t j) -> JoinEntry { return (j - t0 < wn) ? win[j - t0] : join_entry(a, j); };

  // pass 0 counts, pass 1 writes
  uint32_t my_count = 0;
  unsigned long long out = 0;
  for (int pass = 0; pass < 2; ++pass) {
#pragma unroll 1
    for (int k = 0; k < kJoinPerThread; ++k) {
      const uint32_t li = k * kJoinThreads + tid;
      if (li >= kJoinTile || t0 + li >= a.n) continue;
      const JoinEntry ei = win[li];
      if (ei.info >> 24) continue;  // solo launches take no part in the join
      const unsigned long long end_i = ei.start + ei.dur;
      const uint32_t ten_i = (ei.info >> 16) & 0xFFu;
      for (uint64_t j = t0 + li + 1; j < a.n; ++j) {
        const JoinEntry ej = fetch(j);
        if (ej.start >= end_i) break;
        const uint32_t ten_j = (ej.info >> 16) & 0xFFu;
        const unsigned long long end_j = ej.start + ej.dur;
        if ((ej.info >> 24) || ten_j == ten_i || !(ei.start < end_j)) continue;
        if (pass == 0) {
          ++my_count;
        } else {
          if (out < a.capacity) {
            const bool i_is_a = ten_i < ten_j;
            if constexpr (kIndexOutput) {
              a.idx_a[out] = (uint32_t)(i_is_a ? t0 + li : j);
              a.idx_b[out] = (uint32_t)(i_is_a ? j : t0 + li);
            } else {
              const uint32_t kid_i = ei.info & 0xFFFFu, kid_j = ej.info & 0xFFFFu;
              const uint32_t ka = i_is_a ? kid_i : kid_j, kb = i_is_a ? kid_j : kid_i;
              a.skey[out] = nk + ka * nk + kb;
              a.lane0[out] = i_is_a ? ei.dur : ej.dur;
              a.lane1[out] = i_is_a ? ej.dur : ei.dur;
              a.lane2[out] = (uint32_t)(max(end_i, end_j) - ei.start);
            }
          }
          ++out;
        }
      }
    }
    if (pass == 0) {
      // exclusive scan of the per-thread counts, one reservation per CTA
      const uint32_t inc = warp_incl_scan(my_count);
      if (lane == 31) warp_tot[warp] = inc;
      __syncthreads();
      uint32_t off = 0, total = 0;
      for (uint32_t w = 0; w < kJoinThreads / 32; ++w) {
        if (w < warp) off += warp_tot[w];
        total += warp_tot[w];
      }
      if (tid == 0) s_base = total ? atomicAdd(&a.ctl->n_pairs, (unsigned long long)total) : 0ull;
      __syncthreads();
      if (total == 0) return;
      out = s_base + off + inc - my_count;
    }
  }
}

constexpr size_t join_smem_bytes() { return (size_t)(kJoinTile + kJoinAhead) * sizeof(JoinEntry); }

}  // namespace ks
