// ks_reduce.cuh -- K4: segmented reductions over the sorted sample stream, and the final tables.
//
//  k_rows_count / k_rows_scan / k_rows_fill   find where the sort key changes: one row per run (ordered compaction)
//  k_seg_small                                 one warp per row of <= 32 samples: shuffle reductions for sum/min/max and
//                                              a 32-wide bitonic network for the two middle order statistics
//  k_seg_big                                   one CTA per larger row: reductions, then an exact radix select that only
//                                              walks the bits in which the row's minimum and maximum differ
//  k_finalize_keys / k_finalize_pairs          integer statistics -> the float tables (one IEEE division per value)
//
// Everything a row needs from its samples is an integer (durations in ns), so count, min, max and the median are
// exact by construction; the floating-point sum is the exact integer sum divided once.
#pragma once

#include "ks_common.cuh"

namespace ks {

constexpr int kRowsTile = 2048;  // samples per tile of the run-start compaction (256 threads x 8)
constexpr int kLanes = 3;

struct RowStats {
  unsigned long long sum[kLanes];
  uint32_t mn[kLanes], mx[kLanes], lo[kLanes], hi[kLanes];
};

struct RowsArgs {
  const uint32_t* skey;      // sorted sort keys
  const uint32_t* n_dev;     // number of samples in device memory, or nullptr to use n
  uint32_t n;
  uint32_t* tile_cnt;        // [tiles + 1]
  uint32_t* row_start;       // [rows + 1]
  uint32_t* row_key;         // [rows]
  uint32_t* row_of_kid;      // [kMaxKeys + 1], preset to 0xFFFFFFFF
  uint32_t max_tiles;
  uint32_t max_rows;
  Control* ctl;
};

__device__ __forceinline__ bool run_starts_at(const uint32_t* skey, uint32_t i) { return i == 0 || skey[i] != skey[i - 1]; }

__global__ void __launch_bounds__(256) k_rows_count(const RowsArgs a) {
  __shared__ uint32_t warp_tot[8];
  const uint32_t n = a.n_dev ? *a.n_dev : a.n;
  const uint32_t ntiles = (n + kRowsTile - 1) / kRowsTile;
  for (uint32_t tile = blockIdx.x; tile < ntiles && tile < a.max_tiles; tile += gridDim.x) {
    uint32_t c = 0;
#pragma unroll
    for (int k = 0; k < kRowsTile / 256; ++k) {
      const uint32_t i = tile * kRowsTile + k * 256 + threadIdx.x;
      if (i < n) c += run_starts_at(a.skey, i);
    }
    c = warp_sum(c);
    __syncthreads();
    if (lane_id() == 0) warp_tot[threadIdx.x >> 5] = c;
    __syncthreads();
    if (threadIdx.x == 0) {
      uint32_t t = 0;
      for (int w = 0; w < 8; ++w) t += warp_tot[w];
      a.tile_cnt[tile] = t;
    }
  }
}

// one CTA of 1024 threads: exclusive scan of the tile counts in place; total -> Control::n_rows; sentinel row start
__global__ void __launch_bounds__(1024) k_rows_scan(const RowsArgs a) {
  __shared__ uint32_t warp_tot[32];
  __shared__ uint32_t carry;
  const uint32_t n = a.n_dev ? *a.n_dev : a.n;
  const uint32_t ntiles = min((n + kRowsTile - 1) / kRowsTile, a.max_tiles);
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  for (uint32_t base = 0; base < ntiles; base += 1024) {
    const uint32_t i = base + threadIdx.x;
    const uint32_t v = i < ntiles ? a.tile_cnt[i] : 0;
    const uint32_t inc = warp_incl_scan(v);
    if (lane_id() == 31) warp_tot[threadIdx.x >> 5] = inc;
    __syncthreads();
    uint32_t off = carry;
    for (uint32_t w = 0; w < (threadIdx.x >> 5); ++w) off += warp_tot[w];
    if (i < ntiles) a.tile_cnt[i] = off + inc - v;
    __syncthreads();
    if (threadIdx.x == 1023) carry = off + inc;
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    const uint32_t rows = carry;
    a.ctl->n_rows = rows;
    if (rows > a.max_rows) atomicOr(&a.ctl->err, kErrTooLarge);
    else a.row_start[rows] = n;
  }
}

__global__ void __launch_bounds__(256) k_rows_fill(const RowsArgs a) {
  __shared__ uint32_t warp_tot[8];
  const uint32_t n = a.n_dev ? *a.n_dev : a.n;
  const uint32_t nk = a.ctl->n_keys;
  const uint32_t ntiles = min((n + kRowsTile - 1) / kRowsTile, a.max_tiles);
  if (a.ctl->n_rows > a.max_rows) return;
  uint32_t solo_rows = 0;
  for (uint32_t tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
    // thread t owns 8 consecutive samples so that row order = sample order
    const uint32_t i0 = tile * kRowsTile + threadIdx.x * (kRowsTile / 256);
    uint32_t flags = 0, c = 0;
#pragma unroll
    for (int k = 0; k < kRowsTile / 256; ++k) {
      const uint32_t i = i0 + k;
      if (i < n && run_starts_at(a.skey, i)) { flags |= 1u << k; ++c; }
    }
    const uint32_t inc = warp_incl_scan(c);
    __syncthreads();
    if (lane_id() == 31) warp_tot[threadIdx.x >> 5] = inc;
    __syncthreads();
    uint32_t row = a.tile_cnt[tile] + inc - c;
    for (uint32_t w = 0; w < (threadIdx.x >> 5); ++w) row += warp_tot[w];
#pragma unroll
    for (int k = 0; k < kRowsTile / 256; ++k) {
      if (flags & (1u << k)) {
        const uint32_t key = a.skey[i0 + k];
        a.row_start[row] = i0 + k;
        a.row_key[row] = key;
        if (key < nk) { a.row_of_kid[key] = row; ++solo_rows; }
        ++row;
      }
    }
  }
  solo_rows = warp_sum(solo_rows);
  if (lane_id() == 0 && solo_rows) atomicAdd(&a.ctl->ticket2, solo_rows);  // ticket2 = number of solo rows
}

// ---------------------------------------------------------------------------------------------------------
struct SegArgs {
  const uint32_t* lane[kLanes];
  int n_lanes;
  const uint32_t* row_start;
  const uint32_t* n_rows_dev;
  uint32_t max_rows;
  RowStats* stats;
  uint32_t* big_rows;  // [max_rows] rows left to k_seg_big
  Control* ctl;
};

__device__ __forceinline__ uint32_t bitonic_sort32(uint32_t v) {
  const uint32_t lane = lane_id();
#pragma unroll
  for (int k = 2; k <= 32; k <<= 1) {
#pragma unroll
    for (int j = k >> 1; j > 0; j >>= 1) {
      const uint32_t o = __shfl_xor_sync(0xFFFFFFFFu, v, j);
      const bool up = (lane & k) == 0;
      const bool lower = (lane & j) == 0;
      v = (lower == up) ? min(v, o) : max(v, o);
    }
  }
  return v;
}

__global__ void __launch_bounds__(256) k_seg_small(const SegArgs a) {
  const uint32_t n_rows = min(*a.n_rows_dev, a.max_rows);
  const uint32_t lane = lane_id();
  const uint32_t warps = gridDim.x * (blockDim.x >> 5);
  for (uint32_t row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); row < n_rows; row += warps) {
    const uint32_t s = a.row_start[row], cnt = a.row_start[row + 1] - s;
    if (cnt > kSmallSegment) {
      if (lane == 0) a.big_rows[atomicAdd(&a.ctl->n_big, 1u)] = row;
      continue;
    }
    RowStats* st = a.stats + row;
    if (cnt == 0) {  // only the stage API can hand in an empty segment
      if (lane < (uint32_t)a.n_lanes) { st->sum[lane] = 0; st->mn[lane] = 0; st->mx[lane] = 0; st->lo[lane] = 0; st->hi[lane] = 0; }
      continue;
    }
    for (int l = 0; l < a.n_lanes; ++l) {
      const bool have = lane < cnt;
      const uint32_t v = have ? a.lane[l][s + lane] : 0u;
      const unsigned long long sum = warp_sum64(v);
      const uint32_t mx = warp_max(v);
      const uint32_t mn = warp_min(have ? v : 0xFFFFFFFFu);
      const uint32_t sorted = bitonic_sort32(have ? v : 0xFFFFFFFFu);
      const uint32_t lo = __shfl_sync(0xFFFFFFFFu, sorted, (cnt - 1) >> 1);
      const uint32_t hi = __shfl_sync(0xFFFFFFFFu, sorted, cnt >> 1);
      if (lane == 0) { st->sum[l] = sum; st->mn[l] = mn; st->mx[l] = mx; st->lo[l] = lo; st->hi[l] = hi; }
    }
  }
}

// block-wide helpers for k_seg_big (256 threads)
__device__ __forceinline__ unsigned long long block_sum64(unsigned long long v, unsigned long long* sh) {
  v = warp_sum64(v);
  __syncthreads();
  if (lane_id() == 0) sh[threadIdx.x >> 5] = v;
  __syncthreads();
  unsigned long long t = 0;
  for (int w = 0; w < 8; ++w) t += sh[w];
  return t;
}

// value of 0-based rank k among vals[0..cnt) given that all values agree on the bits above `top_bit`
__device__ uint32_t block_radix_select(const uint32_t* vals, uint32_t cnt, uint32_t k, uint32_t common, int top_bit, uint32_t* hist /*[256]*/,
                                       uint32_t* sh_pick /*[2]*/) {
  uint32_t prefix = common;  // bits above the current digit are fixed
  int hi_bit = top_bit;      // highest undecided bit
  while (hi_bit >= 0) {
    const int bits = min(8, hi_bit + 1);
    const int shift = hi_bit + 1 - bits;
    const uint32_t fixed_mask = (hi_bit == 31) ? 0u : ~((2u << hi_bit) - 1u);
    __syncthreads();
    hist[threadIdx.x] = 0;
    __syncthreads();
    for (uint32_t i = threadIdx.x; i < cnt; i += blockDim.x) {
      const uint32_t v = vals[i];
      if ((v & fixed_mask) == (prefix & fixed_mask)) atomicAdd(&hist[(v >> shift) & ((1u << bits) - 1u)], 1u);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      uint32_t acc = 0, d = 0;
      for (; d < (1u << bits); ++d) {
        if (acc + hist[d] > k) break;
        acc += hist[d];
      }
      sh_pick[0] = d;
      sh_pick[1] = acc;
    }
    __syncthreads();
    prefix = (prefix & fixed_mask) | (sh_pick[0] << shift);
    k -= sh_pick[1];
    hi_bit = shift - 1;
  }
  return prefix;
}

__global__ void __launch_bounds__(256) k_seg_big(const SegArgs a) {
  __shared__ unsigned long long sh64[8];
  __shared__ uint32_t sh32[8];
  __shared__ uint32_t hist[256];
  __shared__ uint32_t pick[2];
  const uint32_t n_big = a.ctl->n_big;
  for (uint32_t b = blockIdx.x; b < n_big; b += gridDim.x) {
    const uint32_t row = a.big_rows[b];
    const uint32_t s = a.row_start[row], cnt = a.row_start[row + 1] - s;
    RowStats* st = a.stats + row;
    for (int l = 0; l < a.n_lanes; ++l) {
      const uint32_t* vals = a.lane[l] + s;
      unsigned long long sum = 0;
      uint32_t mn = 0xFFFFFFFFu, mx = 0;
      for (uint32_t i = threadIdx.x; i < cnt; i += blockDim.x) {
        const uint32_t v = vals[i];
        sum += v;
        mn = min(mn, v);
        mx = max(mx, v);
      }
      sum = block_sum64(sum, sh64);
      mn = warp_min(mn);
      mx = warp_max(mx);
      __syncthreads();
      if (lane_id() == 0) sh32[threadIdx.x >> 5] = mn;
      __syncthreads();
      for (int w = 0; w < 8; ++w) mn = min(mn, sh32[w]);
      __syncthreads();
      if (lane_id() == 0) sh32[threadIdx.x >> 5] = mx;
      __syncthreads();
      for (int w = 0; w < 8; ++w) mx = max(mx, sh32[w]);

      uint32_t lo = mn, hi = mn;
      if (mn != mx) {
        const int top_bit = 31 - __clz(mn ^ mx);
        const uint32_t k_lo = (cnt - 1) >> 1, k_hi = cnt >> 1;
        lo = block_radix_select(vals, cnt, k_lo, mn, top_bit, hist, pick);
        hi = lo;
        if (k_hi != k_lo) {
          // hi = x[k_lo + 1]: lo again if more than k_lo + 1 values are <= lo, else the smallest value above lo
          uint32_t le = 0, next = 0xFFFFFFFFu;
          for (uint32_t i = threadIdx.x; i < cnt; i += blockDim.x) {
            const uint32_t v = vals[i];
            le += v <= lo;
            if (v > lo) next = min(next, v);
          }
          const unsigned long long le_tot = block_sum64(le, sh64);
          next = warp_min(next);
          __syncthreads();
          if (lane_id() == 0) sh32[threadIdx.x >> 5] = next;
          __syncthreads();
          for (int w = 0; w < 8; ++w) next = min(next, sh32[w]);
          hi = (le_tot > k_hi) ? lo : next;
        }
      }
      if (threadIdx.x == 0) { st->sum[l] = sum; st->mn[l] = mn; st->mx[l] = mx; st->lo[l] = lo; st->hi[l] = hi; }
      __syncthreads();
    }
  }
}

// ---------------------------------------------------------------------------------------------------------
struct FinalArgs {
  const RowStats* stats;
  const uint32_t* row_start;
  const uint32_t* row_key;
  const uint32_t* row_of_kid;
  const uint32_t* slot_of_kid;
  const unsigned long long* keys_sorted;
  const uint4* dict_words;
  const uint32_t* dict_launches;
  const uint32_t* dict_solo;
  double* solo_ns;        // [kMaxKeys + 1]
  ks_key_row* key_rows;   // [kMaxKeys + 1]
  ks_pair_row* pair_rows; // [max_pair_rows]
  uint32_t max_pair_rows;
  Control* ctl;
};

__global__ void __launch_bounds__(256) k_finalize_keys(const FinalArgs a) {
  const uint32_t nk = min(a.ctl->n_keys, kMaxKeys);
  const uint32_t kid = blockIdx.x * blockDim.x + threadIdx.x;
  if (kid >= nk) return;
  const uint32_t slot = a.slot_of_kid[kid];
  const uint4 w0 = a.dict_words[2 * (size_t)slot], w1 = a.dict_words[2 * (size_t)slot + 1];
  const uint32_t row = a.row_of_kid[kid];
  double solo = __longlong_as_double(0x7FF8000000000000ll);
  if (row != 0xFFFFFFFFu) solo = ((double)a.stats[row].lo[0] + (double)a.stats[row].hi[0]) * 0.5;
  a.solo_ns[kid] = solo;
  ks_key_row r;
  r.key = a.keys_sorted[kid];
  r.name_id = w0.x;
  r.grid[0] = w0.y; r.grid[1] = w0.z; r.grid[2] = w0.w;
  r.block[0] = w1.x; r.block[1] = w1.y; r.block[2] = w1.z;
  r.smem = w1.w & kSmemMask;
  r.tenant = w1.w >> 24;
  r.reserved = 0;
  r.launches = a.dict_launches[slot];
  r.solo_launches = a.dict_solo[slot];
  r.solo_ns = solo;
  a.key_rows[kid] = r;
}

__global__ void __launch_bounds__(256) k_finalize_pairs(const FinalArgs a) {
  const uint32_t n_rows = a.ctl->n_rows, first = a.ctl->ticket2;  // rows [0, first) are the solo rows
  const uint32_t nk = a.ctl->n_keys;
  const double nan = __longlong_as_double(0x7FF8000000000000ll);
  for (uint32_t r = first + blockIdx.x * blockDim.x + threadIdx.x; r < n_rows; r += gridDim.x * blockDim.x) {
    const uint32_t out = r - first;
    if (out >= a.max_pair_rows) { atomicOr(&a.ctl->err, kErrPairTableFull); return; }
    const uint32_t pid = a.row_key[r] - nk;
    const uint32_t ka = pid / nk, kb = pid % nk;
    const RowStats st = a.stats[r];
    const uint32_t cnt = a.row_start[r + 1] - a.row_start[r];
    const double sa = a.solo_ns[ka], sb = a.solo_ns[kb];
    const bool va = sa > 0.0, vb = sb > 0.0;  // false for NaN
    ks_pair_row p;
    p.key_a = a.keys_sorted[ka];
    p.key_b = a.keys_sorted[kb];
    p.count = cnt;
    p.flags = (va ? 1ull : 0ull) | (vb ? 2ull : 0ull);
    if (va) {
      p.sum_a = (double)st.sum[0] / sa;
      p.mean_a = p.sum_a / (double)cnt;
      p.min_a = (double)st.mn[0] / sa;
      p.max_a = (double)st.mx[0] / sa;
      p.median_a = ((double)st.lo[0] / sa + (double)st.hi[0] / sa) * 0.5;
    } else {
      p.sum_a = p.mean_a = p.min_a = p.max_a = p.median_a = nan;
    }
    if (vb) {
      p.sum_b = (double)st.sum[1] / sb;
      p.mean_b = p.sum_b / (double)cnt;
      p.min_b = (double)st.mn[1] / sb;
      p.max_b = (double)st.mx[1] / sb;
      p.median_b = ((double)st.lo[1] / sb + (double)st.hi[1] / sb) * 0.5;
    } else {
      p.sum_b = p.mean_b = p.min_b = p.max_b = p.median_b = nan;
    }
    // efficiency falls as the span grows, so its two middle values come from the span's two middle values
    p.efficiency = (va && vb) ? ((sa + sb) / (double)st.lo[2] + (sa + sb) / (double)st.hi[2]) * 0.5 : nan;
    p.span_sum_ns = st.sum[2];
    a.pair_rows[out] = p;
  }
}

}  // namespace ks
