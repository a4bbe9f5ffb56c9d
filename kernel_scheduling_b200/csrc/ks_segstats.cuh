// ks_segstats.cuh -- K4 core: per row (segment of the sorted sample stream) and per value lane, the exact integer
// statistics  sum, min, max and the two middle order statistics  lo = x[(n-1)/2], hi = x[n/2].
//
// Rows differ in size by six orders of magnitude (most key pairs meet a few times, the hottest pair owns percent of
// all samples), so three size classes share the work:
//
//   tiny   (n <= 4)       k_seg_classify, one thread per row, finishes them in registers (85 % of the rows of a
//                         Zipf-distributed trace) and pushes the other rows onto the work list of their class.
//   small  (n <= 32)      k_seg_small: one warp per row, shuffle reductions and a 32-wide bitonic network.
//   mid    (n <= 2048)    k_seg_mid: one warp per (row, lane).  Reductions, then a radix select over (value - min):
//                         only the bits in which the row's values can differ are walked, 8 per round, with a
//                         256-bin histogram in the warp's own shared memory -- no block-wide barrier anywhere.
//   large  (n > 2048)     the row is cut into chunks of 4096 samples that any CTA may take; k_segL_reduce adds the
//                         chunk's sum/min/max into the row's accumulators, then up to four rounds of
//                         k_segL_hist (chunk histograms of the current digit into the row's global histogram) and
//                         k_segL_resolve (pick the digit that holds the wanted rank) narrow lo and hi separately.
//                         The sample stream of a run is at most a few hundred MB and was just written by the sort,
//                         so these rounds read from L2.
//
// No kernel waits on another CTA; rounds are separate launches.
#pragma once

#include "ks_common.cuh"

namespace ks {

constexpr int kLanes = 3;
constexpr uint32_t kMidMax = 2048;     // largest row the warp-per-(row, lane) kernel takes
constexpr uint32_t kLargeChunk = 4096; // samples per work item of a large row
constexpr int kLargeRounds = 4;        // 8 bits per round: any 32-bit range

struct RowStats {
  unsigned long long sum[kLanes];
  uint32_t mn[kLanes], mx[kLanes], lo[kLanes], hi[kLanes];
};

// accumulators and selection state of one large row; state v = lane * 2 + which (0: lo, 1: hi)
struct LargeRow {
  uint32_t row, start, cnt, pad;
  unsigned long long sum[kLanes];
  uint32_t mn[kLanes], mx[kLanes];
  uint32_t prefix[2 * kLanes];  // decided high bits of (value - min)
  uint32_t k[2 * kLanes];       // rank still to find inside the prefix
  int hi_bit[2 * kLanes];       // highest undecided bit, -1 = resolved
};

struct SegArgs {
  const uint32_t* lane[kLanes];  // value i of lane l is lane[l][i * stride]
  uint32_t stride;
  int n_lanes;
  const uint32_t* row_start;
  const uint32_t* n_rows_dev;
  uint32_t max_rows;
  RowStats* stats;
  uint32_t* small_rows;    // [max_rows]
  uint32_t* mid_rows;      // [max_rows]
  LargeRow* large;         // [max_large]
  uint32_t* chunk_row;     // [max_chunks] index into large[]
  uint32_t* chunk_idx;     // [max_chunks] chunk number inside the row
  uint32_t* large_hist;    // [max_large][2 * kLanes][256]
  uint32_t max_large, max_chunks;
  int round;
  Control* ctl;            // n_big = mid rows, ticket = large rows, scratch0 = chunks, pad[0..3] = unresolved states per round
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

__device__ __forceinline__ int bit_length32(uint32_t v) { return 32 - __clz(v); }

// true if u agrees with prefix on all bits above hi_bit
__device__ __forceinline__ bool matches_prefix(uint32_t u, uint32_t prefix, int hi_bit) {
  return hi_bit >= 31 || (u >> (hi_bit + 1)) == (prefix >> (hi_bit + 1));
}

// One warp, 256 bins in shared memory (8 consecutive bins per lane): the bin that holds rank k and the count below it.
__device__ __forceinline__ void warp_pick_bin(const uint32_t* bins, uint32_t k, uint32_t* digit, uint32_t* below) {
  const uint32_t lane = lane_id();
  uint32_t c[8], tot = 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) { c[i] = bins[lane * 8 + i]; tot += c[i]; }
  const uint32_t inc = warp_incl_scan(tot);
  const uint32_t exc = inc - tot;
  const bool mine = k >= exc && k < inc;
  uint32_t d = 0, b = 0;
  if (mine) {
    uint32_t acc = exc;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (k >= acc && k < acc + c[i]) { d = lane * 8 + i; b = acc; }
      acc += c[i];
    }
  }
  const uint32_t who = __ffs(__ballot_sync(0xFFFFFFFFu, mine)) - 1;
  *digit = __shfl_sync(0xFFFFFFFFu, d, who & 31u);
  *below = __shfl_sync(0xFFFFFFFFu, b, who & 31u);
}

// ---------------------------------------------------------------------------------------------------------
// One thread per row.  Rows of up to four samples (most rows of a Zipf-distributed trace) are finished right here with
// a five-comparator sorting network in registers; the others go to the work list of their size class.
__device__ __forceinline__ void push_row(uint32_t* list, uint32_t* counter, bool mine, uint32_t row) {
  const uint32_t ballot = __ballot_sync(__activemask(), mine);
  if (!mine) return;
  const uint32_t first = __ffs(ballot) - 1;
  uint32_t base = 0;
  if (lane_id() == first) base = atomicAdd(counter, (uint32_t)__popc(ballot));
  base = __shfl_sync(ballot, base, first);
  list[base + __popc(ballot & lanemask_lt())] = row;
}

__global__ void __launch_bounds__(256) k_seg_classify(const SegArgs a) {
  const uint32_t n_rows = min(*a.n_rows_dev, a.max_rows);
  const uint32_t n_round = (n_rows + 31u) & ~31u;  // whole warps take part in the list pushes
  for (uint32_t row = blockIdx.x * blockDim.x + threadIdx.x; row < n_round; row += gridDim.x * blockDim.x) {
    const bool valid = row < n_rows;
    const uint32_t s = valid ? a.row_start[row] : 0, cnt = valid ? a.row_start[row + 1] - s : 0;
    push_row(a.small_rows, &a.ctl->n_small, valid && cnt > 4 && cnt <= kSmallSegment, row);
    push_row(a.mid_rows, &a.ctl->n_big, valid && cnt > kSmallSegment && cnt <= kMidMax, row);
    if (!valid) continue;
    RowStats* st = a.stats + row;
    if (cnt == 0) {  // only the stage API can hand in an empty segment
      for (int l = 0; l < a.n_lanes; ++l) { st->sum[l] = 0; st->mn[l] = 0; st->mx[l] = 0; st->lo[l] = 0; st->hi[l] = 0; }
    } else if (cnt <= 4) {
      for (int l = 0; l < a.n_lanes; ++l) {
        const uint32_t* v = a.lane[l] + (size_t)s * a.stride;
        const uint32_t st1 = a.stride;
        uint32_t x0 = v[0], x1 = cnt > 1 ? v[st1] : 0xFFFFFFFFu, x2 = cnt > 2 ? v[2 * st1] : 0xFFFFFFFFu, x3 = cnt > 3 ? v[3 * st1] : 0xFFFFFFFFu;
        const unsigned long long sum = (unsigned long long)x0 + (cnt > 1 ? x1 : 0u) + (cnt > 2 ? x2 : 0u) + (cnt > 3 ? x3 : 0u);
        uint32_t t;
#define KS_CSWAP(p, q) t = min(p, q); q = max(p, q); p = t;
        KS_CSWAP(x0, x1) KS_CSWAP(x2, x3) KS_CSWAP(x0, x2) KS_CSWAP(x1, x3) KS_CSWAP(x1, x2)
#undef KS_CSWAP
        const uint32_t srt[4] = {x0, x1, x2, x3};
        st->sum[l] = sum;
        st->mn[l] = x0;
        st->mx[l] = srt[cnt - 1];
        st->lo[l] = srt[(cnt - 1) >> 1];
        st->hi[l] = srt[cnt >> 1];
      }
    } else if (cnt > kMidMax) {
      const uint32_t nch = (cnt + kLargeChunk - 1) / kLargeChunk;
      const uint32_t l = atomicAdd(&a.ctl->ticket, 1u);
      const uint32_t cbase = (uint32_t)atomicAdd(&a.ctl->scratch0, (unsigned long long)nch);
      if (l >= a.max_large || cbase + nch > a.max_chunks) { atomicOr(&a.ctl->err, kErrTooLarge); continue; }
      LargeRow* L = a.large + l;
      L->row = row; L->start = s; L->cnt = cnt;
      for (int i = 0; i < kLanes; ++i) { L->sum[i] = 0; L->mn[i] = 0xFFFFFFFFu; L->mx[i] = 0; }
      for (uint32_t c = 0; c < nch; ++c) { a.chunk_row[cbase + c] = l; a.chunk_idx[cbase + c] = c; }
    }
  }
}

// one warp per row of 5..32 samples: shuffle reductions and a 32-wide bitonic network
__global__ void __launch_bounds__(256) k_seg_small(const SegArgs a) {
  const uint32_t n_small = min(a.ctl->n_small, a.max_rows);
  const uint32_t lane = lane_id();
  const uint32_t warps = gridDim.x * (blockDim.x >> 5);
  for (uint32_t t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); t < n_small; t += warps) {
    const uint32_t row = a.small_rows[t];
    const uint32_t s = a.row_start[row], cnt = a.row_start[row + 1] - s;
    RowStats* st = a.stats + row;
    for (int l = 0; l < a.n_lanes; ++l) {
      const bool have = lane < cnt;
      const uint32_t v = have ? a.lane[l][(size_t)(s + lane) * a.stride] : 0u;
      const unsigned long long sum = warp_sum64(v);
      const uint32_t mx = warp_max(v);
      const uint32_t sorted = bitonic_sort32(have ? v : 0xFFFFFFFFu);
      const uint32_t mn = __shfl_sync(0xFFFFFFFFu, sorted, 0);
      const uint32_t lo = __shfl_sync(0xFFFFFFFFu, sorted, (cnt - 1) >> 1);
      const uint32_t hi = __shfl_sync(0xFFFFFFFFu, sorted, cnt >> 1);
      if (lane == 0) { st->sum[l] = sum; st->mn[l] = mn; st->mx[l] = mx; st->lo[l] = lo; st->hi[l] = hi; }
    }
  }
}

// ---------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) k_seg_mid(const SegArgs a) {
  __shared__ uint32_t hist_all[8][256];
  uint32_t* hist = hist_all[threadIdx.x >> 5];
  const uint32_t lane = lane_id();
  const uint32_t n_tasks = min(a.ctl->n_big, a.max_rows) * (uint32_t)a.n_lanes;
  const uint32_t warps = gridDim.x * (blockDim.x >> 5);
  for (uint32_t t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); t < n_tasks; t += warps) {
    const uint32_t row = a.mid_rows[t / a.n_lanes];
    const int l = (int)(t % a.n_lanes);
    const uint32_t s = a.row_start[row], cnt = a.row_start[row + 1] - s;
    const uint32_t* vals = a.lane[l] + (size_t)s * a.stride;
    const uint32_t vs = a.stride;
    unsigned long long sum = 0;
    uint32_t mn = 0xFFFFFFFFu, mx = 0;
    for (uint32_t i = lane; i < cnt; i += 32) {
      const uint32_t v = vals[(size_t)i * vs];
      sum += v;
      mn = min(mn, v);
      mx = max(mx, v);
    }
    sum = warp_sum64(sum);
    mn = warp_min(mn);
    mx = warp_max(mx);
    uint32_t lo = mn, hi = mn;
    if (mn != mx) {
      const uint32_t k_lo = (cnt - 1) >> 1, k_hi = cnt >> 1;
      uint32_t prefix = 0, k = k_lo;
      int hi_bit = bit_length32(mx - mn) - 1;
      while (hi_bit >= 0) {
        const int nb = min(8, hi_bit + 1), shift = hi_bit + 1 - nb;
#pragma unroll
        for (int i = 0; i < 8; ++i) hist[lane * 8 + i] = 0;
        __syncwarp();
        for (uint32_t i = lane; i < cnt; i += 32) {
          const uint32_t u = vals[(size_t)i * vs] - mn;
          if (matches_prefix(u, prefix, hi_bit)) atomicAdd(&hist[(u >> shift) & ((1u << nb) - 1u)], 1u);
        }
        __syncwarp();
        uint32_t d, below;
        warp_pick_bin(hist, k, &d, &below);
        __syncwarp();
        prefix |= d << shift;
        k -= below;
        hi_bit = shift - 1;
      }
      lo = mn + prefix;
      hi = lo;
      if (k_hi != k_lo) {
        // hi = x[k_lo + 1]: lo again if more than k_hi values are <= lo, else the smallest value above lo
        uint32_t le = 0, next = 0xFFFFFFFFu;
        for (uint32_t i = lane; i < cnt; i += 32) {
          const uint32_t v = vals[(size_t)i * vs];
          le += v <= lo;
          if (v > lo) next = min(next, v);
        }
        le = warp_sum(le);
        next = warp_min(next);
        hi = (le > k_hi) ? lo : next;
      }
    }
    if (lane == 0) {
      RowStats* st = a.stats + row;
      st->sum[l] = sum; st->mn[l] = mn; st->mx[l] = mx; st->lo[l] = lo; st->hi[l] = hi;
    }
  }
}

// ---------------------------------------------------------------------------------------------------------
// large rows: chunk work items
__global__ void __launch_bounds__(256) k_segL_reduce(const SegArgs a) {
  __shared__ unsigned long long sh_sum[8];
  __shared__ uint32_t sh_mn[8], sh_mx[8];
  const uint32_t n_chunks = (uint32_t)min(a.ctl->scratch0, (unsigned long long)a.max_chunks);
  for (uint32_t c = blockIdx.x; c < n_chunks; c += gridDim.x) {
    LargeRow* L = a.large + a.chunk_row[c];
    const uint32_t off = a.chunk_idx[c] * kLargeChunk;
    const uint32_t m = min(kLargeChunk, L->cnt - off);
    if (off == 0) {  // the row's first chunk clears the row's histograms for the selection rounds
      uint32_t* gh = a.large_hist + (size_t)a.chunk_row[c] * 2 * kLanes * 256;
      for (uint32_t i = threadIdx.x; i < 2 * kLanes * 256; i += blockDim.x) gh[i] = 0;
    }
    for (int l = 0; l < a.n_lanes; ++l) {
      const uint32_t* vals = a.lane[l] + (size_t)(L->start + off) * a.stride;
      const uint32_t vs = a.stride;
      unsigned long long sum = 0;
      uint32_t mn = 0xFFFFFFFFu, mx = 0;
      for (uint32_t i = threadIdx.x; i < m; i += blockDim.x) {
        const uint32_t v = vals[(size_t)i * vs];
        sum += v;
        mn = min(mn, v);
        mx = max(mx, v);
      }
      sum = warp_sum64(sum);
      mn = warp_min(mn);
      mx = warp_max(mx);
      __syncthreads();
      if (lane_id() == 0) { sh_sum[threadIdx.x >> 5] = sum; sh_mn[threadIdx.x >> 5] = mn; sh_mx[threadIdx.x >> 5] = mx; }
      __syncthreads();
      if (threadIdx.x == 0) {
        for (int w = 1; w < 8; ++w) { sum += sh_sum[w]; mn = min(mn, sh_mn[w]); mx = max(mx, sh_mx[w]); }
        atomicAdd(&L->sum[l], sum);
        atomicMin(&L->mn[l], mn);
        atomicMax(&L->mx[l], mx);
      }
    }
  }
}

// one thread per (large row, state): start the selection
__global__ void __launch_bounds__(256) k_segL_init(const SegArgs a) {
  const uint32_t n_large = min(a.ctl->ticket, a.max_large);
  const uint32_t t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= n_large * 2 * kLanes) return;
  LargeRow* L = a.large + t / (2 * kLanes);
  const int v = (int)(t % (2 * kLanes)), l = v >> 1, which = v & 1;
  if (l >= a.n_lanes) { L->hi_bit[v] = -1; L->prefix[v] = 0; L->k[v] = 0; return; }
  L->prefix[v] = 0;
  L->k[v] = which ? (L->cnt >> 1) : ((L->cnt - 1) >> 1);
  const int hb = (L->mn[l] == L->mx[l]) ? -1 : bit_length32(L->mx[l] - L->mn[l]) - 1;
  L->hi_bit[v] = hb;
  if (hb >= 0) atomicAdd(&a.ctl->pad[0], 1ull);
}

__global__ void __launch_bounds__(256) k_segL_hist(const SegArgs a) {
  __shared__ uint32_t sh[2 * kLanes][256];
  if (a.ctl->pad[a.round] == 0) return;  // nothing left to resolve in this round
  const uint32_t n_chunks = (uint32_t)min(a.ctl->scratch0, (unsigned long long)a.max_chunks);
  for (uint32_t c = blockIdx.x; c < n_chunks; c += gridDim.x) {
    const uint32_t li = a.chunk_row[c];
    const LargeRow* L = a.large + li;
    bool any = false;
    for (int v = 0; v < 2 * a.n_lanes; ++v) any = any || L->hi_bit[v] >= 0;
    if (!any) continue;
    __syncthreads();
    for (uint32_t i = threadIdx.x; i < 2 * kLanes * 256; i += blockDim.x) (&sh[0][0])[i] = 0;
    __syncthreads();
    const uint32_t off = a.chunk_idx[c] * kLargeChunk;
    const uint32_t m = min(kLargeChunk, L->cnt - off);
    for (int l = 0; l < a.n_lanes; ++l) {
      const int hb0 = L->hi_bit[2 * l], hb1 = L->hi_bit[2 * l + 1];
      if (hb0 < 0 && hb1 < 0) continue;
      const uint32_t p0 = L->prefix[2 * l], p1 = L->prefix[2 * l + 1], mn = L->mn[l];
      const int nb0 = min(8, hb0 + 1), sh0 = hb0 + 1 - nb0, nb1 = min(8, hb1 + 1), sh1 = hb1 + 1 - nb1;
      const uint32_t* vals = a.lane[l] + (size_t)(L->start + off) * a.stride;
      const uint32_t vs = a.stride;
      for (uint32_t i = threadIdx.x; i < m; i += blockDim.x) {
        const uint32_t u = vals[(size_t)i * vs] - mn;
        if (hb0 >= 0 && matches_prefix(u, p0, hb0)) atomicAdd(&sh[2 * l][(u >> sh0) & ((1u << nb0) - 1u)], 1u);
        if (hb1 >= 0 && matches_prefix(u, p1, hb1)) atomicAdd(&sh[2 * l + 1][(u >> sh1) & ((1u << nb1) - 1u)], 1u);
      }
    }
    __syncthreads();
    uint32_t* gh = a.large_hist + (size_t)li * 2 * kLanes * 256;
    for (uint32_t i = threadIdx.x; i < 2 * kLanes * 256; i += blockDim.x) {
      const uint32_t x = (&sh[0][0])[i];
      if (x) atomicAdd(&gh[i], x);
    }
  }
}

// one CTA of 2 * kLanes warps per large row: warp v resolves state v, clears its histogram for the next round
__global__ void __launch_bounds__(2 * kLanes * 32) k_segL_resolve(const SegArgs a) {
  __shared__ uint32_t bins[2 * kLanes][256];
  if (a.ctl->pad[a.round] == 0) return;
  const uint32_t n_large = min(a.ctl->ticket, a.max_large);
  const int v = threadIdx.x >> 5;
  const uint32_t lane = lane_id();
  for (uint32_t li = blockIdx.x; li < n_large; li += gridDim.x) {
    LargeRow* L = a.large + li;
    const int hb = L->hi_bit[v];
    if (hb < 0) continue;  // warp-uniform
    uint32_t* gh = a.large_hist + ((size_t)li * 2 * kLanes + v) * 256;
#pragma unroll
    for (int i = 0; i < 8; ++i) { bins[v][lane * 8 + i] = gh[lane * 8 + i]; gh[lane * 8 + i] = 0; }
    __syncwarp();
    uint32_t d, below;
    warp_pick_bin(bins[v], L->k[v], &d, &below);
    __syncwarp();
    if (lane == 0) {
      const int nb = min(8, hb + 1), shift = hb + 1 - nb;
      L->prefix[v] |= d << shift;
      L->k[v] -= below;
      L->hi_bit[v] = shift - 1;
      if (shift - 1 >= 0 && a.round + 1 < kLargeRounds) atomicAdd(&a.ctl->pad[a.round + 1], 1ull);
    }
  }
}

__global__ void __launch_bounds__(256) k_segL_final(const SegArgs a) {
  const uint32_t n_large = min(a.ctl->ticket, a.max_large);
  const uint32_t li = blockIdx.x * blockDim.x + threadIdx.x;
  if (li >= n_large) return;
  const LargeRow* L = a.large + li;
  RowStats* st = a.stats + L->row;
  for (int l = 0; l < a.n_lanes; ++l) {
    st->sum[l] = L->sum[l];
    st->mn[l] = L->mn[l];
    st->mx[l] = L->mx[l];
    st->lo[l] = L->mn[l] + L->prefix[2 * l];
    st->hi[l] = L->mn[l] + L->prefix[2 * l + 1];
    if (L->hi_bit[2 * l] >= 0 || L->hi_bit[2 * l + 1] >= 0) atomicOr(&a.ctl->err, kErrWait);  // cannot happen: 4 x 8 bits
  }
}

}  // namespace ks
