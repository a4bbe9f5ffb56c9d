// ks_segstats.cuh -- K4 core: per row (segment of the sorted sample stream) and per value lane, the exact integer
// statistics  sum, min, max and the two middle order statistics  lo = x[(n-1)/2], hi = x[n/2].
//
// A sample is a 16-byte item {sort key, lane 0, lane 1, lane 2}; every kernel loads an item once (one 128-bit load) and
// feeds all three lanes from it.  The stage entry point ks_segment_stats hands in a plain u32 array instead (one lane).
//
// Rows differ in size by six orders of magnitude (most key pairs meet a few times, the hottest pair owns percent of
// all samples), so five size classes share the work:
//
//   tiny   (n <= 4)       k_seg_classify, one thread per row, finishes them in registers (85 % of the rows of a
//                         Zipf-distributed trace) and pushes the other rows onto the work list of their class.
//   small  (n <= 32)      k_seg_small<W>: W = 8 or 32 lanes per row, shuffle reductions and a W-wide bitonic network.
//   mid    (n <= 512)     k_seg_mid: one warp per row.  The row is read once: its value lanes are staged in the warp's own
//                         shared memory while sum/min/max are taken; then a radix select over (value - min) per lane,
//                         only the bits in which the row's values can differ, 8 per round, with 256-bin histograms in
//                         shared memory -- no block-wide barrier anywhere.
//   big    (n <= 8192)    k_seg_big: one CTA per row, the same scheme with the row staged in 96 KB of shared memory and
//                         block-wide histograms; a row of this size is worth a CTA but not the separate launches of the
//                         large class.
//   large  (n > 8192)     the row is cut into chunks of 4096 samples that any CTA may take; k_segL_reduce adds the
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
constexpr uint32_t kMidMax = 512;      // largest row the warp-per-row kernel takes
constexpr uint32_t kBigMax = 8192;     // largest row the CTA-per-row kernel takes
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
  const uint4* items;      // 16-byte samples (lanes = .y .z .w), or nullptr:
  const uint32_t* plain;   // one lane of plain u32 values
  int n_lanes;             // 3 with items, 1 with plain
  const uint32_t* row_start;
  const uint32_t* n_rows_dev;
  uint32_t max_rows;
  RowStats* stats;
  uint32_t* small_rows;    // [max_rows] rows of 9..32 samples
  uint32_t* small8_rows;   // [max_rows] rows of 5..8 samples
  uint32_t* mid_rows;      // [max_rows]
  uint32_t* big_rows;      // [max_rows] rows of kMidMax+1 .. kBigMax samples
  LargeRow* large;         // [max_large]
  uint32_t* chunk_row;     // [max_chunks] index into large[]
  uint32_t* chunk_idx;     // [max_chunks] chunk number inside the row
  uint32_t* large_hist;    // [max_large][2 * kLanes][256]
  uint32_t max_large, max_chunks;
  int round;
  Control* ctl;            // pad32 / n_small / n_big = rows of 5..8 / 9..32 / mid rows, low word of pad2[1] = big rows,
                           // ticket = large rows, scratch0 = chunks, pad[0..3] = unresolved selection states per round
};

__device__ __forceinline__ uint32_t* big_row_counter(Control* ctl) { return reinterpret_cast<uint32_t*>(&ctl->pad2[1]); }

struct Val3 {
  uint32_t v[kLanes];
};

__device__ __forceinline__ Val3 seg_fetch(const SegArgs& a, size_t i) {
  Val3 r;
  if (a.items) {
    const uint4 it = a.items[i];
    r.v[0] = it.y; r.v[1] = it.z; r.v[2] = it.w;
  } else {
    r.v[0] = a.plain[i]; r.v[1] = 0; r.v[2] = 0;
  }
  return r;
}

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
// One thread per row.  Rows of up to four samples are finished right here with a five-comparator sorting network in
// registers; the others go to the work list of their size class.
__device__ __forceinline__ void push_row(uint32_t* list, uint32_t* counter, bool mine, uint32_t row) {
  const uint32_t ballot = __ballot_sync(__activemask(), mine);
  if (!mine) return;
  const uint32_t first = __ffs(ballot) - 1;
  uint32_t base = 0;
  if (lane_id() == first) base = atomicAdd(counter, (uint32_t)__popc(ballot));
  base = __shfl_sync(ballot, base, first);
  list[base + __popc(ballot & lanemask_lt())] = row;
}

// The large rows (more than kBigMax samples) are found by a kernel of their own, so that their chain of launches can
// start while k_seg_classify and the other classes are still at work on other streams: one thread per row registers the
// row and its chunks.
__global__ void __launch_bounds__(256) k_seg_find_large(const SegArgs a) {
  const uint32_t n_rows = min(*a.n_rows_dev, a.max_rows);
  for (uint32_t row = blockIdx.x * blockDim.x + threadIdx.x; row < n_rows; row += gridDim.x * blockDim.x) {
    const uint32_t s = a.row_start[row], cnt = a.row_start[row + 1] - s;
    if (cnt <= kBigMax) continue;
    const uint32_t nch = (cnt + kLargeChunk - 1) / kLargeChunk;
    const uint32_t l = atomicAdd(&a.ctl->ticket, 1u);
    const uint32_t cbase = (uint32_t)atomicAdd(&a.ctl->scratch0, (unsigned long long)nch);
    if (l >= a.max_large || cbase + nch > a.max_chunks) {
      atomicOr(&a.ctl->err, kErrTooLarge);
    } else {
      LargeRow* L = a.large + l;
      L->row = row; L->start = s; L->cnt = cnt;
      for (int i = 0; i < kLanes; ++i) { L->sum[i] = 0; L->mn[i] = 0xFFFFFFFFu; L->mx[i] = 0; }
      for (uint32_t c = 0; c < nch; ++c) { a.chunk_row[cbase + c] = l; a.chunk_idx[cbase + c] = c; }
    }
  }
}

__global__ void __launch_bounds__(256) k_seg_classify(const SegArgs a) {
  // the statistics of 256 consecutive rows are 18 KB of consecutive memory: staged here, written with coalesced stores
  constexpr int kWords = sizeof(RowStats) / 4;
  __shared__ uint32_t stage[256 * kWords];
  const uint32_t n_rows = min(*a.n_rows_dev, a.max_rows);
  const uint32_t n_round = (n_rows + 255u) & ~255u;  // whole CTAs take part in the staging and the list pushes
  for (uint32_t row0 = blockIdx.x * blockDim.x; row0 < n_round; row0 += gridDim.x * blockDim.x) {
    const uint32_t row = row0 + threadIdx.x;
    const bool valid = row < n_rows;
    const uint32_t s = valid ? a.row_start[row] : 0, cnt = valid ? a.row_start[row + 1] - s : 0;
    push_row(a.small8_rows, &a.ctl->pad32, valid && cnt > 4 && cnt <= 8, row);
    push_row(a.small_rows, &a.ctl->n_small, valid && cnt > 8 && cnt <= kSmallSegment, row);
    push_row(a.mid_rows, &a.ctl->n_big, valid && cnt > kSmallSegment && cnt <= kMidMax, row);
    push_row(a.big_rows, big_row_counter(a.ctl), valid && cnt > kMidMax && cnt <= kBigMax, row);
    RowStats st;
#pragma unroll
    for (int l = 0; l < kLanes; ++l) { st.sum[l] = 0; st.mn[l] = 0; st.mx[l] = 0; st.lo[l] = 0; st.hi[l] = 0; }
    // empty rows (stage API only) and tiny rows are finished here
    if (valid && cnt > 0 && cnt <= 4) {
      Val3 x[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if ((uint32_t)i < cnt) x[i] = seg_fetch(a, (size_t)s + i);
        else { x[i].v[0] = x[i].v[1] = x[i].v[2] = 0xFFFFFFFFu; }
      }
      const uint32_t i_max = cnt - 1, i_lo = (cnt - 1) >> 1, i_hi = cnt >> 1;
#pragma unroll
      for (int l = 0; l < kLanes; ++l) {
        uint32_t x0 = x[0].v[l], x1 = x[1].v[l], x2 = x[2].v[l], x3 = x[3].v[l];
        const unsigned long long sum = (unsigned long long)x0 + (cnt > 1 ? x1 : 0u) + (cnt > 2 ? x2 : 0u) + (cnt > 3 ? x3 : 0u);
        uint32_t t;
#define KS_CSWAP(p, q) t = min(p, q); q = max(p, q); p = t;
        KS_CSWAP(x0, x1) KS_CSWAP(x2, x3) KS_CSWAP(x0, x2) KS_CSWAP(x1, x3) KS_CSWAP(x1, x2)
#undef KS_CSWAP
        auto pick = [&](uint32_t i) { return i == 0 ? x0 : i == 1 ? x1 : i == 2 ? x2 : x3; };
        st.sum[l] = sum;
        st.mn[l] = x0;
        st.mx[l] = pick(i_max);
        st.lo[l] = pick(i_lo);
        st.hi[l] = pick(i_hi);
      }
    }
    // rows of the other classes get zeros now and their statistics from the class kernels, which run after this one
    __syncthreads();
    const uint32_t* w = reinterpret_cast<const uint32_t*>(&st);
#pragma unroll
    for (int i = 0; i < kWords; ++i) stage[threadIdx.x * kWords + i] = w[i];
    __syncthreads();
    const uint32_t rows_here = min(256u, n_rows > row0 ? n_rows - row0 : 0u);
    uint32_t* dst = reinterpret_cast<uint32_t*>(a.stats + row0);
    for (uint32_t i = threadIdx.x; i < rows_here * kWords; i += blockDim.x) dst[i] = stage[i];
  }
}

// W lanes per row (W = 8 for rows of 5..8 samples, 32 for 9..32): a warp takes 32 / W rows at a time; shuffle
// reductions and a W-wide bitonic network inside each group
template <int W>
__device__ __forceinline__ uint32_t bitonic_sort_group(uint32_t v) {
  const uint32_t sub = lane_id() & (W - 1);
#pragma unroll
  for (int k = 2; k <= W; k <<= 1) {
#pragma unroll
    for (int j = k >> 1; j > 0; j >>= 1) {
      const uint32_t o = __shfl_xor_sync(0xFFFFFFFFu, v, j);
      const bool up = (sub & k) == 0;
      const bool lower = (sub & j) == 0;
      v = (lower == up) ? min(v, o) : max(v, o);
    }
  }
  return v;
}

template <int W>
__global__ void __launch_bounds__(256) k_seg_small(const SegArgs a) {
  constexpr uint32_t G = 32 / W;
  const uint32_t* list = W == 8 ? a.small8_rows : a.small_rows;
  const uint32_t n_list = min(W == 8 ? a.ctl->pad32 : a.ctl->n_small, a.max_rows);
  const uint32_t lane = lane_id(), sub = lane & (W - 1), gbase = lane & ~(uint32_t)(W - 1);
  const uint32_t warps = gridDim.x * (blockDim.x >> 5);
  const uint32_t n_round = (n_list + G - 1) / G * G;
  for (uint32_t t0 = (blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * G; t0 < n_round; t0 += warps * G) {
    const uint32_t t = t0 + lane / W;
    const bool valid = t < n_list;
    const uint32_t row = valid ? list[t] : 0;
    const uint32_t s = valid ? a.row_start[row] : 0, cnt = valid ? a.row_start[row + 1] - s : 1;
    const bool have = valid && sub < cnt;
    Val3 x;
    if (have) x = seg_fetch(a, (size_t)s + sub);
    else { x.v[0] = x.v[1] = x.v[2] = 0; }
    RowStats* st = a.stats + row;
#pragma unroll
    for (int l = 0; l < kLanes; ++l) {
      if (l >= a.n_lanes) break;
      const uint32_t v = x.v[l];
      unsigned long long sum = v;
#pragma unroll
      for (int o = W / 2; o; o >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, o);
      const uint32_t sorted = bitonic_sort_group<W>(have ? v : 0xFFFFFFFFu);
      const uint32_t mn = __shfl_sync(0xFFFFFFFFu, sorted, gbase);
      const uint32_t mx = __shfl_sync(0xFFFFFFFFu, sorted, gbase + cnt - 1);
      const uint32_t lo = __shfl_sync(0xFFFFFFFFu, sorted, gbase + ((cnt - 1) >> 1));
      const uint32_t hi = __shfl_sync(0xFFFFFFFFu, sorted, gbase + (cnt >> 1));
      if (valid && sub == 0) { st->sum[l] = sum; st->mn[l] = mn; st->mx[l] = mx; st->lo[l] = lo; st->hi[l] = hi; }
    }
  }
}

// ---------------------------------------------------------------------------------------------------------
// One warp per row of 33..kMidMax samples.  The row is read from global memory ONCE: its three value lanes are staged in
// the warp's own shared memory while sum/min/max are taken, and the selection rounds (and the pass for the upper middle
// value) run over shared memory.  No block-wide barrier anywhere.
constexpr int kMidWarps = 8;
constexpr size_t seg_mid_smem_bytes() { return (size_t)kMidWarps * kLanes * (kMidMax + 256) * sizeof(uint32_t); }

__global__ void __launch_bounds__(kMidWarps * 32, 3) k_seg_mid(const SegArgs a) {
  extern __shared__ __align__(16) uint32_t mid_smem[];
  const uint32_t warp = threadIdx.x >> 5, lane = lane_id();
  uint32_t* vals = mid_smem + (size_t)warp * kLanes * (kMidMax + 256);  // [kLanes][kMidMax]
  uint32_t* hist = vals + kLanes * kMidMax;                              // [kLanes][256]
  const uint32_t n_mid = min(a.ctl->n_big, a.max_rows);
  const uint32_t warps = gridDim.x * kMidWarps;
  const int nl = a.n_lanes;
  for (uint32_t t = blockIdx.x * kMidWarps + warp; t < n_mid; t += warps) {
    const uint32_t row = a.mid_rows[t];
    const uint32_t s = a.row_start[row], cnt = min(a.row_start[row + 1] - s, kMidMax);
    unsigned long long sum[kLanes] = {0, 0, 0};
    uint32_t mn[kLanes] = {0xFFFFFFFFu, 0xFFFFFFFFu, 0xFFFFFFFFu}, mx[kLanes] = {0, 0, 0};
    __syncwarp();  // the previous row's readers of the staging area are done
    for (uint32_t i0 = lane; i0 < cnt; i0 += 128) {
      Val3 xs[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) if (i0 + 32 * u < cnt) xs[u] = seg_fetch(a, (size_t)s + i0 + 32 * u);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (i0 + 32 * u >= cnt) break;
#pragma unroll
        for (int l = 0; l < kLanes; ++l) {
          const uint32_t v = xs[u].v[l];
          vals[l * kMidMax + i0 + 32 * u] = v;
          sum[l] += v; mn[l] = min(mn[l], v); mx[l] = max(mx[l], v);
        }
      }
    }
#pragma unroll
    for (int l = 0; l < kLanes; ++l) { sum[l] = warp_sum64(sum[l]); mn[l] = warp_min(mn[l]); mx[l] = warp_max(mx[l]); }
    __syncwarp();

    const uint32_t k_lo = (cnt - 1) >> 1, k_hi = cnt >> 1;
    uint32_t prefix[kLanes] = {0, 0, 0}, k[kLanes] = {k_lo, k_lo, k_lo};
    int hi_bit[kLanes];
    bool open = false;
#pragma unroll
    for (int l = 0; l < kLanes; ++l) {
      hi_bit[l] = (l < nl && mn[l] != mx[l]) ? bit_length32(mx[l] - mn[l]) - 1 : -1;
      open = open || hi_bit[l] >= 0;
    }
    while (open) {
      int nb[kLanes], shift[kLanes];
#pragma unroll
      for (int l = 0; l < kLanes; ++l) {
        nb[l] = min(8, hi_bit[l] + 1);
        shift[l] = hi_bit[l] + 1 - nb[l];
        if (hi_bit[l] >= 0) {
#pragma unroll
          for (int i = 0; i < 8; ++i) hist[l * 256 + lane * 8 + i] = 0;
        }
      }
      __syncwarp();
#pragma unroll
      for (int l = 0; l < kLanes; ++l) {
        if (hi_bit[l] < 0) continue;
        for (uint32_t i = lane; i < cnt; i += 32) {
          const uint32_t u = vals[l * kMidMax + i] - mn[l];
          if (matches_prefix(u, prefix[l], hi_bit[l])) atomicAdd(&hist[l * 256 + ((u >> shift[l]) & ((1u << nb[l]) - 1u))], 1u);
        }
      }
      __syncwarp();
      open = false;
#pragma unroll
      for (int l = 0; l < kLanes; ++l) {
        if (hi_bit[l] < 0) continue;
        uint32_t d, below;
        warp_pick_bin(hist + l * 256, k[l], &d, &below);
        prefix[l] |= d << shift[l];
        k[l] -= below;
        hi_bit[l] = shift[l] - 1;
        open = open || hi_bit[l] >= 0;
      }
      __syncwarp();
    }
    uint32_t lo[kLanes], hi[kLanes];
#pragma unroll
    for (int l = 0; l < kLanes; ++l) { lo[l] = mn[l] + prefix[l]; hi[l] = lo[l]; }
    if (k_hi != k_lo) {
      // hi = x[k_lo + 1]: lo again if more than k_hi values are <= lo, else the smallest value above lo
#pragma unroll
      for (int l = 0; l < kLanes; ++l) {
        if (l >= nl) continue;
        uint32_t le = 0, next = 0xFFFFFFFFu;
        for (uint32_t i = lane; i < cnt; i += 32) {
          const uint32_t v = vals[l * kMidMax + i];
          le += v <= lo[l];
          if (v > lo[l]) next = min(next, v);
        }
        const uint32_t le_t = warp_sum(le), nx = warp_min(next);
        hi[l] = (le_t > k_hi) ? lo[l] : nx;
      }
    }
    if (lane == 0) {
      RowStats* st = a.stats + row;
      for (int l = 0; l < nl; ++l) { st->sum[l] = sum[l]; st->mn[l] = mn[l]; st->mx[l] = mx[l]; st->lo[l] = lo[l]; st->hi[l] = hi[l]; }
    }
  }
}

// ---------------------------------------------------------------------------------------------------------
// One CTA per row of kMidMax+1 .. kBigMax samples: the same scheme with block-wide reductions and histograms and the
// row's three value lanes staged in the CTA's shared memory (96 KB).  The selection state (prefix, rank, highest open
// bit per lane) is computed redundantly by every thread from shared results, so it stays in registers.
// Two instances: rows up to kBigSmall samples (24 KB of shared memory per CTA, so many CTAs per SM hide each other's
// barriers and loads) and rows up to kBigMax (96 KB).  CAP = the row capacity of the instance; its rows come from its own list.
constexpr uint32_t kBigSmall = 2048;
template <uint32_t CAP>
constexpr size_t seg_big_smem_bytes() { return (size_t)kLanes * CAP * sizeof(uint32_t); }

template <uint32_t CAP>
__global__ void __launch_bounds__(256, CAP <= kBigSmall ? 6 : 2) k_seg_big(const SegArgs a) {
  constexpr uint32_t kBigMax = CAP;  // within this kernel: the capacity of the staging area
  extern __shared__ __align__(16) uint32_t big_vals[];  // [kLanes][CAP]
  __shared__ uint32_t hist[kLanes][256];
  __shared__ unsigned long long sh_sum[8][kLanes];
  __shared__ uint32_t sh_a[8][kLanes], sh_b[8][kLanes];
  __shared__ uint32_t sh_pick[kLanes][2];
  const uint32_t tid = threadIdx.x, lane = lane_id(), warp = tid >> 5;
  const uint32_t* list = CAP <= kBigSmall ? a.mid_rows : a.big_rows;
  const uint32_t n_big = min(big_row_counter(a.ctl)[CAP <= kBigSmall ? 1 : 0], a.max_rows);
  const int nl = a.n_lanes;
  for (uint32_t t = blockIdx.x; t < n_big; t += gridDim.x) {
    const uint32_t row = list[t];
    const uint32_t s = a.row_start[row], cnt = min(a.row_start[row + 1] - s, kBigMax);
    unsigned long long sum[kLanes] = {0, 0, 0};
    uint32_t mn[kLanes] = {0xFFFFFFFFu, 0xFFFFFFFFu, 0xFFFFFFFFu}, mx[kLanes] = {0, 0, 0};
    __syncthreads();  // the previous row's readers of the shared arrays are done
    for (uint32_t i0 = tid; i0 < cnt; i0 += 1024) {
      Val3 xs[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) if (i0 + 256 * u < cnt) xs[u] = seg_fetch(a, (size_t)s + i0 + 256 * u);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (i0 + 256 * u >= cnt) break;
#pragma unroll
        for (int l = 0; l < kLanes; ++l) {
          const uint32_t v = xs[u].v[l];
          big_vals[l * kBigMax + i0 + 256 * u] = v;
          sum[l] += v; mn[l] = min(mn[l], v); mx[l] = max(mx[l], v);
        }
      }
    }
#pragma unroll
    for (int l = 0; l < kLanes; ++l) {
      const unsigned long long s2 = warp_sum64(sum[l]);
      const uint32_t n2 = warp_min(mn[l]), x2 = warp_max(mx[l]);
      if (lane == 0) { sh_sum[warp][l] = s2; sh_a[warp][l] = n2; sh_b[warp][l] = x2; }
    }
    __syncthreads();
#pragma unroll
    for (int l = 0; l < kLanes; ++l) {
      sum[l] = 0; mn[l] = 0xFFFFFFFFu; mx[l] = 0;
      for (int w = 0; w < 8; ++w) { sum[l] += sh_sum[w][l]; mn[l] = min(mn[l], sh_a[w][l]); mx[l] = max(mx[l], sh_b[w][l]); }
    }
    const uint32_t k_lo = (cnt - 1) >> 1, k_hi = cnt >> 1;
    uint32_t prefix[kLanes] = {0, 0, 0}, k[kLanes] = {k_lo, k_lo, k_lo};
    int hi_bit[kLanes];
    bool open = false;
#pragma unroll
    for (int l = 0; l < kLanes; ++l) {
      hi_bit[l] = (l < nl && mn[l] != mx[l]) ? bit_length32(mx[l] - mn[l]) - 1 : -1;
      open = open || hi_bit[l] >= 0;
    }
    while (open) {
      int nb[kLanes], shift[kLanes];
#pragma unroll
      for (int l = 0; l < kLanes; ++l) {
        nb[l] = min(8, hi_bit[l] + 1);
        shift[l] = hi_bit[l] + 1 - nb[l];
        hist[l][tid] = 0;
      }
      __syncthreads();
#pragma unroll
      for (int l = 0; l < kLanes; ++l) {
        if (hi_bit[l] < 0) continue;
        for (uint32_t i = tid; i < cnt; i += 256) {
          const uint32_t v = big_vals[l * kBigMax + i] - mn[l];
          if (matches_prefix(v, prefix[l], hi_bit[l])) atomicAdd(&hist[l][(v >> shift[l]) & ((1u << nb[l]) - 1u)], 1u);
        }
      }
      __syncthreads();
#pragma unroll
      for (int l = 0; l < kLanes; ++l) {  // warp l resolves lane l
        if (warp != (uint32_t)l || hi_bit[l] < 0) continue;
        uint32_t d, below;
        warp_pick_bin(hist[l], k[l], &d, &below);
        if (lane == 0) { sh_pick[l][0] = d; sh_pick[l][1] = below; }
      }
      __syncthreads();
      open = false;
#pragma unroll
      for (int l = 0; l < kLanes; ++l) {
        if (hi_bit[l] < 0) continue;
        prefix[l] |= sh_pick[l][0] << shift[l];
        k[l] -= sh_pick[l][1];
        hi_bit[l] = shift[l] - 1;
        open = open || hi_bit[l] >= 0;
      }
      __syncthreads();  // sh_pick and hist are free again
    }
    uint32_t lo[kLanes], hi[kLanes];
#pragma unroll
    for (int l = 0; l < kLanes; ++l) { lo[l] = mn[l] + prefix[l]; hi[l] = lo[l]; }
    if (k_hi != k_lo) {
      // hi = x[k_lo + 1]: lo again if more than k_hi values are <= lo, else the smallest value above lo
      uint32_t le[kLanes] = {0, 0, 0}, next[kLanes] = {0xFFFFFFFFu, 0xFFFFFFFFu, 0xFFFFFFFFu};
#pragma unroll
      for (int l = 0; l < kLanes; ++l) {
        for (uint32_t i = tid; i < cnt; i += 256) {
          const uint32_t v = big_vals[l * kBigMax + i];
          le[l] += v <= lo[l];
          if (v > lo[l]) next[l] = min(next[l], v);
        }
      }
      __syncthreads();  // every thread has read sh_a / sh_b of the first pass (the select loop may not have run)
#pragma unroll
      for (int l = 0; l < kLanes; ++l) {
        const uint32_t le_w = warp_sum(le[l]), nx_w = warp_min(next[l]);
        if (lane == 0) { sh_a[warp][l] = le_w; sh_b[warp][l] = nx_w; }
      }
      __syncthreads();
#pragma unroll
      for (int l = 0; l < kLanes; ++l) {
        uint32_t le_t = 0, nx = 0xFFFFFFFFu;
        for (int w = 0; w < 8; ++w) { le_t += sh_a[w][l]; nx = min(nx, sh_b[w][l]); }
        hi[l] = (le_t > k_hi) ? lo[l] : nx;
      }
    }
    if (tid == 0) {
      RowStats* st = a.stats + row;
      for (int l = 0; l < nl; ++l) { st->sum[l] = sum[l]; st->mn[l] = mn[l]; st->mx[l] = mx[l]; st->lo[l] = lo[l]; st->hi[l] = hi[l]; }
    }
  }
}

// ---------------------------------------------------------------------------------------------------------
// large rows: chunk work items
__global__ void __launch_bounds__(256) k_segL_reduce(const SegArgs a) {
  __shared__ unsigned long long sh_sum[8][kLanes];
  __shared__ uint32_t sh_mn[8][kLanes], sh_mx[8][kLanes];
  const uint32_t n_chunks = (uint32_t)min(a.ctl->scratch0, (unsigned long long)a.max_chunks);
  for (uint32_t c = blockIdx.x; c < n_chunks; c += gridDim.x) {
    LargeRow* L = a.large + a.chunk_row[c];
    const uint32_t off = a.chunk_idx[c] * kLargeChunk;
    const uint32_t m = min(kLargeChunk, L->cnt - off);
    if (off == 0) {  // the row's first chunk clears the row's histograms for the selection rounds
      uint32_t* gh = a.large_hist + (size_t)a.chunk_row[c] * 2 * kLanes * 256;
      for (uint32_t i = threadIdx.x; i < 2 * kLanes * 256; i += blockDim.x) gh[i] = 0;
    }
    const size_t base = (size_t)L->start + off;
    unsigned long long sum[kLanes] = {0, 0, 0};
    uint32_t mn[kLanes] = {0xFFFFFFFFu, 0xFFFFFFFFu, 0xFFFFFFFFu}, mx[kLanes] = {0, 0, 0};
    for (uint32_t i = threadIdx.x; i < m; i += blockDim.x) {
      const Val3 x = seg_fetch(a, base + i);
#pragma unroll
      for (int l = 0; l < kLanes; ++l) { sum[l] += x.v[l]; mn[l] = min(mn[l], x.v[l]); mx[l] = max(mx[l], x.v[l]); }
    }
    __syncthreads();
#pragma unroll
    for (int l = 0; l < kLanes; ++l) {
      const unsigned long long s2 = warp_sum64(sum[l]);
      const uint32_t n2 = warp_min(mn[l]), x2 = warp_max(mx[l]);
      if (lane_id() == 0) { sh_sum[threadIdx.x >> 5][l] = s2; sh_mn[threadIdx.x >> 5][l] = n2; sh_mx[threadIdx.x >> 5][l] = x2; }
    }
    __syncthreads();
    if (threadIdx.x < (uint32_t)a.n_lanes) {
      const int l = threadIdx.x;
      unsigned long long s2 = 0;
      uint32_t n2 = 0xFFFFFFFFu, x2 = 0;
      for (int w = 0; w < 8; ++w) { s2 += sh_sum[w][l]; n2 = min(n2, sh_mn[w][l]); x2 = max(x2, sh_mx[w][l]); }
      atomicAdd(&L->sum[l], s2);
      atomicMin(&L->mn[l], n2);
      atomicMax(&L->mx[l], x2);
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
    int hb[2 * kLanes], nb[2 * kLanes], shf[2 * kLanes];
    uint32_t pre[2 * kLanes], mn[kLanes];
    bool any = false;
#pragma unroll
    for (int v = 0; v < 2 * kLanes; ++v) {
      hb[v] = L->hi_bit[v];
      pre[v] = L->prefix[v];
      nb[v] = min(8, hb[v] + 1);
      shf[v] = hb[v] + 1 - nb[v];
      any = any || hb[v] >= 0;
    }
#pragma unroll
    for (int l = 0; l < kLanes; ++l) mn[l] = L->mn[l];
    if (!any) continue;
    __syncthreads();
    for (uint32_t i = threadIdx.x; i < 2 * kLanes * 256; i += blockDim.x) (&sh[0][0])[i] = 0;
    __syncthreads();
    const uint32_t off = a.chunk_idx[c] * kLargeChunk;
    const uint32_t m = min(kLargeChunk, L->cnt - off);
    const size_t base = (size_t)L->start + off;
    for (uint32_t i = threadIdx.x; i < m; i += blockDim.x) {
      const Val3 x = seg_fetch(a, base + i);
#pragma unroll
      for (int v = 0; v < 2 * kLanes; ++v) {
        if (hb[v] < 0) continue;
        const uint32_t u = x.v[v >> 1] - mn[v >> 1];
        if (matches_prefix(u, pre[v], hb[v])) atomicAdd(&sh[v][(u >> shf[v]) & ((1u << nb[v]) - 1u)], 1u);
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
