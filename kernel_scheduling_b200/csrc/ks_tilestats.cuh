// ks_tilestats.cuh -- K4 in one read of the sorted sample stream: row detection and the integer statistics of every row
// of up to kTsRowMax samples, fused.
//
// The sorted stream is cut into tiles of kTsTile samples.  A CTA stages its tile plus kTsOver samples behind it in shared
// memory (structure of arrays: sort key and the three value lanes), marks where the sort key changes, numbers the rows
// that START in its tile (row numbers across tiles come from a decoupled look-back over one word per tile, 32 tiles per
// poll), and computes sum / min / max and the two middle order statistics of every such row of at most kTsRowMax
// samples -- straight from shared memory, by size class:
//     1..4 samples     one thread per row, a five-comparator network in registers
//     5..8, 9..16,     one thread per row: the row's values in registers, a bitonic sorting network (fully unrolled, so
//     17..32           every index is static) -- no lane idles the way it does when a warp sorts one short row
//     33..kTsRowMax    one warp per row, radix select over (value - min) for the three value lanes at once, 6 bits per
//                      round, 64 bins per lane of values in the warp's own shared memory
// After the rows of a tile are listed the warps work through the classes on their own (no block-wide barrier until the
// tile is done).  Longer rows, and the rare shorter one that leaves the window, go on the deferred list; k_seg_deferred
// hands them to the CTA-per-row kernel or to the chunked chain of the largest rows (ks_segstats.cuh).
//
// Tiles are taken from a ticket counter, so a tile only ever waits for tiles that already started; the wait is bounded
// (kSpinLimit polls, then kErrWait and a wrong row number -- the host reports the failure).
#pragma once

#include "ks_common.cuh"
#include "ks_segstats.cuh"
#include "ks_sort.cuh"

namespace ks {

constexpr int kTsThreads = 256;
constexpr int kTsWarps = kTsThreads / 32;
constexpr int kTsTile = 2048;
constexpr int kTsOver = 512;
constexpr int kTsWin = kTsTile + kTsOver;
constexpr uint32_t kTsRowMax = 512;  // largest row finished inside a tile
constexpr int kTsDigitBits = 6;
constexpr int kTsBins = 1 << kTsDigitBits;

struct TileStatsArgs {
  const uint4* items;     // sorted samples {sort key, lane 0, lane 1, lane 2}
  const uint32_t* n_dev;  // number of samples in device memory (then n is the bound the buffers were sized for), or nullptr
  uint32_t n;
  uint32_t* tile_state;   // [tiles] look-back words, zeroed: rows starting in the tile | flag << 30
  uint32_t* ticket;       // zeroed
  uint32_t* row_start;    // [max_rows + 1]
  uint32_t* row_key;      // [max_rows]
  uint32_t* row_of_kid;   // [kMaxKeys + 1], preset to 0xFFFFFFFF
  RowStats* stats;        // [max_rows]
  uint32_t* deferred;     // [max_deferred] rows not finished here; count in Control::n_small
  uint32_t max_deferred;
  uint32_t max_rows;
  Control* ctl;           // n_rows, ticket2 = rows with a sort key below n_keys (the solo rows)
};

// rows a tile can hold per class (a row of the class has at least 5 / 9 / 17 / 33 samples)
constexpr int kTsCap8 = kTsTile / 5 + 2, kTsCap16 = kTsTile / 9 + 2, kTsCap32 = kTsTile / 17 + 2, kTsCapW = kTsTile / 33 + 2;

struct TsShared {
  uint32_t key[kTsWin];
  uint32_t val[kLanes][kTsWin];
  uint32_t hist[kTsWarps][kLanes][kTsBins];
  uint16_t rs[kTsTile + 2];  // window position of every row start of the tile, then the end of the last row
  uint16_t list8[kTsCap8], list16[kTsCap16], list32[kTsCap32], listw[kTsCapW];  // local row numbers by class
  uint32_t word_cnt[kTsTile / 32];
  uint32_t n8, n16, n32, nw, qhead;
  uint32_t end_last, tile, row_base, rows_here, n_solo_rows;
};

constexpr size_t tile_stats_smem_bytes() { return sizeof(TsShared); }

__device__ __forceinline__ void ts_store(RowStats* st, int l, unsigned long long sum, uint32_t mn, uint32_t mx, uint32_t lo, uint32_t hi) {
  st->sum[l] = sum; st->mn[l] = mn; st->mx[l] = mx; st->lo[l] = lo; st->hi[l] = hi;
}

// Bitonic sorting network over N registers, ascending.  Every loop is unrolled, so every index and direction is static.
template <int N>
__device__ __forceinline__ void net_sort(uint32_t (&x)[N]) {
#pragma unroll
  for (int k = 2; k <= N; k <<= 1) {
#pragma unroll
    for (int j = k >> 1; j > 0; j >>= 1) {
#pragma unroll
      for (int i = 0; i < N; ++i) {
        const int l = i ^ j;
        if (l > i) {
          const bool up = (i & k) == 0;
          const uint32_t p = x[i], q = x[l];
          x[i] = up ? min(p, q) : max(p, q);
          x[l] = up ? max(p, q) : min(p, q);
        }
      }
    }
  }
}
template <int N>
__device__ __forceinline__ uint32_t net_pick(const uint32_t (&x)[N], uint32_t idx) {
  uint32_t r = x[0];
#pragma unroll
  for (int i = 1; i < N; ++i) r = idx == (uint32_t)i ? x[i] : r;
  return r;
}

// One thread, one row of 1..N samples: the three value lanes one after the other through the network.
template <int N>
__device__ __forceinline__ void ts_thread_row(const TsShared& sh, uint32_t s, uint32_t cnt, RowStats* st) {
  const uint32_t i_lo = (cnt - 1) >> 1, i_hi = cnt >> 1;
#pragma unroll 1
  for (int l = 0; l < kLanes; ++l) {
    const uint32_t* v = sh.val[l] + s;
    uint32_t x[N];
    unsigned long long sum = 0;
#pragma unroll
    for (int i = 0; i < N; ++i) {
      const bool have = (uint32_t)i < cnt;
      x[i] = have ? v[i] : 0xFFFFFFFFu;
      sum += have ? x[i] : 0u;
    }
    net_sort<N>(x);
    ts_store(st, l, sum, x[0], net_pick<N>(x, cnt - 1), net_pick<N>(x, i_lo), net_pick<N>(x, i_hi));
  }
}

// One warp, one row of up to kTsRowMax samples in shared memory: the three value lanes together.
__device__ __forceinline__ void ts_warp_row(TsShared& sh, uint32_t warp, uint32_t s, uint32_t cnt, RowStats* st) {
  const uint32_t lane = lane_id();
  unsigned long long sum[kLanes] = {0, 0, 0};
  uint32_t mn[kLanes] = {0xFFFFFFFFu, 0xFFFFFFFFu, 0xFFFFFFFFu}, mx[kLanes] = {0, 0, 0};
  for (uint32_t i = lane; i < cnt; i += 32) {
#pragma unroll
    for (int l = 0; l < kLanes; ++l) { const uint32_t x = sh.val[l][s + i]; sum[l] += x; mn[l] = min(mn[l], x); mx[l] = max(mx[l], x); }
  }
#pragma unroll
  for (int l = 0; l < kLanes; ++l) { sum[l] = warp_sum64(sum[l]); mn[l] = warp_min(mn[l]); mx[l] = warp_max(mx[l]); }
  const uint32_t k_lo = (cnt - 1) >> 1, k_hi = cnt >> 1;
  uint32_t prefix[kLanes] = {0, 0, 0}, k[kLanes] = {k_lo, k_lo, k_lo};
  int hi_bit[kLanes];
  bool open = false;
#pragma unroll
  for (int l = 0; l < kLanes; ++l) {
    hi_bit[l] = mn[l] != mx[l] ? bit_length32(mx[l] - mn[l]) - 1 : -1;
    open = open || hi_bit[l] >= 0;
  }
  uint32_t (*hist)[kTsBins] = sh.hist[warp];
  while (open) {
    int nb[kLanes], shift[kLanes];
#pragma unroll
    for (int l = 0; l < kLanes; ++l) {
      nb[l] = min(kTsDigitBits, hi_bit[l] + 1);
      shift[l] = hi_bit[l] + 1 - nb[l];
      hist[l][lane] = 0;
      hist[l][lane + 32] = 0;
    }
    __syncwarp();
    for (uint32_t i = lane; i < cnt; i += 32) {
#pragma unroll
      for (int l = 0; l < kLanes; ++l) {
        if (hi_bit[l] < 0) continue;
        const uint32_t u = sh.val[l][s + i] - mn[l];
        if (matches_prefix(u, prefix[l], hi_bit[l])) atomicAdd(&hist[l][(u >> shift[l]) & ((1u << nb[l]) - 1u)], 1u);
      }
    }
    __syncwarp();
    open = false;
#pragma unroll
    for (int l = 0; l < kLanes; ++l) {
      if (hi_bit[l] < 0) continue;  // warp-uniform
      // the bin that holds rank k: lane holds bins 2*lane and 2*lane + 1
      const uint32_t c0 = hist[l][2 * lane], c1 = hist[l][2 * lane + 1];
      const uint32_t inc = warp_incl_scan(c0 + c1), exc = inc - (c0 + c1);
      const bool mine = k[l] >= exc && k[l] < inc;
      const uint32_t who = (uint32_t)(__ffs(__ballot_sync(0xFFFFFFFFu, mine)) - 1) & 31u;
      const uint32_t second = (mine && k[l] >= exc + c0) ? 1u : 0u;
      const uint32_t d = __shfl_sync(0xFFFFFFFFu, 2 * lane + second, who);
      const uint32_t below = __shfl_sync(0xFFFFFFFFu, exc + (second ? c0 : 0u), who);
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
  if (k_hi != k_lo) {  // x[k_lo + 1]: lo again if more than k_hi values are <= lo, else the smallest value above lo
    uint32_t le[kLanes] = {0, 0, 0}, next[kLanes] = {0xFFFFFFFFu, 0xFFFFFFFFu, 0xFFFFFFFFu};
    for (uint32_t i = lane; i < cnt; i += 32) {
#pragma unroll
      for (int l = 0; l < kLanes; ++l) { const uint32_t x = sh.val[l][s + i]; le[l] += x <= lo[l]; if (x > lo[l]) next[l] = min(next[l], x); }
    }
#pragma unroll
    for (int l = 0; l < kLanes; ++l) {
      const uint32_t le_t = warp_sum(le[l]), nx = warp_min(next[l]);
      hi[l] = le_t > k_hi ? lo[l] : nx;
    }
  }
  if (lane == 0) {
#pragma unroll
    for (int l = 0; l < kLanes; ++l) ts_store(st, l, sum[l], mn[l], mx[l], lo[l], hi[l]);
  }
}

__global__ void __launch_bounds__(kTsThreads, 4) k_tile_stats(const TileStatsArgs a) {
  extern __shared__ __align__(16) unsigned char ts_raw[];
  TsShared& sh = *reinterpret_cast<TsShared*>(ts_raw);
  const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
  const uint32_t n = a.n_dev ? min(*a.n_dev, a.n) : a.n;
  const uint32_t ntiles = (n + kTsTile - 1) / kTsTile;
  const uint32_t nk = a.ctl->n_keys;
  if (ntiles == 0) {
    if (blockIdx.x == 0 && tid == 0) { a.ctl->n_rows = 0; a.row_start[0] = 0; }
    return;
  }

  while (true) {
    __syncthreads();  // the previous tile's readers of the shared arrays are done
    if (tid == 0) {
      sh.tile = atomicAdd(a.ticket, 1u);
      sh.n8 = sh.n16 = sh.n32 = sh.nw = 0;
      sh.qhead = 0;
      sh.n_solo_rows = 0;
    }
    __syncthreads();
    const uint32_t tile = sh.tile;
    if (tile >= ntiles) break;
    const uint32_t t0 = tile * kTsTile;
    const uint32_t own = min((uint32_t)kTsTile, n - t0);  // samples whose rows this tile numbers
    const uint32_t wn = min((uint32_t)kTsWin, n - t0);    // staged samples
    if (tid == 0) sh.end_last = wn;

    // ---- stage the window as a structure of arrays (coalesced 128-bit loads, conflict-free 32-bit shared stores)
    for (uint32_t i0 = tid; i0 < wn; i0 += 3 * kTsThreads) {
      uint4 it[3];
#pragma unroll
      for (int u = 0; u < 3; ++u) if (i0 + u * kTsThreads < wn) it[u] = a.items[(size_t)t0 + i0 + u * kTsThreads];
#pragma unroll
      for (int u = 0; u < 3; ++u) {
        const uint32_t i = i0 + u * kTsThreads;
        if (i < wn) { sh.key[i] = it[u].x; sh.val[0][i] = it[u].y; sh.val[1][i] = it[u].z; sh.val[2][i] = it[u].w; }
      }
    }
    const uint32_t prev_key = t0 ? a.items[(size_t)t0 - 1].x : 0u;
    __syncthreads();

    // ---- row starts among the tile's own samples (consecutive lanes, consecutive samples; one ballot per 32 samples)
    uint32_t ballot[kTsTile / kTsThreads];
#pragma unroll
    for (int k = 0; k < kTsTile / kTsThreads; ++k) {
      const uint32_t i = k * kTsThreads + tid;
      bool flag = false;
      if (i < own) flag = (i == 0) ? (t0 == 0 || sh.key[0] != prev_key) : (sh.key[i] != sh.key[i - 1]);
      ballot[k] = __ballot_sync(0xFFFFFFFFu, flag);
      if (lane == 0) sh.word_cnt[k * kTsWarps + warp] = __popc(ballot[k]);
    }
    // where the tile's last row ends: the first change of the sort key behind the tile's own samples
    for (uint32_t j = own + tid; j < wn; j += kTsThreads)
      if (sh.key[j] != sh.key[j - 1]) atomicMin(&sh.end_last, j);
    __syncthreads();
    if (warp == 0) {  // exclusive scan over the 64 words; then the look-back
      const uint32_t c0 = sh.word_cnt[lane], c1 = sh.word_cnt[32 + lane];
      const uint32_t i0 = warp_incl_scan(c0);
      const uint32_t tot0 = __shfl_sync(0xFFFFFFFFu, i0, 31);
      const uint32_t i1 = warp_incl_scan(c1);
      sh.word_cnt[lane] = i0 - c0;
      sh.word_cnt[32 + lane] = tot0 + i1 - c1;
      const uint32_t n_local = tot0 + __shfl_sync(0xFFFFFFFFu, i1, 31);
      // decoupled look-back, 32 earlier tiles per poll: lane l looks at tile - 1 - l
      uint32_t excl = 0;
      if (tile == 0) {
        if (lane == 0) *(volatile uint32_t*)(a.tile_state + tile) = n_local | kFlagPrefix;
      } else {
        if (lane == 0) *(volatile uint32_t*)(a.tile_state + tile) = n_local | kFlagAgg;
        int64_t top = (int64_t)tile - 1;  // the nearest tile not yet added
        uint32_t spins = 0;
        while (true) {
          const int64_t t = top - lane;
          const uint32_t v = t >= 0 ? ld_volatile_u32(a.tile_state + t) : kFlagPrefix;  // in front of tile 0: an empty prefix
          const uint32_t f = v & kFlagMask;
          const uint32_t not_ready = __ballot_sync(0xFFFFFFFFu, f == 0);
          const uint32_t is_prefix = __ballot_sync(0xFFFFFFFFu, f == kFlagPrefix);
          // usable lanes: in front of the first one that is not ready, up to and including the first prefix
          const uint32_t first_bad = not_ready ? (uint32_t)(__ffs(not_ready) - 1) : 32u;
          const uint32_t first_pre = is_prefix ? (uint32_t)(__ffs(is_prefix) - 1) : 32u;
          const uint32_t take = first_pre < first_bad ? first_pre + 1 : first_bad;  // lanes [0, take)
          excl += warp_sum(lane < take ? (v & kCountMask) : 0u);
          if (first_pre < first_bad) break;
          top -= take;
          if (take == 0) {
            if (++spins > kSpinLimit) { if (lane == 0) atomicOr(&a.ctl->err, kErrWait); break; }
            __nanosleep(40);
          }
        }
        if (lane == 0) *(volatile uint32_t*)(a.tile_state + tile) = ((excl + n_local) & kCountMask) | kFlagPrefix;
      }
      if (lane == 0) {
        sh.row_base = excl;
        sh.rows_here = n_local;
        sh.rs[n_local] = (uint16_t)sh.end_last;  // end_last was settled before the barrier above
      }
    }
    __syncthreads();
    // positions of the row starts
#pragma unroll
    for (int k = 0; k < kTsTile / kTsThreads; ++k) {
      if (ballot[k] & (1u << lane)) sh.rs[sh.word_cnt[k * kTsWarps + warp] + __popc(ballot[k] & lanemask_lt())] = (uint16_t)(k * kTsThreads + tid);
    }
    __syncthreads();
    const uint32_t rows_here = sh.rows_here;
    const uint32_t row_base = sh.row_base;
    const uint32_t end_last = sh.end_last;
    const bool last_complete = end_last < wn || t0 + wn >= n;

    // ---- pass 1: one thread per row of the tile: row arrays, rows of up to four samples finished, the others listed by class
    for (uint32_t lr = tid; lr < rows_here; lr += kTsThreads) {
      const uint32_t s = sh.rs[lr], e = sh.rs[lr + 1], cnt = e - s;
      const uint32_t g = row_base + lr;
      const bool complete = lr + 1 < rows_here || last_complete;
      if (g >= a.max_rows) continue;  // more rows than the arrays hold: reported by the last tile
      const uint32_t key = sh.key[s];
      a.row_start[g] = t0 + s;
      a.row_key[g] = key;
      if (key < nk) { a.row_of_kid[key] = g; atomicAdd(&sh.n_solo_rows, 1u); }
      if (!complete || cnt > kTsRowMax) {
        const uint32_t at = atomicAdd(&a.ctl->n_small, 1u);
        if (at < a.max_deferred) a.deferred[at] = g;
        else atomicOr(&a.ctl->err, kErrTooLarge);
      } else if (cnt <= 4) {
        RowStats* st = a.stats + g;
        const uint32_t i_max = cnt - 1, i_lo = (cnt - 1) >> 1, i_hi = cnt >> 1;
#pragma unroll
        for (int l = 0; l < kLanes; ++l) {
          const uint32_t* v = sh.val[l] + s;
          uint32_t x0 = v[0], x1 = cnt > 1 ? v[1] : 0xFFFFFFFFu, x2 = cnt > 2 ? v[2] : 0xFFFFFFFFu, x3 = cnt > 3 ? v[3] : 0xFFFFFFFFu;
          const unsigned long long sum = (unsigned long long)x0 + (cnt > 1 ? x1 : 0u) + (cnt > 2 ? x2 : 0u) + (cnt > 3 ? x3 : 0u);
          uint32_t t;
#define KS_CSWAP(p, q) t = min(p, q); q = max(p, q); p = t;
          KS_CSWAP(x0, x1) KS_CSWAP(x2, x3) KS_CSWAP(x0, x2) KS_CSWAP(x1, x3) KS_CSWAP(x1, x2)
#undef KS_CSWAP
          auto pick = [&](uint32_t i) { return i == 0 ? x0 : i == 1 ? x1 : i == 2 ? x2 : x3; };
          ts_store(st, l, sum, x0, pick(i_max), pick(i_lo), pick(i_hi));
        }
      } else if (cnt <= 8) {
        sh.list8[atomicAdd(&sh.n8, 1u)] = (uint16_t)lr;
      } else if (cnt <= 16) {
        sh.list16[atomicAdd(&sh.n16, 1u)] = (uint16_t)lr;
      } else if (cnt <= 32) {
        sh.list32[atomicAdd(&sh.n32, 1u)] = (uint16_t)lr;
      } else {
        sh.listw[atomicAdd(&sh.nw, 1u)] = (uint16_t)lr;
      }
    }
    __syncthreads();
    if (tid == 0) {
      if (sh.n_solo_rows) atomicAdd(&a.ctl->ticket2, sh.n_solo_rows);
      if (tile == ntiles - 1) {  // the last tile knows the number of rows
        const uint32_t rows = row_base + rows_here;
        if (rows > a.max_rows) {
          atomicOr(&a.ctl->err, kErrTooLarge);
          a.ctl->n_rows = 0;
          a.ctl->pad2[0] = rows;  // so that the host can size the arrays and run again
          a.row_start[0] = 0;
        } else {
          a.ctl->n_rows = rows;
          a.row_start[rows] = n;
        }
      }
    }

    // ---- the listed rows.  Work items, heaviest first: one row of 33..kTsRowMax samples, or 32 rows of a smaller class;
    // no warp waits for another until the tile is done.
    {
      const uint32_t nw = sh.nw, n32 = sh.n32, n16 = sh.n16, n8 = sh.n8;
      const uint32_t c32 = (n32 + 31) >> 5, c16 = (n16 + 31) >> 5, c8 = (n8 + 31) >> 5;
      const uint32_t items_total = nw + c32 + c16 + c8;
      while (true) {  // the warps draw work items from a counter: a warp with a long row does not hold up its share of the short ones
        uint32_t j = 0;
        if (lane == 0) j = atomicAdd(&sh.qhead, 1u);
        j = __shfl_sync(0xFFFFFFFFu, j, 0);
        if (j >= items_total) break;
        if (j < nw) {
          const uint32_t lr = sh.listw[j];
          const uint32_t s = sh.rs[lr], cnt = sh.rs[lr + 1] - s;
          ts_warp_row(sh, warp, s, cnt, a.stats + row_base + lr);
        } else if (j < nw + c32) {
          const uint32_t t = (j - nw) * 32 + lane;
          if (t < n32) { const uint32_t lr = sh.list32[t], s = sh.rs[lr]; ts_thread_row<32>(sh, s, sh.rs[lr + 1] - s, a.stats + row_base + lr); }
        } else if (j < nw + c32 + c16) {
          const uint32_t t = (j - nw - c32) * 32 + lane;
          if (t < n16) { const uint32_t lr = sh.list16[t], s = sh.rs[lr]; ts_thread_row<16>(sh, s, sh.rs[lr + 1] - s, a.stats + row_base + lr); }
        } else {
          const uint32_t t = (j - nw - c32 - c16) * 32 + lane;
          if (t < n8) { const uint32_t lr = sh.list8[t], s = sh.rs[lr]; ts_thread_row<8>(sh, s, sh.rs[lr + 1] - s, a.stats + row_base + lr); }
        }
        __syncwarp();
      }
    }
  }
}

// One thread per deferred row: up to kBigMax samples -> the CTA-per-row list, larger -> a large row and its chunks.
struct DeferredArgs {
  const uint32_t* deferred;
  const uint32_t* row_start;
  uint32_t max_deferred;
  SegArgs seg;
};
__global__ void __launch_bounds__(256) k_seg_deferred(const DeferredArgs a) {
  const SegArgs& s = a.seg;
  const uint32_t n_rows = min(*s.n_rows_dev, s.max_rows);
  if (n_rows == 0) return;  // too many rows for the arrays: the row offsets are not valid
  const uint32_t nd = min(s.ctl->n_small, a.max_deferred);
  for (uint32_t t = blockIdx.x * blockDim.x + threadIdx.x; t < nd; t += gridDim.x * blockDim.x) {
    const uint32_t row = a.deferred[t];
    if (row >= n_rows) continue;
    const uint32_t st = a.row_start[row], cnt = a.row_start[row + 1] - st;
    if (cnt <= kBigSmall) {
      s.mid_rows[atomicAdd(big_row_counter(s.ctl) + 1, 1u)] = row;  // the CTA-per-row kernel with the small staging area
    } else if (cnt <= kBigMax) {
      s.big_rows[atomicAdd(big_row_counter(s.ctl), 1u)] = row;
    } else {
      const uint32_t nch = (cnt + kLargeChunk - 1) / kLargeChunk;
      const uint32_t l = atomicAdd(&s.ctl->ticket, 1u);
      const uint32_t cbase = (uint32_t)atomicAdd(&s.ctl->scratch0, (unsigned long long)nch);
      if (l >= s.max_large || cbase + nch > s.max_chunks) {
        atomicOr(&s.ctl->err, kErrTooLarge);
      } else {
        LargeRow* L = s.large + l;
        L->row = row; L->start = st; L->cnt = cnt;
        for (int i = 0; i < kLanes; ++i) { L->sum[i] = 0; L->mn[i] = 0xFFFFFFFFu; L->mx[i] = 0; }
        for (uint32_t c = 0; c < nch; ++c) { s.chunk_row[cbase + c] = l; s.chunk_idx[cbase + c] = c; }
      }
    }
  }
}

}  // namespace ks
