// ks_update.cuh -- the resident pair table: windows of new launches are merged into statistics that stay in HBM, and the
// table can be read out at any time with exactly the values a build over all launches so far would give.
//
// What makes an exact median incremental.  Everything a table row needs from its samples is an integer (durations and
// spans in ns; the division by the solo time happens when the table is read out), so count, sum, min and max are plain
// accumulators.  For the two middle order statistics a row keeps, per value lane, a WINDOW: the values whose ranks
// surround the median among all values seen so far, in sorted order, and n_below = how many values lie below the window
// (those above follow from the count).  A row of up to 64 samples keeps them all inside its own record; up to 1,024 it
// keeps them all in a block of pool 1; a larger one moves to a block of pool 2 and keeps all values up to 16,384, then
// the central 16,384.  A new value below the window's first value (with n_below > 0) only
// raises n_below, one above its last only the implied count above; any other value is merged into the window, which is
// then cut back to its size, centred on the new median rank.  The window is a contiguous range of ranks of the multiset
// at all times, so the middle values read from it are exact.  Values that were dropped cannot come back: the window
// follows the median only through the new values that fall inside it.  For a stationary distribution the sample median
// wanders among the values by a fraction of sqrt(count) ranks over a row's life (measured: 0.3-0.5 sqrt(count)), so 8,192
// kept values on either side are safe for rows of tens of millions of samples; when the distribution of a row moves
// away from where it was, the median CAN leave the window; the kernel then raises kErrEscaped and the host
// reports KS_ERR_REBUILD instead of returning a wrong table.
//
// Rows are addressed directly: stable dense key ids (order of first appearance, at most kUpdMaxKeys keys) and
// row = id for a key's solo row, kUpdMaxKeys + id_a * kUpdMaxKeys + id_b for a pair row -- the sort key of the samples.
// Launches that are still running when a window ends are carried (as timeline entries) into the next window, where they
// take the halo slots in front of it, so pairs across window borders are found exactly once.
#pragma once

#include "ks_common.cuh"
#include "ks_decode.cuh"
#include "ks_mg.cuh"
#include "ks_segstats.cuh"

namespace ks {

constexpr uint32_t kUpdMaxKeys = 2048;
constexpr uint32_t kUpdWindow = 64;       // values a row keeps inside its own record: rows of up to 64 samples keep them all
constexpr uint32_t kUpdMidWindow = 1024;  // rows of up to 1,024 samples keep them all too, in a block of pool 1
constexpr uint32_t kUpdBigWindow = 16384; // larger rows keep the 16,384 values around the median, in a block of pool 2
constexpr uint32_t kUpdBlockSlots = kUpdBigWindow + 1024;  // per lane in pool 2: the window plus one batch being merged
constexpr uint32_t kErrEscaped = 1u << 7;  // a median left its window: the resident statistics are no longer exact
constexpr size_t kUpdRows = (size_t)kUpdMaxKeys + (size_t)kUpdMaxKeys * kUpdMaxKeys;

struct UpdRow {
  unsigned long long sum[kLanes];
  uint32_t mn[kLanes], mx[kLanes];
  uint32_t cnt;
  uint32_t n_below[kLanes];
  uint32_t win[kLanes][kUpdWindow];  // ranks [n_below, n_below + min(cnt, kUpdWindow)) of the lane's values, ascending
};
static_assert(sizeof(UpdRow) == 64 + kLanes * kUpdWindow * 4, "resident row layout");

struct UpdState {
  UpdRow* rows;                      // [kUpdRows]
  unsigned long long* carry_start;   // [kHaloMax] launches still running at the end of the last window, by start
  unsigned long long* carry_dm;
  uint32_t* scalars;                 // [0] carried launches, [1] key ids handed out, [2..3] start_ns of the last launch seen,
                                     // [4], [5] blocks handed out of pool 1 and 2, [8] scratch counter of the read-out
  uint32_t* pool1;                   // [pool1_blocks][kLanes][kUpdMidWindow]: rows of 65 .. 1,024 samples
  uint32_t* pool2;                   // [pool2_blocks][kLanes][kUpdBlockSlots]: rows with more
  uint32_t pool1_blocks, pool2_blocks;
};

// A row with more than kUpdWindow samples keeps its windows in a pool block; win[0][0] of its record holds the block index.
__device__ __forceinline__ const uint32_t* upd_window(const UpdState& st, const UpdRow* R, int l) {
  if (R->cnt <= kUpdWindow) return R->win[l];
  if (R->cnt <= kUpdMidWindow) return st.pool1 + ((size_t)R->win[0][0] * kLanes + l) * kUpdMidWindow;
  return st.pool2 + ((size_t)R->win[0][0] * kLanes + l) * kUpdBlockSlots;
}

// the control words start a step from zero, except what the session accumulates (longest duration, the id base)
__global__ void k_upd_reset_ctl(Control* ctl) {
  if (threadIdx.x != 0) return;
  const uint32_t max_dur = ctl->max_dur;
  Control c;
  memset(&c, 0, sizeof(c));
  c.min_start = ~0ull;
  c.max_dur = max_dur;
  c.n_keys = kUpdMaxKeys;  // the join forms sort keys as n_keys + id_a * n_keys + id_b
  *ctl = c;
}

// new dictionary entries get the next ids
__global__ void __launch_bounds__(256) k_upd_assign_ids(const unsigned long long* __restrict__ dict_keys, uint32_t* kid_of_slot, uint32_t* slot_of_kid, uint32_t* n_ids,
                                                        Control* ctl) {
  const uint32_t slot = blockIdx.x * blockDim.x + threadIdx.x;
  if (slot >= kDictSlots || dict_keys[slot] == 0ull || kid_of_slot[slot] != 0xFFFFFFFFu) return;
  const uint32_t id = atomicAdd(n_ids, 1u);
  if (id >= kUpdMaxKeys) { atomicOr(&ctl->err, kErrTooManyKeys); return; }
  kid_of_slot[slot] = id;
  slot_of_kid[id] = slot;
}

// One CTA: the carried launches that still run when the new window begins take the last halo slots in front of it, in
// start order; the slots in front of them become inert entries.  Also checks that the window does not start before the
// last launch of the previous one.
__global__ void __launch_bounds__(1024) k_upd_place_carry(const UpdState st, unsigned long long* tl_start, unsigned long long* tl_dm, uint64_t n_window, Control* ctl) {
  __shared__ uint32_t s_warp[32];
  __shared__ uint32_t s_total;
  __shared__ unsigned long long s_min;
  const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
  const unsigned long long first = n_window ? tl_start[kHaloMax] : 0ull;
  const uint32_t n_carry = min(st.scalars[0], kHaloMax);
  if (tid == 0) {
    s_total = 0;
    s_min = ~0ull;
    const unsigned long long last_seen = (unsigned long long)st.scalars[2] | ((unsigned long long)st.scalars[3] << 32);
    if (n_window && first < last_seen) atomicOr(&ctl->err, kErrUnordered);
  }
  __syncthreads();
  uint32_t mine = 0;
  unsigned long long my_min = ~0ull;
  for (uint32_t i = tid; i < n_carry; i += blockDim.x) {
    const unsigned long long s = st.carry_start[i];
    if (s + (uint32_t)st.carry_dm[i] > first) { ++mine; my_min = min(my_min, s); }
  }
  mine = warp_sum(mine);
#pragma unroll
  for (int o = 16; o; o >>= 1) my_min = min(my_min, __shfl_xor_sync(0xFFFFFFFFu, my_min, o));
  if (lane == 0) { if (mine) atomicAdd(&s_total, mine); if (my_min != ~0ull) atomicMin(&s_min, my_min); }
  __syncthreads();
  const uint32_t placed = s_total;
  const unsigned long long filler = placed ? s_min : first;
  for (uint32_t i = tid; i < kHaloMax - placed; i += blockDim.x) {
    tl_start[i] = filler;
    tl_dm[i] = (unsigned long long)kMetaSoloBit << 32;
  }
  uint32_t base = kHaloMax - placed;
  for (uint32_t i0 = 0; i0 < n_carry; i0 += blockDim.x) {
    const uint32_t i = i0 + tid;
    unsigned long long s = 0, dm = 0;
    bool take = false;
    if (i < n_carry) {
      s = st.carry_start[i];
      dm = st.carry_dm[i];
      take = s + (uint32_t)dm > first;
    }
    const uint32_t ballot = __ballot_sync(0xFFFFFFFFu, take);
    if (lane == 0) s_warp[warp] = __popc(ballot);
    __syncthreads();
    uint32_t before = 0, chunk = 0;
    for (uint32_t w = 0; w < blockDim.x / 32; ++w) { if (w < warp) before += s_warp[w]; chunk += s_warp[w]; }
    if (take) {
      const uint32_t at = base + before + __popc(ballot & lanemask_lt());
      tl_start[at] = s;
      tl_dm[at] = dm;
    }
    base += chunk;
    __syncthreads();
  }
}

// the launches picked by k_tail_select (indices into [halo slots | window]) become the new carry
__global__ void __launch_bounds__(256) k_upd_save_carry(const UpdState st, const unsigned long long* __restrict__ tl_start, const unsigned long long* __restrict__ tl_dm,
                                                        const uint32_t* __restrict__ idx, const uint32_t* __restrict__ count, uint64_t n_total, Control* ctl) {
  const uint32_t found = *count;
  const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i == 0) {
    if (found > kHaloMax) atomicOr(&ctl->err, kErrTooLarge);
    st.scalars[0] = min(found, kHaloMax);
    if (n_total > kHaloMax) {
      const unsigned long long last = tl_start[n_total - 1];
      st.scalars[2] = (uint32_t)last;
      st.scalars[3] = (uint32_t)(last >> 32);
    }
  }
  if (i < min(found, kHaloMax)) {
    st.carry_start[i] = tl_start[idx[i]];
    st.carry_dm[i] = tl_dm[idx[i]];
  }
}

struct UpdArgs {
  UpdState st;
  const uint4* items;          // the step's samples, sorted by row
  const uint32_t* row_start;   // runs of equal row in items
  const uint32_t* row_key;
  const uint32_t* n_rows_dev;
  uint32_t max_rows;
  uint32_t* big_list;          // [max_rows] rows left to k_upd_big_rows
  Control* ctl;
};

constexpr uint32_t kUpdBatch = 1024;  // new values of one row merged in one go
constexpr int kUpdWarps = 4;          // warps per CTA of k_upd_rows: 8 KB of shared memory each
constexpr int kUpdBigThreads = 256;   // threads of the CTA that merges into one row of the largest kind

// The merge is written for a GROUP of G threads that own the row: a warp (G = 32) for rows that keep all their values,
// a whole CTA (G = 256) for rows with a 16,384-value window.
template <int G>
__device__ __forceinline__ void grp_sync() {
  if (G == 32) __syncwarp(); else __syncthreads();
}

// bitonic sort of the first n words (n a power of two, 32..kUpdBatch) of the group's shared-memory buffer
template <int G>
__device__ __forceinline__ void grp_sort_pow2(uint32_t* buf, uint32_t n, uint32_t tid) {
  for (uint32_t k = 2; k <= n; k <<= 1) {
    for (uint32_t j = k >> 1; j > 0; j >>= 1) {
      for (uint32_t t = tid; t < n; t += G) {
        const uint32_t o = t ^ j;
        if (o > t) {
          const uint32_t x = buf[t], y = buf[o];
          const bool up = (t & k) == 0;
          if ((x > y) == up) { buf[t] = y; buf[o] = x; }
        }
      }
      grp_sync<G>();
    }
  }
}

// Merges mb <= kUpdBatch new values of one lane of a row (items[j].lane, j < mb) into the sorted window vals[0 .. wlen) that
// holds the ranks [n_below, n_below + wlen) of the cnt values seen before.  trim_to = the most values the window keeps
// (0: the window keeps everything, its caller makes sure there is room).  The window has room for wlen + mb values.
// Returns the new n_below.  Shared memory of the group: buf, dest (kUpdBatch words each), ctr (2 words).
template <int G>
__device__ __forceinline__ uint32_t upd_merge(uint32_t* vals, uint32_t wlen, uint32_t trim_to, uint32_t cnt, const uint4* items, int l, uint32_t mb,
                                              uint32_t n_below, uint32_t* buf, uint32_t* dest, uint32_t* ctr, Control* ctl, uint32_t tid) {
  const uint32_t n_above = cnt - n_below - wlen;
  const uint32_t w_first = wlen ? vals[0] : 0u, w_last = wlen ? vals[wlen - 1] : 0u;
  grp_sync<G>();
  if (tid == 0) { ctr[0] = 0; ctr[1] = 0; }
  grp_sync<G>();
  // the values that enter the window -> buf (in any order: they are sorted next)
  for (uint32_t j = tid; j < mb; j += G) {
    const uint4 it = items[j];
    const uint32_t x = l == 0 ? it.y : l == 1 ? it.z : it.w;
    if (wlen && n_below && x < w_first) atomicAdd(&ctr[1], 1u);
    else if (wlen && n_above && x > w_last) { }
    else buf[atomicAdd(&ctr[0], 1u)] = x;
  }
  grp_sync<G>();
  const uint32_t k = ctr[0];
  n_below += ctr[1];
  if (k) {
    uint32_t p2 = 32;
    while (p2 < k) p2 <<= 1;
    for (uint32_t j = k + tid; j < p2; j += G) buf[j] = 0xFFFFFFFFu;
    grp_sync<G>();
    grp_sort_pow2<G>(buf, p2, tid);
    // where each entering value goes: old values <= it stay in front of it
    for (uint32_t j = tid; j < k; j += G) {
      const uint32_t x = buf[j];
      uint32_t lo = 0, hi = wlen;
      while (lo < hi) {
        const uint32_t mid = (lo + hi) >> 1;
        if (vals[mid] <= x) lo = mid + 1; else hi = mid;
      }
      dest[j] = lo + j;
    }
    grp_sync<G>();
    // open the gaps: every old value moves up by the number of entering values smaller than it; tiles from the top down,
    // so a value is always read before its slot is written.  Old values in front of the first entering one do not move.
    const uint32_t first_moved = dest[0];
    const uint32_t tiles = (wlen + G - 1) / G;
    for (uint32_t t = tiles; t-- > first_moved / G;) {
      const uint32_t p = t * G + tid;
      uint32_t v = 0, sh = 0;
      if (p < wlen) {
        v = vals[p];
        uint32_t lo = 0, hi = k;
        while (lo < hi) {
          const uint32_t mid = (lo + hi) >> 1;
          if (buf[mid] < v) lo = mid + 1; else hi = mid;
        }
        sh = lo;
      }
      grp_sync<G>();
      if (p < wlen && sh) vals[p + sh] = v;
      grp_sync<G>();
    }
    for (uint32_t j = tid; j < k; j += G) vals[dest[j]] = buf[j];
    grp_sync<G>();
  }
  const uint32_t L = wlen + k, cnt_new = cnt + mb;
  const long long idx_lo = (long long)((cnt_new - 1) >> 1) - (long long)n_below, idx_hi = (long long)(cnt_new >> 1) - (long long)n_below;
  if (idx_lo < 0 || idx_hi >= (long long)L) {
    if (tid == 0) atomicOr(&ctl->err, kErrEscaped);
  }
  if (trim_to && L > trim_to) {  // cut back to trim_to values centred on the median: `start` go at the bottom, the rest at the top
    long long want = idx_lo - (long long)(trim_to / 2 - 1);
    want = max(want, 0ll);
    want = min(want, (long long)(L - trim_to));
    const uint32_t start = (uint32_t)want;
    if (start) {
      for (uint32_t t = 0; t < (trim_to + G - 1) / G; ++t) {
        const uint32_t p = t * G + tid;
        const uint32_t v = p < trim_to ? vals[p + start] : 0u;
        grp_sync<G>();
        if (p < trim_to) vals[p] = v;
        grp_sync<G>();
      }
    }
    n_below += start;
  }
  return n_below;
}

// where a row of cnt samples keeps its windows: 0 = inside its record, 1 = a block of pool 1, 2 = a block of pool 2
__device__ __forceinline__ int upd_tier(uint32_t cnt) { return cnt <= kUpdWindow ? 0 : cnt <= kUpdMidWindow ? 1 : 2; }

__device__ __forceinline__ uint32_t* upd_block(const UpdState& st, int tier, uint32_t block, int l) {
  return tier == 1 ? st.pool1 + ((size_t)block * kLanes + l) * kUpdMidWindow : st.pool2 + ((size_t)block * kLanes + l) * kUpdBlockSlots;
}

// The step's samples of one row (items[0 .. m), all of one row) merged into the row by a group of G threads.
// Shared memory of the group: buf, dest (kUpdBatch words each), ctr (2 words), red (3 * G / 32 64-bit words for G > 32).
template <int G>
__device__ __forceinline__ void upd_row(const UpdState& st, UpdRow* R, int nl, const uint4* items, uint32_t m, uint32_t* buf, uint32_t* dest, uint32_t* ctr,
                                        unsigned long long* red, Control* ctl, uint32_t tid) {
  uint32_t cnt = R->cnt;
  uint32_t nb[kLanes];  // values below the window, per lane (kept in registers over the batches)
#pragma unroll
  for (int l = 0; l < kLanes; ++l) nb[l] = R->n_below[l];
  int tier = upd_tier(cnt);
  uint32_t block = tier ? R->win[0][0] : 0u;
  // accumulators
  for (int l = 0; l < nl; ++l) {
    unsigned long long add = 0;
    uint32_t lo_new = 0xFFFFFFFFu, hi_new = 0;
    for (uint32_t j = tid; j < m; j += G) {
      const uint4 it = items[j];
      const uint32_t x = l == 0 ? it.y : l == 1 ? it.z : it.w;
      add += x; lo_new = min(lo_new, x); hi_new = max(hi_new, x);
    }
    add = warp_sum64(add); lo_new = warp_min(lo_new); hi_new = warp_max(hi_new);
    if (G > 32) {
      grp_sync<G>();
      if ((tid & 31u) == 0) { red[3 * (tid >> 5)] = add; red[3 * (tid >> 5) + 1] = lo_new; red[3 * (tid >> 5) + 2] = hi_new; }
      grp_sync<G>();
      if (tid == 0) {
        add = 0; lo_new = 0xFFFFFFFFu; hi_new = 0;
        for (int w = 0; w < G / 32; ++w) { add += red[3 * w]; lo_new = min(lo_new, (uint32_t)red[3 * w + 1]); hi_new = max(hi_new, (uint32_t)red[3 * w + 2]); }
      }
    }
    if (tid == 0) {
      R->sum[l] += add;
      R->mn[l] = cnt ? min(R->mn[l], lo_new) : lo_new;
      R->mx[l] = cnt ? max(R->mx[l], hi_new) : hi_new;
    }
  }
  for (uint32_t c0 = 0; c0 < m; c0 += kUpdBatch) {
    const uint32_t mb = min(kUpdBatch, m - c0);
    const int want = upd_tier(cnt + mb);
    if (want != tier) {
      // the row outgrows where it lives: its values (all of them: it is complete up to kUpdMidWindow) move to a block of
      // the next pool
      grp_sync<G>();
      if (tid == 0) ctr[0] = atomicAdd(st.scalars + (want == 1 ? 4 : 5), 1u);
      grp_sync<G>();
      const uint32_t got = ctr[0];
      if (got >= (want == 1 ? st.pool1_blocks : st.pool2_blocks)) {  // a pool ran out: the row cannot be kept exact
        if (tid == 0) atomicOr(&ctl->err, kErrPairTableFull);
        return;
      }
      for (int l = 0; l < kLanes; ++l) {
        const uint32_t* src = tier == 0 ? R->win[l] : upd_block(st, tier, block, l);
        uint32_t* dst = upd_block(st, want, got, l);
        for (uint32_t i = tid; i < cnt; i += G) dst[i] = src[i];
      }
      grp_sync<G>();
      tier = want;
      block = got;
      if (tid == 0) R->win[0][0] = got;
      grp_sync<G>();
    }
#pragma unroll
    for (int l = 0; l < kLanes; ++l) {
      if (l >= nl) continue;
      uint32_t* vals = tier == 0 ? R->win[l] : upd_block(st, tier, block, l);
      const uint32_t cap = tier == 0 ? kUpdWindow : tier == 1 ? kUpdMidWindow : kUpdBigWindow;
      nb[l] = upd_merge<G>(vals, min(cnt, cap), tier == 2 ? kUpdBigWindow : 0u, cnt, items + c0, l, mb, nb[l], buf, dest, ctr, ctl, tid);
    }
    cnt += mb;
  }
  if (tid == 0) {
    R->cnt = cnt;
#pragma unroll
    for (int l = 0; l < kLanes; ++l) R->n_below[l] = nb[l];
  }
  grp_sync<G>();
}

// One warp per row touched by the step.  Rows that have or will get a 16,384-value window are left to k_upd_big_rows
// (one CTA per row): their list goes to big_list, its length to scalars[6].
__global__ void __launch_bounds__(kUpdWarps * 32) k_upd_rows(const UpdArgs a) {
  __shared__ uint32_t bufs[kUpdWarps][2 * kUpdBatch];
  __shared__ uint32_t ctrs[kUpdWarps][2];
  const uint32_t warp = threadIdx.x >> 5, lane = lane_id();
  const uint32_t n_rows = min(*a.n_rows_dev, a.max_rows);
  const uint32_t warps = gridDim.x * kUpdWarps;
  for (uint32_t t = blockIdx.x * kUpdWarps + warp; t < n_rows; t += warps) {
    const uint32_t key = a.row_key[t];
    if ((size_t)key >= kUpdRows) { if (lane == 0) atomicOr(&a.ctl->err, kErrTooManyKeys); continue; }
    UpdRow* R = a.st.rows + key;
    const uint32_t s = a.row_start[t], m = a.row_start[t + 1] - s;
    if (upd_tier(R->cnt + m) == 2) {
      if (lane == 0) a.big_list[atomicAdd(a.st.scalars + 6, 1u)] = t;
      continue;
    }
    upd_row<32>(a.st, R, key < kUpdMaxKeys ? 1 : kLanes, a.items + s, m, bufs[warp], bufs[warp] + kUpdBatch, ctrs[warp], nullptr, a.ctl, lane);
  }
}

// one CTA per row of the largest kind
__global__ void __launch_bounds__(kUpdBigThreads) k_upd_big_rows(const UpdArgs a) {
  __shared__ uint32_t buf[2 * kUpdBatch];
  __shared__ uint32_t ctr[2];
  __shared__ unsigned long long red[3 * kUpdBigThreads / 32];
  const uint32_t n_big = min(a.st.scalars[6], a.max_rows);
  for (uint32_t i = blockIdx.x; i < n_big; i += gridDim.x) {
    const uint32_t t = a.big_list[i];
    const uint32_t key = a.row_key[t];
    UpdRow* R = a.st.rows + key;
    const uint32_t s = a.row_start[t], m = a.row_start[t + 1] - s;
    upd_row<kUpdBigThreads>(a.st, R, key < kUpdMaxKeys ? 1 : kLanes, a.items + s, m, buf, buf + kUpdBatch, ctr, red, a.ctl, threadIdx.x);
    __syncthreads();
  }
}

// ---- reading the table out -----------------------------------------------------------------------------------------
__device__ __forceinline__ void upd_middle(const UpdState& st, const UpdRow* R, int l, uint32_t* lo, uint32_t* hi) {
  const uint32_t cnt = R->cnt, nb = R->n_below[l];
  const uint32_t* w = upd_window(st, R, l);
  *lo = w[((cnt - 1) >> 1) - nb];
  *hi = w[(cnt >> 1) - nb];
}

// the key of every id, for the host to rank
__global__ void __launch_bounds__(256) k_upd_keys_by_id(const unsigned long long* __restrict__ dict_keys, const uint32_t* __restrict__ slot_of_kid, uint32_t n_ids,
                                                        unsigned long long* __restrict__ out) {
  const uint32_t id = blockIdx.x * blockDim.x + threadIdx.x;
  if (id < n_ids) out[id] = dict_keys[slot_of_kid[id]];
}

// pair rows that hold samples: (rank_a * kUpdMaxKeys + rank_b, id_a * kUpdMaxKeys + id_b), in no particular order
__global__ void __launch_bounds__(256) k_upd_collect(const UpdRow* __restrict__ rows, const uint32_t* __restrict__ rank_of_id, uint32_t n_ids, uint32_t* __restrict__ sort_key,
                                                     uint32_t* __restrict__ pair_id, uint32_t* counter, uint32_t capacity) {
  const uint64_t total = (uint64_t)n_ids * n_ids;
  for (uint64_t base = (uint64_t)blockIdx.x * blockDim.x; base < total; base += (uint64_t)gridDim.x * blockDim.x) {
    const uint64_t t = base + threadIdx.x;
    bool mine = false;
    uint32_t ia = 0, ib = 0;
    if (t < total) {
      ia = (uint32_t)(t / n_ids);
      ib = (uint32_t)(t % n_ids);
      mine = rows[(size_t)kUpdMaxKeys + (size_t)ia * kUpdMaxKeys + ib].cnt != 0;
    }
    const uint32_t ballot = __ballot_sync(0xFFFFFFFFu, mine);
    if (!ballot) continue;
    uint32_t at = 0;
    const uint32_t leader = __ffs(ballot) - 1;
    if (lane_id() == leader) at = atomicAdd(counter, (uint32_t)__popc(ballot));
    at = __shfl_sync(0xFFFFFFFFu, at, leader) + __popc(ballot & lanemask_lt());
    if (mine && at < capacity) {
      sort_key[at] = rank_of_id[ia] * kUpdMaxKeys + rank_of_id[ib];
      pair_id[at] = ia * kUpdMaxKeys + ib;
    }
  }
}

struct UpdEmitArgs {
  UpdState st;
  const UpdRow* rows;
  const uint32_t* pair_id;     // sorted by (rank_a, rank_b)
  uint32_t n_pairs;
  const uint32_t* id_by_rank;  // [n_ids]
  const uint32_t* slot_of_kid;
  const unsigned long long* dict_keys;
  const uint4* dict_words;
  const uint32_t* dict_launches;
  const uint32_t* dict_solo;
  uint32_t n_ids;
  ks_key_row* key_rows;
  ks_pair_row* pair_rows;
};

__device__ __forceinline__ double upd_solo_ns(const UpdState& st, uint32_t id) {
  const UpdRow* R = st.rows + id;
  if (R->cnt == 0) return __longlong_as_double(0x7FF8000000000000ll);
  uint32_t lo, hi;
  upd_middle(st, R, 0, &lo, &hi);
  return ((double)lo + (double)hi) * 0.5;
}

__global__ void __launch_bounds__(256) k_upd_emit_keys(const UpdEmitArgs a) {
  const uint32_t r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= a.n_ids) return;
  const uint32_t id = a.id_by_rank[r], slot = a.slot_of_kid[id];
  const uint4 w0 = a.dict_words[2 * (size_t)slot], w1 = a.dict_words[2 * (size_t)slot + 1];
  ks_key_row k;
  k.key = a.dict_keys[slot];
  k.name_id = w0.x;
  k.grid[0] = w0.y; k.grid[1] = w0.z; k.grid[2] = w0.w;
  k.block[0] = w1.x; k.block[1] = w1.y; k.block[2] = w1.z;
  k.smem = w1.w & kSmemMask;
  k.tenant = w1.w >> 24;
  k.reserved = 0;
  k.launches = a.dict_launches[slot];
  k.solo_launches = a.dict_solo[slot];
  k.solo_ns = upd_solo_ns(a.st, id);
  a.key_rows[r] = k;
}

// the same arithmetic as k_finalize_pairs, from the resident statistics
__global__ void __launch_bounds__(256) k_upd_emit_pairs(const UpdEmitArgs a) {
  const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= a.n_pairs) return;
  const uint32_t pid = a.pair_id[i], ia = pid / kUpdMaxKeys, ib = pid % kUpdMaxKeys;
  const UpdRow* R = a.rows + (size_t)kUpdMaxKeys + pid;
  const double nan = __longlong_as_double(0x7FF8000000000000ll);
  const double sa = upd_solo_ns(a.st, ia), sb = upd_solo_ns(a.st, ib);
  const bool va = sa > 0.0, vb = sb > 0.0;
  uint32_t lo[kLanes], hi[kLanes];
  for (int l = 0; l < kLanes; ++l) upd_middle(a.st, R, l, &lo[l], &hi[l]);
  const uint32_t cnt = R->cnt;
  ks_pair_row p;
  p.key_a = a.dict_keys[a.slot_of_kid[ia]];
  p.key_b = a.dict_keys[a.slot_of_kid[ib]];
  p.count = cnt;
  p.flags = (va ? 1ull : 0ull) | (vb ? 2ull : 0ull);
  if (va) {
    p.sum_a = (double)R->sum[0] / sa;
    p.mean_a = p.sum_a / (double)cnt;
    p.min_a = (double)R->mn[0] / sa;
    p.max_a = (double)R->mx[0] / sa;
    p.median_a = ((double)lo[0] / sa + (double)hi[0] / sa) * 0.5;
  } else {
    p.sum_a = p.mean_a = p.min_a = p.max_a = p.median_a = nan;
  }
  if (vb) {
    p.sum_b = (double)R->sum[1] / sb;
    p.mean_b = p.sum_b / (double)cnt;
    p.min_b = (double)R->mn[1] / sb;
    p.max_b = (double)R->mx[1] / sb;
    p.median_b = ((double)lo[1] / sb + (double)hi[1] / sb) * 0.5;
  } else {
    p.sum_b = p.mean_b = p.min_b = p.max_b = p.median_b = nan;
  }
  p.efficiency = (va && vb) ? ((sa + sb) / (double)lo[2] + (sa + sb) / (double)hi[2]) * 0.5 : nan;
  p.span_sum_ns = R->sum[2];
  a.pair_rows[i] = p;
}

}  // namespace ks
