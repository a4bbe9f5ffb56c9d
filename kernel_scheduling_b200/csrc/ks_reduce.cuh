// ks_reduce.cuh -- K4: the rows of the sorted sample stream, and the final tables.
//
//  k_rows_count / k_rows_scan / k_rows_fill   find where the sort key changes: one row per run (ordered compaction); the
//                                              resident-table update uses these, the table builds find their rows inside
//                                              the statistics kernel (ks_tilestats.cuh)
//  (ks_tilestats.cuh, ks_segstats.cuh)         the integer statistics of every row
//  k_finalize_keys / k_finalize_pairs          integer statistics -> the float tables (one IEEE division per value)
//
// Everything a row needs from its samples is an integer (durations in ns), so count, min, max and the median are
// exact by construction; the floating-point sum is the exact integer sum divided once.
#pragma once

#include "ks_common.cuh"
#include "ks_segstats.cuh"

namespace ks {

constexpr int kRowsTile = 2048;  // samples per tile of the run-start compaction (256 threads x 8)
struct RowsArgs {
  const uint32_t* skey;      // sorted sort keys, one every key_stride words
  uint32_t key_stride;
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

__device__ __forceinline__ bool run_starts_at(const uint32_t* skey, uint32_t stride, uint32_t i) {
  return i == 0 || skey[(size_t)i * stride] != skey[(size_t)(i - 1) * stride];
}

__global__ void __launch_bounds__(256) k_rows_count(const RowsArgs a) {
  __shared__ uint32_t warp_tot[8];
  const uint32_t n = a.n_dev ? min(*a.n_dev, a.n) : a.n;
  const uint32_t ntiles = (n + kRowsTile - 1) / kRowsTile;
  for (uint32_t tile = blockIdx.x; tile < ntiles && tile < a.max_tiles; tile += gridDim.x) {
    uint32_t c = 0;
#pragma unroll
    for (int k = 0; k < kRowsTile / 256; ++k) {
      const uint32_t i = tile * kRowsTile + k * 256 + threadIdx.x;
      if (i < n) c += run_starts_at(a.skey, a.key_stride, i);
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
  const uint32_t n = a.n_dev ? min(*a.n_dev, a.n) : a.n;
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
    if (rows > a.max_rows) {
      // more rows than the arrays hold: report it and leave NO rows, so that no later kernel walks stale row offsets
      atomicOr(&a.ctl->err, kErrTooLarge);
      a.ctl->n_rows = 0;
      a.ctl->pad2[0] = rows;  // how many rows there are, so that the host can size the arrays and run again
      a.row_start[0] = 0;
    } else {
      a.ctl->n_rows = rows;
      a.row_start[rows] = n;
    }
  }
}

__global__ void __launch_bounds__(256) k_rows_fill(const RowsArgs a) {
  __shared__ uint32_t word_base[kRowsTile / 32];  // run starts in front of each 32-sample word of the tile
  const uint32_t n = a.n_dev ? min(*a.n_dev, a.n) : a.n;
  const uint32_t nk = a.ctl->n_keys;
  const uint32_t ntiles = min((n + kRowsTile - 1) / kRowsTile, a.max_tiles);
  if (a.ctl->err & kErrTooLarge) return;  // the scan found more rows than the arrays hold
  const uint32_t lane = lane_id(), warp = threadIdx.x >> 5;
  uint32_t solo_rows = 0;
  for (uint32_t tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
    // consecutive lanes look at consecutive samples; a ballot per 32 samples marks the run starts
    uint32_t key[kRowsTile / 256], ballot[kRowsTile / 256];
#pragma unroll
    for (int k = 0; k < kRowsTile / 256; ++k) {
      const uint32_t i = tile * kRowsTile + k * 256 + threadIdx.x;
      bool flag = false;
      key[k] = 0;
      if (i < n) {
        key[k] = a.skey[(size_t)i * a.key_stride];
        flag = i == 0 || key[k] != a.skey[(size_t)(i - 1) * a.key_stride];
      }
      ballot[k] = __ballot_sync(0xFFFFFFFFu, flag);
      if (lane == 0) word_base[k * 8 + warp] = __popc(ballot[k]);
    }
    __syncthreads();
    if (warp == 0) {  // exclusive scan over the 64 words
      const uint32_t c0 = word_base[lane], c1 = word_base[32 + lane];
      const uint32_t i0 = warp_incl_scan(c0);
      const uint32_t tot0 = __shfl_sync(0xFFFFFFFFu, i0, 31);
      const uint32_t i1 = warp_incl_scan(c1);
      word_base[lane] = i0 - c0;
      word_base[32 + lane] = tot0 + i1 - c1;
    }
    __syncthreads();
    const uint32_t tile_row = a.tile_cnt[tile];
#pragma unroll
    for (int k = 0; k < kRowsTile / 256; ++k) {
      if (ballot[k] & (1u << lane)) {
        const uint32_t row = tile_row + word_base[k * 8 + warp] + __popc(ballot[k] & lanemask_lt());
        a.row_start[row] = tile * kRowsTile + k * 256 + threadIdx.x;
        a.row_key[row] = key[k];
        if (key[k] < nk) { a.row_of_kid[key[k]] = row; ++solo_rows; }
      }
    }
    __syncthreads();
  }
  solo_rows = warp_sum(solo_rows);
  if (lane == 0 && solo_rows) atomicAdd(&a.ctl->ticket2, solo_rows);  // ticket2 = number of solo rows
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
  int solo_given;         // 1: solo_ns already holds every key's solo time (multi-GPU: merged over the ranks)
  ks_key_row* key_rows;   // [kMaxKeys + 1]
  ks_pair_row* pair_rows; // [max_pair_rows]
  uint32_t max_pair_rows;
  Control* ctl;
  // multi-GPU, peer memory: the rows are ALSO written to the same place in these tables (the other ranks' copies of the
  // whole table, plain stores over NVLink), so the table needs no exchange afterwards
  uint32_t n_peer_tables;
  ks_pair_row* peer_rows[15];
};

__global__ void __launch_bounds__(256) k_finalize_keys(const FinalArgs a) {
  const uint32_t nk = min(a.ctl->n_keys, kMaxKeys);
  const uint32_t kid = blockIdx.x * blockDim.x + threadIdx.x;
  if (kid >= nk) return;
  const uint32_t slot = a.slot_of_kid[kid];
  const uint4 w0 = a.dict_words[2 * (size_t)slot], w1 = a.dict_words[2 * (size_t)slot + 1];
  const uint32_t row = a.row_of_kid[kid];
  double solo = __longlong_as_double(0x7FF8000000000000ll);
  if (a.solo_given) solo = a.solo_ns[kid];
  else if (row != 0xFFFFFFFFu) solo = ((double)a.stats[row].lo[0] + (double)a.stats[row].hi[0]) * 0.5;
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
  // 256 consecutive rows per CTA and iteration: their statistics (18 KB) come in and their table rows (32 KB) go out as
  // consecutive memory, staged through shared memory so that every global access is coalesced
  constexpr int kInWords = sizeof(RowStats) / 4, kOutWords = sizeof(ks_pair_row) / 4;
  constexpr int kRowVec = kOutWords / 4 + 1;  // 16-byte vectors per staged row, one of padding: conflict-free 128-bit stores
  __shared__ __align__(16) uint32_t stage[256 * kRowVec * 4];
  const uint32_t n_rows = a.ctl->n_rows, first = a.ctl->ticket2;  // rows [0, first) are the solo rows
  const uint32_t nk = a.ctl->n_keys;
  const double nan = __longlong_as_double(0x7FF8000000000000ll);
  const uint32_t n_out = n_rows > first ? n_rows - first : 0;
  for (uint32_t out0 = blockIdx.x * 256u; out0 < n_out; out0 += gridDim.x * 256u) {
    const uint32_t here = min(256u, n_out - out0);
    if (out0 + here > a.max_pair_rows) { if (threadIdx.x == 0) atomicOr(&a.ctl->err, kErrPairTableFull); return; }
    __syncthreads();
    const uint32_t* src = reinterpret_cast<const uint32_t*>(a.stats + first + out0);
    for (uint32_t i = threadIdx.x; i < here * kInWords; i += 256) stage[i] = src[i];
    __syncthreads();
    ks_pair_row p;
    const bool mine = threadIdx.x < here;
    if (mine) {
      const uint32_t r = first + out0 + threadIdx.x;
      RowStats st;
      uint32_t* w = reinterpret_cast<uint32_t*>(&st);
#pragma unroll
      for (int i = 0; i < kInWords; ++i) w[i] = stage[threadIdx.x * kInWords + i];
      // A row behind the solo rows holds a pair key >= nk.  When a caller's size guess was wrong (the sort covered too
      // few key bits) rows are out of order and this does not hold: such a table is thrown away by the host, but its
      // rows must still index inside the key arrays.
      const uint32_t rk = a.row_key[r];
      const bool sane = nk != 0 && rk >= nk && (rk - nk) / nk < nk;
      const uint32_t pid = sane ? rk - nk : 0u;
      const uint32_t ka = sane ? pid / nk : 0u, kb = sane ? pid % nk : 0u;
      const uint32_t cnt = a.row_start[r + 1] - a.row_start[r];
      const double sa = a.solo_ns[ka], sb = a.solo_ns[kb];
      const bool va = sa > 0.0, vb = sb > 0.0;  // false for NaN
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
    }
    __syncthreads();
    if (mine) {
      const uint4* q = reinterpret_cast<const uint4*>(&p);
      uint4* d = reinterpret_cast<uint4*>(stage) + threadIdx.x * kRowVec;
#pragma unroll
      for (int i = 0; i < kOutWords / 4; ++i) d[i] = q[i];
    }
    __syncthreads();
    uint4* dst = reinterpret_cast<uint4*>(a.pair_rows + out0);
    const uint4* sv = reinterpret_cast<const uint4*>(stage);
    for (uint32_t i = threadIdx.x; i < here * (kOutWords / 4); i += 256) {
      const uint4 v = sv[(i / (kOutWords / 4)) * kRowVec + i % (kOutWords / 4)];
      dst[i] = v;
      for (uint32_t q = 0; q < a.n_peer_tables; ++q) reinterpret_cast<uint4*>(a.peer_rows[q] + out0)[i] = v;
    }
  }
}

}  // namespace ks
