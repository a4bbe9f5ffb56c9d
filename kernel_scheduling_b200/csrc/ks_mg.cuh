// ks_mg.cuh -- small kernels of the multi-GPU path (one process per GPU, each owning one time window of the trace).
//
// Windows are cut by record position in the start-ordered trace.  A pair of overlapping launches belongs to the window
// of its LATER member, so a rank also needs the launches of the previous window that are still running when its own
// window begins (the halo); k_tail_select picks, on the previous rank, the launches that end after that rank's last
// start -- a superset of what the next window can overlap.  Keys are made global by inserting every rank's distinct
// keys into every rank's dictionary (same key set => same dense ids everywhere).  Samples are range-partitioned over the
// ranks by sort key with splitters chosen from a coarse global histogram, so the rank-order concatenation of the ranks'
// tables is the sorted table.
#pragma once

#include "ks_common.cuh"
#include "ks_decode.cuh"
#include "ks_segstats.cuh"

namespace ks {

constexpr uint32_t kHaloMax = 4096;      // timeline entries reserved in front of a window for the halo
constexpr uint32_t kKeyHistBins = 4096;  // coarse histogram of sample sort keys for the splitters

// one CTA: indices (into the window's timeline, ascending = start order) of the co-run launches that end after the
// window's last start
__global__ void __launch_bounds__(1024) k_tail_select(const unsigned long long* __restrict__ tl_start, const unsigned long long* __restrict__ tl_dm,
                                                      uint32_t n, uint32_t* __restrict__ idx_out, uint32_t capacity, uint32_t* __restrict__ count, Control* ctl) {
  __shared__ uint32_t s_first, s_count;
  __shared__ uint32_t list[kHaloMax];
  if (n == 0) return;
  const unsigned long long last = tl_start[n - 1];
  for (uint32_t i = threadIdx.x; i < kHaloMax; i += blockDim.x) list[i] = 0xFFFFFFFFu;
  if (threadIdx.x == 0) {
    s_count = 0;
    const unsigned long long reach = ctl->max_dur;  // no launch starting before last - max_dur can still be running
    const unsigned long long from = last > reach ? last - reach : 0ull;
    uint32_t lo = 0, hi = n;
    while (lo < hi) {
      const uint32_t mid = (lo + hi) >> 1;
      if (tl_start[mid] < from) lo = mid + 1; else hi = mid;
    }
    s_first = lo;
  }
  __syncthreads();
  for (uint32_t i = s_first + threadIdx.x; i < n; i += blockDim.x) {
    const unsigned long long dm = tl_dm[i];
    const bool solo = ((uint32_t)(dm >> 32) & kMetaSoloBit) != 0;
    if (!solo && tl_start[i] + (uint32_t)dm > last) {
      const uint32_t at = atomicAdd(&s_count, 1u);
      if (at < kHaloMax) list[at] = i;
    }
  }
  __syncthreads();
  const uint32_t found = s_count;
  if (threadIdx.x == 0) *count = found;
  if (found > kHaloMax || found > capacity) return;  // the host reports the overflow
  // bitonic sort of the list (padded with 0xFFFFFFFF to a power of two) in shared memory
  uint32_t width = 2;
  while (width < found) width <<= 1;
  for (uint32_t k = 2; k <= width; k <<= 1) {
    for (uint32_t j = k >> 1; j > 0; j >>= 1) {
      for (uint32_t t = threadIdx.x; t < width; t += blockDim.x) {
        const uint32_t o = t ^ j;
        if (o > t) {
          const uint32_t x = list[t], y = list[o];
          const bool up = (t & k) == 0;
          if ((x > y) == up) { list[t] = y; list[o] = x; }
        }
      }
      __syncthreads();
    }
  }
  for (uint32_t i = threadIdx.x; i < found; i += blockDim.x) idx_out[i] = list[i];
}

// gathers 48-byte records by index (three 16-byte vectors each); thread per vector
__global__ void __launch_bounds__(256) k_gather_records(const uint4* __restrict__ records, const uint32_t* __restrict__ idx, uint32_t n, uint4* __restrict__ out) {
  const uint32_t t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= n * 3) return;
  out[t] = records[(size_t)idx[t / 3] * 3 + t % 3];
}

// distinct keys of this rank with the launch fields behind them (for the other ranks' dictionaries)
__global__ void __launch_bounds__(256) k_export_keys(const unsigned long long* __restrict__ dkeys, const uint32_t* __restrict__ dslot, const uint4* __restrict__ dict_words,
                                                     uint32_t n, unsigned long long* __restrict__ keys_out, uint4* __restrict__ words_out) {
  const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  keys_out[i] = dkeys[i];
  words_out[2 * (size_t)i] = dict_words[2 * (size_t)dslot[i]];
  words_out[2 * (size_t)i + 1] = dict_words[2 * (size_t)dslot[i] + 1];
}

// inserts keys gathered from all ranks into this rank's dictionary
__global__ void __launch_bounds__(256) k_dict_insert(const unsigned long long* __restrict__ keys, const uint4* __restrict__ words, uint32_t n,
                                                     unsigned long long* dict_keys, uint4* dict_words, Control* ctl) {
  const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n || keys[i] == 0ull) return;
  bool inserted;
  const uint32_t slot = dict_find_or_insert(dict_keys, keys[i], &inserted);
  if (slot >= kDictSlots) { atomicOr(&ctl->err, kErrTooManyKeys); return; }
  if (inserted) {
    dict_words[2 * (size_t)slot] = words[2 * (size_t)i];
    dict_words[2 * (size_t)slot + 1] = words[2 * (size_t)i + 1];
  }
}

// per-key launch counts by dense key id, out of and back into the dictionary (they are summed over the ranks in between)
__global__ void __launch_bounds__(256) k_counts_by_kid(const uint32_t* __restrict__ slot_of_kid, uint32_t* dict_launches, uint32_t* dict_solo, uint32_t nk,
                                                       unsigned long long* launches, unsigned long long* solo, int import) {
  const uint32_t kid = blockIdx.x * blockDim.x + threadIdx.x;
  if (kid >= nk) return;
  const uint32_t slot = slot_of_kid[kid];
  if (import) { dict_launches[slot] = (uint32_t)launches[kid]; dict_solo[slot] = (uint32_t)solo[kid]; }
  else { launches[kid] = dict_launches[slot]; solo[kid] = dict_solo[slot]; }
}

// coarse histogram of the samples' sort keys: bin = key >> shift
__global__ void __launch_bounds__(256) k_key_hist(const uint4* __restrict__ samples, uint32_t n, uint32_t shift, unsigned long long* __restrict__ hist) {
  __shared__ uint32_t sh[kKeyHistBins];
  for (uint32_t i = threadIdx.x; i < kKeyHistBins; i += blockDim.x) sh[i] = 0;
  __syncthreads();
  for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) atomicAdd(&sh[min(samples[i].x >> shift, kKeyHistBins - 1)], 1u);
  __syncthreads();
  for (uint32_t i = threadIdx.x; i < kKeyHistBins; i += blockDim.x)
    if (sh[i]) atomicAdd(&hist[i], (unsigned long long)sh[i]);
}

// solo time of the keys whose solo row this rank reduced; NaN for the others
__global__ void __launch_bounds__(256) k_solo_ns(const RowStats* __restrict__ stats, const uint32_t* __restrict__ row_of_kid, uint32_t nk, double* __restrict__ solo_ns) {
  const uint32_t kid = blockIdx.x * blockDim.x + threadIdx.x;
  if (kid >= nk) return;
  const uint32_t row = row_of_kid[kid];
  solo_ns[kid] = row == 0xFFFFFFFFu ? __longlong_as_double(0x7FF8000000000000ll) : ((double)stats[row].lo[0] + (double)stats[row].hi[0]) * 0.5;
}

}  // namespace ks
