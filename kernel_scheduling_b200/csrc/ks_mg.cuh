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

// ---------------------------------------------------------------------------------------------------------
// Kernels of the native driver (ks_mg_build): the same phases, but every count a later kernel needs is read on the
// device, so the host waits only three times per table (after the three header exchanges).

// First 256 bytes of every exchanged block: the sender's control words and the counts the other ranks need.
struct MgHeader {
  Control ctl;
  uint32_t n_tail;                 // launches in the sender's tail
  uint32_t n_halo;                 // launches of earlier windows that reach into the sender's window (from block 2 on)
  unsigned long long capacity;     // sample capacity of the sender (block 2): n_pairs above it means "grow and repeat"
  unsigned long long first_start;  // start_ns of the sender's first record
  // peer-memory mode: the buffer the other ranks store into next (block 2: the sample receive buffer, block 4: the table)
  unsigned char ipc[64];           // cudaIpcMemHandle_t
  unsigned long long buf_gen;      // changes whenever the sender replaced the buffer
  unsigned long long buf_cap;      // its size in bytes
  uint32_t n_local_keys;           // distinct keys of the sender's own window
  uint32_t reserved0;
  unsigned char pad[256 - sizeof(Control) - 24 - 64 - 16 - 8];
};
struct MgIpc {
  unsigned char handle[64];
  unsigned long long gen, cap;
};
static_assert(sizeof(MgHeader) == 256, "exchange header is 256 bytes");

// counts: {tail, halo, keys of the own window} on the device, or null
__global__ void k_mg_header(MgHeader* out, const Control* ctl, const uint32_t* counts, const unsigned char* records, uint64_t n_owned, uint64_t capacity,
                            const MgIpc ipc) {
  const uint32_t t = threadIdx.x;
  const uint32_t* src = reinterpret_cast<const uint32_t*>(ctl);
  uint32_t* dst = reinterpret_cast<uint32_t*>(&out->ctl);
  if (t < sizeof(Control) / 4) dst[t] = src[t];
  if (t == 0) {
    out->n_tail = counts ? counts[0] : 0u;
    out->n_halo = counts ? counts[1] : 0u;
    out->n_local_keys = counts ? counts[2] : 0u;
    out->reserved0 = 0;
    out->capacity = capacity;
    out->first_start = n_owned ? *reinterpret_cast<const unsigned long long*>(records + 32) : 0ull;
    out->buf_gen = ipc.gen;
    out->buf_cap = ipc.cap;
  }
  if (t < 16) reinterpret_cast<uint32_t*>(out->ipc)[t] = reinterpret_cast<const uint32_t*>(ipc.handle)[t];
}

// every rank's exported keys into this rank's dictionary, counts from the gathered headers (blockIdx.y = source rank)
__global__ void __launch_bounds__(256) k_dict_insert_gathered(const unsigned char* __restrict__ gathered, size_t stride, size_t off_keys, size_t off_words, uint32_t capacity,
                                                              unsigned long long* dict_keys, uint4* dict_words, Control* ctl) {
  const unsigned char* block = gathered + blockIdx.y * stride;
  const uint32_t n = min(reinterpret_cast<const MgHeader*>(block)->ctl.n_keys, capacity);
  const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const unsigned long long key = reinterpret_cast<const unsigned long long*>(block + off_keys)[i];
  if (key == 0ull) return;
  const uint4* words = reinterpret_cast<const uint4*>(block + off_words);
  bool inserted;
  const uint32_t slot = dict_find_or_insert(dict_keys, key, &inserted);
  if (slot >= kDictSlots) { atomicOr(&ctl->err, kErrTooManyKeys); return; }
  if (inserted) {
    dict_words[2 * (size_t)slot] = words[2 * (size_t)i];
    dict_words[2 * (size_t)slot + 1] = words[2 * (size_t)i + 1];
  }
}

// k_gather_records with the count on the device
__global__ void __launch_bounds__(256) k_gather_records_dev(const uint4* __restrict__ records, const uint32_t* __restrict__ idx, const uint32_t* __restrict__ n_dev,
                                                            uint32_t capacity, uint4* __restrict__ out) {
  const uint32_t n = min(*n_dev, capacity);
  const uint32_t t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= n * 3) return;
  out[t] = records[(size_t)idx[t / 3] * 3 + t % 3];
}

// k_export_keys with the count on the device (ctl->n_keys, clamped to what the block holds)
__global__ void __launch_bounds__(256) k_export_keys_dev(const unsigned long long* __restrict__ dkeys, const uint32_t* __restrict__ dslot, const uint4* __restrict__ dict_words,
                                                         const Control* __restrict__ ctl, uint32_t capacity, unsigned long long* __restrict__ keys_out, uint4* __restrict__ words_out) {
  const uint32_t n = min(ctl->n_keys, capacity);
  const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  keys_out[i] = dkeys[i];
  words_out[2 * (size_t)i] = dict_words[2 * (size_t)dslot[i]];
  words_out[2 * (size_t)i + 1] = dict_words[2 * (size_t)dslot[i] + 1];
}

// The halo of this rank, straight from the gathered blocks onto the timeline: of the tails of all earlier ranks, the
// launches that end after this window's first start, in start order, placed in the last entries of the kHaloMax timeline
// slots in front of the window.  The unused slots in front of them become inert entries (solo flag, no duration, a start
// no later than any halo start), so the join always sees exactly kHaloMax halo slots and needs no count from the host.
struct HaloArgs {
  const unsigned char* gathered;  // block 1 of every rank, `stride` bytes apart; tails start 256 bytes into a block
  size_t stride;
  uint32_t rank;
  const unsigned char* own_records;
  uint64_t n_owned;
  unsigned long long* dict_keys;
  int type_mode;
  unsigned long long* tl_start;  // timeline set 0, entries [0, kHaloMax) are the halo slots
  unsigned long long* tl_dm;
  uint32_t* n_halo;              // out: launches found (above kHaloMax: nothing was placed)
  Control* ctl;
};

__global__ void __launch_bounds__(1024) k_halo_place(const HaloArgs a) {
  __shared__ uint32_t s_warp[32];
  __shared__ uint32_t s_total;
  __shared__ unsigned long long s_min;
  const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
  const unsigned long long first = a.n_owned ? *reinterpret_cast<const unsigned long long*>(a.own_records + 32) : 0ull;
  if (tid == 0) { s_total = 0; s_min = ~0ull; }
  __syncthreads();
  auto tail_count = [&](uint32_t q) { return min(reinterpret_cast<const MgHeader*>(a.gathered + q * a.stride)->n_tail, kHaloMax); };
  auto tail_rec = [&](uint32_t q, uint32_t i) { return a.gathered + q * a.stride + sizeof(MgHeader) + (size_t)i * 48; };
  // pass 1: how many, and the earliest start among them
  uint32_t mine = 0;
  unsigned long long my_min = ~0ull;
  if (a.n_owned) {
    for (uint32_t q = 0; q < a.rank; ++q) {
      const uint32_t nq = tail_count(q);
      for (uint32_t i = tid; i < nq; i += blockDim.x) {
        const unsigned long long* se = reinterpret_cast<const unsigned long long*>(tail_rec(q, i) + 32);
        if (se[1] > first) { ++mine; my_min = min(my_min, se[0]); }
      }
    }
  }
  mine = warp_sum(mine);
#pragma unroll
  for (int o = 16; o; o >>= 1) my_min = min(my_min, __shfl_xor_sync(0xFFFFFFFFu, my_min, o));
  if (lane == 0) { if (mine) atomicAdd(&s_total, mine); if (my_min != ~0ull) atomicMin(&s_min, my_min); }
  __syncthreads();
  const uint32_t total = s_total;
  if (tid == 0) *a.n_halo = total;
  const uint32_t placed = total <= kHaloMax ? total : 0u;
  const unsigned long long filler_start = placed ? s_min : first;
  for (uint32_t i = tid; i < kHaloMax - placed; i += blockDim.x) {
    a.tl_start[i] = filler_start;
    a.tl_dm[i] = (unsigned long long)kMetaSoloBit << 32;
  }
  if (!placed) return;
  // pass 2: ordered placement (ranks ascending, tails are in start order, windows are ordered in time)
  uint32_t base = kHaloMax - placed, max_dur = 0, err = 0;
  for (uint32_t q = 0; q < a.rank; ++q) {
    const uint32_t nq = tail_count(q);
    for (uint32_t i0 = 0; i0 < nq; i0 += blockDim.x) {
      const uint32_t i = i0 + tid;
      bool take = false;
      uint4 w0 = make_uint4(0, 0, 0, 0), w1 = w0, w2 = w0;
      if (i < nq) {
        const uint4* rp = reinterpret_cast<const uint4*>(tail_rec(q, i));
        w2 = rp[2];
        const unsigned long long end = (unsigned long long)w2.z | ((unsigned long long)w2.w << 32);
        take = end > first;
        if (take) { w0 = rp[0]; w1 = rp[1]; }
      }
      const uint32_t ballot = __ballot_sync(0xFFFFFFFFu, take);
      if (lane == 0) s_warp[warp] = __popc(ballot);
      __syncthreads();
      uint32_t before = 0, chunk = 0;
      for (uint32_t w = 0; w < blockDim.x / 32; ++w) { if (w < warp) before += s_warp[w]; chunk += s_warp[w]; }
      if (take) {
        const uint32_t at = base + before + __popc(ballot & lanemask_lt());
        const unsigned long long start = (unsigned long long)w2.x | ((unsigned long long)w2.y << 32);
        const unsigned long long end = (unsigned long long)w2.z | ((unsigned long long)w2.w << 32);
        const uint64_t key = kernel_key(w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w, a.type_mode != 0);
        bool inserted = false;
        uint32_t slot = dict_find_or_insert(a.dict_keys, key, &inserted);
        if (slot >= kDictSlots || inserted) { err |= kErrTooManyKeys; slot = 0; }  // every halo key came with its owner's key list
        const uint32_t dur = (uint32_t)(end - start);
        a.tl_start[at] = start;
        a.tl_dm[at] = (unsigned long long)dur | ((unsigned long long)(slot | (w1.w & (kMetaSoloBit | 0xFF000000u))) << 32);
        max_dur = max(max_dur, dur);
      }
      base += chunk;
      __syncthreads();
    }
  }
  max_dur = warp_max(max_dur);
  err = __reduce_or_sync(0xFFFFFFFFu, err);
  if (lane == 0) { if (max_dur) atomicMax(&a.ctl->max_dur, max_dur); if (err) atomicOr(&a.ctl->err, err); }
}

// per-key launch counts by dense key id out of the dictionary, count on the device
__global__ void __launch_bounds__(256) k_counts_export_dev(const uint32_t* __restrict__ slot_of_kid, const uint32_t* __restrict__ dict_launches,
                                                           const uint32_t* __restrict__ dict_solo, const Control* __restrict__ ctl, uint32_t capacity,
                                                           unsigned long long* __restrict__ launches, unsigned long long* __restrict__ solo) {
  const uint32_t nk = min(ctl->n_keys, capacity);
  const uint32_t kid = blockIdx.x * blockDim.x + threadIdx.x;
  if (kid >= nk) return;
  const uint32_t slot = slot_of_kid[kid];
  launches[kid] = dict_launches[slot];
  solo[kid] = dict_solo[slot];
}

// the counts of all ranks summed, back into the dictionary (blocks `stride` bytes apart, counts at the given offsets)
__global__ void __launch_bounds__(256) k_counts_sum_import(const unsigned char* __restrict__ gathered, size_t stride, uint32_t world, size_t off_launches, size_t off_solo,
                                                           const uint32_t* __restrict__ slot_of_kid, uint32_t nk, uint32_t* dict_launches, uint32_t* dict_solo) {
  const uint32_t kid = blockIdx.x * blockDim.x + threadIdx.x;
  if (kid >= nk) return;
  unsigned long long l = 0, s = 0;
  for (uint32_t q = 0; q < world; ++q) {
    l += reinterpret_cast<const unsigned long long*>(gathered + q * stride + off_launches)[kid];
    s += reinterpret_cast<const unsigned long long*>(gathered + q * stride + off_solo)[kid];
  }
  const uint32_t slot = slot_of_kid[kid];
  dict_launches[slot] = (uint32_t)l;
  dict_solo[slot] = (uint32_t)s;
}

// k_key_hist with the sample count and the key count on the device: bin = sort key >> shift, shift from the key count
__device__ __forceinline__ uint32_t key_hist_shift(unsigned long long nk) {
  const unsigned long long top = nk + nk * nk;
  const int bits = top ? 64 - __clzll(top) : 0;
  return bits > 12 ? (uint32_t)(bits - 12) : 0u;
}
__global__ void __launch_bounds__(256) k_key_hist_dev(const uint4* __restrict__ samples, const Control* __restrict__ ctl, uint64_t capacity, unsigned long long* __restrict__ hist) {
  __shared__ uint32_t sh[kKeyHistBins];
  const uint32_t n = (uint32_t)min((unsigned long long)capacity, ctl->n_pairs);
  const uint32_t shift = key_hist_shift(ctl->n_keys);
  for (uint32_t i = threadIdx.x; i < kKeyHistBins; i += blockDim.x) sh[i] = 0;
  __syncthreads();
  const uint32_t gstride = gridDim.x * blockDim.x;
  for (uint32_t i0 = blockIdx.x * blockDim.x + threadIdx.x; i0 < n; i0 += 4 * gstride) {  // four loads in flight per thread
    uint32_t k[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const uint32_t i = i0 + u * gstride;
      k[u] = i < n ? samples[i].x : 0xFFFFFFFFu;
    }
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (i0 + u * gstride < n) atomicAdd(&sh[min(k[u] >> shift, kKeyHistBins - 1)], 1u);
  }
  __syncthreads();
  for (uint32_t i = threadIdx.x; i < kKeyHistBins; i += blockDim.x)
    if (sh[i]) atomicAdd(&hist[i], (unsigned long long)sh[i]);
}

// The histogram bins that hold a cut between two key ranges, counted again in 1 << sub_bits sub-bins each:
// out[cut index << sub_bits | sub-bin] += 1 for every sample whose bin is bin[cut index].
struct KeySubHistArgs {
  uint32_t n_cut;
  uint32_t sub_bits;
  uint32_t bin[31];  // ascending
};
__global__ void __launch_bounds__(256) k_key_subhist_dev(const uint4* __restrict__ samples, const Control* __restrict__ ctl, uint64_t capacity, const KeySubHistArgs a,
                                                         unsigned long long* __restrict__ out) {
  __shared__ uint32_t sh[31 * 256];
  __shared__ unsigned char cut_of_bin[kKeyHistBins];
  const uint32_t n = (uint32_t)min((unsigned long long)capacity, ctl->n_pairs);
  const uint32_t shift = key_hist_shift(ctl->n_keys);
  const uint32_t words = a.n_cut << a.sub_bits;
  for (uint32_t i = threadIdx.x; i < words; i += blockDim.x) sh[i] = 0;
  for (uint32_t i = threadIdx.x; i < kKeyHistBins; i += blockDim.x) cut_of_bin[i] = 0xFF;
  __syncthreads();
  if (threadIdx.x < a.n_cut) cut_of_bin[a.bin[threadIdx.x]] = (unsigned char)threadIdx.x;
  __syncthreads();
  const uint32_t sub_shift = shift - a.sub_bits, sub_mask = (1u << a.sub_bits) - 1u;  // sub_bits <= shift
  const uint32_t gstride = gridDim.x * blockDim.x;
  for (uint32_t i0 = blockIdx.x * blockDim.x + threadIdx.x; i0 < n; i0 += 4 * gstride) {  // four loads in flight per thread
    uint32_t k[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const uint32_t i = i0 + u * gstride;
      k[u] = i < n ? samples[i].x : 0xFFFFFFFFu;
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      if (i0 + u * gstride >= n) continue;
      const uint32_t c = cut_of_bin[min(k[u] >> shift, kKeyHistBins - 1)];
      if (c != 0xFF) atomicAdd(&sh[(c << a.sub_bits) | ((k[u] >> sub_shift) & sub_mask)], 1u);
    }
  }
  __syncthreads();
  for (uint32_t i = threadIdx.x; i < words; i += blockDim.x)
    if (sh[i]) atomicAdd(&out[i], (unsigned long long)sh[i]);
}

// every key's solo time: the rank that reduced the key's solo row has a number, the others NaN
__global__ void __launch_bounds__(256) k_solo_merge(const unsigned char* __restrict__ gathered, size_t stride, uint32_t world, size_t off_solo, uint32_t nk,
                                                    double* __restrict__ solo_ns) {
  const uint32_t kid = blockIdx.x * blockDim.x + threadIdx.x;
  if (kid >= nk) return;
  double best = __longlong_as_double(0x7FF8000000000000ll);
  for (uint32_t q = 0; q < world; ++q) {
    const double v = reinterpret_cast<const double*>(gathered + q * stride + off_solo)[kid];
    if (v == v && !(best >= v)) best = v;  // the maximum of the numbers
  }
  solo_ns[kid] = best;
}

}  // namespace ks
