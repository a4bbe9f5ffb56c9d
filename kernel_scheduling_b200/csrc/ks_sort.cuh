// ks_sort.cuh -- K2: stable least-significant-digit radix sort, one sweep over the data per 8-bit digit.
//
// Per pass every CTA takes tiles of 256 x ITEMS keys from a ticket counter (so a tile only ever waits for tiles
// that already started), ranks the keys of a tile by digit with warp ballots (one per digit bit) and per-warp digit
// counters in shared memory, learns the number of equal digits in all earlier tiles by decoupled look-back over
// a per-tile status array (aggregate / inclusive-prefix words with the flag in the top two bits), stages keys
// and payload lanes in shared memory in digit order and writes them out in runs.  One histogram kernel in front
// reads the keys once and counts the digits of every pass.
//
// Every wait is bounded (kSpinLimit polls); a wait that runs out sets kErrWait in the error word and the CTA
// carries on with a wrong offset, so the kernel always terminates and the host reports the failure.
//
// The element count may live in device memory (n_dev != nullptr), so a sort can be queued behind the kernel that
// produces its input without a host round trip.
#pragma once

#include "ks_common.cuh"

namespace ks {

constexpr int kSortThreads = 256;
constexpr int kSortWarps = kSortThreads / 32;
constexpr uint32_t kFlagAgg = 1u << 30;
constexpr uint32_t kFlagPrefix = 2u << 30;
constexpr uint32_t kFlagMask = 3u << 30;
constexpr uint32_t kCountMask = ~kFlagMask;
constexpr uint64_t kSortMaxItems = 1ull << 30;

template <typename KeyT, typename ValT, int NV>
struct SortPassArgs {
  const KeyT* kin;
  KeyT* kout;
  const ValT* vin[NV > 0 ? NV : 1];
  ValT* vout[NV > 0 ? NV : 1];
  const uint32_t* n_dev;  // element count in device memory, or nullptr to use n
  uint32_t n;
  int shift;
  int bits;                // 1..8
  const uint32_t* gbase;   // [256] exclusive digit offsets of this pass
  uint32_t* lookback;      // [tiles][256], zeroed before the pass
  uint32_t* ticket;        // zeroed before the pass
  uint32_t* err;
};

template <typename KeyT>
__device__ __forceinline__ uint32_t digit_of(KeyT k, int shift, uint32_t mask) {
  return (uint32_t)(k >> shift) & mask;
}

// Lanes of the warp whose digit equals this lane's digit, among the lanes of `valid_lanes`.  One ballot per digit
// bit: the vote unit keeps up with the issue rate, the match instruction does not.
template <int BITS = 8>
__device__ __forceinline__ uint32_t match_digit(uint32_t d, uint32_t valid_lanes) {
  uint32_t same = valid_lanes;
#pragma unroll
  for (int b = 0; b < BITS; ++b) {
    const bool bit = (d >> b) & 1u;
    const uint32_t vote = __ballot_sync(0xFFFFFFFFu, bit);
    same &= bit ? vote : ~vote;
  }
  return same;
}

// ---- histogram of every pass's digits in one read of the keys
template <typename KeyT>
__global__ void __launch_bounds__(256) k_radix_hist(const KeyT* __restrict__ keys, uint32_t stride, const uint32_t* n_dev, uint32_t n, int begin_bit,
                                                    int end_bit, uint32_t* __restrict__ hist /*[passes][256]*/) {
  __shared__ uint32_t sh[8 * 256];
  if (n_dev) n = min(*n_dev, n);  // n is then the bound the buffers were sized for
  const int passes = (end_bit - begin_bit + 7) / 8;
  for (int i = threadIdx.x; i < passes * 256; i += blockDim.x) sh[i] = 0;
  __syncthreads();
  const uint32_t gstride = gridDim.x * blockDim.x;
  // four independent loads per thread and iteration (the loop is bound by load latency); plain shared-memory atomics:
  // they cost a few cycles per distinct digit of a warp, less than grouping the lanes by digit first
  for (uint32_t i0 = blockIdx.x * blockDim.x + threadIdx.x; i0 < n; i0 += 4 * gstride) {
    KeyT k[4];
    bool valid[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const uint32_t i = i0 + u * gstride;
      valid[u] = i < n;
      k[u] = valid[u] ? keys[(size_t)i * stride] : (KeyT)0;
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      if (!valid[u]) continue;
      for (int p = 0; p < passes; ++p) {
        const int shift = begin_bit + 8 * p;
        const int bits = min(8, end_bit - shift);
        atomicAdd(&sh[p * 256 + digit_of(k[u], shift, (1u << bits) - 1u)], 1u);
      }
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < passes * 256; i += blockDim.x)
    if (sh[i]) atomicAdd(&hist[i], sh[i]);
}

// ---- exclusive scan of each pass's 256 counters (one CTA of 256 threads)
__global__ void __launch_bounds__(256) k_radix_scan_hist(const uint32_t* __restrict__ hist, uint32_t* __restrict__ gbase, int passes) {
  __shared__ uint32_t warp_tot[8];
  for (int p = 0; p < passes; ++p) {
    const uint32_t v = hist[p * 256 + threadIdx.x];
    const uint32_t inc = warp_incl_scan(v);
    if (lane_id() == 31) warp_tot[threadIdx.x >> 5] = inc;
    __syncthreads();
    uint32_t off = 0;
    for (uint32_t w = 0; w < (threadIdx.x >> 5); ++w) off += warp_tot[w];
    gbase[p * 256 + threadIdx.x] = off + inc - v;
    __syncthreads();
  }
}

// ---- one pass
template <typename KeyT, typename ValT, int NV, int ITEMS>
__global__ void __launch_bounds__(kSortThreads) k_onesweep_pass(const SortPassArgs<KeyT, ValT, NV> a) {
  constexpr int TILE = kSortThreads * ITEMS;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  uint32_t* warp_hist = reinterpret_cast<uint32_t*>(smem_raw);             // [warps][256]
  uint32_t* s_gpos = warp_hist + kSortWarps * 256;                          // [256] global position of staged index 0 of a digit
  uint32_t* s_misc = s_gpos + 256;                                          // [16]
  KeyT* s_keys = reinterpret_cast<KeyT*>(s_misc + 16);                      // [TILE]
  ValT* s_vals = reinterpret_cast<ValT*>(s_keys + TILE);                    // [TILE]

  const uint32_t n = a.n_dev ? *a.n_dev : a.n;
  const uint32_t ntiles = (n + TILE - 1) / TILE;
  const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
  const uint32_t dmask = (1u << a.bits) - 1u;

  while (true) {
    __syncthreads();
    if (tid == 0) s_misc[0] = atomicAdd(a.ticket, 1u);
    for (int i = tid; i < kSortWarps * 256; i += kSortThreads) warp_hist[i] = 0;
    __syncthreads();
    const uint32_t tile = s_misc[0];
    if (tile >= ntiles) break;
    const uint32_t tile_base = tile * TILE;
    const uint32_t tile_n = min((uint32_t)TILE, n - tile_base);

    // -- load keys, warp-striped: item i of lane l of warp w sits at w*32*ITEMS + i*32 + l
    KeyT key[ITEMS];
    uint32_t rank[ITEMS];
    const uint32_t wbase = warp * 32 * ITEMS;
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
      const uint32_t li = wbase + i * 32 + lane;
      key[i] = li < tile_n ? a.kin[tile_base + li] : (KeyT)0;
    }
    // -- rank within the warp, digit by digit in item order (keeps the sort stable)
    uint32_t* wh = warp_hist + warp * 256;
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
      const uint32_t li = wbase + i * 32 + lane;
      const bool valid = li < tile_n;
      const uint32_t d = digit_of(key[i], a.shift, dmask);
      const uint32_t same = match_digit(d, __ballot_sync(0xFFFFFFFFu, valid));
      const uint32_t before = __popc(same & lanemask_lt());
      uint32_t pre = 0;
      if (valid) pre = wh[d];
      __syncwarp();
      if (valid && before == 0) wh[d] = pre + __popc(same);
      __syncwarp();
      rank[i] = pre + before;
    }
    __syncthreads();

    // -- per digit (thread d): exclusive offsets of the warps, the tile's count, look-back
    {
      const uint32_t d = tid;
      uint32_t acc = 0;
#pragma unroll
      for (int w = 0; w < kSortWarps; ++w) {
        const uint32_t t = warp_hist[w * 256 + d];
        warp_hist[w * 256 + d] = acc;
        acc += t;
      }
      uint32_t excl = 0;
      volatile uint32_t* lb = a.lookback + (size_t)tile * 256 + d;
      if (tile == 0) {
        *lb = acc | kFlagPrefix;
      } else {
        *lb = acc | kFlagAgg;
        uint32_t t = tile - 1, spins = 0;
        while (true) {
          const uint32_t v = ld_volatile_u32(a.lookback + (size_t)t * 256 + d);
          const uint32_t f = v & kFlagMask;
          if (f == 0) {
            if (++spins > kSpinLimit) { atomicOr(a.err, kErrWait); break; }
            __nanosleep(20);
            continue;
          }
          excl += v & kCountMask;
          if (f == kFlagPrefix || t == 0) break;
          --t;
        }
        *lb = ((excl + acc) & kCountMask) | kFlagPrefix;
      }
      // exclusive scan of the tile counts over the digits -> where each digit starts in the staging buffer
      const uint32_t inc = warp_incl_scan(acc);
      if (lane == 31) s_misc[1 + warp] = inc;
      __syncthreads();
      uint32_t off = 0;
      for (uint32_t w = 0; w < warp; ++w) off += s_misc[1 + w];
      const uint32_t dstart = off + inc - acc;
      s_gpos[d] = a.gbase[d] + excl - dstart;
      // fold the digit start into the warp offsets so the item loop needs one lookup
#pragma unroll
      for (int w = 0; w < kSortWarps; ++w) warp_hist[w * 256 + d] += dstart;
    }
    __syncthreads();

    // -- stage keys in digit order
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
      const uint32_t li = wbase + i * 32 + lane;
      if (li < tile_n) {
        const uint32_t d = digit_of(key[i], a.shift, dmask);
        rank[i] += wh[d];
        s_keys[rank[i]] = key[i];
      }
    }
    __syncthreads();
    uint32_t outpos[ITEMS];
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
      const uint32_t si = i * kSortThreads + tid;
      if (si < tile_n) {
        const KeyT k = s_keys[si];
        outpos[i] = s_gpos[digit_of(k, a.shift, dmask)] + si;
        a.kout[outpos[i]] = k;
      }
    }
    // -- payload lanes through the same permutation
    if constexpr (NV > 0) {
#pragma unroll
      for (int v = 0; v < NV; ++v) {
        __syncthreads();
#pragma unroll
        for (int i = 0; i < ITEMS; ++i) {
          const uint32_t li = wbase + i * 32 + lane;
          if (li < tile_n) s_vals[rank[i]] = a.vin[v][tile_base + li];
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < ITEMS; ++i) {
          const uint32_t si = i * kSortThreads + tid;
          if (si < tile_n) a.vout[v][outpos[i]] = s_vals[si];
        }
      }
    }
  }
}

// ---- one pass over 16-byte items {key, three payload words}: the sample stream of the pair table.  Same scheme as
// above; an item travels as one 128-bit load, one 128-bit shared-memory staging store and one 128-bit store, so even a
// run of two equal digits fills a whole 32-byte sector.  Digits are up to kSort16MaxBits wide (a 25-bit sort key takes
// three passes, not four); the look-back reads four earlier tiles per round trip.
constexpr int kSort16MaxBits = 9;
constexpr int kSort16Bins = 1 << kSort16MaxBits;  // look-back words per tile, counters per pass
constexpr int kSort16Threads = 512;               // threads per CTA of the sample sort
constexpr int kSort16Items = 8;                   // items per thread: tiles of kSort16Threads x kSort16Items samples
constexpr int kSort16CtasPerSm = 2;

// Digits of a sort over end_bit key bits in `passes` passes: as equal as possible, the wider ones first.
__host__ __device__ __forceinline__ void digit_layout(int end_bit, int passes, int pass, int* shift, int* bits) {
  const int base = end_bit / passes, rem = end_bit % passes;
  *bits = base + (pass < rem ? 1 : 0);
  *shift = pass * base + (pass < rem ? pass : rem);
}
__host__ __device__ __forceinline__ int sort_key_bits(uint64_t nk) {  // bits of the largest sample sort key, nk + nk * nk
  uint64_t v = nk + nk * nk;
  int b = 0;
  while (v) { ++b; v >>= 1; }
  return b;
}

constexpr int kMaxDest = 32;  // destinations of a partition pass (by_dest)

struct SortPass16Args {
  // by_dest != 0: the "digit" is the destination rank of the item = number of splitters <= (key >> split_shift)
  // by_dest == 2: the items of destination d go to dest[d] (this rank's place in rank d's receive buffer, peer memory for
  // d != own rank: plain stores over NVLink) instead of out + gbase[d]
  uint32_t by_dest;
  uint32_t n_split;
  uint32_t split_shift;
  uint32_t split[kMaxDest - 1];
  const uint4* in;
  uint4* out;
  const uint32_t* n_dev;
  uint32_t n;
  // the digit of this pass: shift / bits as given, or -- nk_dev != nullptr -- pass `pass` of `passes` over the bits of the
  // largest sort key of *nk_dev keys (the key count may still be in flight when the pass is queued)
  int shift;
  int bits;
  const uint32_t* nk_dev;
  int pass, passes;
  uint32_t key_base;       // the digits are those of key - key_base (a key range that starts at key_base sorts over fewer bits)
  int unstable;            // 1: equal digits may change their order inside a tile (the first pass of a sort)
  uint32_t spin_limit;     // polls before a look-back gives up; 0 = kSpinLimit
  const uint32_t* gbase;   // [kSort16Bins]
  uint32_t* lookback;      // [tiles][kSort16Bins], zeroed before the pass
  uint32_t* ticket;
  uint32_t* err;
  uint4* dest[kMaxDest];
};

__device__ __forceinline__ void pass_digit(const SortPass16Args& a, int* shift, int* bits) {
  *shift = a.shift;
  *bits = a.bits;
  if (a.nk_dev) {
    const int end_bit = min(sort_key_bits(*a.nk_dev), a.passes * kSort16MaxBits);  // beyond: the caller's guess failed, it reruns
    digit_layout(end_bit, a.passes, a.pass, shift, bits);
  }
}

__device__ __forceinline__ uint32_t digit16(const SortPass16Args& a, uint32_t key, int shift, uint32_t dmask) {
  if (!a.by_dest) return ((key - a.key_base) >> shift) & dmask;
  const uint32_t b = key >> a.split_shift;
  uint32_t d = 0;
  for (uint32_t i = 0; i < a.n_split; ++i) d += a.split[i] <= b;
  return d;
}

// lanes with this lane's digit among valid_lanes: one ballot per digit bit, `bits` of them (warp-uniform)
__device__ __forceinline__ uint32_t match_digit_n(uint32_t d, uint32_t valid_lanes, int bits) {
  uint32_t same = valid_lanes;
#pragma unroll
  for (int b = 0; b < kSort16MaxBits; ++b) {
    if (b < bits) {
      const bool bit = (d >> b) & 1u;
      const uint32_t vote = __ballot_sync(0xFFFFFFFFu, bit);
      same &= bit ? vote : ~vote;
    }
  }
  return same;
}

// histogram of the destination digit (multi-GPU partition): hist[kMaxDest]
__global__ void __launch_bounds__(256) k_dest_hist(const SortPass16Args a, uint32_t* __restrict__ hist) {
  __shared__ uint32_t sh[kMaxDest];
  if (threadIdx.x < kMaxDest) sh[threadIdx.x] = 0;
  __syncthreads();
  const uint32_t n = a.n_dev ? *a.n_dev : a.n;
  for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) atomicAdd(&sh[digit16(a, a.in[i].x, 0, 0xFFu)], 1u);
  __syncthreads();
  if (threadIdx.x < kMaxDest && sh[threadIdx.x]) atomicAdd(&hist[threadIdx.x], sh[threadIdx.x]);
}

// the digit counts of every pass in one read of the sort keys: hist[passes][kSort16Bins]
__global__ void __launch_bounds__(256) k_radix_hist16(const uint4* __restrict__ items, const uint32_t* n_dev, uint32_t n, int end_bit, int passes,
                                                      const uint32_t* nk_dev, uint32_t* __restrict__ hist, uint32_t key_base) {
  __shared__ uint32_t sh[4 * kSort16Bins];
  if (n_dev) n = min(*n_dev, n);
  if (nk_dev) end_bit = min(sort_key_bits(*nk_dev), passes * kSort16MaxBits);
  int shift[4], bits[4];
#pragma unroll
  for (int p = 0; p < 4; ++p) { shift[p] = 0; bits[p] = 0; if (p < passes) digit_layout(end_bit, passes, p, &shift[p], &bits[p]); }
  for (int i = threadIdx.x; i < passes * kSort16Bins; i += blockDim.x) sh[i] = 0;
  __syncthreads();
  const uint32_t gstride = gridDim.x * blockDim.x;
  for (uint32_t i0 = blockIdx.x * blockDim.x + threadIdx.x; i0 < n; i0 += 4 * gstride) {
    uint32_t k[4];
    bool valid[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const uint32_t i = i0 + u * gstride;
      valid[u] = i < n;
      k[u] = valid[u] ? items[i].x - key_base : 0u;
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      if (!valid[u]) continue;
#pragma unroll
      for (int p = 0; p < 4; ++p)
        if (p < passes) atomicAdd(&sh[p * kSort16Bins + ((k[u] >> shift[p]) & ((1u << bits[p]) - 1u))], 1u);
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < passes * kSort16Bins; i += blockDim.x)
    if (sh[i]) atomicAdd(&hist[i], sh[i]);
}

// exclusive scan of each pass's kSort16Bins counters (one CTA of kSort16Bins threads)
__global__ void __launch_bounds__(kSort16Bins) k_radix_scan_hist16(const uint32_t* __restrict__ hist, uint32_t* __restrict__ gbase, int passes) {
  __shared__ uint32_t warp_tot[kSort16Bins / 32];
  for (int p = 0; p < passes; ++p) {
    const uint32_t v = hist[p * kSort16Bins + threadIdx.x];
    const uint32_t inc = warp_incl_scan(v);
    if (lane_id() == 31) warp_tot[threadIdx.x >> 5] = inc;
    __syncthreads();
    uint32_t off = 0;
    for (uint32_t w = 0; w < (threadIdx.x >> 5); ++w) off += warp_tot[w];
    gbase[p * kSort16Bins + threadIdx.x] = off + inc - v;
    __syncthreads();
  }
}

template <int ITEMS, int THREADS>
__global__ void __launch_bounds__(THREADS, kSort16CtasPerSm) k_onesweep_pass16(const SortPass16Args a) {
  constexpr int TILE = THREADS * ITEMS;
  constexpr int WARPS = THREADS / 32;
  constexpr int SLOTS = (kSort16Bins + THREADS - 1) / THREADS;  // digits per thread
  extern __shared__ __align__(16) unsigned char smem_raw[];
  uint4* s_items = reinterpret_cast<uint4*>(smem_raw);                       // [TILE]
  uint32_t* warp_hist = reinterpret_cast<uint32_t*>(s_items + TILE);          // [warps][kSort16Bins]
  uint32_t* s_gpos = warp_hist + WARPS * kSort16Bins;                         // [kSort16Bins]
  uint32_t* s_misc = s_gpos + kSort16Bins;                                    // [2] ticket, [SLOTS][warps] scan totals
  uint32_t* s_acc = s_misc + 2 + SLOTS * WARPS + 14;                          // [kSort16Bins] the tile's count of every digit

  const uint32_t n = a.n_dev ? min(*a.n_dev, a.n) : a.n;  // with n_dev, a.n is the bound the buffers were sized for
  const uint32_t ntiles = (n + TILE - 1) / TILE;
  const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
  int shift, bits;
  pass_digit(a, &shift, &bits);
  const uint32_t dmask = (1u << bits) - 1u;
  const uint32_t nd = a.by_dest ? (uint32_t)kMaxDest : (1u << bits);  // digits in use

  while (true) {
    // A ticket is drawn only when its tile is started: a tile that is reserved ahead of time keeps every later tile waiting
    // in its look-back.
    if (tid == 0) s_misc[0] = atomicAdd(a.ticket, 1u);
    for (uint32_t i = tid; i < WARPS * kSort16Bins / 4; i += THREADS) reinterpret_cast<uint4*>(warp_hist)[i] = make_uint4(0, 0, 0, 0);
    __syncthreads();
    const uint32_t tile = s_misc[0];
    if (tile >= ntiles) break;
    const uint32_t tile_base = tile * TILE;
    const uint32_t tile_n = min((uint32_t)TILE, n - tile_base);

    uint4 item[ITEMS];
    uint32_t rank[ITEMS];
    const uint32_t wbase = warp * 32 * ITEMS;
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
      const uint32_t li = wbase + i * 32 + lane;
      item[i] = li < tile_n ? a.in[tile_base + li] : make_uint4(0, 0, 0, 0);
    }
    // The first pass of a sort has no earlier order to keep, so it may rank the items of a tile in any order: one
    // shared-memory atomic per item on the CTA's counters (row 0) instead of a ballot per digit bit and per-warp counters.
    uint32_t* wh = warp_hist + (a.unstable ? 0u : warp * kSort16Bins);
    if (a.unstable) {
#pragma unroll
      for (int i = 0; i < ITEMS; ++i) {
        const uint32_t li = wbase + i * 32 + lane;
        rank[i] = li < tile_n ? atomicAdd(&wh[digit16(a, item[i].x, shift, dmask)], 1u) : 0u;
      }
    } else {
#pragma unroll
      for (int i = 0; i < ITEMS; ++i) {
        const uint32_t li = wbase + i * 32 + lane;
        const bool valid = li < tile_n;
        const uint32_t d = digit16(a, item[i].x, shift, dmask);
        const uint32_t same = __match_any_sync(0xFFFFFFFFu, valid ? d : 0xFFFFFFFFu);  // the lanes with this lane's digit
        const uint32_t before = __popc(same & lanemask_lt());
        uint32_t pre = 0;
        if (valid) pre = wh[d];
        __syncwarp();
        if (valid && before == 0) wh[d] = pre + __popc(same);
        __syncwarp();
        rank[i] = pre + before;
      }
    }
    __syncthreads();
    {
      // ---- thread t owns digits t, t + THREADS, ...: the tile's count of the digit and the exclusive offsets of the warps;
      // the count is published for the tiles behind this one
      uint32_t acc[SLOTS], inc[SLOTS];
#pragma unroll
      for (int q = 0; q < SLOTS; ++q) {
        const uint32_t d = tid + q * THREADS;
        acc[q] = 0;
        if (d < nd) {
#pragma unroll
          for (int w = 0; w < WARPS; ++w) {
            const uint32_t t = warp_hist[w * kSort16Bins + d];
            warp_hist[w * kSort16Bins + d] = acc[q];
            acc[q] += t;
          }
          s_acc[d] = acc[q];
          *(volatile uint32_t*)(a.lookback + (size_t)tile * kSort16Bins + d) = acc[q] | (tile == 0 ? kFlagPrefix : kFlagAgg);
        }
        inc[q] = warp_incl_scan(acc[q]);
        if (lane == 31) s_misc[2 + q * WARPS + warp] = inc[q];
      }
      __syncthreads();
      // exclusive scan of the tile counts over the digits -> where each digit starts in the staging buffer
      uint32_t carry = 0;
#pragma unroll
      for (int q = 0; q < SLOTS; ++q) {
        const uint32_t d = tid + q * THREADS;
        uint32_t off2 = carry;
        for (uint32_t w = 0; w < WARPS; ++w) {
          const uint32_t t = s_misc[2 + q * WARPS + w];
          if (w < warp) off2 += t;
          carry += t;
        }
        if (d < nd) {
          const uint32_t dstart = off2 + inc[q] - acc[q];
          s_gpos[d] = (a.by_dest == 2 ? 0u : a.gbase[d]) - dstart;  // + the count in all earlier tiles, below
#pragma unroll
          for (int w = 0; w < WARPS; ++w) warp_hist[w * kSort16Bins + d] += dstart;
        }
      }
    }
    __syncthreads();
    // ---- the items go to the staging buffer in digit order (the registers that held them are free for the look-back)
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
      const uint32_t li = wbase + i * 32 + lane;
      if (li < tile_n) s_items[rank[i] + wh[digit16(a, item[i].x, shift, dmask)]] = item[i];
    }
    {
      // ---- the look-back, thread t for digits t, t + THREADS, ...: four earlier tiles per round trip, all of the thread's
      // digits in flight together
      uint32_t excl[SLOTS], left[SLOTS];  // left: tiles [0, left) are still to be added; 0 = done
      bool open = false;
#pragma unroll
      for (int q = 0; q < SLOTS; ++q) {
        excl[q] = 0;
        left[q] = (tid + q * THREADS < nd) ? tile : 0u;
        open = open || left[q] != 0;
      }
      uint32_t spins = 0;
      const uint32_t spin_limit = a.spin_limit ? a.spin_limit : kSpinLimit;
      while (open) {
        uint32_t v[SLOTS][4];
#pragma unroll
        for (int q = 0; q < SLOTS; ++q) {
          const uint32_t d = tid + q * THREADS;
#pragma unroll
          for (uint32_t u = 0; u < 4; ++u) v[q][u] = left[q] > u ? ld_volatile_u32(a.lookback + (size_t)(left[q] - 1 - u) * kSort16Bins + d) : kFlagPrefix;  // in front of tile 0: nothing
        }
        open = false;
        bool progress = false;
#pragma unroll
        for (int q = 0; q < SLOTS; ++q) {
          if (left[q] == 0) continue;
          uint32_t used = 0;
          bool done = false;
#pragma unroll
          for (uint32_t u = 0; u < 4; ++u) {
            if (done || used != u) continue;  // stop at the first word that is not there yet
            const uint32_t f = v[q][u] & kFlagMask;
            if (f == 0) continue;
            excl[q] += v[q][u] & kCountMask;
            used = u + 1;
            if (f == kFlagPrefix) done = true;
          }
          progress = progress || used != 0;
          left[q] = done ? 0u : left[q] - min(left[q], used);
          open = open || left[q] != 0;
        }
        if (open && !progress) {
          if (++spins > spin_limit) { atomicOr(a.err, kErrWait); break; }
          __nanosleep(20);
        }
      }
#pragma unroll
      for (int q = 0; q < SLOTS; ++q) {
        const uint32_t d = tid + q * THREADS;
        if (d < nd) {
          if (tile != 0) *(volatile uint32_t*)(a.lookback + (size_t)tile * kSort16Bins + d) = ((excl[q] + s_acc[d]) & kCountMask) | kFlagPrefix;
          s_gpos[d] += excl[q];
        }
      }
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
      const uint32_t si = i * THREADS + tid;
      if (si < tile_n) {
        const uint4 it = s_items[si];
        const uint32_t d = digit16(a, it.x, shift, dmask);
        uint4* o = a.by_dest == 2 ? a.dest[d] : a.out;
        o[s_gpos[d] + si] = it;
      }
    }
    __syncthreads();  // everyone is done with the ticket word, the counters and the staged items
  }
}

template <int ITEMS, int THREADS>
constexpr size_t sort16_smem_bytes() {
  return (size_t)THREADS * ITEMS * sizeof(uint4) + ((THREADS / 32) * kSort16Bins + 2 * kSort16Bins + 2 + ((kSort16Bins + THREADS - 1) / THREADS) * (THREADS / 32) + 14) * sizeof(uint32_t);
}

template <typename KeyT, typename ValT, int ITEMS>
constexpr size_t sort_smem_bytes() {
  return (kSortWarps * 256 + 256 + 16) * sizeof(uint32_t) + (size_t)kSortThreads * ITEMS * (sizeof(KeyT) + sizeof(ValT));
}

}  // namespace ks
