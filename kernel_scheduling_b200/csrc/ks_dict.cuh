// ks_dict.cuh -- turns the open-addressing key dictionary into dense key ids.
//
// The decode kernel leaves the distinct keys scattered over kDictSlots slots.  Here they are compacted, ranked by
// key value (kid = number of smaller keys, so kid order = key order and every later table comes out sorted without
// looking at the 64-bit keys again), and the solo launches are turned into the first entries of the sample stream.
#pragma once

#include "ks_common.cuh"

namespace ks {

struct DictArgs {
  const unsigned long long* dict_keys;  // [kDictSlots]
  unsigned long long* dkeys;            // [kMaxKeys + 1] compacted keys (arbitrary order)
  uint32_t* dslot;                      // [kMaxKeys + 1] their slots
  uint32_t* drank;                      // [kMaxKeys + 1] zeroed; rank of dkeys[i]
  uint32_t* kid_of_slot;                // [kDictSlots]
  uint32_t* slot_of_kid;                // [kMaxKeys + 1]
  unsigned long long* keys_sorted;      // [kMaxKeys + 1]
  Control* ctl;
};

__global__ void __launch_bounds__(256) k_dict_compact(const DictArgs a) {
  const uint32_t slot = blockIdx.x * blockDim.x + threadIdx.x;
  const unsigned long long k = slot < kDictSlots ? a.dict_keys[slot] : 0ull;
  const uint32_t ballot = __ballot_sync(0xFFFFFFFFu, k != 0ull);
  if (!ballot) return;
  uint32_t base = 0;
  const uint32_t first = __ffs(ballot) - 1;
  if (lane_id() == first) base = atomicAdd(&a.ctl->n_keys, (uint32_t)__popc(ballot));
  base = __shfl_sync(0xFFFFFFFFu, base, first);
  if (k != 0ull) {
    const uint32_t i = base + __popc(ballot & lanemask_lt());
    if (i < kMaxKeys) {
      a.dkeys[i] = k;
      a.dslot[i] = slot;
    } else {
      atomicOr(&a.ctl->err, kErrTooManyKeys);
    }
  }
}

// rank by counting: grid (ceil(kMaxKeys/256), kRankSplit); CTA (x, y) counts, for its 256 keys, the smaller keys among
// slice y of the list and adds the partial count.
constexpr int kRankSplit = 8;
__global__ void __launch_bounds__(256) k_dict_rank(const DictArgs a) {
  __shared__ unsigned long long tile[256];
  const uint32_t nk = min(a.ctl->n_keys, kMaxKeys);
  const uint32_t i = blockIdx.x * 256 + threadIdx.x;
  if (blockIdx.x * 256 >= nk) return;
  const unsigned long long mine = i < nk ? a.dkeys[i] : ~0ull;
  const uint32_t per = (nk + kRankSplit - 1) / kRankSplit;
  const uint32_t j0 = blockIdx.y * per, j1 = min(nk, j0 + per);
  uint32_t cnt = 0;
  for (uint32_t j = j0; j < j1; j += 256) {
    __syncthreads();
    tile[threadIdx.x] = (j + threadIdx.x < j1) ? a.dkeys[j + threadIdx.x] : ~0ull;
    __syncthreads();
    const uint32_t m = min(256u, j1 - j);
    for (uint32_t t = 0; t < m; ++t) cnt += tile[t] < mine;
  }
  if (i < nk && cnt) atomicAdd(&a.drank[i], cnt);
}

__global__ void __launch_bounds__(256) k_dict_place(const DictArgs a) {
  const uint32_t nk = min(a.ctl->n_keys, kMaxKeys);
  const uint32_t i = blockIdx.x * 256 + threadIdx.x;
  if (i >= nk) return;
  const uint32_t r = a.drank[i], slot = a.dslot[i];
  a.kid_of_slot[slot] = r;
  a.slot_of_kid[r] = slot;
  a.keys_sorted[r] = a.dkeys[i];
}

// The solo launches become samples [0, n_solo) of the sample stream: sort key = kid, lane 0 = duration.
// Also starts the pair counter behind them.
struct SoloArgs {
  const unsigned long long* solo_stream;
  const uint32_t* kid_of_slot;
  uint4* samples;  // {sort key, lane 0, lane 1, lane 2}
  uint64_t capacity;
  Control* ctl;
};
__global__ void __launch_bounds__(256) k_solo_samples(const SoloArgs a) {
  const uint32_t ns = a.ctl->n_solo;
  if (blockIdx.x == 0 && threadIdx.x == 0) a.ctl->n_pairs = ns;  // pairs are appended behind the solo samples
  for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < ns && i < a.capacity; i += gridDim.x * blockDim.x) {
    const unsigned long long e = a.solo_stream[i];
    a.samples[i] = make_uint4(a.kid_of_slot[(uint32_t)e & kMetaSlotMask], (uint32_t)(e >> 32), 0u, 0u);
  }
}

}  // namespace ks
