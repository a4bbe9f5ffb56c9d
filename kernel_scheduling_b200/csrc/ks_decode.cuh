// ks_decode.cuh -- K1: record decode, kernel-key hash and key dictionary in one read of the trace.
//
// A CTA streams tiles of 512 records (24,576 contiguous bytes) into shared memory with bulk asynchronous copies
// (cp.async.bulk, completion on an mbarrier, two tiles in flight), so global memory is read as whole 128-byte
// lines although a record is 48 bytes; each thread then takes its record from shared memory as three 128-bit
// loads (a 48-byte stride is conflict-free for 128-bit shared loads).  Per record it
//   * computes the 64-bit kernel key (ks_common.cuh kernel_key),
//   * finds the key's slot in the open-addressing dictionary (2^18 slots, 2 MB: the probes are L2 hits),
//   * writes the compact timeline entry  start_ns (u64) | duration (u32) | meta (u32: slot, solo, tenant),
//   * appends solo launches to the solo stream (slot | duration << 32) with one warp-aggregated counter update,
//   * checks the record (end >= start, duration < 2^31 ns so that a pair's span fits 32 bits) and whether start_ns is non-decreasing.
// Per-key launch counts are accumulated in a small per-CTA shared-memory table and flushed once, so hot keys do
// not turn into a queue of same-address global atomics.
#pragma once

#include "ks_common.cuh"

namespace ks {

constexpr int kDecodeThreads = 256;
constexpr int kDecodeStages = 2;
constexpr int kDecodePerThread = 2;  // two records per thread: two dictionary probes in flight
constexpr int kDecodeTile = kDecodeThreads * kDecodePerThread;
constexpr int kDecodeTileBytes = kDecodeTile * 48;
constexpr int kCtaCountBits = 10;
constexpr int kDecodeCtasPerSm = 3;  // 61 KB of shared memory per CTA; four CTAs with a 512-slot count cache measured the same
constexpr uint32_t kCountFlushTiles = 32;       // the count cache is flushed and emptied every so many tiles of a CTA
constexpr uint32_t kCtaCountSlots = 1u << kCtaCountBits;  // per-CTA launch-count cache (open addressing on the dictionary slot)

struct DecodeArgs {
  const unsigned char* records;
  uint64_t n;
  int type_mode;
  // dictionary
  unsigned long long* dict_keys;  // [kDictSlots], 0 = empty
  uint4* dict_words;              // [kDictSlots][2] the launch fields behind a key (written by the inserting thread)
  uint32_t* dict_launches;        // [kDictSlots]
  uint32_t* dict_solo;            // [kDictSlots]
  // outputs
  unsigned long long* tl_start;   // [n]
  unsigned long long* tl_dm;      // [n] duration | meta << 32
  unsigned long long* solo_stream;  // [n] slot | duration << 32, first Control::n_solo entries valid
  unsigned long long* keys_out;   // optional [n]: the key of every record
  int halo;                       // 1: records of a neighbouring time window -- keyed and placed on the timeline, but not counted
  Control* ctl;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst)), "l"(src),
               "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait; false if the copy never arrived.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity) {
  for (uint32_t spins = 0; spins < kSpinLimit; ++spins) {
    if (mbar_try_wait(bar, parity)) return true;
  }
  return false;
}

// Dictionary lookup / insert of one key; returns the slot, or kDictSlots if the table is full.
__device__ __forceinline__ uint32_t dict_find_or_insert(unsigned long long* dict_keys, uint64_t key, bool* inserted) {
  uint32_t slot = dict_home(key);
  *inserted = false;
  for (uint32_t probe = 0; probe < kDictSlots; ++probe) {
    const uint64_t cur = ld_volatile_u64(reinterpret_cast<const uint64_t*>(dict_keys + slot));
    if (cur == key) return slot;
    if (cur == 0) {
      const unsigned long long old = atomicCAS(dict_keys + slot, 0ull, (unsigned long long)key);
      if (old == 0ull) { *inserted = true; return slot; }
      if (old == key) return slot;
    }
    slot = (slot + 1) & (kDictSlots - 1);
  }
  return kDictSlots;
}

__global__ void __launch_bounds__(kDecodeThreads, kDecodeCtasPerSm) k_decode_hash(const DecodeArgs a) {
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* tiles = smem;                                                           // [stages][tile bytes]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kDecodeStages * kDecodeTileBytes);  // [stages]
  uint32_t* cc_slot = reinterpret_cast<uint32_t*>(bars + kDecodeStages + 1);              // [kCtaCountSlots] dictionary slot + 1
  uint32_t* cc_cnt = cc_slot + kCtaCountSlots;                                             // launches
  uint32_t* cc_solo = cc_cnt + kCtaCountSlots;                                             // solo launches

  const uint32_t tid = threadIdx.x, lane = tid & 31u;
  const uint64_t ntiles = (a.n + kDecodeTile - 1) / kDecodeTile;
  for (uint32_t i = tid; i < kCtaCountSlots; i += kDecodeThreads) { cc_slot[i] = 0; cc_cnt[i] = 0; cc_solo[i] = 0; }
  if (tid == 0) {
    for (int s = 0; s < kDecodeStages; ++s) mbar_init(&bars[s], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncthreads();

  auto issue = [&](uint64_t tile, int stage) {
    const uint64_t first = tile * kDecodeTile;
    const uint32_t cnt = (uint32_t)min((uint64_t)kDecodeTile, a.n - first);
    const uint32_t bytes = cnt * 48u;
    mbar_expect_tx(&bars[stage], bytes);
    bulk_load(tiles + stage * kDecodeTileBytes, a.records + first * 48ull, bytes, &bars[stage]);
  };
  // prologue: fill the pipeline
  if (tid == 0) {
    for (int s = 0; s < kDecodeStages; ++s) {
      const uint64_t t = blockIdx.x + (uint64_t)s * gridDim.x;
      if (t < ntiles) issue(t, s);
    }
  }

  uint32_t err = 0, max_dur = 0;
  uint32_t it = 0;
  for (uint64_t tile = blockIdx.x; tile < ntiles; tile += gridDim.x, ++it) {
    const int stage = it % kDecodeStages;
    const uint32_t parity = (it / kDecodeStages) & 1u;
    if (!mbar_wait_bounded(&bars[stage], parity)) err |= kErrWait;  // carry on: the CTA still terminates

    // ---- phase 1, both records of the thread: fields, key, and the first dictionary probe of each is put in flight
    uint4 w0[kDecodePerThread], w1[kDecodePerThread];
    unsigned long long start[kDecodePerThread], end[kDecodePerThread], prev[kDecodePerThread], key[kDecodePerThread], seen[kDecodePerThread];
    uint64_t r[kDecodePerThread];
    bool valid[kDecodePerThread];
#pragma unroll
    for (int u = 0; u < kDecodePerThread; ++u) {
      const uint32_t li = u * kDecodeThreads + tid;  // consecutive lanes, consecutive records
      r[u] = tile * kDecodeTile + li;
      valid[u] = r[u] < a.n;
      const unsigned char* rp = tiles + stage * kDecodeTileBytes + li * 48;
      uint4 w2 = make_uint4(0, 0, 0, 0);
      w0[u] = w2; w1[u] = w2;
      prev[u] = 0;
      if (valid[u]) {
        w0[u] = *reinterpret_cast<const uint4*>(rp);
        w1[u] = *reinterpret_cast<const uint4*>(rp + 16);
        w2 = *reinterpret_cast<const uint4*>(rp + 32);
        if (li > 0) prev[u] = *reinterpret_cast<const unsigned long long*>(rp - 48 + 32);
        else if (r[u] > 0) prev[u] = *reinterpret_cast<const unsigned long long*>(a.records + (r[u] - 1) * 48ull + 32);
      }
      start[u] = (unsigned long long)w2.x | ((unsigned long long)w2.y << 32);
      end[u] = (unsigned long long)w2.z | ((unsigned long long)w2.w << 32);
      key[u] = kernel_key(w0[u].x, w0[u].y, w0[u].z, w0[u].w, w1[u].x, w1[u].y, w1[u].z, w1[u].w, a.type_mode != 0);
      seen[u] = valid[u] ? ld_volatile_u64(reinterpret_cast<const uint64_t*>(a.dict_keys + dict_home(key[u]))) : 0ull;
    }

    // ---- phase 2: finish the lookups (keys of a warp are mostly distinct, so every lane probes for itself; the
    // dictionary is 2 MB and lives in L2), count, write
#pragma unroll
    for (int u = 0; u < kDecodePerThread; ++u) {
      const bool solo = (w1[u].w & kMetaSoloBit) != 0;
      const uint32_t solo_ballot = __ballot_sync(0xFFFFFFFFu, valid[u] && solo && !a.halo);
      uint32_t slot = 0;
      if (valid[u]) {
        bool inserted = false;
        slot = dict_home(key[u]);
        if (seen[u] != key[u]) slot = dict_find_or_insert(a.dict_keys, key[u], &inserted);
        if (slot >= kDictSlots) { err |= kErrTooManyKeys; slot = 0; inserted = false; }
        if (inserted) {
          uint4 k0 = w0[u], k1 = w1[u];
          k1.w &= ~kMetaSoloBit;
          if (a.type_mode) { k0.y = k0.z = k0.w = 0; k1.w &= 0xFF000000u; }
          a.dict_words[2 * (size_t)slot] = k0;
          a.dict_words[2 * (size_t)slot + 1] = k1;
        }
        if (!a.halo) {
          // launch counts: CTA-local cache first (a plain load finds the key's entry once it exists), global atomics
          // when the cache is crowded
          uint32_t h = (slot * 2654435761u) >> (32 - kCtaCountBits);
          bool cached = false;
          for (int probe = 0; probe < 8; ++probe) {
            uint32_t cur = cc_slot[h];
            if (cur == 0u) cur = atomicCAS(&cc_slot[h], 0u, slot + 1);
            if (cur == 0u || cur == slot + 1) {
              atomicAdd(&cc_cnt[h], 1u);
              if (solo) atomicAdd(&cc_solo[h], 1u);
              cached = true;
              break;
            }
            h = (h + 1) & (kCtaCountSlots - 1);
          }
          if (!cached) {
            atomicAdd(&a.dict_launches[slot], 1u);
            if (solo) atomicAdd(&a.dict_solo[slot], 1u);
          }
        }
        if (end[u] < start[u] || end[u] - start[u] >= 0x80000000ull) err |= kErrRecord;
        if (start[u] < prev[u] && !(a.halo && r[u] == 0)) err |= kErrUnordered;
        const uint32_t dur = (uint32_t)(end[u] - start[u]);
        const uint32_t meta = slot | (w1[u].w & (kMetaSoloBit | 0xFF000000u));
        a.tl_start[r[u]] = start[u];
        a.tl_dm[r[u]] = (unsigned long long)dur | ((unsigned long long)meta << 32);
        if (a.keys_out) a.keys_out[r[u]] = key[u];
        max_dur = max(max_dur, dur);
        // Control::min_start / max_start: of an ordered trace they are the first and the last start.  An unordered one
        // gets them from a pass of its own (the host runs it when the order flag comes back set).
        if (r[u] == 0) atomicMin(&a.ctl->min_start, start[u]);
        if (r[u] == a.n - 1) atomicMax(&a.ctl->max_start, start[u]);
      }
      // solo stream: one counter update per warp
      if (solo_ballot) {
        uint32_t base = 0;
        const uint32_t first = __ffs(solo_ballot) - 1;
        if (lane == first) base = atomicAdd(&a.ctl->n_solo, (uint32_t)__popc(solo_ballot));
        base = __shfl_sync(0xFFFFFFFFu, base, first);
        if (valid[u] && solo) {
          const uint32_t dur = (uint32_t)(end[u] - start[u]);
          a.solo_stream[base + __popc(solo_ballot & lanemask_lt())] = (unsigned long long)slot | ((unsigned long long)dur << 32);
        }
      }
    }

    __syncthreads();  // everyone is done with this stage's tile
    if (tid == 0) {
      const uint64_t next = tile + (uint64_t)kDecodeStages * gridDim.x;
      if (next < ntiles) issue(next, stage);
    }
    // The count cache takes keys first come, first served.  A trace whose key mix changes (one tenant's solo run, then
    // another's, then all of them together) would leave it full of keys that no longer occur, and the hottest keys of the
    // later mix would all go to the same few global counters.  So it is emptied every kCountFlushTiles tiles and refills
    // with the keys of the stretch at hand, the frequent ones first.
    if ((it + 1) % kCountFlushTiles == 0) {
      for (uint32_t i = tid; i < kCtaCountSlots; i += kDecodeThreads) {
        const uint32_t s = cc_slot[i];
        if (s) {
          atomicAdd(&a.dict_launches[s - 1], cc_cnt[i]);
          if (cc_solo[i]) atomicAdd(&a.dict_solo[s - 1], cc_solo[i]);
          cc_slot[i] = 0; cc_cnt[i] = 0; cc_solo[i] = 0;
        }
      }
      __syncthreads();
    }
  }

  // flush per-thread reductions and the CTA's launch counts
  err = __reduce_or_sync(0xFFFFFFFFu, err);
  max_dur = warp_max(max_dur);
  if (lane == 0) {
    if (err) atomicOr(&a.ctl->err, err);
    if (max_dur) atomicMax(&a.ctl->max_dur, max_dur);
  }
  __syncthreads();
  for (uint32_t i = tid; i < kCtaCountSlots; i += kDecodeThreads) {
    const uint32_t s = cc_slot[i];
    if (s) {
      atomicAdd(&a.dict_launches[s - 1], cc_cnt[i]);
      if (cc_solo[i]) atomicAdd(&a.dict_solo[s - 1], cc_solo[i]);
    }
  }
}

constexpr size_t decode_smem_bytes() { return kDecodeStages * kDecodeTileBytes + (kDecodeStages + 1) * 8 + 3 * kCtaCountSlots * 4; }

}  // namespace ks
