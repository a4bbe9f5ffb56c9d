// ks_common.cuh -- layouts, the key hash and small device helpers shared by every stage.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/ks_b200.h"

namespace ks {

// ---------------------------------------------------------------------------------------------------------
// Sizes fixed at compile time
// ---------------------------------------------------------------------------------------------------------
constexpr uint32_t kDictSlots = 1u << 18;      // open-addressing slots of the key dictionary (load <= 25 %)
constexpr uint32_t kMaxKeys = 65535;           // dense key ids are 16 bits; pair id = kid_a * n_keys + kid_b < 2^32
constexpr uint32_t kEmptyPair = 0xFFFFFFFFu;   // empty slot of the pair dictionary
constexpr uint32_t kSpinLimit = 1u << 22;      // iteration bound of every device-side wait
constexpr uint32_t kSmallSegment = 32;         // segments up to this size are reduced by one warp

constexpr uint32_t kMetaSlotMask = 0x003FFFFFu;  // meta word of a timeline entry: bits 0..21 dictionary slot,
constexpr uint32_t kMetaSoloBit = 1u << 23;      // bit 23 solo, bits 24..31 tenant (same places as smem_word)
constexpr uint32_t kSmemMask = 0x007FFFFFu;

// Error bits set by kernels in Control::err
enum : uint32_t {
  kErrRecord = 1u << 0,      // end < start or duration >= 2^31 ns
  kErrUnordered = 1u << 1,   // start_ns decreases somewhere (information unless the caller asserted order)
  kErrTooManyKeys = 1u << 2,
  kErrPairTableFull = 1u << 3,
  kErrWait = 1u << 4,
  kErrDuplicate = 1u << 5,
  kErrTooLarge = 1u << 6,
};

// Counters and flags of one run, in device memory; copied to pinned host memory at the sync points.
struct Control {
  uint32_t err;
  uint32_t n_keys;
  uint32_t n_solo;       // solo launches appended by the decode kernel
  uint32_t n_rows;       // distinct key pairs
  uint32_t n_big;        // segments handed to the CTA-per-segment kernel
  uint32_t max_dur;
  uint32_t ticket;       // work counters for persistent kernels
  uint32_t ticket2;
  unsigned long long n_pairs;
  unsigned long long min_start;
  unsigned long long max_start;
  unsigned long long scratch0;
  unsigned long long batches_both;  // ks_count_batches
  unsigned long long pad[4];         // large-row selection: unresolved states per round
  uint32_t n_small;      // rows handed to the warp-per-row kernel
  uint32_t pad32;
  unsigned long long pad2[2];
};

// ---------------------------------------------------------------------------------------------------------
// Key hash.  splitmix64's output function chained over four 64-bit lanes of the launch fields.
// ---------------------------------------------------------------------------------------------------------
__host__ __device__ __forceinline__ uint64_t mix64(uint64_t x) {
  x ^= x >> 30;
  x *= 0xBF58476D1CE4E5B9ull;
  x ^= x >> 27;
  x *= 0x94D049BB133111EBull;
  x ^= x >> 31;
  return x;
}

// w[0..7] = the first eight 32-bit words of a record.  type_mode drops grid and dynamic smem from the key.
__host__ __device__ __forceinline__ uint64_t kernel_key(uint32_t name, uint32_t gx, uint32_t gy, uint32_t gz, uint32_t bx, uint32_t by,
                                                        uint32_t bz, uint32_t smem_word, bool type_mode) {
  uint32_t w = smem_word & ~kMetaSoloBit;
  if (type_mode) { gx = gy = gz = 0; w &= 0xFF000000u; }
  const uint64_t G = 0x9E3779B97F4A7C15ull;
  const uint64_t q0 = (uint64_t)name | ((uint64_t)gx << 32);
  const uint64_t q1 = (uint64_t)gy | ((uint64_t)gz << 32);
  const uint64_t q2 = (uint64_t)bx | ((uint64_t)by << 32);
  const uint64_t q3 = (uint64_t)bz | ((uint64_t)w << 32);
  uint64_t h = mix64(q0 + G);
  h = mix64((h ^ q1) + G);
  h = mix64((h ^ q2) + G);
  h = mix64((h ^ q3) + G);
  return h ? h : 1ull;
}

__host__ __device__ __forceinline__ uint32_t dict_home(uint64_t key) { return (uint32_t)((key * 0x9E3779B97F4A7C15ull) >> (64 - 18)); }
__host__ __device__ __forceinline__ uint32_t pair_home(uint32_t pair, uint32_t log2_slots) {
  return (uint32_t)(((uint64_t)pair * 0x9E3779B97F4A7C15ull) >> (64 - log2_slots));
}

// ---------------------------------------------------------------------------------------------------------
// Small device helpers
// ---------------------------------------------------------------------------------------------------------
#ifdef __CUDACC__
__device__ __forceinline__ uint32_t lane_id() { return threadIdx.x & 31u; }
__device__ __forceinline__ uint32_t lanemask_lt() {
  uint32_t m;
  asm("mov.u32 %0, %%lanemask_lt;" : "=r"(m));
  return m;
}
__device__ __forceinline__ uint32_t ld_volatile_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ uint64_t ld_volatile_u64(const uint64_t* p) {
  uint64_t v;
  asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ uint32_t warp_sum(uint32_t v) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
  return v;
}
__device__ __forceinline__ uint32_t warp_max(uint32_t v) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v = max(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
  return v;
}
__device__ __forceinline__ uint32_t warp_min(uint32_t v) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v = min(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
  return v;
}
__device__ __forceinline__ unsigned long long warp_sum64(unsigned long long v) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
  return v;
}
__device__ __forceinline__ uint32_t warp_incl_scan(uint32_t v) {
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    uint32_t t = __shfl_up_sync(0xFFFFFFFFu, v, o);
    if (lane_id() >= (uint32_t)o) v += t;
  }
  return v;
}
#endif

}  // namespace ks
