// ks_misc.cuh -- the two computations the reference's Python scripts do implement, as kernels.
//
//  * batch counter of scheduler/postprocess.py:17-41: after both files' start_ns are sorted, duplicates inside a
//    file are adjacent (the reference's asserts), and a start_ns of file 1 that also occurs in file 2 is a pair.
//  * combine_duplicates of postprocess/profile_postprocess.py:5-27: rows sorted by group (stable), then one thread
//    per (group, column) adds value * launches and launches over the non-NaN cells in row order with the same
//    compensated (Kahan) accumulation pandas' group sum uses, and divides.
#pragma once

#include "ks_common.cuh"

namespace ks {

// min / max of a u64 array into Control::min_start / max_start (preset to ~0 / 0)
__global__ void __launch_bounds__(256) k_minmax_u64(const unsigned long long* __restrict__ v, uint64_t n, Control* ctl) {
  unsigned long long mn = ~0ull, mx = 0ull;
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
    const unsigned long long x = v[i];
    mn = min(mn, x);
    mx = max(mx, x);
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) {
    mn = min(mn, __shfl_xor_sync(0xFFFFFFFFu, mn, o));
    mx = max(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
  }
  if (lane_id() == 0 && mn != ~0ull) {
    atomicMin(&ctl->min_start, mn);
    atomicMax(&ctl->max_start, mx);
  }
}

// s1, s2 sorted.  Flags duplicates inside either array; counts the s1 values present in s2.
__global__ void __launch_bounds__(256) k_count_batches(const unsigned long long* __restrict__ s1, uint64_t n1, const unsigned long long* __restrict__ s2,
                                                       uint64_t n2, Control* ctl) {
  unsigned long long both = 0;
  bool dup = false;
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n1 || i < n2; i += stride) {
    if (i < n2 && i > 0 && s2[i] == s2[i - 1]) dup = true;
    if (i < n1) {
      const unsigned long long x = s1[i];
      if (i > 0 && x == s1[i - 1]) dup = true;
      uint64_t lo = 0, hi = n2;  // first position with s2 >= x
      while (lo < hi) {
        const uint64_t mid = (lo + hi) >> 1;
        if (s2[mid] < x) lo = mid + 1; else hi = mid;
      }
      if (lo < n2 && s2[lo] == x) ++both;
    }
  }
  both = warp_sum64(both);
  if (lane_id() == 0 && both) atomicAdd(&ctl->batches_both, both);
  if (dup) atomicOr(&ctl->err, kErrDuplicate);
}

// order[] = row indices sorted by group (stable); seg[g] .. seg[g+1] = the rows of group g in order[].
__global__ void __launch_bounds__(256) k_group_offsets(const uint32_t* __restrict__ sorted_group, uint32_t rows, uint32_t n_groups, uint32_t* __restrict__ seg) {
  const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i > rows) return;
  // seg[g] = first position whose group is >= g
  const uint32_t g_here = i < rows ? sorted_group[i] : n_groups;
  const uint32_t g_prev = i > 0 ? sorted_group[i - 1] + 1 : 0;
  for (uint32_t g = g_prev; g <= g_here && g <= n_groups; ++g) seg[g] = i;
}

__global__ void __launch_bounds__(256) k_combine_duplicates(const uint32_t* __restrict__ order, const uint32_t* __restrict__ seg, const double* __restrict__ launches,
                                                            const double* __restrict__ values, uint32_t cols, uint32_t n_groups, double* __restrict__ out_total,
                                                            double* __restrict__ out_means) {
  const uint64_t t = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= (uint64_t)n_groups * (cols + 1)) return;
  const uint32_t g = (uint32_t)(t / (cols + 1)), c = (uint32_t)(t % (cols + 1));
  const uint32_t r0 = seg[g], r1 = seg[g + 1];
  if (c == cols) {  // the group's total launches (profile_postprocess.py:25): plain sum over every row
    double s = 0.0, comp = 0.0;
    for (uint32_t r = r0; r < r1; ++r) {
      const double y = launches[order[r]] - comp;
      const double tt = s + y;
      comp = (tt - s) - y;
      s = tt;
    }
    out_total[g] = s;
    return;
  }
  double ws = 0.0, wc = 0.0, wt = 0.0, tc = 0.0;
  bool any = false;
  for (uint32_t r = r0; r < r1; ++r) {
    const uint32_t row = order[r];
    const double v = values[(uint64_t)row * cols + c];
    if (v != v) continue;  // NaN cell: left out of numerator and weight (:10-22)
    any = true;
    const double w = launches[row];
    double y = v * w - wc;
    double tt = ws + y;
    wc = (tt - ws) - y;
    ws = tt;
    y = w - tc;
    tt = wt + y;
    tc = (tt - wt) - y;
    wt = tt;
  }
  out_means[(uint64_t)g * cols + c] = any ? ws / wt : __longlong_as_double(0x7FF8000000000000ll);
}

// Pooling of per-launch profiler metrics (profiling/ncu-bench/ncu_summary.py:185-245): per group and column the mean and
// the SAMPLE standard deviation (n - 1; 0 for a single value) over the cells that hold a value (NaN = the launch has no
// such metric), and the number of launches of the group.  One thread per (group, column); two passes (mean, then
// squared deviations from it), both compensated.
__global__ void __launch_bounds__(256) k_pool_launches(const uint32_t* __restrict__ order, const uint32_t* __restrict__ seg, const double* __restrict__ values,
                                                       uint32_t cols, uint32_t n_groups, unsigned long long* __restrict__ out_launches,
                                                       double* __restrict__ out_mean, double* __restrict__ out_std) {
  const uint64_t t = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= (uint64_t)n_groups * (cols + 1)) return;
  const uint32_t g = (uint32_t)(t / (cols + 1)), c = (uint32_t)(t % (cols + 1));
  const uint32_t r0 = seg[g], r1 = seg[g + 1];
  if (c == cols) { out_launches[g] = r1 - r0; return; }
  const double nan = __longlong_as_double(0x7FF8000000000000ll);
  double s = 0.0, comp = 0.0;
  uint32_t n = 0;
  for (uint32_t r = r0; r < r1; ++r) {
    const double v = values[(uint64_t)order[r] * cols + c];
    if (v != v) continue;
    ++n;
    const double y = v - comp, tt = s + y;
    comp = (tt - s) - y;
    s = tt;
  }
  if (n == 0) { out_mean[(uint64_t)g * cols + c] = nan; out_std[(uint64_t)g * cols + c] = nan; return; }
  const double mean = s / (double)n;
  double ss = 0.0, d1 = 0.0;
  comp = 0.0;
  for (uint32_t r = r0; r < r1; ++r) {
    const double v = values[(uint64_t)order[r] * cols + c];
    if (v != v) continue;
    const double d = v - mean;
    d1 += d;  // the residual of the rounded mean, for the correction below
    const double y = d * d - comp, tt = ss + y;
    comp = (tt - ss) - y;
    ss = tt;
  }
  ss -= d1 * d1 / (double)n;
  out_mean[(uint64_t)g * cols + c] = mean;
  out_std[(uint64_t)g * cols + c] = n > 1 ? sqrt(fmax(ss, 0.0) / (double)(n - 1)) : 0.0;
}

__global__ void __launch_bounds__(256) k_iota(uint32_t* v, uint32_t n) {
  const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) v[i] = i;
}

__global__ void __launch_bounds__(256) k_offsets_to_u32(const unsigned long long* off, uint32_t n, uint32_t* out) {
  const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = (uint32_t)off[i];
}

}  // namespace ks
