// ks_synth.cpp -- seeded synthetic launch traces with the shapes of the benchmark configurations, written on the
// host's cores straight into the caller's (pinned) record buffer.  Host code only; no counterpart in the reference,
// whose traces come from live model servers (scheduler/agent.cpp:643-709).
//
// The workload model is the one of kernel_scheduling_b200/trace.py: every tenant is one process with at most one launch
// in flight; per launch a key drawn from the tenant's Zipf table, a duration = the key's typical duration x lognormal
// jitter (x 1 + |N(0, s)| when co-running), an exponential idle gap in front; solo launches run one at a time in a phase
// of their own before the co-run phase.  Every random number is a pure function of (seed, tenant, launch index), so the
// trace does not depend on the number of threads, and any stretch of it can be regenerated without the rest.
#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

#include "../../include/ks_b200.h"

namespace {

inline uint64_t smix(uint64_t x) {
  x ^= x >> 30;
  x *= 0xBF58476D1CE4E5B9ull;
  x ^= x >> 27;
  x *= 0x94D049BB133111EBull;
  x ^= x >> 31;
  return x;
}
// j-th uniform in (0, 1) of launch i of tenant t
struct LaunchRng {
  uint64_t base;
  LaunchRng(uint64_t seed, uint32_t tenant, uint64_t i) : base(smix(seed ^ smix(((uint64_t)tenant << 56) ^ (i + 0x9E3779B97F4A7C15ull)))) {}
  double uniform(uint32_t j) const { return ((double)(smix(base + (uint64_t)(j + 1) * 0xD1B54A32D192ED03ull) >> 11) + 0.5) * (1.0 / 9007199254740992.0); }
};

struct Launch {
  uint32_t key;
  uint32_t dur;
  bool solo;
  uint64_t gap;
};

struct Model {
  double solo_fraction, jitter_sigma, corun_slowdown;
  uint64_t seed;
  bool interleave;  // solo launches take their turn on their tenant's timeline instead of a phase of their own
};

inline Launch make_launch(const ks_synth_tenant& T, const Model& m, uint64_t i) {
  const LaunchRng r(m.seed, T.tenant, i);
  Launch L;
  const double* c = T.cdf;
  L.key = (uint32_t)std::min<size_t>((size_t)(std::lower_bound(c, c + T.n_keys, r.uniform(0)) - c), T.n_keys - 1);
  L.solo = r.uniform(1) < m.solo_fraction;
  const double rad = std::sqrt(-2.0 * std::log(r.uniform(2))), ang = 6.283185307179586 * r.uniform(3);
  const double z1 = rad * std::cos(ang), z2 = rad * std::sin(ang);
  double d = T.dur_ns[L.key] * std::exp(m.jitter_sigma * z1);
  if (!L.solo) d *= 1.0 + std::fabs(m.corun_slowdown * z2);
  d = std::nearbyint(d);
  L.dur = (uint32_t)std::min(std::max(d, 200.0), 2147483647.0);
  L.gap = (uint64_t)std::nearbyint(-T.gap_mean_ns * std::log(r.uniform(4))) + 1;
  return L;
}

template <typename F>
void parallel_for(uint64_t n, unsigned threads, F&& fn) {
  if (threads <= 1 || n <= 1) {
    for (uint64_t i = 0; i < n; ++i) fn(i);
    return;
  }
  std::atomic<uint64_t> next{0};
  std::vector<std::thread> pool;
  for (unsigned t = 0; t < std::min<uint64_t>(threads, n); ++t)
    pool.emplace_back([&] {
      for (uint64_t i; (i = next.fetch_add(1)) < n;) fn(i);
    });
  for (auto& th : pool) th.join();
}

struct CoLaunch {
  uint64_t start;
  uint32_t key, dur;  // bit 31 of key: a solo launch (interleaved traces only)
};

inline void write_record(ks_record* o, const ks_synth_tenant& T, uint32_t key, bool solo, uint64_t start, uint32_t dur) {
  o->name_id = T.name_id[key];
  for (int d = 0; d < 3; ++d) { o->grid[d] = T.grid[3 * key + d]; o->block[d] = T.block[3 * key + d]; }
  o->smem_word = (T.smem[key] & 0x007FFFFFu) | (solo ? 0x00800000u : 0u) | (T.tenant << 24);
  o->start_ns = start;
  o->end_ns = start + dur;
}

constexpr uint64_t kChunk = 1u << 18;

}  // namespace

extern "C" int64_t ks_synth_trace(const ks_synth_tenant* tenants, uint32_t n_tenants, double solo_fraction, double jitter_sigma, double corun_slowdown,
                                  uint64_t seed, uint64_t t0_ns, ks_record* out, uint64_t capacity, uint32_t threads, uint32_t flags) {
  if (!tenants || !n_tenants || n_tenants > 256 || (!out && capacity)) return -KS_ERR_ARG;
  uint64_t total = 0;
  for (uint32_t t = 0; t < n_tenants; ++t) {
    const ks_synth_tenant& T = tenants[t];
    if (!T.n_keys || !T.name_id || !T.grid || !T.block || !T.smem || !T.dur_ns || !T.cdf || T.tenant > 255 || !(T.gap_mean_ns >= 0.0)) return -KS_ERR_ARG;
    total += T.n_launches;
  }
  if (total > capacity) return -KS_ERR_CAPACITY;
  if (!threads) threads = std::max(1u, std::thread::hardware_concurrency());
  if (flags & ~KS_SYNTH_INTERLEAVE_SOLO) return -KS_ERR_ARG;
  const Model m{solo_fraction, jitter_sigma, corun_slowdown, seed, (flags & KS_SYNTH_INTERLEAVE_SOLO) != 0};

  // ---- pass A: per chunk of every tenant, the number of solo launches, their time, the co-run launches and their steps
  struct Chunk {
    uint32_t tenant;
    uint64_t first, count;
    uint64_t n_solo = 0, solo_time = 0, n_co = 0, co_step = 0;  // sums over the chunk, then exclusive prefixes
  };
  std::vector<Chunk> chunks;
  for (uint32_t t = 0; t < n_tenants; ++t)
    for (uint64_t f = 0; f < tenants[t].n_launches; f += kChunk) {
      Chunk c;
      c.tenant = t;
      c.first = f;
      c.count = std::min<uint64_t>(kChunk, tenants[t].n_launches - f);
      chunks.push_back(c);
    }
  parallel_for(chunks.size(), threads, [&](uint64_t ci) {
    Chunk& c = chunks[ci];
    const ks_synth_tenant& T = tenants[c.tenant];
    for (uint64_t i = c.first; i < c.first + c.count; ++i) {
      const Launch L = make_launch(T, m, i);
      if (L.solo && !m.interleave) { ++c.n_solo; c.solo_time += (uint64_t)L.dur + 500; }
      else { ++c.n_co; c.co_step += L.gap + L.dur; }
    }
  });
  // exclusive prefixes: solo launches are numbered and timed across ALL tenants (one at a time, tenant after tenant),
  // co-run launches per tenant
  uint64_t solo_count = 0, solo_time = 0;
  std::vector<uint64_t> co_count(n_tenants, 0);
  {
    std::vector<uint64_t> co_time(n_tenants, 0);
    for (Chunk& c : chunks) {
      const uint64_t ns = c.n_solo, st = c.solo_time, nc = c.n_co, cs = c.co_step;
      c.n_solo = solo_count; c.solo_time = solo_time; c.n_co = co_count[c.tenant]; c.co_step = co_time[c.tenant];
      solo_count += ns; solo_time += st; co_count[c.tenant] += nc; co_time[c.tenant] += cs;
    }
  }
  const uint64_t phase2 = t0_ns + solo_time + 1000000;

  // ---- pass B: the solo launches go straight to their place (they start before every co-run launch); the co-run
  // launches of a tenant become one start-ordered list
  std::vector<std::vector<CoLaunch>> co(n_tenants);
  for (uint32_t t = 0; t < n_tenants; ++t) co[t].resize(co_count[t]);
  parallel_for(chunks.size(), threads, [&](uint64_t ci) {
    const Chunk& c = chunks[ci];
    const ks_synth_tenant& T = tenants[c.tenant];
    uint64_t si = c.n_solo, st = c.solo_time, cj = c.n_co, ct = c.co_step;
    for (uint64_t i = c.first; i < c.first + c.count; ++i) {
      const Launch L = make_launch(T, m, i);
      if (L.solo && !m.interleave) {
        write_record(out + si, T, L.key, true, t0_ns + st, L.dur);
        ++si;
        st += (uint64_t)L.dur + 500;
      } else {
        ct += L.gap + L.dur;  // gap, launch, gap, launch ...
        co[c.tenant][cj++] = CoLaunch{phase2 + ct - L.dur, L.key | (L.solo ? 0x80000000u : 0u), L.dur};
      }
    }
  });

  // ---- pass C: merge the tenants' lists by start time, in slices of time that are merged independently
  uint64_t lo_t = ~0ull, hi_t = 0;
  for (uint32_t t = 0; t < n_tenants; ++t)
    if (!co[t].empty()) { lo_t = std::min(lo_t, co[t].front().start); hi_t = std::max(hi_t, co[t].back().start); }
  const uint64_t n_co_total = total - solo_count;
  if (n_co_total) {
    const uint64_t slices = std::max<uint64_t>(1, std::min<uint64_t>(n_co_total / 65536 + 1, 1u << 16));
    const long double width = (long double)(hi_t - lo_t + 1) / (long double)slices;
    // cut[s][t] = first launch of tenant t at or behind the start of slice s
    std::vector<uint64_t> cut((slices + 1) * n_tenants);
    parallel_for(slices + 1, threads, [&](uint64_t s) {
      const uint64_t edge = s == slices ? hi_t + 1 : lo_t + (uint64_t)(width * (long double)s);
      for (uint32_t t = 0; t < n_tenants; ++t) {
        const auto& v = co[t];
        cut[s * n_tenants + t] = (uint64_t)(std::lower_bound(v.begin(), v.end(), edge, [](const CoLaunch& a, uint64_t e) { return a.start < e; }) - v.begin());
      }
    });
    for (uint32_t t = 0; t < n_tenants; ++t) cut[t] = 0;  // slice 0 starts at the lists' heads whatever the rounding
    parallel_for(slices, threads, [&](uint64_t s) {
      uint64_t pos[256], end[256], o = solo_count;
      for (uint32_t t = 0; t < n_tenants; ++t) {
        pos[t] = cut[s * n_tenants + t];
        end[t] = cut[(s + 1) * n_tenants + t];
        o += pos[t];
      }
      while (true) {
        int best = -1;
        uint64_t bs = 0;
        for (uint32_t t = 0; t < n_tenants; ++t)
          if (pos[t] < end[t] && (best < 0 || co[t][pos[t]].start < bs)) { best = (int)t; bs = co[t][pos[t]].start; }  // ties: lower tenant first
        if (best < 0) break;
        const CoLaunch& L = co[best][pos[best]++];
        write_record(out + o++, tenants[best], L.key & 0x7FFFFFFFu, (L.key >> 31) != 0, L.start, L.dur);
      }
    });
  }
  return (int64_t)total;
}
