// ks_tsv.cuh -- the agent's timing log (tab separated text) to 48-byte launch records, on the device.
//
// Input: the bytes of one agent_<pid>_timing.tsv as the reference's agent writes it (scheduler/agent.cpp:692-705): a
// header line, then one line per launch with 17 columns, of which the path needs kernel_name (column 8), start_ns (9),
// end_ns (10, blank when no completion callback was seen, agent.cpp:702 -- such rows are dropped), block (14), model
// (15) and grid (16); dimensions are "(x, y, z)" or "x,y,z".
//
//   k_tsv_nl_count / k_tsv_nl_scan / k_tsv_nl_fill   line starts: an ordered compaction of the newline positions
//   k_tsv_parse          one thread per line: walks the tabs, parses the numeric fields, hashes the kernel symbol and the
//                        model string (64-bit FNV-1a) and enters both into small open-addressing string dictionaries
//                        (first occurrence wins: offset and length of the text), writes a record and a valid flag
//   k_tsv_valid_count / (k_rows_scan-style scan) / k_tsv_compact   drop invalid lines, keeping the file's order
//   k_tsv_finish         replaces dictionary slots by the ids the host assigned (name -> canonical name id,
//                        model -> tenant), sets the solo flag
//
// Strings are canonicalised on the host (ks_function_base needs the C++ demangler), once per DISTINCT symbol.
#pragma once

#include "ks_common.cuh"

namespace ks {

constexpr uint32_t kTsvTile = 4096;          // bytes per tile of the newline scan
constexpr uint32_t kTsvNameSlots = 1u << 16; // distinct kernel symbols per file (open addressing)
constexpr uint32_t kTsvModelSlots = 256;

struct TsvArgs {
  const unsigned char* text;
  uint64_t n_bytes;
  uint32_t* tile_cnt;            // [tiles + 1]
  unsigned long long* line_start; // [lines + 1]
  uint64_t max_lines;
  ks_record* parsed;             // [lines] one per line (valid or not)
  unsigned char* valid;          // [lines]
  uint32_t* vtile_cnt;           // [line tiles + 1]
  ks_record* out;                // compacted records
  uint64_t out_capacity;
  unsigned long long* name_hash; // [kTsvNameSlots] 0 = empty
  unsigned long long* name_where; // [kTsvNameSlots] offset << 20 | length
  unsigned long long* model_hash; // [kTsvModelSlots]
  unsigned long long* model_where;
  const uint32_t* name_map;      // k_tsv_finish: slot -> name id
  const uint32_t* model_map;     // slot -> tenant
  uint32_t solo;
  uint32_t* kernel_id;           // [lines] column 0 (the agent's running launch number), 0xFFFFFFFF if absent
  const unsigned char* row_solo; // [lines] per-row solo flag from a pairprof log (ks_tsv_label), or null: `solo` for all
  Control* ctl;                  // scratch0 = lines, n_pairs = valid records, max_start = largest kernel_id
};

__device__ __forceinline__ uint64_t fnv1a(const unsigned char* p, uint32_t n) {
  uint64_t h = 0xCBF29CE484222325ull;
  for (uint32_t i = 0; i < n; ++i) { h ^= p[i]; h *= 0x100000001B3ull; }
  return h ? h : 1ull;
}

__device__ __forceinline__ uint32_t tsv_dict_insert(unsigned long long* hashes, unsigned long long* where, uint32_t slots, uint64_t h, uint64_t off, uint32_t len,
                                                    Control* ctl) {
  uint32_t s = (uint32_t)((h * 0x9E3779B97F4A7C15ull) >> 40) & (slots - 1);
  for (uint32_t probe = 0; probe < slots; ++probe) {
    unsigned long long cur = ld_volatile_u64(reinterpret_cast<const uint64_t*>(hashes + s));
    if (cur == 0ull) {
      cur = atomicCAS(hashes + s, 0ull, (unsigned long long)h);
      if (cur == 0ull) cur = h;
    }
    if (cur == h) {
      // keep the FIRST occurrence in the text (lines are parsed in no particular order): minimum of offset << 20 | length
      const unsigned long long packed = (off << 20) | len;
      if (packed < ld_volatile_u64(reinterpret_cast<const uint64_t*>(where + s))) atomicMin(where + s, packed);
      return s;
    }
    s = (s + 1) & (slots - 1);
  }
  atomicOr(&ctl->err, kErrTooManyKeys);
  return 0;
}

// ---- line starts
__global__ void __launch_bounds__(256) k_tsv_nl_count(const TsvArgs a) {
  __shared__ uint32_t warp_tot[8];
  const uint64_t ntiles = (a.n_bytes + kTsvTile - 1) / kTsvTile;
  for (uint64_t tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
    uint32_t c = 0;
    for (uint32_t k = threadIdx.x; k < kTsvTile; k += 256) {
      const uint64_t i = tile * kTsvTile + k;
      if (i < a.n_bytes) c += a.text[i] == '\n';
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

// one CTA of 1024 threads: exclusive scan of per-tile counts in place; total -> *total_out
// (text != nullptr: the total counts newlines; one more line if the text does not end with a newline)
__global__ void __launch_bounds__(1024) k_tsv_scan(uint32_t* cnt, uint64_t ntiles, unsigned long long* total_out, const unsigned char* text, uint64_t n_bytes) {
  __shared__ uint32_t warp_tot[32];
  __shared__ uint32_t carry;
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  for (uint64_t base = 0; base < ntiles; base += 1024) {
    const uint64_t i = base + threadIdx.x;
    const uint32_t v = i < ntiles ? cnt[i] : 0;
    const uint32_t inc = warp_incl_scan(v);
    if (lane_id() == 31) warp_tot[threadIdx.x >> 5] = inc;
    __syncthreads();
    uint32_t off = carry;
    for (uint32_t w = 0; w < (threadIdx.x >> 5); ++w) off += warp_tot[w];
    if (i < ntiles) cnt[i] = off + inc - v;
    __syncthreads();
    if (threadIdx.x == 1023) carry = off + inc;
    __syncthreads();
  }
  if (threadIdx.x == 0) *total_out = carry + ((text && n_bytes && text[n_bytes - 1] != '\n') ? 1u : 0u);
}

// line k (k >= 1) starts behind the k-th newline; line 0 starts at 0
__global__ void __launch_bounds__(256) k_tsv_nl_fill(const TsvArgs a) {
  __shared__ uint32_t word_base[kTsvTile / 32];
  const uint64_t ntiles = (a.n_bytes + kTsvTile - 1) / kTsvTile;
  const uint32_t lane = lane_id(), warp = threadIdx.x >> 5;
  if (blockIdx.x == 0 && threadIdx.x == 0) a.line_start[0] = 0;
  for (uint64_t tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
    uint32_t ballot[kTsvTile / 256];
#pragma unroll
    for (int k = 0; k < (int)(kTsvTile / 256); ++k) {
      const uint64_t i = tile * kTsvTile + k * 256 + threadIdx.x;
      ballot[k] = __ballot_sync(0xFFFFFFFFu, i < a.n_bytes && a.text[i] == '\n');
      if (lane == 0) word_base[k * 8 + warp] = __popc(ballot[k]);
    }
    __syncthreads();
    if (warp == 0) {  // exclusive scan over the 128 words
      uint32_t run = 0;
      for (int q = 0; q < (int)(kTsvTile / 32 / 32); ++q) {
        const uint32_t c = word_base[q * 32 + lane];
        const uint32_t inc = warp_incl_scan(c);
        word_base[q * 32 + lane] = run + inc - c;
        run += __shfl_sync(0xFFFFFFFFu, inc, 31);
      }
    }
    __syncthreads();
    const uint64_t tile_line = a.tile_cnt[tile];
#pragma unroll
    for (int k = 0; k < (int)(kTsvTile / 256); ++k) {
      if (ballot[k] & (1u << lane)) {
        const uint64_t line = 1 + tile_line + word_base[k * 8 + warp] + __popc(ballot[k] & lanemask_lt());
        if (line <= a.max_lines) a.line_start[line] = tile * kTsvTile + k * 256 + threadIdx.x + 1;
      }
    }
    __syncthreads();
  }
}

// ---- per-line parse
__device__ __forceinline__ bool tsv_u64(const unsigned char* p, uint32_t n, unsigned long long* out) {
  if (n == 0) return false;
  unsigned long long v = 0;
  uint32_t i = 0;
  for (; i < n && p[i] >= '0' && p[i] <= '9'; ++i) v = v * 10ull + (p[i] - '0');
  if (i == 0) return false;
  if (i < n) {  // a float rendering of an integer ("123.0"), as written for a column that also holds blanks
    if (p[i] != '.') return false;
    for (++i; i < n; ++i) if (p[i] != '0') return false;
  }
  *out = v;
  return true;
}

__device__ __forceinline__ bool tsv_dims(const unsigned char* p, uint32_t n, uint32_t out[3]) {
  uint32_t found = 0, i = 0;
  while (i < n && found < 3) {
    if (p[i] >= '0' && p[i] <= '9') {
      uint32_t v = 0;
      for (; i < n && p[i] >= '0' && p[i] <= '9'; ++i) v = v * 10u + (p[i] - '0');
      out[found++] = v;
    } else {
      ++i;
    }
  }
  return found == 3;
}

__global__ void __launch_bounds__(256) k_tsv_parse(const TsvArgs a) {
  const uint64_t n_lines = min(a.ctl->scratch0, (unsigned long long)a.max_lines);
  for (uint64_t line = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; line < n_lines; line += (uint64_t)gridDim.x * blockDim.x) {
    const uint64_t b = a.line_start[line];
    uint64_t e = (line + 1 < n_lines || (a.n_bytes && a.text[a.n_bytes - 1] == '\n')) ? a.line_start[line + 1] - 1 : a.n_bytes;
    if (e > b && a.text[e - 1] == '\r') --e;
    ks_record r;
    r.name_id = 0; r.smem_word = 0; r.start_ns = 0; r.end_ns = 0;
    for (int i = 0; i < 3; ++i) { r.grid[i] = 0; r.block[i] = 0; }
    bool ok = e > b && line > 0;  // line 0 is the header
    // field boundaries: walk the tabs
    uint64_t fs = b;
    int col = 0;
    uint64_t name_off = 0, model_off = 0;
    uint32_t name_len = 0, model_len = 0, kid = 0xFFFFFFFFu;
    bool have_name = false, have_model = false, have_start = false, have_end = false, have_block = false, have_grid = false;
    for (uint64_t i = b; ok && i <= e; ++i) {
      if (i == e || a.text[i] == '\t') {
        const unsigned char* f = a.text + fs;
        const uint32_t fl = (uint32_t)(i - fs);
        if (col == 0) { unsigned long long v; if (tsv_u64(f, fl, &v) && v < 0xFFFFFFFFull) kid = (uint32_t)v; }
        else if (col == 8) { name_off = fs; name_len = fl; have_name = fl > 0; }
        else if (col == 9) have_start = tsv_u64(f, fl, reinterpret_cast<unsigned long long*>(&r.start_ns));
        else if (col == 10) have_end = tsv_u64(f, fl, reinterpret_cast<unsigned long long*>(&r.end_ns));
        else if (col == 14) have_block = tsv_dims(f, fl, r.block);
        else if (col == 15) { model_off = fs; model_len = fl; have_model = true; }
        else if (col == 16) have_grid = tsv_dims(f, fl, r.grid);
        fs = i + 1;
        ++col;
      }
    }
    ok = ok && have_name && have_start && have_end && have_block && have_grid && have_model && name_len < (1u << 20);
    if (ok) {  // only rows that are kept enter the dictionaries: models and names are numbered over the kept rows
      r.name_id = tsv_dict_insert(a.name_hash, a.name_where, kTsvNameSlots, fnv1a(a.text + name_off, name_len), name_off, name_len, a.ctl);
      const uint32_t model_slot = tsv_dict_insert(a.model_hash, a.model_where, kTsvModelSlots, fnv1a(a.text + model_off, model_len), model_off, model_len, a.ctl);
      r.smem_word = model_slot << 24;  // replaced by the tenant id in k_tsv_finish
    }
    a.parsed[line] = r;
    a.valid[line] = ok ? 1 : 0;
    a.kernel_id[line] = kid;
    if (ok && kid != 0xFFFFFFFFu) atomicMax(&a.ctl->max_start, (unsigned long long)kid);
  }
}

// ---- generic column extraction: any tab-separated log with a header line (the daemon's decision log,
// scheduler_daemon.cpp:674-676; the agent's timing log).  One thread per data line walks the tabs once; every requested
// column becomes one 64-bit word per line:
//   KS_COL_U64    decimal integer ("123", also "123.0"); blank or malformed -> all ones
//   KS_COL_MILLI  decimal with up to three fraction digits, as printf("%.3f") writes it -> the value x 1000; blank -> all ones
//   KS_COL_DIMS   "(x, y, z)" or "x,y,z" -> x | y << 21 | z << 42 (each below 2^21); malformed -> all ones
//   KS_COL_HASH   64-bit FNV-1a of the field's bytes (an empty field hashes like any other)
//   KS_COL_SPAN   offset of the field in the text << 20 | its length (to read a string back on the host)
constexpr uint32_t kTsvMaxCols = 16;
struct TsvExtractArgs {
  const unsigned char* text;
  uint64_t n_bytes;
  const unsigned long long* line_start;
  uint64_t n_lines;  // including the header line
  uint32_t n_cols;
  uint32_t col[kTsvMaxCols], kind[kTsvMaxCols];
  unsigned long long* out;  // [n_cols][capacity]
  uint64_t capacity;
};

__device__ __forceinline__ unsigned long long tsv_field(const unsigned char* f, uint32_t fl, uint64_t off, uint32_t kind) {
  const unsigned long long none = ~0ull;
  if (kind == KS_COL_U64) {
    unsigned long long v;
    return tsv_u64(f, fl, &v) ? v : none;
  }
  if (kind == KS_COL_MILLI) {
    if (fl == 0) return none;
    unsigned long long v = 0;
    uint32_t i = 0, frac = 0;
    for (; i < fl && f[i] >= '0' && f[i] <= '9'; ++i) v = v * 10ull + (f[i] - '0');
    if (i == 0) return none;
    if (i < fl) {
      if (f[i] != '.') return none;
      for (++i; i < fl && frac < 3; ++i, ++frac) {
        if (f[i] < '0' || f[i] > '9') return none;
        v = v * 10ull + (f[i] - '0');
      }
      for (; i < fl; ++i) if (f[i] < '0' || f[i] > '9') return none;  // further digits are cut off
    }
    for (; frac < 3; ++frac) v *= 10ull;
    return v;
  }
  if (kind == KS_COL_DIMS) {
    uint32_t d[3];
    if (!tsv_dims(f, fl, d) || d[0] >= (1u << 21) || d[1] >= (1u << 21) || d[2] >= (1u << 21)) return none;
    return (unsigned long long)d[0] | ((unsigned long long)d[1] << 21) | ((unsigned long long)d[2] << 42);
  }
  if (kind == KS_COL_HASH) return fnv1a(f, fl);
  return (off << 20) | (fl & 0xFFFFFu);  // KS_COL_SPAN
}

__global__ void __launch_bounds__(256) k_tsv_extract(const TsvExtractArgs a) {
  for (uint64_t line = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x + 1; line < a.n_lines; line += (uint64_t)gridDim.x * blockDim.x) {  // line 0: header
    const uint64_t row = line - 1;
    if (row >= a.capacity) continue;
    const uint64_t b = a.line_start[line];
    uint64_t e = (line + 1 < a.n_lines || (a.n_bytes && a.text[a.n_bytes - 1] == '\n')) ? a.line_start[line + 1] - 1 : a.n_bytes;
    if (e > b && a.text[e - 1] == '\r') --e;
    for (uint32_t c = 0; c < a.n_cols; ++c) a.out[(size_t)c * a.capacity + row] = a.kind[c] == KS_COL_HASH ? fnv1a(a.text, 0) : ~0ull;  // a missing column
    uint64_t fs = b;
    uint32_t col = 0;
    for (uint64_t i = b; i <= e; ++i) {
      if (i == e || a.text[i] == '\t') {
        for (uint32_t c = 0; c < a.n_cols; ++c)
          if (a.col[c] == col) a.out[(size_t)c * a.capacity + row] = tsv_field(a.text + fs, (uint32_t)(i - fs), fs, a.kind[c]);
        fs = i + 1;
        ++col;
      }
    }
  }
}

// histogram of the values of every segment: log2 bins (bin = bit length of the value, 0..32) or linear bins (value, clamped)
__global__ void __launch_bounds__(256) k_segment_hist(const uint32_t* __restrict__ values, const unsigned long long* __restrict__ offsets, uint64_t n_segments,
                                                      uint32_t n_bins, uint32_t log2_bins, uint32_t* __restrict__ out) {
  const uint32_t lane = lane_id();
  const uint64_t warps = (uint64_t)gridDim.x * (blockDim.x >> 5);
  for (uint64_t s = (uint64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); s < n_segments; s += warps) {
    const unsigned long long lo = offsets[s], hi = offsets[s + 1];
    for (unsigned long long i = lo + lane; i < hi; i += 32) {
      const uint32_t v = values[i];
      const uint32_t bin = min(log2_bins ? (uint32_t)(32 - __clz(v)) : v, n_bins - 1);
      atomicAdd(&out[s * n_bins + bin], 1u);
    }
  }
}

// ---- labels from the profiling daemon's log (profiling/pairprof_daemon.cpp:266 header, :317-318 rows):
// batch_id, kind, pid, kernel_id, model, kernel, block, rep, grid -- one row per released kernel; kernel_id is the agent
// log's kernel_id of process pid.  kind "alone" / "alone_other_waits" = the kernel had the GPU to itself (a solo sample),
// "gang_profile" / "gang_filler" = released together with a kernel of the other model.
struct TsvLabelArgs {
  const unsigned char* text;
  uint64_t n_bytes;
  const unsigned long long* line_start;
  uint64_t n_lines;
  unsigned long long pid;
  unsigned char* label;  // [label_cap] by kernel_id: 0 = not in the log, 1 = alone, 2 = gang
  uint64_t label_cap;
};

__global__ void __launch_bounds__(256) k_pplog_parse(const TsvLabelArgs a) {
  for (uint64_t line = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x + 1; line < a.n_lines; line += (uint64_t)gridDim.x * blockDim.x) {  // line 0: header
    const uint64_t b = a.line_start[line];
    uint64_t e = (line + 1 < a.n_lines || (a.n_bytes && a.text[a.n_bytes - 1] == '\n')) ? a.line_start[line + 1] - 1 : a.n_bytes;
    if (e > b && a.text[e - 1] == '\r') --e;
    uint64_t fs = b;
    int col = 0;
    unsigned char kind = 0;
    unsigned long long pid = ~0ull, kid = ~0ull;
    for (uint64_t i = b; i <= e && col <= 3; ++i) {
      if (i == e || a.text[i] == '\t') {
        const unsigned char* f = a.text + fs;
        const uint32_t fl = (uint32_t)(i - fs);
        if (col == 1) kind = (fl >= 5 && f[0] == 'a' && f[1] == 'l' && f[2] == 'o' && f[3] == 'n' && f[4] == 'e') ? 1 : (fl >= 4 && f[0] == 'g' && f[1] == 'a' && f[2] == 'n' && f[3] == 'g') ? 2 : 0;
        else if (col == 2) { if (!tsv_u64(f, fl, &pid)) pid = ~0ull; }
        else if (col == 3) { if (!tsv_u64(f, fl, &kid)) kid = ~0ull; }
        fs = i + 1;
        ++col;
      }
    }
    if (kind && pid == a.pid && kid < a.label_cap) a.label[kid] = kind;
  }
}

// rows the log does not mention are dropped (launches of the warm-up, which the profiler does not register); the others
// get their own solo flag
__global__ void __launch_bounds__(256) k_tsv_apply_labels(const TsvArgs a, const unsigned char* __restrict__ label, uint64_t label_cap, unsigned char* __restrict__ row_solo) {
  const uint64_t n_lines = min(a.ctl->scratch0, (unsigned long long)a.max_lines);
  for (uint64_t line = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; line < n_lines; line += (uint64_t)gridDim.x * blockDim.x) {
    if (!a.valid[line]) continue;
    const uint32_t kid = a.kernel_id[line];
    const unsigned char lab = kid < label_cap ? label[kid] : 0;
    if (!lab) a.valid[line] = 0;
    row_solo[line] = lab == 1;
  }
}

__global__ void __launch_bounds__(256) k_tsv_valid_count(const TsvArgs a) {
  __shared__ uint32_t warp_tot[8];
  const uint64_t n_lines = min(a.ctl->scratch0, (unsigned long long)a.max_lines);
  const uint64_t ntiles = (n_lines + 255) / 256;
  for (uint64_t tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
    const uint64_t i = tile * 256 + threadIdx.x;
    uint32_t c = (i < n_lines && a.valid[i]) ? 1u : 0u;
    c = warp_sum(c);
    __syncthreads();
    if (lane_id() == 0) warp_tot[threadIdx.x >> 5] = c;
    __syncthreads();
    if (threadIdx.x == 0) {
      uint32_t t = 0;
      for (int w = 0; w < 8; ++w) t += warp_tot[w];
      a.vtile_cnt[tile] = t;
    }
  }
}

// order-preserving compaction + dictionary slots -> ids
__global__ void __launch_bounds__(256) k_tsv_compact(const TsvArgs a) {
  __shared__ uint32_t warp_tot[8];
  const uint64_t n_lines = min(a.ctl->scratch0, (unsigned long long)a.max_lines);
  const uint64_t ntiles = (n_lines + 255) / 256;
  for (uint64_t tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
    const uint64_t i = tile * 256 + threadIdx.x;
    const bool v = i < n_lines && a.valid[i];
    const uint32_t ballot = __ballot_sync(0xFFFFFFFFu, v);
    __syncthreads();
    if (lane_id() == 0) warp_tot[threadIdx.x >> 5] = __popc(ballot);
    __syncthreads();
    uint64_t pos = a.vtile_cnt[tile] + __popc(ballot & lanemask_lt());
    for (uint32_t w = 0; w < (threadIdx.x >> 5); ++w) pos += warp_tot[w];
    if (v && pos < a.out_capacity) {
      ks_record r = a.parsed[i];
      r.name_id = a.name_map[r.name_id];
      const bool solo = a.row_solo ? a.row_solo[i] != 0 : a.solo != 0;
      r.smem_word = (a.model_map[r.smem_word >> 24] << 24) | (solo ? kMetaSoloBit : 0u);
      a.out[pos] = r;
    }
  }
}

}  // namespace ks
