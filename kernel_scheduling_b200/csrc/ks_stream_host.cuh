// ks_stream_host.cuh -- ks_build_table_streamed: the pair table of a trace whose overlapping pairs do not fit one call.
// Part of ks_api.cu (included behind the handle and the stage drivers); not a translation unit of its own.
//
// One call of ks_build_table sorts all samples of the trace at once: fewer than 2^30 of them, twice in memory.  A trace
// of 10^9 launches from eight tenants has three times that.  Here the trace is still decoded once (the timeline of 10^9
// launches is 16 GB), but it is JOINED window after window: the samples of a window are cut into key ranges
// ("parts", the partition pass of the multi-GPU exchange with all destinations in this GPU's memory) and appended to
// the parts' stores; when the last window is done every part is sorted and reduced on its own and its rows are appended
// to the table.  A pair belongs to the window of its EARLIER launch (the join reads the timeline behind the window's
// end), so nothing is carried between windows.  The splitters come from the sort-key histogram of a window in the
// middle of the trace, joined once in advance; a part's store holds what that window predicts for the whole trace plus
// a margin, and when a part outgrows it anyway the store is enlarged and the parts are moved.
//
// Solo samples have the smallest sort keys: they all land in part 0, which is reduced first and gives the solo times
// the other parts divide by.
#pragma once

#include <algorithm>
#include <vector>

namespace {

// a buffer that keeps its content when it grows
int ensure_keep(ks_handle* h, DevBuf& b, size_t bytes, size_t used) {
  if (bytes <= b.cap) return 0;
  const size_t want = (std::max(bytes, b.cap + b.cap / 2) + 255) & ~(size_t)255;
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, want);
  if (e != cudaSuccess) return fail(h, KS_ERR_CUDA, "cudaMalloc of " + std::to_string(want) + " bytes: " + cudaGetErrorString(e));
  if (b.p && used) {
    e = cudaMemcpyAsync(p, b.p, used, cudaMemcpyDeviceToDevice, h->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(h->stream);
    if (e != cudaSuccess) { cudaFree(p); return fail(h, KS_ERR_CUDA, std::string("cudaMemcpyAsync: ") + cudaGetErrorString(e)); }
  }
  if (b.p) cudaFree(b.p);
  b.p = p;
  b.cap = want;
  return 0;
}

struct StreamParts {
  uint32_t n_parts = 1, shift = 0;
  uint32_t splitters[16] = {0};
  uint64_t off[17] = {0};   // where a part's store begins (samples)
  uint64_t fill[16] = {0};  // samples in it
};

// n samples at `in` go to their parts' stores
int stream_partition(ks_handle* h, StreamParts& P, const uint4* in, uint64_t n) {
  if (!n) return 0;
  constexpr int ITEMS = kSort16Items;
  constexpr int THREADS = kSort16Threads;
  constexpr int TILE = THREADS * ITEMS;
  const uint32_t ntiles = (uint32_t)((n + TILE - 1) / TILE);
  const size_t lb_bytes = ((size_t)ntiles * kSort16Bins + 64) * sizeof(uint32_t);
  KS_ENSURE(h, h->lookback, lb_bytes);
  KS_ENSURE(h, h->hist, 2 * 4 * kSort16Bins * sizeof(uint32_t));
  uint32_t* hist = as<uint32_t>(h->hist);
  KS_CUDA(h, cudaMemsetAsync(hist, 0, 256 * sizeof(uint32_t), h->stream));
  KS_CUDA(h, cudaMemsetAsync(h->lookback.p, 0, lb_bytes, h->stream));
  SortPass16Args a{};
  a.by_dest = 2;
  a.n_split = P.n_parts - 1;
  a.split_shift = P.shift;
  for (uint32_t i = 0; i + 1 < P.n_parts; ++i) a.split[i] = P.splitters[i];
  a.in = in;
  a.n = (uint32_t)n;
  a.bits = 8;
  a.lookback = as<uint32_t>(h->lookback);
  a.ticket = as<uint32_t>(h->lookback) + (size_t)ntiles * kSort16Bins;
  a.err = &h->d_ctl->err;
  // how many samples every part receives: counted first, so that an overflow is refused before anything is written
  k_dest_hist<<<h->sm_count * 2, 256, 0, h->stream>>>(a, hist);
  uint32_t cnt[16];
  KS_CUDA(h, cudaMemcpyAsync(cnt, hist, sizeof(cnt), cudaMemcpyDeviceToHost, h->stream));
  KS_CUDA(h, cudaStreamSynchronize(h->stream));
  bool grow = false;
  for (uint32_t d = 0; d < P.n_parts; ++d) grow = grow || P.fill[d] + cnt[d] > P.off[d + 1] - P.off[d];
  if (grow) {
    // a key range outgrew what the first window predicted for it: a larger store, the ranges moved over
    uint64_t off2[17] = {0};
    for (uint32_t d = 0; d < P.n_parts; ++d) {
      const uint64_t have = P.off[d + 1] - P.off[d], need = P.fill[d] + cnt[d];
      const uint64_t c = need > have ? need + need / 2 + (1u << 16) : have;
      if (c >= kSortMaxItems) return fail(h, KS_ERR_TOO_LARGE, "ks_build_table_streamed: a key range of 2^30 samples or more: use more parts");
      off2[d + 1] = off2[d] + c;
    }
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, off2[P.n_parts] * 16);
    if (e != cudaSuccess) return fail(h, KS_ERR_CUDA, "ks_build_table_streamed: cudaMalloc of " + std::to_string(off2[P.n_parts] * 16) + " bytes: " + cudaGetErrorString(e));
    for (uint32_t d = 0; d < P.n_parts && e == cudaSuccess; ++d)
      if (P.fill[d]) e = cudaMemcpyAsync(static_cast<uint4*>(p) + off2[d], as<uint4>(h->stream_store) + P.off[d], P.fill[d] * 16, cudaMemcpyDeviceToDevice, h->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(h->stream);
    if (e != cudaSuccess) { cudaFree(p); return fail(h, KS_ERR_CUDA, std::string("ks_build_table_streamed: moving the key ranges: ") + cudaGetErrorString(e)); }
    cudaFree(h->stream_store.p);
    h->stream_store.p = p;
    h->stream_store.cap = off2[P.n_parts] * 16;
    for (uint32_t d = 0; d <= P.n_parts; ++d) P.off[d] = off2[d];
  }
  for (uint32_t d = 0; d < P.n_parts; ++d) {
    a.dest[d] = as<uint4>(h->stream_store) + P.off[d] + P.fill[d];
    P.fill[d] += cnt[d];
  }
  constexpr size_t smem = sort16_smem_bytes<ITEMS, THREADS>();
  if (!h->attr_sort16) {
    KS_CUDA(h, cudaFuncSetAttribute(k_onesweep_pass16<ITEMS, THREADS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    h->attr_sort16 = true;
  }
  k_onesweep_pass16<ITEMS, THREADS><<<(int)std::min<uint32_t>(ntiles, (uint32_t)h->sm_count * kSort16CtasPerSm), THREADS, smem, h->stream>>>(a);
  h->launches += 2;
  KS_CUDA(h, cudaGetLastError());
  return 0;
}

}  // namespace

extern "C" int64_t ks_build_table_streamed(ks_handle* h, const void* records, uint64_t n, uint32_t flags, uint64_t window_records, uint32_t n_parts,
                                           ks_table_info* info) {
  if (!h) return -KS_ERR_ARG;
  if ((!records && n) || (flags & ~(KS_ON_DEVICE | KS_KEY_TYPE)) || n_parts > 16) return fail(h, KS_ERR_ARG, "ks_build_table_streamed: bad argument");
  if (n >= kSortMaxItems) return fail(h, KS_ERR_TOO_LARGE, "ks_build_table_streamed: 2^30 records or more");
  KS_CUDA(h, cudaSetDevice(h->device));
  if (!n_parts) n_parts = 16;
  if (!window_records) window_records = 1ull << 26;
  h->n_pair_rows = h->n_key_rows = 0;
  cudaEvent_t* ev = h->ev;
  cudaEventRecord(ev[0], h->stream);
  const unsigned char* d_rec = nullptr;
  { int r = stage_in<unsigned char>(h, h->records, reinterpret_cast<const unsigned char*>(records), n * 48, (flags & KS_ON_DEVICE) != 0, &d_rec); if (r) return r; }
  { int r = reset_run(h); if (r) return r; }
  cudaEventRecord(ev[1], h->stream);

  // ---- K1 over the whole trace, the dictionary, the solo samples
  { int r = run_decode(h, d_rec, n, flags, nullptr); if (r) return r; }
  cudaEventRecord(ev[2], h->stream);
  { int r = run_dict(h); if (r) return r; }
  { int r = read_ctl(h); if (r) return r; }
  {
    const int st = status_of_err(h->h_ctl->err, true);  // the trace must be in start order: the join reads behind a window's end
    if (st) return fail(h, st, std::string("ks_build_table_streamed: ") + ks_status_string(st));
  }
  const uint64_t nk = h->h_ctl->n_keys, n_solo = h->h_ctl->n_solo;
  const uint32_t max_dur = h->h_ctl->max_dur;
  const unsigned long long min_start = h->h_ctl->min_start, max_start = h->h_ctl->max_start;
  const int key_bits = bit_length(nk + nk * nk);
  uint64_t cap = std::max<uint64_t>({sample_capacity(h), 3 * std::min(window_records, n), n_solo, 1u << 16});
  { int r = ensure_samples(h, cap); if (r) return r; }
  cudaEventRecord(ev[3], h->stream);

  StreamParts P;
  P.n_parts = n_parts;
  P.shift = key_bits > 12 ? (uint32_t)(key_bits - 12) : 0u;
  uint64_t n_pairs_total = 0;
  KS_ENSURE(h, h->tmp[3], (size_t)kKeyHistBins * 8);
  unsigned long long* d_hist = as<unsigned long long>(h->tmp[3]);
  std::vector<unsigned long long> solo_hist(kKeyHistBins, 0), first_hist(kKeyHistBins, 0);
  auto key_histogram = [&](const uint4* smp, uint64_t cnt, std::vector<unsigned long long>& out) -> int {
    KS_CUDA(h, cudaMemsetAsync(d_hist, 0, (size_t)kKeyHistBins * 8, h->stream));
    if (cnt) { k_key_hist<<<h->sm_count * 2, 256, 0, h->stream>>>(smp, (uint32_t)cnt, P.shift, d_hist); ++h->launches; }
    KS_CUDA(h, cudaMemcpyAsync(out.data(), d_hist, (size_t)kKeyHistBins * 8, cudaMemcpyDeviceToHost, h->stream));
    KS_CUDA(h, cudaStreamSynchronize(h->stream));
    return 0;
  };
  // The splitters and the stores' sizes: what the first window holds, scaled to the whole trace, plus the solo samples.
  auto make_store = [&](double scale) -> int {
    std::vector<double> expect(kKeyHistBins);
    double all = 0;
    for (uint32_t b = 0; b < kKeyHistBins; ++b) { expect[b] = (double)first_hist[b] * scale + (double)solo_hist[b]; all += expect[b]; }
    uint32_t edge[17];
    edge[0] = 0;
    double before = 0;
    uint32_t b = 0;
    const uint32_t solo_bins = nk ? (uint32_t)std::min<uint64_t>(((nk - 1) >> P.shift) + 1, kKeyHistBins) : 0u;  // bins that hold sort keys below nk
    for (uint32_t r = 1; r < P.n_parts; ++r) {
      const double target = all * r / P.n_parts;
      while (b < kKeyHistBins && (before < target || b < solo_bins)) before += expect[b++];  // every solo key stays in part 0
      edge[r] = b;
      P.splitters[r - 1] = b;
    }
    edge[P.n_parts] = kKeyHistBins;
    for (uint32_t r = 0; r < P.n_parts; ++r) {
      double sum = 0;
      for (uint32_t q = edge[r]; q < edge[r + 1]; ++q) sum += expect[q];
      const uint64_t c = (uint64_t)(sum * 1.25) + (1u << 16);  // a quarter of margin for what the first window does not show
      if (c >= kSortMaxItems) return fail(h, KS_ERR_TOO_LARGE, "ks_build_table_streamed: a key range of 2^30 samples or more: use more parts");
      P.off[r + 1] = P.off[r] + c;
    }
    KS_ENSURE(h, h->stream_store, P.off[P.n_parts] * 16);
    return 0;
  };

  // ---- the solo samples wait in a buffer of their own until the splitters are known
  {
    SoloArgs s{};
    s.solo_stream = as<unsigned long long>(h->solo_stream);
    s.kid_of_slot = h->kid_of_slot;
    s.samples = as<uint4>(h->samples[0]);
    s.capacity = cap;
    s.ctl = h->d_ctl;
    k_solo_samples<<<h->sm_count * 4, 256, 0, h->stream>>>(s);
    ++h->launches;
    KS_ENSURE(h, h->tmp[4], std::max<size_t>(n_solo * 16, 16));
    if (n_solo) KS_CUDA(h, cudaMemcpyAsync(h->tmp[4].p, h->samples[0].p, n_solo * 16, cudaMemcpyDeviceToDevice, h->stream));
    { int r = key_histogram(as<uint4>(h->tmp[4]), n_solo, solo_hist); if (r) return r; }
  }
  // the pairs whose earlier launch lies in [lo, hi) -> sample set 0; the join reads the timeline behind hi for their later launches
  auto join_window = [&](uint64_t lo, uint64_t hi, uint64_t* n_out) -> int {
    for (int attempt = 0; attempt < 2; ++attempt) {
      KS_CUDA(h, cudaMemsetAsync(&h->d_ctl->n_pairs, 0, 8, h->stream));
      { int r = run_join(h, 0, n - lo, cap, nullptr, nullptr, lo, 0, hi - lo); if (r) return r; }
      { int r = read_ctl(h); if (r) return r; }
      const int st = status_of_err(h->h_ctl->err, true);
      if (st) return fail(h, st, std::string("ks_build_table_streamed: ") + ks_status_string(st));
      *n_out = h->h_ctl->n_pairs;
      if (*n_out <= cap) return 0;
      if (*n_out >= kSortMaxItems) return fail(h, KS_ERR_TOO_LARGE, "ks_build_table_streamed: 2^30 samples or more in one window: use smaller windows");
      cap = *n_out + *n_out / 16;
      { int r = ensure_samples(h, cap); if (r) return r; }
    }
    return fail(h, KS_ERR_CAPACITY, "ks_build_table_streamed: sample stream still too small");
  };
  // A window from the middle of the trace is joined once in advance, only for its sort-key histogram: the splitters and
  // the stores' sizes come from it (the beginning of a trace is often unlike the rest: a solo phase, a warm-up).
  {
    const uint64_t plo = n > window_records ? n / 2 : 0, phi = std::min(n, plo + window_records);
    uint64_t n_probe = 0;
    if (phi > plo) { int r = join_window(plo, phi, &n_probe); if (r) return r; }
    { int r = key_histogram(as<uint4>(h->samples[0]), n_probe, first_hist); if (r) return r; }
    { int r = make_store(phi > plo ? (double)n / (double)(phi - plo) : 1.0); if (r) return r; }
    { int r = stream_partition(h, P, as<uint4>(h->tmp[4]), n_solo); if (r) return r; }
  }
  for (uint64_t lo = 0; lo < n; lo += window_records) {
    const uint64_t hi = std::min(n, lo + window_records);
    uint64_t n_batch = 0;
    { int r = join_window(lo, hi, &n_batch); if (r) return r; }
    n_pairs_total += n_batch;
    { int r = stream_partition(h, P, as<uint4>(h->samples[0]), n_batch); if (r) return r; }
  }
  cudaEventRecord(ev[4], h->stream);
  // the timeline and the solo stream are not needed any more; a long trace needs their room for the parts' scratch
  if (n > (1ull << 27)) {
    KS_CUDA(h, cudaStreamSynchronize(h->stream));
    for (DevBuf* b : {&h->tl_start[0], &h->tl_dm[0], &h->solo_stream, &h->tmp[4]}) {
      if (b->p) cudaFree(b->p);
      b->p = nullptr;
      b->cap = 0;
    }
  }
  // ---- every part: sort, rows, statistics, table rows.  Part 0 first: it holds the solo rows.
  uint64_t rows_total = 0;
  uint64_t max_part = 0;
  for (uint32_t r = 0; r < P.n_parts; ++r) max_part = std::max(max_part, P.fill[r]);
  { int r = ensure_samples(h, std::max<uint64_t>(max_part, 16)); if (r) return r; }
  for (uint32_t part = 0; part < P.n_parts; ++part) {
    const uint64_t np = P.fill[part];
    for (int attempt = 0;; ++attempt) {
      { int r = mg_zero_u32(h, &h->d_ctl->n_rows, 2); if (r) return r; }
      { int r = mg_zero_u32(h, &h->d_ctl->ticket, 2); if (r) return r; }
      { int r = mg_zero_u32(h, &h->d_ctl->ticket2, 1); if (r) return r; }
      KS_CUDA(h, cudaMemsetAsync(&h->d_ctl->scratch0, 0, 8, h->stream));
      KS_CUDA(h, cudaMemsetAsync(&h->d_ctl->pad[0], 0, 4 * 8 + 8, h->stream));
      KS_CUDA(h, cudaMemsetAsync(&h->d_ctl->pad2[0], 0, 16, h->stream));
      KS_CUDA(h, cudaMemsetAsync(h->row_of_kid, 0xFF, (size_t)(kMaxKeys + 1) * 4, h->stream));
      // the range's keys lie in [splitter << shift, next splitter << shift): sorted over the bits of that width only
      const uint64_t key_end = nk + nk * nk + 1;
      const uint64_t key_lo = part ? std::min<uint64_t>((uint64_t)P.splitters[part - 1] << P.shift, key_end) : 0;
      const uint64_t key_hi = part + 1 < P.n_parts ? std::min<uint64_t>((uint64_t)P.splitters[part] << P.shift, key_end) : key_end;
      const int cur = key_hi > key_lo ? radix_sort16(h, np, std::max(1, bit_length(key_hi - key_lo - 1)), nullptr, as<uint4>(h->stream_store) + P.off[part], nullptr, (uint32_t)key_lo)
                                      : radix_sort16(h, np, key_bits, nullptr, as<uint4>(h->stream_store) + P.off[part]);
      if (cur < 0) return cur;
      const uint32_t max_rows = (uint32_t)std::min<uint64_t>(np, (uint64_t)h->cfg.max_pair_rows + nk) + 1;
      { int r = run_rows_and_stats(h, np ? as<uint4>(h->samples[cur]) : as<uint4>(h->samples[0]), np, max_rows); if (r) return r; }
      if (part == 0 && nk) {
        k_solo_ns<<<(unsigned)((nk + 255) / 256), 256, 0, h->stream>>>(as<RowStats>(h->stats), h->row_of_kid, (uint32_t)nk, h->solo_ns);
        ++h->launches;
      }
      { int r = read_ctl(h); if (r) return r; }
      if ((h->h_ctl->err & kErrTooLarge) && attempt == 0 && h->rows_auto && h->h_ctl->pad2[0] > h->cfg.max_pair_rows && h->h_ctl->pad2[0] < (1ull << 31)) {
        // more rows in this key range than the row arrays were sized for: size them for it and do the range again
        h->cfg.max_pair_rows = (uint32_t)std::min<uint64_t>(h->h_ctl->pad2[0] + h->h_ctl->pad2[0] / 8, 0x7FFFFFFFull);
        KS_CUDA(h, cudaMemsetAsync(&h->d_ctl->err, 0, 4, h->stream));
        continue;
      }
      const int st = status_of_err(h->h_ctl->err, true);
      if (st) return fail(h, st, std::string("ks_build_table_streamed: ") + ks_status_string(st));
      break;
    }
    const uint64_t rows_here = h->h_ctl->n_rows - h->h_ctl->ticket2;  // without the solo rows
    { int r = ensure_keep(h, h->pair_rows, (rows_total + rows_here + 1) * sizeof(ks_pair_row), rows_total * sizeof(ks_pair_row)); if (r) return r; }
    h->mg_nk = nk;
    if (part == 0) {
      { int r = mg_finalize_queue(h, as<ks_pair_row>(h->pair_rows) + rows_total, (uint32_t)rows_here + 1); if (r) return r; }
    } else if (rows_here) {
      FinalArgs f{};
      f.stats = as<RowStats>(h->stats);
      f.row_start = as<uint32_t>(h->row_start);
      f.row_key = as<uint32_t>(h->row_key);
      f.row_of_kid = h->row_of_kid;
      f.slot_of_kid = h->slot_of_kid;
      f.keys_sorted = h->keys_sorted;
      f.dict_words = h->dict_words;
      f.dict_launches = h->dict_launches;
      f.dict_solo = h->dict_solo;
      f.solo_ns = h->solo_ns;
      f.solo_given = 1;
      f.key_rows = h->key_rows;
      f.pair_rows = as<ks_pair_row>(h->pair_rows) + rows_total;
      f.max_pair_rows = (uint32_t)rows_here + 1;
      f.ctl = h->d_ctl;
      k_finalize_pairs<<<h->sm_count * 4, 256, 0, h->stream>>>(f);
      ++h->launches;
      KS_CUDA(h, cudaGetLastError());
    }
    rows_total += rows_here;
  }
  cudaEventRecord(ev[5], h->stream);
  { int r = read_ctl(h); if (r) return r; }
  {
    const int st = status_of_err(h->h_ctl->err, true);
    if (st) return fail(h, st, std::string("ks_build_table_streamed: ") + ks_status_string(st));
  }
  KS_CUDA(h, cudaGetLastError());
  h->hint_valid = false;
  h->n_key_rows = nk;
  h->n_pair_rows = rows_total;
  h->pair_rows_src = h->pair_rows.p;
  if (info) {
    std::memset(info, 0, sizeof(*info));
    info->n_records = n;
    info->n_keys = nk;
    info->n_solo = n_solo;
    info->n_pairs = n_pairs_total;
    info->n_rows = rows_total;
    info->max_duration_ns = max_dur;
    info->min_start_ns = n ? min_start : 0;
    info->max_start_ns = max_start;
    info->was_time_ordered = 1;
    info->ms_stage_in = ev_ms(ev[0], ev[1]);
    info->ms_decode = ev_ms(ev[1], ev[2]);
    info->ms_dict = ev_ms(ev[2], ev[3]);
    info->ms_join = ev_ms(ev[3], ev[4]);    // the windows: join + partition into the parts' stores
    info->ms_reduce = ev_ms(ev[4], ev[5]);  // the parts: sort, statistics, table rows
    info->ms_total = ev_ms(ev[0], ev[5]);
    info->sort_passes = (uint32_t)h->sort_passes;
  }
  return (int64_t)rows_total;
}
