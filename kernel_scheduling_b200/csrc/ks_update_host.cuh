// ks_update_host.cuh -- host side of the resident pair table (kernels and the method: ks_update.cuh).  Part of ks_api.cu
// (included behind the handle and the stage drivers); not a translation unit of its own.
//
//   ks_update_begin   clears the dictionary and the resident statistics: an empty table
//   ks_update         one window of new launches (start order, not before the previous window): K1 over the window, the
//                     launches carried over from earlier windows in the halo slots, K3, a small K2, then k_upd_rows merges
//                     the window's samples into the rows they belong to.  Two host waits (sample count, error bits).
//   ks_update_table   reads the table out (key rows by key, pair rows by (key_a, key_b)) for ks_copy_*_rows
//   ks_update_end     frees the resident statistics
#pragma once

#include <algorithm>
#include <numeric>

namespace {

UpdState upd_state(ks_handle* h) {
  UpdState st{};
  st.rows = as<UpdRow>(h->upd_rows);
  st.carry_start = as<unsigned long long>(h->upd_carry);
  st.carry_dm = st.carry_start + kHaloMax;
  st.scalars = as<uint32_t>(h->upd_scalars);
  st.pool1 = as<uint32_t>(h->upd_pool);
  st.pool2 = as<uint32_t>(h->upd_pool2);
  st.pool1_blocks = h->upd_pool_blocks;
  st.pool2_blocks = h->upd_pool2_blocks;
  return st;
}

int upd_status(ks_handle* h, uint32_t err, const char* what) {
  if (err & kErrEscaped) {
    h->upd_broken = true;
    return fail(h, KS_ERR_REBUILD, std::string(what) + ": a median left its window (the distribution of a row jumped); begin again and replay the launches");
  }
  const int st = status_of_err(err, true);
  if (st) {
    h->upd_broken = true;  // the window may have been merged in part
    return fail(h, st, std::string(what) + ": " + ks_status_string(st));
  }
  return 0;
}

}  // namespace

extern "C" {

int64_t ks_update_begin(ks_handle* h, uint32_t flags) {
  if (!h || (flags & ~KS_KEY_TYPE)) return -KS_ERR_ARG;
  KS_CUDA(h, cudaSetDevice(h->device));
  { int r = reset_run(h); if (r) return r; }  // empty dictionary, zero launch counts
  KS_ENSURE(h, h->upd_rows, kUpdRows * sizeof(UpdRow));
  KS_ENSURE(h, h->upd_carry, 2 * (size_t)kHaloMax * 8);
  KS_ENSURE(h, h->upd_scalars, 64);
  // the windows of the rows with more than 64 samples: pool 1 (rows of up to 1,024 samples, 12 KB each) and pool 2 (larger
  // rows, 204 KB each).  Sized for the full-length run of the online configuration (a 1,200 x 800 pair table after
  // 10,000 windows of 65,536 launches: about 290,000 rows above 64 samples, 33,000 above 1,024): 4.8 GB + 8.6 GB.
  h->upd_pool_blocks = 393216;
  h->upd_pool2_blocks = 40960;
  KS_ENSURE(h, h->upd_pool, (size_t)h->upd_pool_blocks * kLanes * kUpdMidWindow * 4);
  KS_ENSURE(h, h->upd_pool2, (size_t)h->upd_pool2_blocks * kLanes * kUpdBlockSlots * 4);
  KS_CUDA(h, cudaMemsetAsync(h->upd_rows.p, 0, kUpdRows * sizeof(UpdRow), h->stream));
  KS_CUDA(h, cudaMemsetAsync(h->upd_scalars.p, 0, 64, h->stream));
  KS_CUDA(h, cudaMemsetAsync(h->kid_of_slot, 0xFF, (size_t)kDictSlots * 4, h->stream));
  KS_CUDA(h, cudaStreamSynchronize(h->stream));
  h->upd_active = true;
  h->upd_broken = false;
  h->upd_flags = flags;
  h->upd_windows = 0;
  h->upd_records = 0;
  h->n_pair_rows = h->n_key_rows = 0;
  return KS_OK;
}

int64_t ks_update_end(ks_handle* h) {
  if (!h) return -KS_ERR_ARG;
  cudaSetDevice(h->device);
  if (h->stream) cudaStreamSynchronize(h->stream);
  for (DevBuf* b : {&h->upd_rows, &h->upd_carry, &h->upd_scalars, &h->upd_list[0], &h->upd_list[1], &h->upd_list[2], &h->upd_list[3], &h->upd_ranks, &h->upd_pool, &h->upd_pool2, &h->upd_big}) {
    if (b->p) cudaFree(b->p);
    b->p = nullptr;
    b->cap = 0;
  }
  h->upd_active = false;
  return KS_OK;
}

int64_t ks_update(ks_handle* h, const void* records, uint64_t n, uint32_t flags, ks_table_info* info) {
  if (!h || (!records && n) || (flags & ~KS_ON_DEVICE)) return -KS_ERR_ARG;
  if (!h->upd_active) return fail(h, KS_ERR_ARG, "ks_update: no resident table (ks_update_begin)");
  if (h->upd_broken) return fail(h, KS_ERR_REBUILD, "ks_update: the resident table is no longer valid after an earlier error; begin again");
  if (n + kHaloMax >= kSortMaxItems) return fail(h, KS_ERR_TOO_LARGE, "ks_update: too many records in one window");
  KS_CUDA(h, cudaSetDevice(h->device));
  if (n == 0) return 0;
  cudaEvent_t* ev = h->ev;
  cudaEventRecord(ev[0], h->stream);
  const unsigned char* d_rec = nullptr;
  { int r = stage_in<unsigned char>(h, h->records, reinterpret_cast<const unsigned char*>(records), n * 48, (flags & KS_ON_DEVICE) != 0, &d_rec); if (r) return r; }
  if (reinterpret_cast<uintptr_t>(d_rec) & 15u) return fail(h, KS_ERR_ARG, "ks_update: device records must be 16-byte aligned");
  const UpdState st = upd_state(h);
  k_upd_reset_ctl<<<1, 32, 0, h->stream>>>(h->d_ctl);
  // K1 over the window, behind the halo slots; the dictionary and its launch counts persist over the windows
  { int r = run_decode(h, d_rec, n, h->upd_flags, nullptr, kHaloMax, 2 * (uint64_t)kHaloMax, 0); if (r) return r; }
  unsigned long long* tl_start = as<unsigned long long>(h->tl_start[0]);
  unsigned long long* tl_dm = as<unsigned long long>(h->tl_dm[0]);
  k_upd_assign_ids<<<kDictSlots / 256, 256, 0, h->stream>>>(h->dict_keys, h->kid_of_slot, h->slot_of_kid, st.scalars + 1, h->d_ctl);
  k_upd_place_carry<<<1, 1024, 0, h->stream>>>(st, tl_start, tl_dm, n, h->d_ctl);
  h->launches += 3;
  // samples of the window: its solo launches, then the pairs whose later launch is in the window
  const uint64_t n_tl = n + kHaloMax;
  uint64_t cap = sample_capacity(h);
  if (cap < std::max<uint64_t>(4 * n_tl, 1u << 16)) {
    cap = std::max<uint64_t>(4 * n_tl, 1u << 16);
    int r = ensure_samples(h, cap);
    if (r) return r;
  }
  uint64_t n_samples = 0;
  for (int attempt = 0;; ++attempt) {
    SoloArgs s{};
    s.solo_stream = as<unsigned long long>(h->solo_stream);
    s.kid_of_slot = h->kid_of_slot;
    s.samples = as<uint4>(h->samples[0]);
    s.capacity = cap;
    s.ctl = h->d_ctl;
    k_solo_samples<<<h->sm_count * 4, 256, 0, h->stream>>>(s);
    ++h->launches;
    { int r = run_join(h, 0, n_tl, cap, nullptr, nullptr, 0, kHaloMax); if (r) return r; }
    { int r = read_ctl(h); if (r) return r; }                                                         // ---- wait 1
    { int r = upd_status(h, h->h_ctl->err, "ks_update"); if (r) return r; }  // the dictionary already counted the window: the session is over
    n_samples = h->h_ctl->n_pairs;
    if (n_samples <= cap) break;
    if (n_samples >= kSortMaxItems) return fail(h, KS_ERR_TOO_LARGE, "ks_update: 2^30 samples or more in one window");
    if (attempt == 1) return fail(h, KS_ERR_CAPACITY, "ks_update: sample stream still too small");
    cap = n_samples + n_samples / 16;
    { int r = ensure_samples(h, cap); if (r) return r; }
  }
  // the launches still running at the end of the window are carried into the next one
  KS_ENSURE(h, h->tmp[0], (size_t)kHaloMax * 4 + 16);
  uint32_t* tail_idx = as<uint32_t>(h->tmp[0]);
  uint32_t* tail_count = tail_idx + kHaloMax;
  KS_CUDA(h, cudaMemsetAsync(tail_count, 0, 4, h->stream));
  k_tail_select<<<1, 1024, 0, h->stream>>>(tl_start, tl_dm, (uint32_t)n_tl, tail_idx, kHaloMax, tail_count, h->d_ctl);
  k_upd_save_carry<<<(kHaloMax + 255) / 256, 256, 0, h->stream>>>(st, tl_start, tl_dm, tail_idx, tail_count, n_tl, h->d_ctl);
  h->launches += 2;
  // K2 by row, the runs of equal row, and the merge into the resident rows
  if (n_samples) {
    { int r = mg_zero_u32(h, &h->d_ctl->n_rows, 1); if (r) return r; }
    { int r = mg_zero_u32(h, &h->d_ctl->ticket, 2); if (r) return r; }
    KS_CUDA(h, cudaMemsetAsync(h->row_of_kid, 0xFF, (size_t)(kMaxKeys + 1) * 4, h->stream));
    const int cur = radix_sort16(h, n_samples, bit_length((uint64_t)kUpdMaxKeys + (uint64_t)kUpdMaxKeys * kUpdMaxKeys));
    if (cur < 0) return cur;
    const uint32_t max_rows = (uint32_t)n_samples + 1;
    const uint32_t max_tiles = (uint32_t)((n_samples + kRowsTile - 1) / kRowsTile);
    KS_ENSURE(h, h->tile_cnt, ((size_t)max_tiles + 1) * 4);
    KS_ENSURE(h, h->row_start, ((size_t)max_rows + 2) * 4);
    KS_ENSURE(h, h->row_key, ((size_t)max_rows + 2) * 4);
    RowsArgs r{};
    r.skey = reinterpret_cast<const uint32_t*>(h->samples[cur].p);
    r.key_stride = 4;
    r.n = (uint32_t)n_samples;
    r.tile_cnt = as<uint32_t>(h->tile_cnt);
    r.row_start = as<uint32_t>(h->row_start);
    r.row_key = as<uint32_t>(h->row_key);
    r.row_of_kid = h->row_of_kid;
    r.max_tiles = max_tiles;
    r.max_rows = max_rows;
    r.ctl = h->d_ctl;
    const int grid = (int)std::max<uint32_t>(1, std::min<uint32_t>(max_tiles, (uint32_t)h->sm_count * 8));
    k_rows_count<<<grid, 256, 0, h->stream>>>(r);
    k_rows_scan<<<1, 1024, 0, h->stream>>>(r);
    k_rows_fill<<<grid, 256, 0, h->stream>>>(r);
    KS_ENSURE(h, h->upd_big, ((size_t)max_rows + 1) * 4);
    KS_CUDA(h, cudaMemsetAsync(st.scalars + 6, 0, 4, h->stream));
    UpdArgs u{};
    u.st = st;
    u.big_list = as<uint32_t>(h->upd_big);
    u.items = as<uint4>(h->samples[cur]);
    u.row_start = as<uint32_t>(h->row_start);
    u.row_key = as<uint32_t>(h->row_key);
    u.n_rows_dev = &h->d_ctl->n_rows;
    u.max_rows = max_rows;
    u.ctl = h->d_ctl;
    k_upd_rows<<<(int)std::min<uint64_t>((n_samples + kUpdWarps - 1) / kUpdWarps, (uint64_t)h->sm_count * 16), kUpdWarps * 32, 0, h->stream>>>(u);
    k_upd_big_rows<<<h->sm_count * 4, kUpdBigThreads, 0, h->stream>>>(u);
    h->launches += 5;
    KS_CUDA(h, cudaGetLastError());
  }
  cudaEventRecord(ev[1], h->stream);
  { int r = read_ctl(h); if (r) return r; }                                                           // ---- wait 2
  { int r = upd_status(h, h->h_ctl->err, "ks_update"); if (r) return r; }
  ++h->upd_windows;
  h->upd_records += n;
  if (info) {
    memset(info, 0, sizeof(*info));
    info->n_records = n;
    info->n_solo = h->h_ctl->n_solo;
    info->n_pairs = n_samples - h->h_ctl->n_solo;
    info->n_rows = h->h_ctl->n_rows;  // rows touched by this window
    info->max_duration_ns = h->h_ctl->max_dur;
    info->min_start_ns = h->h_ctl->min_start;
    info->max_start_ns = h->h_ctl->max_start;
    info->was_time_ordered = 1;
    info->ms_total = ev_ms(ev[0], ev[1]);
  }
  return (int64_t)n_samples;
}

int64_t ks_update_table(ks_handle* h) {
  if (!h) return -KS_ERR_ARG;
  if (!h->upd_active) return fail(h, KS_ERR_ARG, "ks_update_table: no resident table (ks_update_begin)");
  if (h->upd_broken) return fail(h, KS_ERR_REBUILD, "ks_update_table: the resident table is no longer valid after an earlier error; begin again");
  KS_CUDA(h, cudaSetDevice(h->device));
  const UpdState st = upd_state(h);
  uint32_t n_ids = 0;
  KS_CUDA(h, cudaMemcpyAsync(&n_ids, st.scalars + 1, 4, cudaMemcpyDeviceToHost, h->stream));
  KS_CUDA(h, cudaStreamSynchronize(h->stream));
  n_ids = std::min(n_ids, kUpdMaxKeys);
  h->n_key_rows = h->n_pair_rows = 0;
  h->pair_rows_src = h->pair_rows.p;
  if (n_ids == 0) return 0;
  // rank the ids by key on the host (a few thousand keys)
  KS_ENSURE(h, h->upd_ranks, (size_t)kUpdMaxKeys * (8 + 4 + 4));
  unsigned long long* d_keys = as<unsigned long long>(h->upd_ranks);
  uint32_t* d_rank_of_id = reinterpret_cast<uint32_t*>(d_keys + kUpdMaxKeys);
  uint32_t* d_id_by_rank = d_rank_of_id + kUpdMaxKeys;
  k_upd_keys_by_id<<<(n_ids + 255) / 256, 256, 0, h->stream>>>(h->dict_keys, h->slot_of_kid, n_ids, d_keys);
  std::vector<unsigned long long> keys(n_ids);
  KS_CUDA(h, cudaMemcpyAsync(keys.data(), d_keys, (size_t)n_ids * 8, cudaMemcpyDeviceToHost, h->stream));
  KS_CUDA(h, cudaStreamSynchronize(h->stream));
  std::vector<uint32_t> id_by_rank(n_ids), rank_of_id(n_ids);
  std::iota(id_by_rank.begin(), id_by_rank.end(), 0u);
  std::sort(id_by_rank.begin(), id_by_rank.end(), [&](uint32_t x, uint32_t y) { return keys[x] < keys[y]; });
  for (uint32_t r = 0; r < n_ids; ++r) rank_of_id[id_by_rank[r]] = r;
  KS_CUDA(h, cudaMemcpyAsync(d_rank_of_id, rank_of_id.data(), (size_t)n_ids * 4, cudaMemcpyHostToDevice, h->stream));
  KS_CUDA(h, cudaMemcpyAsync(d_id_by_rank, id_by_rank.data(), (size_t)n_ids * 4, cudaMemcpyHostToDevice, h->stream));
  // the pair rows that hold samples, ordered by (rank_a, rank_b)
  const uint64_t slots = (uint64_t)n_ids * n_ids;
  for (int i = 0; i < 4; ++i) KS_ENSURE(h, h->upd_list[i], std::max<size_t>(slots * 4, 16));
  uint32_t* k[2] = {as<uint32_t>(h->upd_list[0]), as<uint32_t>(h->upd_list[1])};
  uint32_t* v[2][1] = {{as<uint32_t>(h->upd_list[2])}, {as<uint32_t>(h->upd_list[3])}};
  uint32_t* counter = st.scalars + 8;
  KS_CUDA(h, cudaMemsetAsync(counter, 0, 4, h->stream));
  k_upd_collect<<<(int)std::min<uint64_t>((slots + 255) / 256, (uint64_t)h->sm_count * 16), 256, 0, h->stream>>>(st.rows, d_rank_of_id, n_ids, k[0], v[0][0], counter,
                                                                                                             (uint32_t)slots);
  uint32_t n_pairs = 0;
  KS_CUDA(h, cudaMemcpyAsync(&n_pairs, counter, 4, cudaMemcpyDeviceToHost, h->stream));
  KS_CUDA(h, cudaStreamSynchronize(h->stream));
  const int cur = radix_sort<uint32_t, uint32_t, 1, 16>(h, k, v, n_pairs, nullptr, 0, bit_length((uint64_t)kUpdMaxKeys * kUpdMaxKeys));
  if (cur < 0) return cur;
  KS_ENSURE(h, h->pair_rows, std::max<size_t>(n_pairs, 1) * sizeof(ks_pair_row));
  UpdEmitArgs e{};
  e.st = st;
  e.rows = st.rows;
  e.pair_id = v[cur][0];
  e.n_pairs = n_pairs;
  e.id_by_rank = d_id_by_rank;
  e.slot_of_kid = h->slot_of_kid;
  e.dict_keys = h->dict_keys;
  e.dict_words = h->dict_words;
  e.dict_launches = h->dict_launches;
  e.dict_solo = h->dict_solo;
  e.n_ids = n_ids;
  e.key_rows = h->key_rows;
  e.pair_rows = as<ks_pair_row>(h->pair_rows);
  k_upd_emit_keys<<<(n_ids + 255) / 256, 256, 0, h->stream>>>(e);
  if (n_pairs) k_upd_emit_pairs<<<(n_pairs + 255) / 256, 256, 0, h->stream>>>(e);
  h->launches += 4;
  KS_CUDA(h, cudaGetLastError());
  KS_CUDA(h, cudaStreamSynchronize(h->stream));
  h->n_key_rows = n_ids;
  h->n_pair_rows = n_pairs;
  h->pair_rows_src = h->pair_rows.p;
  return (int64_t)n_pairs;
}

}  // extern "C"
