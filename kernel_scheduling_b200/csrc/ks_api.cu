// ks_api.cu -- the handle, the host-side orchestration of the stages and the extern "C" layer (include/ks_b200.h).
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "ks_common.cuh"
#include "ks_decode.cuh"
#include "ks_dict.cuh"
#include "ks_join.cuh"
#include "ks_mg.cuh"
#include "ks_misc.cuh"
#include "ks_reduce.cuh"
#include "ks_sort.cuh"
#include "ks_tilestats.cuh"
#include "ks_tsv.cuh"
#include "ks_update.cuh"

using namespace ks;

namespace {

struct DevBuf {
  void* p = nullptr;
  size_t cap = 0;
};

}  // namespace

struct ks_handle {
  int device = 0;
  int sm_count = 148;
  cudaStream_t stream = nullptr;
  bool own_stream = false;
  std::string last_error;
  ks_config cfg{};
  bool rows_auto = true;  // max_pair_rows was not given: the row arrays grow to what a trace needs

  Control* d_ctl = nullptr;
  Control* h_ctl = nullptr;  // pinned

  // dictionary (fixed size)
  unsigned long long* dict_keys = nullptr;
  uint4* dict_words = nullptr;
  uint32_t *dict_launches = nullptr, *dict_solo = nullptr;
  unsigned long long* dkeys = nullptr;
  uint32_t *dslot = nullptr, *drank = nullptr, *kid_of_slot = nullptr, *slot_of_kid = nullptr, *row_of_kid = nullptr;
  unsigned long long* keys_sorted = nullptr;
  double* solo_ns = nullptr;
  ks_key_row* key_rows = nullptr;

  // growable
  DevBuf records, tl_start[2], tl_dm[2], solo_stream, keys_tmp;
  DevBuf samples[2];  // the sample stream, 16-byte items {sort key, lane 0, lane 1, lane 2}; two sets for the sort
  DevBuf lookback, hist, tile_cnt, row_start, row_key, stats, big_rows, pair_rows;
  DevBuf large_rows, chunk_row, chunk_idx, large_hist, small_rows, small8_rows, cta_rows;
  DevBuf tmp[6];
  DevBuf stream_store;  // ks_build_table_streamed: the samples of all windows, one region per key range
  // ks_mg_build in stages: the copy engines carry the table rows of a stage to the peers on this stream while the next
  // stage is sorted and reduced on the handle's stream
  cudaStream_t mg_side[1]{};
  cudaEvent_t mg_side_ev[2]{};   // [0]: the rows are written; [1]: the copies are done
  DevBuf tsv_text, tsv_lines, tsv_parsed, tsv_valid, tsv_cnt, tsv_vcnt, tsv_dict, tsv_maps;
  DevBuf tsv_kid, tsv_rowsolo, tsv_label, tsv_logtext, tsv_loglines, tsv_logcnt;
  uint64_t tsv_n_lines = 0, tsv_n_valid = 0, tsv_n_bytes = 0, tsv_max_kid = 0;
  bool tsv_labelled = false;  // ks_tsv_label ran on the parsed text: the solo flag is per row

  // resident table (ks_update_*)
  DevBuf upd_rows, upd_carry, upd_scalars, upd_list[4], upd_ranks, upd_pool, upd_pool2, upd_big;
  uint32_t upd_pool_blocks = 0, upd_pool2_blocks = 0;
  bool upd_active = false, upd_broken = false;
  uint32_t upd_flags = 0;
  uint64_t upd_windows = 0, upd_records = 0;
  const unsigned char* tsv_dev_text = nullptr;

  // results of the last ks_build_table
  uint64_t n_pair_rows = 0, n_key_rows = 0;
  const void* pair_rows_src = nullptr;  // where the last build left its pair rows (ks_copy_pair_rows reads here)
  uint64_t launches = 0;  // kernels launched so far (cumulative)

  // multi-GPU session state (ks_mg_*)
  const unsigned char* mg_rec = nullptr;
  uint64_t mg_n_owned = 0, mg_n_halo = 0, mg_nk = 0, mg_n_samples = 0;
  uint64_t mg_rows_hint = 0;  // rows of the last table of ks_mg_build: sizes the table before the last stage's rows are known
  uint32_t mg_flags = 0;
  int mg_cur = 0;

  // native multi-GPU driver (ks_mg_comm_init / ks_mg_build): an NCCL communicator of this handle's own
  void* mg_comm = nullptr;
  int mg_rank = 0, mg_world = 1;
  uint32_t mg_key_cap = 4096;  // keys per rank that fit the first exchange; grows on every rank alike
  DevBuf mg_block, mg_gathered, mg_recv;
  // peer memory (one process per GPU, buffers shared through CUDA IPC): the sample exchange and the table exchange become
  // plain stores into the other ranks' buffers from the kernels that produce the data
  bool mg_p2p = false;
  struct Exported { void* p = nullptr; size_t cap = 0; unsigned long long gen = 0; cudaIpcMemHandle_t handle{}; } mg_recv_x, mg_table_x;
  struct Imported { void* p = nullptr; unsigned long long gen = 0; } mg_peer_recv[16], mg_peer_table[16];
  std::vector<void*> mg_retired;  // exported buffers that were replaced by larger ones: freed when the session ends
  unsigned char* mg_bar = nullptr;  // device: 16 bytes to send, 16 per rank to receive (the barrier behind peer stores)
  uint32_t* mg_counts = nullptr;        // device: [0] launches in the tail, [1] launches in the halo
  unsigned char* mg_host = nullptr;     // pinned: the headers (and histograms) of all ranks
  size_t mg_host_cap = 0;

  // what the last ks_build_table saw: lets the next call queue every stage without reading counts back in between
  bool attr_sort16 = false, attr_decode = false, attr_seg = false, attr_tile = false;  // kernel attributes set on this handle's device
  bool hint_valid = false;
  uint64_t hint_samples = 0, hint_nk = 0, hint_rows = 0;
  cudaEvent_t ev[12]{};
  cudaEvent_t ev_sort[2]{};  // around the passes of the last sample sort
  int sort_passes = 0;
  // the three size classes of K4 are independent of one another: they run side by side on two helper streams
  cudaStream_t aux[2]{};
  cudaEvent_t fork_ev{}, classify_ev{}, join_ev[2]{};
};

namespace {

thread_local std::string g_null_error;

int fail(ks_handle* h, int code, const std::string& msg) {
  if (h) h->last_error = msg;
  return -code;
}

#define KS_CUDA(h, call)                                                                                            \
  do {                                                                                                              \
    cudaError_t e__ = (call);                                                                                       \
    if (e__ != cudaSuccess) return fail((h), KS_ERR_CUDA, std::string(#call) + ": " + cudaGetErrorString(e__));     \
  } while (0)

int ensure(ks_handle* h, DevBuf& b, size_t bytes) {
  if (bytes <= b.cap) return 0;
  if (b.p) {
    cudaError_t e = cudaFree(b.p);
    b.p = nullptr;
    b.cap = 0;
    if (e != cudaSuccess) return fail(h, KS_ERR_CUDA, std::string("cudaFree: ") + cudaGetErrorString(e));
  }
  const size_t want = (bytes + 255) & ~(size_t)255;
  cudaError_t e = cudaMalloc(&b.p, want);
  if (e != cudaSuccess) return fail(h, KS_ERR_CUDA, "cudaMalloc of " + std::to_string(want) + " bytes: " + cudaGetErrorString(e));
  b.cap = want;
  return 0;
}
#define KS_ENSURE(h, buf, bytes)              \
  do {                                        \
    int r__ = ensure((h), (buf), (bytes));    \
    if (r__) return r__;                      \
  } while (0)

template <typename T>
T* as(const DevBuf& b) { return reinterpret_cast<T*>(b.p); }


int bit_length(uint64_t v) {
  int b = 0;
  while (v) { ++b; v >>= 1; }
  return b;
}

int status_of_err(uint32_t err, bool assume_ordered) {
  if (err & kErrWait) return KS_ERR_WAIT;
  if (err & kErrRecord) return KS_ERR_RECORD;
  if (err & kErrTooManyKeys) return KS_ERR_TOO_MANY_KEYS;
  if ((err & kErrUnordered) && assume_ordered) return KS_ERR_NOT_ORDERED;
  if (err & kErrPairTableFull) return KS_ERR_TABLE_FULL;
  if (err & kErrTooLarge) return KS_ERR_TOO_LARGE;
  if (err & kErrDuplicate) return KS_ERR_DUPLICATE;
  return KS_OK;
}

int read_ctl(ks_handle* h) {
  KS_CUDA(h, cudaMemcpyAsync(h->h_ctl, h->d_ctl, sizeof(Control), cudaMemcpyDeviceToHost, h->stream));
  KS_CUDA(h, cudaStreamSynchronize(h->stream));
  return 0;
}

// ---- K2 driver: sorts (keys, NV payload arrays) on key bits [begin_bit, end_bit); ping-pongs between the given
// buffer sets; returns the index (0/1) of the set that holds the result, or a negative status.
template <typename KeyT, typename ValT, int NV, int ITEMS>
int radix_sort(ks_handle* h, KeyT* keys[2], ValT* vals[2][NV > 0 ? NV : 1], uint64_t n, const uint32_t* n_dev, int begin_bit, int end_bit) {
  if (n >= kSortMaxItems) return fail(h, KS_ERR_TOO_LARGE, "radix sort of 2^30 items or more");
  const int passes = (end_bit - begin_bit + 7) / 8;
  if (passes <= 0 || n == 0) return 0;
  constexpr int TILE = kSortThreads * ITEMS;
  const uint32_t ntiles = (uint32_t)((n + TILE - 1) / TILE);
  const size_t lb_bytes = ((size_t)ntiles * 256 + 64) * sizeof(uint32_t);  // + ticket
  KS_ENSURE(h, h->lookback, lb_bytes);
  KS_ENSURE(h, h->hist, 2 * 8 * 256 * sizeof(uint32_t));
  uint32_t* hist = as<uint32_t>(h->hist);
  uint32_t* gbase = hist + 8 * 256;
  KS_CUDA(h, cudaMemsetAsync(hist, 0, 8 * 256 * sizeof(uint32_t), h->stream));
  const int hist_grid = (int)std::min<uint64_t>((n + 256 * 16 - 1) / (256 * 16), (uint64_t)h->sm_count * 6);
  k_radix_hist<KeyT><<<hist_grid, 256, 0, h->stream>>>(keys[0], 1u, n_dev, (uint32_t)n, begin_bit, end_bit, hist);
  k_radix_scan_hist<<<1, 256, 0, h->stream>>>(hist, gbase, passes);
  h->launches += 2 + passes;
  auto kern = k_onesweep_pass<KeyT, ValT, NV, ITEMS>;
  constexpr size_t smem = sort_smem_bytes<KeyT, ValT, ITEMS>();
  KS_CUDA(h, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));  // per device: set every time
  int cur = 0;
  const int grid = (int)std::min<uint64_t>(ntiles, (uint64_t)h->sm_count * 4);
  for (int p = 0; p < passes; ++p) {
    KS_CUDA(h, cudaMemsetAsync(h->lookback.p, 0, lb_bytes, h->stream));
    SortPassArgs<KeyT, ValT, NV> a{};
    a.kin = keys[cur];
    a.kout = keys[cur ^ 1];
    for (int v = 0; v < NV; ++v) { a.vin[v] = vals[cur][v]; a.vout[v] = vals[cur ^ 1][v]; }
    a.n_dev = n_dev;
    a.n = (uint32_t)n;
    a.shift = begin_bit + 8 * p;
    a.bits = std::min(8, end_bit - a.shift);
    a.gbase = gbase + p * 256;
    a.lookback = as<uint32_t>(h->lookback);
    a.ticket = as<uint32_t>(h->lookback) + (size_t)ntiles * 256;
    a.err = &h->d_ctl->err;
    kern<<<grid, kSortThreads, smem, h->stream>>>(a);
    cur ^= 1;
  }
  KS_CUDA(h, cudaGetLastError());
  return cur;
}

// K2 driver for the 16-byte sample stream: sorts set 0/1 of h->samples on key bits [0, end_bit); returns the set that
// holds the result.  nk_dev: the key count in device memory -- the passes then split the bits of ITS largest sort key
// among them (end_bit only fixes the number of passes; kernels read the count when they run).
// key_base: every key is at least key_base and end_bit counts the bits of key - key_base (a key range of a larger sort)
int radix_sort16(ks_handle* h, uint64_t n, int end_bit, const uint32_t* n_dev = nullptr, const uint4* first_in = nullptr, const uint32_t* nk_dev = nullptr,
                 uint32_t key_base = 0) {
  constexpr int ITEMS = kSort16Items;
  constexpr int THREADS = kSort16Threads;
  constexpr int TILE = THREADS * ITEMS;
  if (n >= kSortMaxItems) return fail(h, KS_ERR_TOO_LARGE, "radix sort of 2^30 items or more");
  const int passes = (end_bit + kSort16MaxBits - 1) / kSort16MaxBits;
  h->sort_passes = passes;
  if (passes <= 0 || n == 0) return 0;
  const uint32_t ntiles = (uint32_t)((n + TILE - 1) / TILE);
  const size_t lb_bytes = ((size_t)ntiles * kSort16Bins + 64) * sizeof(uint32_t);
  KS_ENSURE(h, h->lookback, lb_bytes);
  KS_ENSURE(h, h->hist, 2 * 4 * kSort16Bins * sizeof(uint32_t));
  uint32_t* hist = as<uint32_t>(h->hist);
  uint32_t* gbase = hist + 4 * kSort16Bins;
  KS_CUDA(h, cudaMemsetAsync(hist, 0, 4 * kSort16Bins * sizeof(uint32_t), h->stream));
  const int hist_grid = (int)std::min<uint64_t>((n + 256 * 16 - 1) / (256 * 16), (uint64_t)h->sm_count * 6);
  // first_in: the unsorted items live outside the two sets (a receive buffer); the first pass reads them from there
  const uint4* src0 = first_in ? first_in : as<uint4>(h->samples[0]);
  k_radix_hist16<<<hist_grid, 256, 0, h->stream>>>(src0, n_dev, (uint32_t)n, end_bit, passes, nk_dev, hist, key_base);
  k_radix_scan_hist16<<<1, kSort16Bins, 0, h->stream>>>(hist, gbase, passes);
  h->launches += 2 + passes;
  constexpr size_t smem = sort16_smem_bytes<ITEMS, THREADS>();
  if (!h->attr_sort16) {  // the attribute is per device, so it is remembered per handle
    KS_CUDA(h, cudaFuncSetAttribute(k_onesweep_pass16<ITEMS, THREADS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    h->attr_sort16 = true;
  }
  int cur = 0;
  const int grid = (int)std::min<uint64_t>(ntiles, (uint64_t)h->sm_count * kSort16CtasPerSm);
  for (int p = 0; p < passes; ++p) {
    KS_CUDA(h, cudaMemsetAsync(h->lookback.p, 0, lb_bytes, h->stream));
    if (p == 0 && h->ev_sort[0]) cudaEventRecord(h->ev_sort[0], h->stream);
    SortPass16Args a{};
    a.in = p == 0 ? src0 : as<uint4>(h->samples[cur]);
    a.out = as<uint4>(h->samples[cur ^ 1]);
    a.n_dev = n_dev;
    a.n = (uint32_t)n;
    digit_layout(end_bit, passes, p, &a.shift, &a.bits);
    a.nk_dev = nk_dev;
    a.key_base = key_base;
    a.pass = p;
    a.passes = passes;
    a.unstable = p == 0;
    a.gbase = gbase + p * kSort16Bins;
    a.lookback = as<uint32_t>(h->lookback);
    a.ticket = as<uint32_t>(h->lookback) + (size_t)ntiles * kSort16Bins;
    a.err = &h->d_ctl->err;
    k_onesweep_pass16<ITEMS, THREADS><<<grid, THREADS, smem, h->stream>>>(a);
    if (p == passes - 1 && h->ev_sort[1]) cudaEventRecord(h->ev_sort[1], h->stream);
    cur ^= 1;
  }
  KS_CUDA(h, cudaGetLastError());
  return cur;
}

// stage a host or device input into a device pointer
template <typename T>
int stage_in(ks_handle* h, DevBuf& buf, const T* src, uint64_t count, bool on_device, const T** out) {
  if (on_device) { *out = src; return 0; }
  KS_ENSURE(h, buf, std::max<size_t>(count * sizeof(T), 16));
  KS_CUDA(h, cudaMemcpyAsync(buf.p, src, count * sizeof(T), cudaMemcpyHostToDevice, h->stream));
  *out = as<const T>(buf);
  return 0;
}

int copy_out(ks_handle* h, void* dst, const void* src_dev, size_t bytes, bool on_device) {
  if (bytes == 0) return 0;
  KS_CUDA(h, cudaMemcpyAsync(dst, src_dev, bytes, on_device ? cudaMemcpyDeviceToDevice : cudaMemcpyDeviceToHost, h->stream));
  return 0;
}

int reset_run(ks_handle* h) {
  Control init{};
  init.min_start = ~0ull;
  *h->h_ctl = init;
  KS_CUDA(h, cudaMemcpyAsync(h->d_ctl, h->h_ctl, sizeof(Control), cudaMemcpyHostToDevice, h->stream));
  KS_CUDA(h, cudaMemsetAsync(h->dict_keys, 0, (size_t)kDictSlots * 8, h->stream));
  KS_CUDA(h, cudaMemsetAsync(h->dict_launches, 0, (size_t)kDictSlots * 4, h->stream));
  KS_CUDA(h, cudaMemsetAsync(h->dict_solo, 0, (size_t)kDictSlots * 4, h->stream));
  KS_CUDA(h, cudaMemsetAsync(h->drank, 0, (size_t)(kMaxKeys + 1) * 4, h->stream));
  KS_CUDA(h, cudaMemsetAsync(h->row_of_kid, 0xFF, (size_t)(kMaxKeys + 1) * 4, h->stream));
  return 0;
}

// K1 over device records -> timeline set 0, solo stream, dictionary.  keys_out optional (device).
int run_decode(ks_handle* h, const void* d_records, uint64_t n, uint32_t flags, unsigned long long* keys_out, uint64_t out_offset = 0, uint64_t reserve = 0,
               int halo = 0) {
  KS_ENSURE(h, h->tl_start[0], std::max<size_t>((n + reserve) * 8, 16));
  KS_ENSURE(h, h->tl_dm[0], std::max<size_t>((n + reserve) * 8, 16));
  KS_ENSURE(h, h->solo_stream, std::max<size_t>((n + reserve) * 8, 16));
  if (n == 0) return 0;
  // the bulk copies of K1 read whole 16-byte units: an unaligned source (a slice of a byte buffer) would be a misaligned-
  // address fault on the device, so it is refused here, for every entry point that decodes records
  if (reinterpret_cast<uintptr_t>(d_records) & 15u) return fail(h, KS_ERR_ARG, "records on the device must be 16-byte aligned");
  DecodeArgs a{};
  a.records = reinterpret_cast<const unsigned char*>(d_records);
  a.n = n;
  a.type_mode = (flags & KS_KEY_TYPE) ? 1 : 0;
  a.dict_keys = h->dict_keys;
  a.dict_words = h->dict_words;
  a.dict_launches = h->dict_launches;
  a.dict_solo = h->dict_solo;
  a.tl_start = as<unsigned long long>(h->tl_start[0]) + out_offset;
  a.tl_dm = as<unsigned long long>(h->tl_dm[0]) + out_offset;
  a.halo = halo;
  a.solo_stream = as<unsigned long long>(h->solo_stream);
  a.keys_out = keys_out;
  a.ctl = h->d_ctl;
  if (!h->attr_decode) {
    KS_CUDA(h, cudaFuncSetAttribute(k_decode_hash, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)decode_smem_bytes()));
    h->attr_decode = true;
  }
  const uint64_t ntiles = (n + kDecodeTile - 1) / kDecodeTile;
  const int grid = (int)std::min<uint64_t>(ntiles, (uint64_t)h->sm_count * kDecodeCtasPerSm);
  k_decode_hash<<<grid, kDecodeThreads, decode_smem_bytes(), h->stream>>>(a);
  ++h->launches;
  KS_CUDA(h, cudaGetLastError());
  return 0;
}

// The decode kernel records only the first and the last start in Control::min_start / max_start: the range of an ordered
// trace.  For an unordered one this pass over the timeline extends them to the real range (and reads the control words back).
int start_range_of_unordered(ks_handle* h, const unsigned long long* tl_start, uint64_t n) {
  k_minmax_u64<<<h->sm_count * 2, 256, 0, h->stream>>>(tl_start, n, h->d_ctl);
  ++h->launches;
  KS_CUDA(h, cudaGetLastError());
  return read_ctl(h);
}

// sorts timeline set 0 by start_ns if the decode found it unordered; returns the set that holds the ordered timeline
int order_timeline(ks_handle* h, uint64_t n, bool* was_ordered) {
  *was_ordered = !(h->h_ctl->err & kErrUnordered);
  if (*was_ordered || n < 2) return 0;
  KS_ENSURE(h, h->tl_start[1], n * 8);
  KS_ENSURE(h, h->tl_dm[1], n * 8);
  unsigned long long* keys[2] = {as<unsigned long long>(h->tl_start[0]), as<unsigned long long>(h->tl_start[1])};
  unsigned long long* vals[2][1] = {{as<unsigned long long>(h->tl_dm[0])}, {as<unsigned long long>(h->tl_dm[1])}};
  { int r = start_range_of_unordered(h, keys[0], n); if (r) return r; }
  const int end_bit = bit_length(h->h_ctl->min_start ^ h->h_ctl->max_start);
  return radix_sort<unsigned long long, unsigned long long, 1, 8>(h, keys, vals, n, nullptr, 0, end_bit);
}

int run_dict(ks_handle* h) {
  DictArgs d{};
  d.dict_keys = h->dict_keys;
  d.dkeys = h->dkeys;
  d.dslot = h->dslot;
  d.drank = h->drank;
  d.kid_of_slot = h->kid_of_slot;
  d.slot_of_kid = h->slot_of_kid;
  d.keys_sorted = h->keys_sorted;
  d.ctl = h->d_ctl;
  k_dict_compact<<<kDictSlots / 256, 256, 0, h->stream>>>(d);
  k_dict_rank<<<dim3((kMaxKeys + 255) / 256, kRankSplit), 256, 0, h->stream>>>(d);
  k_dict_place<<<(kMaxKeys + 255) / 256, 256, 0, h->stream>>>(d);
  h->launches += 3;
  KS_CUDA(h, cudaGetLastError());
  return 0;
}

int ensure_samples(ks_handle* h, uint64_t cap) {
  for (int s = 0; s < 2; ++s) {
    KS_ENSURE(h, h->samples[s], cap * 16);
  }
  return 0;
}

uint64_t sample_capacity(ks_handle* h) {
  return std::min<uint64_t>(h->samples[0].cap, h->samples[1].cap) / 16;
}

int run_join(ks_handle* h, int tl, uint64_t n, uint64_t capacity, uint32_t* idx_a, uint32_t* idx_b, uint64_t tl_offset = 0, uint64_t n_halo = 0,
             uint64_t n_own = 0) {
  if (n == 0) return 0;
  JoinArgs j{};
  j.tl_start = as<unsigned long long>(h->tl_start[tl]) + tl_offset;
  j.tl_dm = as<unsigned long long>(h->tl_dm[tl]) + tl_offset;
  j.n_halo = n_halo;
  j.kid_of_slot = h->kid_of_slot;
  j.n = n;
  j.samples = as<uint4>(h->samples[0]);
  j.idx_a = idx_a;
  j.idx_b = idx_b;
  j.capacity = capacity;
  j.ctl = h->d_ctl;
  j.n_own = n_own;
  const unsigned grid = (unsigned)(((n_own ? std::min(n_own, n) : n) + kJoinTile - 1) / kJoinTile);
  if (idx_a) k_join<true><<<grid, kJoinThreads, join_smem_bytes(), h->stream>>>(j);
  else k_join<false><<<grid, kJoinThreads, join_smem_bytes(), h->stream>>>(j);
  ++h->launches;
  KS_CUDA(h, cudaGetLastError());
  return 0;
}

// K4 core: integer statistics of every row (three size classes, see ks_segstats.cuh)
int run_segment_stats(ks_handle* h, const uint4* items, const uint32_t* plain, uint64_t n_values, uint32_t max_rows) {
  const uint32_t max_large = (uint32_t)(n_values / kBigMax) + 1;
  const uint32_t max_chunks = (uint32_t)(n_values / kLargeChunk) + max_large + 1;
  KS_ENSURE(h, h->stats, ((size_t)max_rows + 257) * sizeof(RowStats));
  KS_ENSURE(h, h->big_rows, ((size_t)max_rows + 1) * 4);
  KS_ENSURE(h, h->small_rows, ((size_t)max_rows + 1) * 4);
  KS_ENSURE(h, h->small8_rows, ((size_t)max_rows + 1) * 4);
  KS_ENSURE(h, h->cta_rows, ((size_t)(n_values / kMidMax) + 2) * 4);
  KS_ENSURE(h, h->large_rows, (size_t)max_large * sizeof(LargeRow));
  KS_ENSURE(h, h->chunk_row, (size_t)max_chunks * 4);
  KS_ENSURE(h, h->chunk_idx, (size_t)max_chunks * 4);
  KS_ENSURE(h, h->large_hist, (size_t)max_large * 2 * kLanes * 256 * 4);
  SegArgs s{};
  s.items = items;
  s.plain = plain;
  s.n_lanes = items ? kLanes : 1;
  s.row_start = as<uint32_t>(h->row_start);
  s.n_rows_dev = &h->d_ctl->n_rows;
  s.max_rows = max_rows;
  s.stats = as<RowStats>(h->stats);
  s.mid_rows = as<uint32_t>(h->big_rows);
  s.small_rows = as<uint32_t>(h->small_rows);
  s.small8_rows = as<uint32_t>(h->small8_rows);
  s.big_rows = as<uint32_t>(h->cta_rows);
  s.large = as<LargeRow>(h->large_rows);
  s.chunk_row = as<uint32_t>(h->chunk_row);
  s.chunk_idx = as<uint32_t>(h->chunk_idx);
  s.large_hist = as<uint32_t>(h->large_hist);
  s.max_large = max_large;
  s.max_chunks = max_chunks;
  s.ctl = h->d_ctl;
  const int cgrid = (int)std::max<uint32_t>(1, std::min<uint32_t>((max_rows + 255) / 256, (uint32_t)h->sm_count * 8));
  if (!h->attr_seg) {  // per device, so remembered per handle
    KS_CUDA(h, cudaFuncSetAttribute(k_seg_mid, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)seg_mid_smem_bytes()));
    KS_CUDA(h, cudaFuncSetAttribute(k_seg_big<kBigMax>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)seg_big_smem_bytes<kBigMax>()));
    h->attr_seg = true;
  }
  // Three streams.  The chain of launches of the large rows is the longest path, so it starts first and stays on the main
  // stream; the classification and the other classes run beside it: aux[0] classify, rows of 5..32, big rows; aux[1]
  // (behind the classification) mid rows.  k_segL_final also waits for the classification, which writes zeros into the
  // statistics of every row it does not finish itself.
  KS_CUDA(h, cudaEventRecord(h->fork_ev, h->stream));
  KS_CUDA(h, cudaStreamWaitEvent(h->aux[0], h->fork_ev, 0));
  k_seg_classify<<<cgrid, 256, 0, h->aux[0]>>>(s);
  KS_CUDA(h, cudaEventRecord(h->classify_ev, h->aux[0]));
  KS_CUDA(h, cudaStreamWaitEvent(h->aux[1], h->classify_ev, 0));
  k_seg_mid<<<h->sm_count * 3, kMidWarps * 32, seg_mid_smem_bytes(), h->aux[1]>>>(s);
  k_seg_small<8><<<h->sm_count * 4, 256, 0, h->aux[0]>>>(s);
  k_seg_small<32><<<h->sm_count * 4, 256, 0, h->aux[0]>>>(s);
  k_seg_big<kBigMax><<<h->sm_count * 2, 256, seg_big_smem_bytes<kBigMax>(), h->aux[0]>>>(s);
  KS_CUDA(h, cudaEventRecord(h->join_ev[0], h->aux[0]));
  KS_CUDA(h, cudaEventRecord(h->join_ev[1], h->aux[1]));
  const int lgrid = (int)std::max<uint32_t>(1, std::min<uint32_t>(max_chunks, (uint32_t)h->sm_count * 4));
  k_seg_find_large<<<cgrid, 256, 0, h->stream>>>(s);
  k_segL_reduce<<<lgrid, 256, 0, h->stream>>>(s);
  k_segL_init<<<(max_large * 2 * kLanes + 255) / 256, 256, 0, h->stream>>>(s);
  for (int r = 0; r < kLargeRounds; ++r) {
    s.round = r;
    k_segL_hist<<<lgrid, 256, 0, h->stream>>>(s);
    k_segL_resolve<<<(int)std::min<uint32_t>(max_large, (uint32_t)h->sm_count * 8), 2 * kLanes * 32, 0, h->stream>>>(s);
  }
  KS_CUDA(h, cudaStreamWaitEvent(h->stream, h->classify_ev, 0));
  k_segL_final<<<(max_large + 255) / 256, 256, 0, h->stream>>>(s);
  KS_CUDA(h, cudaStreamWaitEvent(h->stream, h->join_ev[0], 0));
  KS_CUDA(h, cudaStreamWaitEvent(h->stream, h->join_ev[1], 0));
  h->launches += 9 + 2 * kLargeRounds;
  KS_CUDA(h, cudaGetLastError());
  return 0;
}

// rows + segment statistics over sorted samples, n samples (or the count in device memory, bounded by n): one fused pass
// (ks_tilestats.cuh) finishes every row that fits a tile's window; the rows that do not are handed to the CTA-per-row kernel
// (up to kBigMax samples, on a helper stream) and to the chunked chain of the largest rows
int run_rows_and_stats(ks_handle* h, const uint4* items, uint64_t n, uint32_t max_rows, const uint32_t* n_dev = nullptr) {
  const uint32_t max_tiles = (uint32_t)((n + kTsTile - 1) / kTsTile);
  const uint32_t max_large = (uint32_t)(n / kBigMax) + 1;
  const uint32_t max_chunks = (uint32_t)(n / kLargeChunk) + max_large + 1;
  const size_t state_bytes = ((size_t)max_tiles + 64) * 4;  // look-back words + ticket
  KS_ENSURE(h, h->tile_cnt, state_bytes);
  KS_ENSURE(h, h->row_start, ((size_t)max_rows + 2) * 4);
  KS_ENSURE(h, h->row_key, ((size_t)max_rows + 2) * 4);
  KS_ENSURE(h, h->stats, ((size_t)max_rows + 257) * sizeof(RowStats));
  const uint32_t max_deferred = (uint32_t)(n / kTsRowMax) + max_tiles + 2;  // rows above kTsRowMax, and one row per tile that may leave its window
  KS_ENSURE(h, h->small_rows, (size_t)max_deferred * 4);
  KS_ENSURE(h, h->cta_rows, (size_t)max_deferred * 4);
  KS_ENSURE(h, h->big_rows, (size_t)max_deferred * 4);
  KS_ENSURE(h, h->large_rows, (size_t)max_large * sizeof(LargeRow));
  KS_ENSURE(h, h->chunk_row, (size_t)max_chunks * 4);
  KS_ENSURE(h, h->chunk_idx, (size_t)max_chunks * 4);
  KS_ENSURE(h, h->large_hist, (size_t)max_large * 2 * kLanes * 256 * 4);
  if (!h->attr_tile) {  // per device, so remembered per handle
    KS_CUDA(h, cudaFuncSetAttribute(k_tile_stats, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tile_stats_smem_bytes()));
    KS_CUDA(h, cudaFuncSetAttribute(k_seg_big<kBigMax>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)seg_big_smem_bytes<kBigMax>()));
    KS_CUDA(h, cudaFuncSetAttribute(k_seg_big<kBigSmall>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)seg_big_smem_bytes<kBigSmall>()));
    h->attr_tile = true;
  }
  KS_CUDA(h, cudaMemsetAsync(h->tile_cnt.p, 0, state_bytes, h->stream));
  TileStatsArgs t{};
  t.items = items;
  t.n_dev = n_dev;
  t.n = (uint32_t)n;
  t.tile_state = as<uint32_t>(h->tile_cnt);
  t.ticket = as<uint32_t>(h->tile_cnt) + max_tiles + 32;
  t.row_start = as<uint32_t>(h->row_start);
  t.row_key = as<uint32_t>(h->row_key);
  t.row_of_kid = h->row_of_kid;
  t.stats = as<RowStats>(h->stats);
  t.deferred = as<uint32_t>(h->small_rows);
  t.max_deferred = max_deferred;
  t.max_rows = max_rows;
  t.ctl = h->d_ctl;
  const int grid = (int)std::max<uint32_t>(1, std::min<uint32_t>(max_tiles, (uint32_t)h->sm_count * 4));
  k_tile_stats<<<grid, kTsThreads, tile_stats_smem_bytes(), h->stream>>>(t);
  DeferredArgs d{};
  SegArgs& s = d.seg;
  s.items = items;
  s.plain = nullptr;
  s.n_lanes = kLanes;
  s.row_start = as<uint32_t>(h->row_start);
  s.n_rows_dev = &h->d_ctl->n_rows;
  s.max_rows = max_rows;
  s.stats = as<RowStats>(h->stats);
  s.big_rows = as<uint32_t>(h->cta_rows);
  s.mid_rows = as<uint32_t>(h->big_rows);  // rows of up to kBigSmall samples: the CTA-per-row kernel with the small staging area
  s.large = as<LargeRow>(h->large_rows);
  s.chunk_row = as<uint32_t>(h->chunk_row);
  s.chunk_idx = as<uint32_t>(h->chunk_idx);
  s.large_hist = as<uint32_t>(h->large_hist);
  s.max_large = max_large;
  s.max_chunks = max_chunks;
  s.ctl = h->d_ctl;
  d.deferred = as<uint32_t>(h->small_rows);
  d.row_start = as<uint32_t>(h->row_start);
  d.max_deferred = max_deferred;
  k_seg_deferred<<<(int)std::max<uint32_t>(1, std::min<uint32_t>((max_deferred + 255) / 256, (uint32_t)h->sm_count * 4)), 256, 0, h->stream>>>(d);
  // the CTA-per-row kernel beside the chain of the largest rows
  KS_CUDA(h, cudaEventRecord(h->fork_ev, h->stream));
  KS_CUDA(h, cudaStreamWaitEvent(h->aux[0], h->fork_ev, 0));
  k_seg_big<kBigSmall><<<h->sm_count * 6, 256, seg_big_smem_bytes<kBigSmall>(), h->aux[0]>>>(s);
  KS_CUDA(h, cudaEventRecord(h->join_ev[0], h->aux[0]));
  KS_CUDA(h, cudaStreamWaitEvent(h->aux[1], h->fork_ev, 0));
  k_seg_big<kBigMax><<<h->sm_count * 2, 256, seg_big_smem_bytes<kBigMax>(), h->aux[1]>>>(s);
  KS_CUDA(h, cudaEventRecord(h->join_ev[1], h->aux[1]));
  const int lgrid = (int)std::max<uint32_t>(1, std::min<uint32_t>(max_chunks, (uint32_t)h->sm_count * 4));
  k_segL_reduce<<<lgrid, 256, 0, h->stream>>>(s);
  k_segL_init<<<(max_large * 2 * kLanes + 255) / 256, 256, 0, h->stream>>>(s);
  for (int r = 0; r < kLargeRounds; ++r) {
    s.round = r;
    k_segL_hist<<<lgrid, 256, 0, h->stream>>>(s);
    k_segL_resolve<<<(int)std::min<uint32_t>(max_large, (uint32_t)h->sm_count * 8), 2 * kLanes * 32, 0, h->stream>>>(s);
  }
  k_segL_final<<<(max_large + 255) / 256, 256, 0, h->stream>>>(s);
  KS_CUDA(h, cudaStreamWaitEvent(h->stream, h->join_ev[0], 0));
  KS_CUDA(h, cudaStreamWaitEvent(h->stream, h->join_ev[1], 0));
  h->launches += 7 + 2 * kLargeRounds;
  KS_CUDA(h, cudaGetLastError());
  return 0;
}

__global__ void k_stats_to_u64(const RowStats* stats, const uint32_t* row_start, uint32_t n_rows, unsigned long long* out) {
  const uint32_t r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= n_rows) return;
  const RowStats st = stats[r];
  out[6 * (size_t)r + 0] = row_start[r + 1] - row_start[r];
  out[6 * (size_t)r + 1] = st.sum[0];
  out[6 * (size_t)r + 2] = st.mn[0];
  out[6 * (size_t)r + 3] = st.mx[0];
  out[6 * (size_t)r + 4] = st.lo[0];
  out[6 * (size_t)r + 5] = st.hi[0];
}

void mg_native_release(ks_handle* h, bool orderly);  // ks_mg_native.cuh

float ev_ms(cudaEvent_t a, cudaEvent_t b) {
  float ms = 0.f;
  if (cudaEventElapsedTime(&ms, a, b) != cudaSuccess) {  // an event of a stage that did not run in this call: no time, and no
    cudaGetLastError();                                   // error left behind for the next call to trip over
    ms = 0.f;
  }
  return ms;
}

}  // namespace

// =========================================================================================================
extern "C" {

int ks_version(void) { return KS_VERSION; }

const char* ks_status_string(int status) {
  switch (status < 0 ? -status : status) {
    case KS_OK: return "ok";
    case KS_ERR_ARG: return "bad argument";
    case KS_ERR_CUDA: return "CUDA error";
    case KS_ERR_RECORD: return "record with end_ns < start_ns or a duration of 2^31 ns or more";
    case KS_ERR_NOT_ORDERED: return "records are not ordered by start_ns";
    case KS_ERR_TOO_MANY_KEYS: return "more than 65,535 distinct kernel keys";
    case KS_ERR_TABLE_FULL: return "more pair rows than max_pair_rows";
    case KS_ERR_CAPACITY: return "output buffer too small";
    case KS_ERR_WAIT: return "a bounded device-side wait ran out";
    case KS_ERR_DUPLICATE: return "duplicate start_ns inside one file";
    case KS_ERR_TOO_LARGE: return "too many items for one call";
    case KS_ERR_COMM: return "NCCL missing or failed";
    case KS_ERR_REBUILD: return "the resident table is no longer exact: begin again and replay";
    default: return "unknown status";
  }
}

ks_handle* ks_create(int device, void* stream, const ks_config* cfg) {
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess || device < 0 || device >= count) {
    g_null_error = "no such CUDA device";
    return nullptr;
  }
  if (cudaSetDevice(device) != cudaSuccess) return nullptr;
  ks_handle* h = new ks_handle();
  h->device = device;
  cudaDeviceGetAttribute(&h->sm_count, cudaDevAttrMultiProcessorCount, device);
  if (cfg) h->cfg = *cfg;
  h->rows_auto = h->cfg.max_pair_rows == 0;
  if (h->cfg.max_pair_rows == 0) h->cfg.max_pair_rows = 1u << 22;
  bool ok = true;
  if (stream) {
    h->stream = reinterpret_cast<cudaStream_t>(stream);
  } else {
    ok = ok && cudaStreamCreateWithFlags(&h->stream, cudaStreamNonBlocking) == cudaSuccess;
    h->own_stream = true;
  }
  auto alloc = [&](auto** p, size_t bytes) { ok = ok && cudaMalloc(reinterpret_cast<void**>(p), bytes) == cudaSuccess; };
  alloc(&h->d_ctl, sizeof(Control));
  ok = ok && cudaMallocHost(reinterpret_cast<void**>(&h->h_ctl), sizeof(Control)) == cudaSuccess;
  alloc(&h->dict_keys, (size_t)kDictSlots * 8);
  alloc(&h->dict_words, (size_t)kDictSlots * 32);
  alloc(&h->dict_launches, (size_t)kDictSlots * 4);
  alloc(&h->dict_solo, (size_t)kDictSlots * 4);
  alloc(&h->kid_of_slot, (size_t)kDictSlots * 4);
  alloc(&h->dkeys, (size_t)(kMaxKeys + 1) * 8);
  alloc(&h->dslot, (size_t)(kMaxKeys + 1) * 4);
  alloc(&h->drank, (size_t)(kMaxKeys + 1) * 4);
  alloc(&h->slot_of_kid, (size_t)(kMaxKeys + 1) * 4);
  alloc(&h->row_of_kid, (size_t)(kMaxKeys + 1) * 4);
  alloc(&h->keys_sorted, (size_t)(kMaxKeys + 1) * 8);
  alloc(&h->solo_ns, (size_t)(kMaxKeys + 1) * 8);
  alloc(&h->key_rows, (size_t)(kMaxKeys + 1) * sizeof(ks_key_row));
  for (auto& e : h->ev) ok = ok && cudaEventCreate(&e) == cudaSuccess;
  for (auto& e : h->ev_sort) ok = ok && cudaEventCreate(&e) == cudaSuccess;
  for (auto& st : h->aux) ok = ok && cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking) == cudaSuccess;
  for (auto& st : h->mg_side) ok = ok && cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking) == cudaSuccess;
  for (auto& e : h->mg_side_ev) ok = ok && cudaEventCreateWithFlags(&e, cudaEventDisableTiming) == cudaSuccess;
  ok = ok && cudaEventCreateWithFlags(&h->fork_ev, cudaEventDisableTiming) == cudaSuccess;
  ok = ok && cudaEventCreateWithFlags(&h->classify_ev, cudaEventDisableTiming) == cudaSuccess;
  for (auto& e : h->join_ev) ok = ok && cudaEventCreateWithFlags(&e, cudaEventDisableTiming) == cudaSuccess;
  if (ok && h->cfg.max_records) {
    const size_t n = h->cfg.max_records;
    ok = ok && !ensure(h, h->tl_start[0], n * 8) && !ensure(h, h->tl_dm[0], n * 8) && !ensure(h, h->solo_stream, n * 8);
  }
  if (ok && h->cfg.max_pairs) ok = !ensure_samples(h, h->cfg.max_pairs);
  if (!ok) {
    g_null_error = std::string("ks_create: ") + cudaGetErrorString(cudaGetLastError());
    ks_destroy(h);
    return nullptr;
  }
  return h;
}

void ks_destroy(ks_handle* h) {
  if (!h) return;
  cudaSetDevice(h->device);
  if (h->stream) cudaStreamSynchronize(h->stream);
  mg_native_release(h, false);
  auto fr = [](void* p) { if (p) cudaFree(p); };
  for (auto& st : h->mg_side) if (st) cudaStreamSynchronize(st);
  fr(h->d_ctl); fr(h->dict_keys); fr(h->dict_words); fr(h->dict_launches); fr(h->dict_solo); fr(h->kid_of_slot);
  fr(h->dkeys); fr(h->dslot); fr(h->drank); fr(h->slot_of_kid); fr(h->row_of_kid); fr(h->keys_sorted); fr(h->solo_ns); fr(h->key_rows);
  if (h->h_ctl) cudaFreeHost(h->h_ctl);
  DevBuf* bufs[] = {&h->records, &h->tl_start[0], &h->tl_start[1], &h->tl_dm[0], &h->tl_dm[1], &h->solo_stream, &h->keys_tmp,
                    &h->samples[0], &h->samples[1], &h->lookback, &h->hist, &h->tile_cnt, &h->row_start, &h->row_key, &h->stats,
                    &h->big_rows, &h->pair_rows, &h->large_rows, &h->chunk_row, &h->chunk_idx, &h->large_hist, &h->small_rows, &h->small8_rows, &h->cta_rows, &h->tsv_text, &h->tsv_lines, &h->tsv_parsed, &h->tsv_valid, &h->tsv_cnt, &h->tsv_vcnt, &h->tsv_dict, &h->tsv_maps, &h->tsv_kid, &h->tsv_rowsolo, &h->tsv_label, &h->tsv_logtext, &h->tsv_loglines, &h->tsv_logcnt, &h->upd_rows, &h->upd_carry, &h->upd_scalars, &h->upd_list[0], &h->upd_list[1], &h->upd_list[2], &h->upd_list[3], &h->upd_ranks, &h->upd_pool, &h->upd_pool2, &h->upd_big, &h->tmp[0], &h->tmp[1], &h->tmp[2], &h->tmp[3], &h->tmp[4], &h->tmp[5], &h->stream_store};
  for (DevBuf* b : bufs) fr(b->p);
  for (auto& e : h->ev) if (e) cudaEventDestroy(e);
  for (auto& e : h->ev_sort) if (e) cudaEventDestroy(e);
  for (auto& st : h->aux) if (st) { cudaStreamSynchronize(st); cudaStreamDestroy(st); }
  for (auto& st : h->mg_side) if (st) cudaStreamDestroy(st);
  for (auto& e : h->mg_side_ev) if (e) cudaEventDestroy(e);
  if (h->fork_ev) cudaEventDestroy(h->fork_ev);
  if (h->classify_ev) cudaEventDestroy(h->classify_ev);
  for (auto& e : h->join_ev) if (e) cudaEventDestroy(e);
  if (h->own_stream && h->stream) cudaStreamDestroy(h->stream);
  delete h;
}

uint64_t ks_kernel_key(uint32_t name_id, const uint32_t grid[3], const uint32_t block[3], uint32_t smem, uint32_t tenant, uint32_t flags) {
  const uint32_t smem_word = (smem & kSmemMask) | (tenant << 24);
  return kernel_key(name_id, grid[0], grid[1], grid[2], block[0], block[1], block[2], smem_word, (flags & KS_KEY_TYPE) != 0);
}

const char* ks_last_error(ks_handle* h) { return h ? h->last_error.c_str() : g_null_error.c_str(); }
void* ks_stream(ks_handle* h) { return h ? reinterpret_cast<void*>(h->stream) : nullptr; }
uint64_t ks_launch_count(ks_handle* h) { return h ? h->launches : 0; }

// page-locked host memory for inputs and outputs that cross PCIe every call (pageable memory halves the copy rate)
void* ks_pinned_alloc(uint64_t bytes) {
  void* p = nullptr;
  if (cudaMallocHost(&p, bytes ? bytes : 1) != cudaSuccess) { g_null_error = "ks_pinned_alloc: cudaMallocHost failed"; return nullptr; }
  return p;
}
void ks_pinned_free(void* p) { if (p) cudaFreeHost(p); }

// ---------------------------------------------------------------------------------------------------------
int64_t ks_build_table(ks_handle* h, const void* records, uint64_t n, uint32_t flags, ks_table_info* info) {
  if (!h) return -KS_ERR_ARG;
  if ((!records && n) || (flags & ~(KS_ON_DEVICE | KS_ASSUME_TIME_ORDERED | KS_KEY_TYPE))) return fail(h, KS_ERR_ARG, "ks_build_table: bad argument");
  if (n >= kSortMaxItems) return fail(h, KS_ERR_TOO_LARGE, "ks_build_table: 2^30 records or more in one call");
  KS_CUDA(h, cudaSetDevice(h->device));
  const bool assume_ordered = (flags & KS_ASSUME_TIME_ORDERED) != 0;
  // With the caller vouching for the order and the previous call's counts as a guide, every stage is queued without a
  // host round trip; the kernels take the actual counts from device memory, clamped to the bounds the buffers were
  // sized for, and the bounds are checked at the end (a violated guess reruns the call the slow way).
  const bool hinted = assume_ordered && h->hint_valid;
  h->n_pair_rows = h->n_key_rows = 0;
  cudaEvent_t* ev = h->ev;

  cudaEventRecord(ev[0], h->stream);
  const unsigned char* d_rec = nullptr;
  { int r = stage_in<unsigned char>(h, h->records, reinterpret_cast<const unsigned char*>(records), n * 48, (flags & KS_ON_DEVICE) != 0, &d_rec); if (r) return r; }
  if (n && (reinterpret_cast<uintptr_t>(d_rec) & 15u)) return fail(h, KS_ERR_ARG, "ks_build_table: device records must be 16-byte aligned");
  { int r = reset_run(h); if (r) return r; }
  cudaEventRecord(ev[1], h->stream);
  { int r = run_decode(h, d_rec, n, flags, nullptr); if (r) return r; }
  cudaEventRecord(ev[2], h->stream);

  // order the timeline (needs the decode's flags on the host unless the caller vouches for the order)
  int tl = 0;
  bool was_ordered = true;
  if (!assume_ordered) {
    { int r = read_ctl(h); if (r) return r; }
    const int st = status_of_err(h->h_ctl->err, false);
    if (st) return fail(h, st, std::string("ks_build_table: ") + ks_status_string(st));
    tl = order_timeline(h, n, &was_ordered);
    if (tl < 0) return tl;
  }
  cudaEventRecord(ev[3], h->stream);

  { int r = run_dict(h); if (r) return r; }
  cudaEventRecord(ev[4], h->stream);

  // samples: solo launches first, pairs appended by the join; grow and redo if the stream was too small
  uint64_t cap = sample_capacity(h);
  if (cap < std::max<uint64_t>(2 * n, 1u << 16)) {
    cap = std::max<uint64_t>(2 * n, 1u << 16);
    int r = ensure_samples(h, cap);
    if (r) return r;
  }
  uint64_t n_samples = 0;
  for (int attempt = 0; attempt < 2; ++attempt) {
    SoloArgs s{};
    s.solo_stream = as<unsigned long long>(h->solo_stream);
    s.kid_of_slot = h->kid_of_slot;
    s.samples = as<uint4>(h->samples[0]);
    s.capacity = cap;
    s.ctl = h->d_ctl;
    k_solo_samples<<<h->sm_count * 4, 256, 0, h->stream>>>(s);
    ++h->launches;
    if (attempt == 0) cudaEventRecord(ev[5], h->stream);
    { int r = run_join(h, tl, n, cap, nullptr, nullptr); if (r) return r; }
    cudaEventRecord(ev[6], h->stream);
    if (hinted) { n_samples = std::min<uint64_t>(cap, h->hint_samples + h->hint_samples / 4 + 4096); break; }  // a bound, not the count
    { int r = read_ctl(h); if (r) return r; }
    const int st = status_of_err(h->h_ctl->err, assume_ordered);
    if (st) return fail(h, st, std::string("ks_build_table: ") + ks_status_string(st));
    n_samples = h->h_ctl->n_pairs;
    if (n_samples <= cap) break;
    if (n_samples >= kSortMaxItems) return fail(h, KS_ERR_TOO_LARGE, "ks_build_table: 2^30 samples or more");
    if (attempt == 1) return fail(h, KS_ERR_CAPACITY, "ks_build_table: sample stream still too small");
    cap = n_samples + n_samples / 16;
    int r = ensure_samples(h, cap);
    if (r) return r;
  }
  cudaEventRecord(ev[10], h->stream);
  const uint64_t nk = hinted ? h->hint_nk : h->h_ctl->n_keys;
  const uint32_t* n_dev = hinted ? reinterpret_cast<const uint32_t*>(&h->d_ctl->n_pairs) : nullptr;

  // K2: group the samples by sort key.  When the key count is only the previous call's, it fixes the number of passes and
  // the kernels split the bits of the actual largest sort key among them.
  const int end_bit = bit_length(nk + nk * nk);
  const int sort_capacity_bits = ((end_bit + kSort16MaxBits - 1) / kSort16MaxBits) * kSort16MaxBits;
  const int cur = radix_sort16(h, n_samples, end_bit, n_dev, nullptr, hinted ? &h->d_ctl->n_keys : nullptr);
  if (cur < 0) return cur;
  cudaEventRecord(ev[7], h->stream);

  // K4: rows, statistics, tables
  uint32_t max_rows = (uint32_t)std::min<uint64_t>(n_samples, (uint64_t)h->cfg.max_pair_rows + nk) + 1;
  if (hinted) max_rows = (uint32_t)std::min<uint64_t>(max_rows, h->hint_rows + h->hint_rows / 4 + 4096);
  { int r = run_rows_and_stats(h, as<uint4>(h->samples[cur]), n_samples, max_rows, n_dev); if (r) return r; }
  cudaEventRecord(ev[8], h->stream);
  KS_ENSURE(h, h->pair_rows, (size_t)max_rows * sizeof(ks_pair_row));
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
  f.key_rows = h->key_rows;
  f.pair_rows = as<ks_pair_row>(h->pair_rows);
  f.max_pair_rows = max_rows;
  f.ctl = h->d_ctl;
  const uint64_t nk_launch = hinted ? kMaxKeys : nk;  // the kernel clamps to the key count in device memory
  if (nk_launch) k_finalize_keys<<<(unsigned)((nk_launch + 255) / 256), 256, 0, h->stream>>>(f);
  k_finalize_pairs<<<h->sm_count * 4, 256, 0, h->stream>>>(f);
  h->launches += nk_launch ? 2 : 1;
  KS_CUDA(h, cudaGetLastError());
  cudaEventRecord(ev[9], h->stream);
  { int r = read_ctl(h); if (r) return r; }
  if (hinted) {
    const Control& g = *h->h_ctl;
    const bool guess_held = g.n_pairs <= n_samples && bit_length((uint64_t)g.n_keys + (uint64_t)g.n_keys * g.n_keys) <= sort_capacity_bits && g.n_rows <= max_rows &&
                            !(g.err & (kErrTooLarge | kErrPairTableFull));
    if (!guess_held) {  // the trace changed shape: do it again, reading the counts back between the stages
      h->hint_valid = false;
      return ks_build_table(h, records, n, flags, info);
    }
  }
  if ((h->h_ctl->err & kErrTooLarge) && h->rows_auto && h->h_ctl->pad2[0] > h->cfg.max_pair_rows && h->h_ctl->pad2[0] < (1ull << 31)) {
    // more table rows than the arrays were sized for, and no limit was asked for: size them for this trace and run again
    h->cfg.max_pair_rows = (uint32_t)std::min<uint64_t>(h->h_ctl->pad2[0] + h->h_ctl->pad2[0] / 8, 0x7FFFFFFFull);
    h->hint_valid = false;
    return ks_build_table(h, records, n, flags, info);
  }
  const int st = status_of_err(h->h_ctl->err, assume_ordered);
  if (st) { h->hint_valid = false; return fail(h, st, std::string("ks_build_table: ") + ks_status_string(st)); }
  h->hint_valid = true;
  h->hint_samples = h->h_ctl->n_pairs;
  h->hint_nk = h->h_ctl->n_keys;
  h->hint_rows = h->h_ctl->n_rows;
  const uint64_t n_solo = h->h_ctl->n_solo;
  n_samples = h->h_ctl->n_pairs;

  const Control& c = *h->h_ctl;
  h->n_key_rows = c.n_keys;
  h->n_pair_rows = c.n_rows - c.ticket2;
  h->pair_rows_src = h->pair_rows.p;
  if (info) {
    std::memset(info, 0, sizeof(*info));
    info->n_records = n;
    info->n_keys = c.n_keys;
    info->n_solo = n_solo;
    info->n_pairs = n_samples - n_solo;
    info->n_rows = h->n_pair_rows;
    info->max_duration_ns = c.max_dur;
    info->min_start_ns = n ? c.min_start : 0;
    info->max_start_ns = c.max_start;
    info->was_time_ordered = was_ordered && !(c.err & kErrUnordered);
    info->ms_stage_in = ev_ms(ev[0], ev[1]);
    info->ms_decode = ev_ms(ev[1], ev[2]);
    info->ms_order = ev_ms(ev[2], ev[3]);
    info->ms_dict = ev_ms(ev[3], ev[5]);
    info->ms_join = ev_ms(ev[5], ev[6]);
    info->ms_sort = ev_ms(ev[10], ev[7]);
    info->ms_reduce = ev_ms(ev[7], ev[8]);
    info->ms_finalize = ev_ms(ev[8], ev[9]);
    info->ms_total = ev_ms(ev[0], ev[9]);
    info->sort_passes = (uint32_t)h->sort_passes;
    info->ms_sort_pass = h->sort_passes > 0 && n_samples ? ev_ms(h->ev_sort[0], h->ev_sort[1]) / (float)h->sort_passes : 0.f;
  }
  return (int64_t)h->n_pair_rows;
}

// A sort pass whose first tile is never started (the ticket counter begins at 1): the second tile's look-back finds no
// word of tile 0, runs out of polls, sets the error bit and the kernel ends.  What the host then reports is returned.
int64_t ks_selftest_bounded_wait(ks_handle* h) {
  if (!h) return -KS_ERR_ARG;
  KS_CUDA(h, cudaSetDevice(h->device));
  constexpr int ITEMS = kSort16Items;
  constexpr int THREADS = kSort16Threads;
  const uint64_t n = 2 * (uint64_t)THREADS * ITEMS;
  { int r = reset_run(h); if (r) return r; }
  { int r = ensure_samples(h, std::max<uint64_t>(n, sample_capacity(h))); if (r) return r; }
  const size_t lb_bytes = ((size_t)2 * kSort16Bins + 64) * sizeof(uint32_t);
  KS_ENSURE(h, h->lookback, lb_bytes);
  KS_ENSURE(h, h->hist, 2 * 4 * kSort16Bins * sizeof(uint32_t));
  KS_CUDA(h, cudaMemsetAsync(h->lookback.p, 0, lb_bytes, h->stream));
  KS_CUDA(h, cudaMemsetAsync(h->hist.p, 0, 2 * 4 * kSort16Bins * sizeof(uint32_t), h->stream));
  KS_CUDA(h, cudaMemsetAsync(h->samples[0].p, 0, n * 16, h->stream));
  SortPass16Args a{};
  a.in = as<uint4>(h->samples[0]);
  a.out = as<uint4>(h->samples[1]);
  a.n = (uint32_t)n;
  a.bits = 8;
  a.gbase = as<uint32_t>(h->hist);
  a.lookback = as<uint32_t>(h->lookback);
  a.ticket = as<uint32_t>(h->lookback) + (size_t)2 * kSort16Bins;
  a.err = &h->d_ctl->err;
  a.spin_limit = 1u << 12;
  const uint32_t one = 1;
  KS_CUDA(h, cudaMemcpyAsync(a.ticket, &one, 4, cudaMemcpyHostToDevice, h->stream));  // tile 0 is handed to nobody
  constexpr size_t smem = sort16_smem_bytes<ITEMS, THREADS>();
  if (!h->attr_sort16) {
    KS_CUDA(h, cudaFuncSetAttribute(k_onesweep_pass16<ITEMS, THREADS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    h->attr_sort16 = true;
  }
  k_onesweep_pass16<ITEMS, THREADS><<<1, THREADS, smem, h->stream>>>(a);
  ++h->launches;
  KS_CUDA(h, cudaGetLastError());
  { int r = read_ctl(h); if (r) return r; }
  const int st = status_of_err(h->h_ctl->err, true);
  if (st) return fail(h, st, std::string("ks_selftest_bounded_wait: ") + ks_status_string(st));
  return 0;
}

int64_t ks_copy_pair_rows(ks_handle* h, ks_pair_row* dst, uint64_t capacity_rows, uint32_t flags) {
  if (!h || (!dst && h->n_pair_rows)) return -KS_ERR_ARG;
  if (capacity_rows < h->n_pair_rows) return fail(h, KS_ERR_CAPACITY, "ks_copy_pair_rows: buffer too small");
  KS_CUDA(h, cudaSetDevice(h->device));
  { int r = copy_out(h, dst, h->pair_rows_src, h->n_pair_rows * sizeof(ks_pair_row), (flags & KS_ON_DEVICE) != 0); if (r) return r; }
  if (!(flags & KS_ON_DEVICE)) KS_CUDA(h, cudaStreamSynchronize(h->stream));  // device destinations are ordered by the stream
  return (int64_t)h->n_pair_rows;
}

int64_t ks_copy_key_rows(ks_handle* h, ks_key_row* dst, uint64_t capacity_rows, uint32_t flags) {
  if (!h || (!dst && h->n_key_rows)) return -KS_ERR_ARG;
  if (capacity_rows < h->n_key_rows) return fail(h, KS_ERR_CAPACITY, "ks_copy_key_rows: buffer too small");
  KS_CUDA(h, cudaSetDevice(h->device));
  { int r = copy_out(h, dst, h->key_rows, h->n_key_rows * sizeof(ks_key_row), (flags & KS_ON_DEVICE) != 0); if (r) return r; }
  if (!(flags & KS_ON_DEVICE)) KS_CUDA(h, cudaStreamSynchronize(h->stream));
  return (int64_t)h->n_key_rows;
}

// ---------------------------------------------------------------------------------------------------------
int64_t ks_hash_keys(ks_handle* h, const void* records, uint64_t n, uint32_t flags, uint64_t* keys_out) {
  if (!h || ((!records || !keys_out) && n)) return -KS_ERR_ARG;
  KS_CUDA(h, cudaSetDevice(h->device));
  const bool dev = (flags & KS_ON_DEVICE) != 0;
  const unsigned char* d_rec = nullptr;
  { int r = stage_in<unsigned char>(h, h->records, reinterpret_cast<const unsigned char*>(records), n * 48, dev, &d_rec); if (r) return r; }
  unsigned long long* d_keys = reinterpret_cast<unsigned long long*>(keys_out);
  if (!dev) { KS_ENSURE(h, h->keys_tmp, std::max<size_t>(n * 8, 16)); d_keys = as<unsigned long long>(h->keys_tmp); }
  { int r = reset_run(h); if (r) return r; }
  { int r = run_decode(h, d_rec, n, flags, d_keys); if (r) return r; }
  if (!dev) { int r = copy_out(h, keys_out, d_keys, n * 8, false); if (r) return r; }
  { int r = read_ctl(h); if (r) return r; }
  const int st = status_of_err(h->h_ctl->err & (kErrRecord | kErrWait | kErrTooManyKeys), false);
  if (st) return fail(h, st, std::string("ks_hash_keys: ") + ks_status_string(st));
  return (int64_t)n;
}

}  // extern "C"

template <typename KeyT, int ITEMS>
static int64_t sort_pairs_impl(ks_handle* h, KeyT* keys, KeyT* vals, uint64_t n, int begin_bit, int end_bit, uint32_t flags) {
  const int width = (int)sizeof(KeyT) * 8;
  if (!h || (!keys && n) || begin_bit < 0 || end_bit > width || begin_bit > end_bit) return -KS_ERR_ARG;
  KS_CUDA(h, cudaSetDevice(h->device));
  if (n == 0 || begin_bit == end_bit) return (int64_t)n;
  const bool dev = (flags & KS_ON_DEVICE) != 0;
  const size_t bytes = n * sizeof(KeyT);
  KeyT* k[2];
  KeyT* v[2][1];
  KS_ENSURE(h, h->tmp[1], bytes);
  k[1] = as<KeyT>(h->tmp[1]);
  if (dev) { k[0] = keys; }
  else { KS_ENSURE(h, h->tmp[0], bytes); k[0] = as<KeyT>(h->tmp[0]); KS_CUDA(h, cudaMemcpyAsync(k[0], keys, bytes, cudaMemcpyHostToDevice, h->stream)); }
  v[0][0] = v[1][0] = nullptr;
  if (vals) {
    KS_ENSURE(h, h->tmp[3], bytes);
    v[1][0] = as<KeyT>(h->tmp[3]);
    if (dev) { v[0][0] = vals; }
    else { KS_ENSURE(h, h->tmp[2], bytes); v[0][0] = as<KeyT>(h->tmp[2]); KS_CUDA(h, cudaMemcpyAsync(v[0][0], vals, bytes, cudaMemcpyHostToDevice, h->stream)); }
  }
  { int r = reset_run(h); if (r) return r; }
  int cur;
  if (vals) cur = radix_sort<KeyT, KeyT, 1, ITEMS>(h, k, v, n, nullptr, begin_bit, end_bit);
  else cur = radix_sort<KeyT, KeyT, 0, ITEMS>(h, k, v, n, nullptr, begin_bit, end_bit);
  if (cur < 0) return cur;
  if (!dev || cur == 1) {
    KS_CUDA(h, cudaMemcpyAsync(keys, k[cur], bytes, dev ? cudaMemcpyDeviceToDevice : cudaMemcpyDeviceToHost, h->stream));
    if (vals) KS_CUDA(h, cudaMemcpyAsync(vals, v[cur][0], bytes, dev ? cudaMemcpyDeviceToDevice : cudaMemcpyDeviceToHost, h->stream));
  }
  { int r = read_ctl(h); if (r) return r; }
  const int st = status_of_err(h->h_ctl->err, false);
  if (st) return fail(h, st, std::string("ks_sort_pairs: ") + ks_status_string(st));
  return (int64_t)n;
}

extern "C" {

int64_t ks_sort_pairs_u64(ks_handle* h, uint64_t* keys, uint64_t* vals, uint64_t n, int begin_bit, int end_bit, uint32_t flags) {
  return sort_pairs_impl<unsigned long long, 8>(h, reinterpret_cast<unsigned long long*>(keys), reinterpret_cast<unsigned long long*>(vals), n, begin_bit, end_bit, flags);
}
int64_t ks_sort_pairs_u32(ks_handle* h, uint32_t* keys, uint32_t* vals, uint64_t n, int begin_bit, int end_bit, uint32_t flags) {
  return sort_pairs_impl<uint32_t, 16>(h, keys, vals, n, begin_bit, end_bit, flags);
}

int64_t ks_sort_launches(ks_handle* h, const void* records, uint64_t n, uint32_t flags, uint64_t* keys_out, uint64_t* start_out) {
  if (!h || ((!records || !keys_out || !start_out) && n)) return -KS_ERR_ARG;
  KS_CUDA(h, cudaSetDevice(h->device));
  const bool dev = (flags & KS_ON_DEVICE) != 0;
  const unsigned char* d_rec = nullptr;
  { int r = stage_in<unsigned char>(h, h->records, reinterpret_cast<const unsigned char*>(records), n * 48, dev, &d_rec); if (r) return r; }
  KS_ENSURE(h, h->keys_tmp, std::max<size_t>(n * 8, 16));
  KS_ENSURE(h, h->tmp[4], std::max<size_t>(n * 8, 16));
  KS_ENSURE(h, h->tl_start[1], std::max<size_t>(n * 8, 16));
  { int r = reset_run(h); if (r) return r; }
  { int r = run_decode(h, d_rec, n, flags, as<unsigned long long>(h->keys_tmp)); if (r) return r; }
  { int r = read_ctl(h); if (r) return r; }
  { const int st = status_of_err(h->h_ctl->err & (kErrRecord | kErrWait | kErrTooManyKeys), false); if (st) return fail(h, st, std::string("ks_sort_launches: ") + ks_status_string(st)); }
  // by start_ns first (payload: the key), then stably by key: (key, start_ns) order
  unsigned long long* a[2] = {as<unsigned long long>(h->tl_start[0]), as<unsigned long long>(h->tl_start[1])};
  unsigned long long* b[2][1] = {{as<unsigned long long>(h->keys_tmp)}, {as<unsigned long long>(h->tmp[4])}};
  int cur = 0;
  if ((h->h_ctl->err & kErrUnordered) && n > 1) {
    { int r = start_range_of_unordered(h, a[0], n); if (r) return r; }
    cur = radix_sort<unsigned long long, unsigned long long, 1, 8>(h, a, b, n, nullptr, 0, bit_length(h->h_ctl->min_start ^ h->h_ctl->max_start));
    if (cur < 0) return cur;
  }
  unsigned long long* k2[2] = {b[cur][0], b[cur ^ 1][0]};
  unsigned long long* v2[2][1] = {{a[cur]}, {a[cur ^ 1]}};
  const int cur2 = radix_sort<unsigned long long, unsigned long long, 1, 8>(h, k2, v2, n, nullptr, 0, 64);
  if (cur2 < 0) return cur2;
  { int r = copy_out(h, keys_out, k2[cur2], n * 8, dev); if (r) return r; }
  { int r = copy_out(h, start_out, v2[cur2][0], n * 8, dev); if (r) return r; }
  { int r = read_ctl(h); if (r) return r; }
  { const int st = status_of_err(h->h_ctl->err & kErrWait, false); if (st) return fail(h, st, "ks_sort_launches: bounded wait ran out"); }
  return (int64_t)n;
}

int64_t ks_join_overlaps(ks_handle* h, const void* records, uint64_t n, uint32_t flags, uint32_t* idx_a, uint32_t* idx_b, uint64_t capacity) {
  if (!h || (!records && n) || (capacity && (!idx_a || !idx_b))) return -KS_ERR_ARG;
  if (n >= kSortMaxItems) return fail(h, KS_ERR_TOO_LARGE, "ks_join_overlaps: 2^30 records or more");
  KS_CUDA(h, cudaSetDevice(h->device));
  const bool dev = (flags & KS_ON_DEVICE) != 0;
  const unsigned char* d_rec = nullptr;
  { int r = stage_in<unsigned char>(h, h->records, reinterpret_cast<const unsigned char*>(records), n * 48, dev, &d_rec); if (r) return r; }
  { int r = reset_run(h); if (r) return r; }
  { int r = run_decode(h, d_rec, n, flags, nullptr); if (r) return r; }
  { int r = read_ctl(h); if (r) return r; }
  { const int st = status_of_err(h->h_ctl->err, false); if (st) return fail(h, st, std::string("ks_join_overlaps: ") + ks_status_string(st)); }
  bool was_ordered;
  const int tl = order_timeline(h, n, &was_ordered);
  if (tl < 0) return tl;
  { int r = run_dict(h); if (r) return r; }
  uint32_t *da = idx_a, *db = idx_b;
  if (!dev) {
    KS_ENSURE(h, h->tmp[0], std::max<size_t>(capacity * 4, 16));
    KS_ENSURE(h, h->tmp[1], std::max<size_t>(capacity * 4, 16));
    da = as<uint32_t>(h->tmp[0]);
    db = as<uint32_t>(h->tmp[1]);
  } else if (!capacity) {
    KS_ENSURE(h, h->tmp[0], 16);
    da = db = as<uint32_t>(h->tmp[0]);
  }
  { int r = run_join(h, tl, n, capacity, da, db); if (r) return r; }
  { int r = read_ctl(h); if (r) return r; }
  const uint64_t p = h->h_ctl->n_pairs;
  if (!dev && p <= capacity) {
    { int r = copy_out(h, idx_a, da, p * 4, false); if (r) return r; }
    { int r = copy_out(h, idx_b, db, p * 4, false); if (r) return r; }
    KS_CUDA(h, cudaStreamSynchronize(h->stream));
  }
  return (int64_t)p;
}

int64_t ks_segment_stats(ks_handle* h, const uint32_t* values, const uint64_t* offsets, uint64_t n_segments, uint32_t flags, uint64_t* out) {
  if (!h || !offsets || (n_segments && !out)) return -KS_ERR_ARG;
  if (n_segments >= (1ull << 31)) return fail(h, KS_ERR_TOO_LARGE, "ks_segment_stats: too many segments");
  KS_CUDA(h, cudaSetDevice(h->device));
  if (n_segments == 0) return 0;
  const bool dev = (flags & KS_ON_DEVICE) != 0;
  uint64_t n_values;
  const unsigned long long* d_off = nullptr;
  { int r = stage_in<unsigned long long>(h, h->tmp[0], reinterpret_cast<const unsigned long long*>(offsets), n_segments + 1, dev, &d_off); if (r) return r; }
  if (dev) { KS_CUDA(h, cudaMemcpyAsync(&n_values, offsets + n_segments, 8, cudaMemcpyDeviceToHost, h->stream)); KS_CUDA(h, cudaStreamSynchronize(h->stream)); }
  else n_values = offsets[n_segments];
  if (n_values >= (1ull << 32)) return fail(h, KS_ERR_TOO_LARGE, "ks_segment_stats: 2^32 values or more");
  if (!values && n_values) return -KS_ERR_ARG;
  const uint32_t* d_val = nullptr;
  { int r = stage_in<uint32_t>(h, h->tmp[1], values, n_values, dev, &d_val); if (r) return r; }
  { int r = reset_run(h); if (r) return r; }
  const uint32_t rows = (uint32_t)n_segments;
  KS_ENSURE(h, h->row_start, ((size_t)rows + 2) * 4);
  KS_ENSURE(h, h->tmp[2], (size_t)rows * 48);
  k_offsets_to_u32<<<(rows + 1 + 255) / 256, 256, 0, h->stream>>>(d_off, rows + 1, as<uint32_t>(h->row_start));
  h->h_ctl->n_rows = rows;
  KS_CUDA(h, cudaMemcpyAsync(&h->d_ctl->n_rows, &h->h_ctl->n_rows, 4, cudaMemcpyHostToDevice, h->stream));
  { int r = run_segment_stats(h, nullptr, d_val, n_values, rows); if (r) return r; }
  unsigned long long* d_out = dev ? reinterpret_cast<unsigned long long*>(out) : as<unsigned long long>(h->tmp[2]);
  k_stats_to_u64<<<(rows + 255) / 256, 256, 0, h->stream>>>(as<RowStats>(h->stats), as<uint32_t>(h->row_start), rows, d_out);
  KS_CUDA(h, cudaGetLastError());
  if (!dev) { int r = copy_out(h, out, d_out, (size_t)rows * 48, false); if (r) return r; }
  KS_CUDA(h, cudaStreamSynchronize(h->stream));
  return (int64_t)n_segments;
}

int64_t ks_count_batches(ks_handle* h, const uint64_t* start1, uint64_t n1, const uint64_t* start2, uint64_t n2, uint32_t flags, uint64_t out[2]) {
  if (!h || !out || (!start1 && n1) || (!start2 && n2)) return -KS_ERR_ARG;
  KS_CUDA(h, cudaSetDevice(h->device));
  const bool dev = (flags & KS_ON_DEVICE) != 0;
  { int r = reset_run(h); if (r) return r; }
  // private copies: the sort works in place
  unsigned long long* s[2][2];
  const uint64_t* src[2] = {start1, start2};
  const uint64_t cnt[2] = {n1, n2};
  for (int f = 0; f < 2; ++f) {
    KS_ENSURE(h, h->tmp[2 * f], std::max<size_t>(cnt[f] * 8, 16));
    KS_ENSURE(h, h->tmp[2 * f + 1], std::max<size_t>(cnt[f] * 8, 16));
    s[f][0] = as<unsigned long long>(h->tmp[2 * f]);
    s[f][1] = as<unsigned long long>(h->tmp[2 * f + 1]);
    if (cnt[f]) KS_CUDA(h, cudaMemcpyAsync(s[f][0], src[f], cnt[f] * 8, dev ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice, h->stream));
    if (cnt[f]) k_minmax_u64<<<h->sm_count * 2, 256, 0, h->stream>>>(s[f][0], cnt[f], h->d_ctl);
  }
  { int r = read_ctl(h); if (r) return r; }
  const int end_bit = bit_length(h->h_ctl->min_start ^ h->h_ctl->max_start);
  const unsigned long long* sorted[2];
  for (int f = 0; f < 2; ++f) {
    unsigned long long* k[2] = {s[f][0], s[f][1]};
    unsigned long long* v[2][1] = {{nullptr}, {nullptr}};
    const int cur = radix_sort<unsigned long long, unsigned long long, 0, 8>(h, k, v, cnt[f], nullptr, 0, end_bit);
    if (cur < 0) return cur;
    sorted[f] = k[cur];
  }
  if (n1 || n2) k_count_batches<<<h->sm_count * 4, 256, 0, h->stream>>>(sorted[0], n1, sorted[1], n2, h->d_ctl);
  KS_CUDA(h, cudaGetLastError());
  { int r = read_ctl(h); if (r) return r; }
  const int st = status_of_err(h->h_ctl->err, false);
  if (st) return fail(h, st, std::string("ks_count_batches: ") + ks_status_string(st));
  const uint64_t both = h->h_ctl->batches_both;
  out[0] = n1 + n2 - 2 * both;
  out[1] = both;
  return (int64_t)(out[0] + out[1]);
}

int64_t ks_combine_duplicates(ks_handle* h, const uint32_t* group, const double* launches, const double* values, uint64_t rows, uint32_t cols,
                              uint32_t n_groups, uint32_t flags, double* out_total, double* out_means) {
  if (!h || ((!group || !launches) && rows) || (!values && rows && cols) || (n_groups && (!out_total || (!out_means && cols)))) return -KS_ERR_ARG;
  if (rows >= kSortMaxItems) return fail(h, KS_ERR_TOO_LARGE, "ks_combine_duplicates: too many rows");
  KS_CUDA(h, cudaSetDevice(h->device));
  if (n_groups == 0) return 0;
  const bool dev = (flags & KS_ON_DEVICE) != 0;
  { int r = reset_run(h); if (r) return r; }
  // sort row indices by group (stable) -> order[]
  const size_t rb = std::max<size_t>(rows * 4, 16);
  DevBuf* t = h->tmp;
  KS_ENSURE(h, t[0], rb); KS_ENSURE(h, t[1], rb); KS_ENSURE(h, t[2], rb); KS_ENSURE(h, t[3], rb);
  uint32_t* k[2] = {as<uint32_t>(t[0]), as<uint32_t>(t[1])};
  uint32_t* v[2][1] = {{as<uint32_t>(t[2])}, {as<uint32_t>(t[3])}};
  if (rows) {
    KS_CUDA(h, cudaMemcpyAsync(k[0], group, rows * 4, dev ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice, h->stream));
    k_iota<<<(unsigned)((rows + 255) / 256), 256, 0, h->stream>>>(v[0][0], (uint32_t)rows);
  }
  const int cur = radix_sort<uint32_t, uint32_t, 1, 16>(h, k, v, rows, nullptr, 0, bit_length(n_groups ? n_groups - 1 : 0));
  if (cur < 0) return cur;
  KS_ENSURE(h, t[4], ((size_t)n_groups + 2) * 4);
  uint32_t* seg = as<uint32_t>(t[4]);
  k_group_offsets<<<(unsigned)((rows + 1 + 255) / 256), 256, 0, h->stream>>>(k[cur], (uint32_t)rows, n_groups, seg);
  const double *d_l = nullptr, *d_v = nullptr;
  { int r = stage_in<double>(h, h->keys_tmp, launches, rows, dev, &d_l); if (r) return r; }
  { int r = stage_in<double>(h, h->tl_start[1], values, rows * cols, dev, &d_v); if (r) return r; }
  double *d_tot = out_total, *d_mean = out_means;
  if (!dev) {
    KS_ENSURE(h, t[5], ((size_t)n_groups * (cols + 1)) * 8 + 16);
    d_tot = as<double>(t[5]);
    d_mean = d_tot + n_groups;
  }
  const uint64_t threads = (uint64_t)n_groups * (cols + 1);
  k_combine_duplicates<<<(unsigned)((threads + 255) / 256), 256, 0, h->stream>>>(v[cur][0], seg, d_l, d_v, cols, n_groups, d_tot, d_mean);
  KS_CUDA(h, cudaGetLastError());
  if (!dev) {
    { int r = copy_out(h, out_total, d_tot, (size_t)n_groups * 8, false); if (r) return r; }
    { int r = copy_out(h, out_means, d_mean, (size_t)n_groups * cols * 8, false); if (r) return r; }
  }
  { int r = read_ctl(h); if (r) return r; }
  const int st = status_of_err(h->h_ctl->err, false);
  if (st) return fail(h, st, std::string("ks_combine_duplicates: ") + ks_status_string(st));
  return (int64_t)n_groups;
}

int64_t ks_pool_launches(ks_handle* h, const uint32_t* group, const double* values, uint64_t rows, uint32_t cols, uint32_t n_groups, uint32_t flags,
                         uint64_t* out_launches, double* out_mean, double* out_std) {
  if (!h || (!group && rows) || (!values && rows && cols) || (n_groups && (!out_launches || ((!out_mean || !out_std) && cols)))) return -KS_ERR_ARG;
  if (rows >= kSortMaxItems) return fail(h, KS_ERR_TOO_LARGE, "ks_pool_launches: too many rows");
  KS_CUDA(h, cudaSetDevice(h->device));
  if (n_groups == 0) return 0;
  const bool dev = (flags & KS_ON_DEVICE) != 0;
  { int r = reset_run(h); if (r) return r; }
  // sort row indices by group (stable) -> order[]
  const size_t rb = std::max<size_t>(rows * 4, 16);
  DevBuf* t = h->tmp;
  KS_ENSURE(h, t[0], rb); KS_ENSURE(h, t[1], rb); KS_ENSURE(h, t[2], rb); KS_ENSURE(h, t[3], rb);
  uint32_t* k[2] = {as<uint32_t>(t[0]), as<uint32_t>(t[1])};
  uint32_t* v[2][1] = {{as<uint32_t>(t[2])}, {as<uint32_t>(t[3])}};
  if (rows) {
    KS_CUDA(h, cudaMemcpyAsync(k[0], group, rows * 4, dev ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice, h->stream));
    k_iota<<<(unsigned)((rows + 255) / 256), 256, 0, h->stream>>>(v[0][0], (uint32_t)rows);
  }
  const int cur = radix_sort<uint32_t, uint32_t, 1, 16>(h, k, v, rows, nullptr, 0, bit_length(n_groups ? n_groups - 1 : 0));
  if (cur < 0) return cur;
  KS_ENSURE(h, t[4], ((size_t)n_groups + 2) * 4);
  uint32_t* seg = as<uint32_t>(t[4]);
  k_group_offsets<<<(unsigned)((rows + 1 + 255) / 256), 256, 0, h->stream>>>(k[cur], (uint32_t)rows, n_groups, seg);
  const double* d_v = nullptr;
  { int r = stage_in<double>(h, h->tl_start[1], values, rows * cols, dev, &d_v); if (r) return r; }
  unsigned long long* d_cnt = reinterpret_cast<unsigned long long*>(out_launches);
  double *d_mean = out_mean, *d_std = out_std;
  if (!dev) {
    KS_ENSURE(h, t[5], ((size_t)n_groups * (2 * (size_t)cols + 1)) * 8 + 16);
    d_cnt = as<unsigned long long>(t[5]);
    d_mean = reinterpret_cast<double*>(d_cnt + n_groups);
    d_std = d_mean + (size_t)n_groups * cols;
  }
  const uint64_t threads = (uint64_t)n_groups * (cols + 1);
  k_pool_launches<<<(unsigned)((threads + 255) / 256), 256, 0, h->stream>>>(v[cur][0], seg, d_v, cols, n_groups, d_cnt, d_mean, d_std);
  ++h->launches;
  KS_CUDA(h, cudaGetLastError());
  if (!dev) {
    { int r = copy_out(h, out_launches, d_cnt, (size_t)n_groups * 8, false); if (r) return r; }
    { int r = copy_out(h, out_mean, d_mean, (size_t)n_groups * cols * 8, false); if (r) return r; }
    { int r = copy_out(h, out_std, d_std, (size_t)n_groups * cols * 8, false); if (r) return r; }
  }
  { int r = read_ctl(h); if (r) return r; }
  const int st = status_of_err(h->h_ctl->err, false);
  if (st) return fail(h, st, std::string("ks_pool_launches: ") + ks_status_string(st));
  return (int64_t)n_groups;
}

}  // extern "C"

// =========================================================================================================
// Multi-GPU session: one handle per rank, the caller (kernel_scheduling_b200/parallel.py) runs the collectives between
// the phases.  All pointers are DEVICE pointers on the handle's device.
namespace {

int mg_zero_u32(ks_handle* h, uint32_t* field, size_t count = 1) {
  KS_CUDA(h, cudaMemsetAsync(field, 0, count * sizeof(uint32_t), h->stream));
  return 0;
}

int mg_status(ks_handle* h, const char* what) {
  const int st = status_of_err(h->h_ctl->err, true);
  if (st) return fail(h, st, std::string(what) + ": " + ks_status_string(st));
  return 0;
}

// K2 + K4 over the n samples in sample set 0 (this rank's key range), then the solo times of the keys reduced here.
// Queues only; the caller reads the control words back.
// [key_lo, key_hi): the sort keys the samples can have (0, 0: any), so that a key range is sorted over the bits of its width
int mg_reduce_queue(ks_handle* h, uint64_t n, const uint4* first_in = nullptr, bool solo = true, uint64_t key_lo = 0, uint64_t key_hi = 0) {
  // counters of the row / statistics kernels start from zero
  { int r = mg_zero_u32(h, &h->d_ctl->n_rows, 2); if (r) return r; }
  { int r = mg_zero_u32(h, &h->d_ctl->ticket, 2); if (r) return r; }
  KS_CUDA(h, cudaMemsetAsync(&h->d_ctl->scratch0, 0, 8, h->stream));
  KS_CUDA(h, cudaMemsetAsync(&h->d_ctl->pad[0], 0, 4 * 8 + 8, h->stream));
  KS_CUDA(h, cudaMemsetAsync(&h->d_ctl->pad2[1], 0, 8, h->stream));
  KS_CUDA(h, cudaMemsetAsync(h->row_of_kid, 0xFF, (size_t)(kMaxKeys + 1) * 4, h->stream));
  const uint64_t nk = h->mg_nk;
  const int cur = key_hi > key_lo ? radix_sort16(h, n, std::max(1, bit_length(key_hi - key_lo - 1)), nullptr, first_in, nullptr, (uint32_t)key_lo)
                                  : radix_sort16(h, n, bit_length(nk + nk * nk), nullptr, first_in);
  if (cur < 0) return cur;
  h->mg_cur = cur;
  h->mg_n_samples = n;
  const uint32_t max_rows = (uint32_t)std::min<uint64_t>(n, (uint64_t)h->cfg.max_pair_rows + nk) + 1;
  { int r = run_rows_and_stats(h, as<uint4>(h->samples[cur]), n, max_rows); if (r) return r; }
  if (nk && solo) {  // (a range known to hold no solo rows leaves the solo times alone: another stream may be reading them)
    k_solo_ns<<<(unsigned)((nk + 255) / 256), 256, 0, h->stream>>>(as<RowStats>(h->stats), h->row_of_kid, (uint32_t)nk, h->solo_ns);
    ++h->launches;
  }
  return 0;
}

// key rows of every key (keys = true) and the pair rows of this rank's range (written to `out`, room for max_rows)
int mg_finalize_queue(ks_handle* h, ks_pair_row* out, uint32_t max_rows, uint32_t n_peers = 0, ks_pair_row* const* peers = nullptr, bool keys = true) {
  const uint64_t nk = h->mg_nk;
  cudaStream_t stream = h->stream;
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
  f.pair_rows = out;
  f.max_pair_rows = max_rows;
  f.ctl = h->d_ctl;
  f.n_peer_tables = n_peers;
  for (uint32_t q = 0; q < n_peers; ++q) f.peer_rows[q] = peers[q];
  if (nk && keys) k_finalize_keys<<<(unsigned)((nk + 255) / 256), 256, 0, stream>>>(f);
  k_finalize_pairs<<<h->sm_count * 4, 256, 0, stream>>>(f);
  h->launches += nk && keys ? 2 : 1;
  KS_CUDA(h, cudaGetLastError());
  return 0;
}

}  // namespace

extern "C" {

int64_t ks_mg_begin(ks_handle* h, const void* records, uint64_t n_owned, uint32_t flags) {
  if (!h || (!records && n_owned) || (flags & ~KS_KEY_TYPE)) return -KS_ERR_ARG;
  if (n_owned + kHaloMax >= kSortMaxItems) return fail(h, KS_ERR_TOO_LARGE, "ks_mg_begin: too many records for one rank");
  KS_CUDA(h, cudaSetDevice(h->device));
  if (n_owned && (reinterpret_cast<uintptr_t>(records) & 15u)) return fail(h, KS_ERR_ARG, "ks_mg_begin: records must be 16-byte aligned");
  h->mg_rec = reinterpret_cast<const unsigned char*>(records);
  h->mg_n_owned = n_owned;
  h->mg_n_halo = 0;
  h->mg_flags = flags;
  h->n_pair_rows = h->n_key_rows = 0;
  { int r = reset_run(h); if (r) return r; }
  // sized once for window + halo so that the halo decode cannot trigger a (content-losing) regrowth
  return run_decode(h, records, n_owned, flags, nullptr, kHaloMax, 2 * (uint64_t)kHaloMax, 0);
}

int64_t ks_mg_tail(ks_handle* h, void* out_records, uint64_t capacity) {
  if (!h || (!out_records && capacity)) return -KS_ERR_ARG;
  KS_CUDA(h, cudaSetDevice(h->device));
  KS_ENSURE(h, h->tmp[0], (size_t)kHaloMax * 4 + 16);
  uint32_t* idx = as<uint32_t>(h->tmp[0]);
  uint32_t* count = idx + kHaloMax;
  { int r = mg_zero_u32(h, count); if (r) return r; }
  if (h->mg_n_owned) {
    k_tail_select<<<1, 1024, 0, h->stream>>>(as<unsigned long long>(h->tl_start[0]) + kHaloMax, as<unsigned long long>(h->tl_dm[0]) + kHaloMax,
                                             (uint32_t)h->mg_n_owned, idx, kHaloMax, count, h->d_ctl);
    ++h->launches;
  }
  uint32_t n_tail = 0;
  KS_CUDA(h, cudaMemcpyAsync(&n_tail, count, 4, cudaMemcpyDeviceToHost, h->stream));
  { int r = read_ctl(h); if (r) return r; }
  { int r = mg_status(h, "ks_mg_tail"); if (r) return r; }
  if (n_tail > kHaloMax || n_tail > capacity) return fail(h, KS_ERR_CAPACITY, "ks_mg_tail: more launches reach into the next window than the halo can hold");
  if (n_tail) {
    k_gather_records<<<(n_tail * 3 + 255) / 256, 256, 0, h->stream>>>(reinterpret_cast<const uint4*>(h->mg_rec), idx, n_tail, reinterpret_cast<uint4*>(out_records));
    ++h->launches;
  }
  return (int64_t)n_tail;
}

int64_t ks_mg_halo(ks_handle* h, const void* halo_records, uint64_t n_halo) {
  if (!h || (!halo_records && n_halo)) return -KS_ERR_ARG;
  if (n_halo > kHaloMax) return fail(h, KS_ERR_CAPACITY, "ks_mg_halo: halo larger than the reserve");
  KS_CUDA(h, cudaSetDevice(h->device));
  h->mg_n_halo = n_halo;
  if (!n_halo) return 0;
  // the halo records must be in start order themselves; the tail selection emits them unordered, so sort is the caller's job
  return run_decode(h, halo_records, n_halo, h->mg_flags, nullptr, kHaloMax - n_halo, h->mg_n_owned + 2 * (uint64_t)kHaloMax - n_halo, 1);
}

int64_t ks_mg_local_keys(ks_handle* h, uint64_t* keys_out, void* words_out, uint64_t capacity) {
  if (!h || !keys_out || !words_out) return -KS_ERR_ARG;
  KS_CUDA(h, cudaSetDevice(h->device));
  { int r = mg_zero_u32(h, &h->d_ctl->n_keys); if (r) return r; }
  DictArgs d{};
  d.dict_keys = h->dict_keys; d.dkeys = h->dkeys; d.dslot = h->dslot; d.drank = h->drank; d.kid_of_slot = h->kid_of_slot;
  d.slot_of_kid = h->slot_of_kid; d.keys_sorted = h->keys_sorted; d.ctl = h->d_ctl;
  k_dict_compact<<<kDictSlots / 256, 256, 0, h->stream>>>(d);
  ++h->launches;
  { int r = read_ctl(h); if (r) return r; }
  { int r = mg_status(h, "ks_mg_local_keys"); if (r) return r; }
  const uint32_t nk = h->h_ctl->n_keys;
  if (nk > capacity) return fail(h, KS_ERR_CAPACITY, "ks_mg_local_keys: buffer too small");
  if (nk) {
    k_export_keys<<<(nk + 255) / 256, 256, 0, h->stream>>>(h->dkeys, h->dslot, h->dict_words, nk, reinterpret_cast<unsigned long long*>(keys_out),
                                                           reinterpret_cast<uint4*>(words_out));
    ++h->launches;
  }
  return (int64_t)nk;
}

int64_t ks_mg_global_keys(ks_handle* h, const uint64_t* keys, const void* words, uint64_t n) {
  if (!h || ((!keys || !words) && n)) return -KS_ERR_ARG;
  KS_CUDA(h, cudaSetDevice(h->device));
  if (n) {
    k_dict_insert<<<(unsigned)((n + 255) / 256), 256, 0, h->stream>>>(reinterpret_cast<const unsigned long long*>(keys), reinterpret_cast<const uint4*>(words),
                                                                      (uint32_t)n, h->dict_keys, h->dict_words, h->d_ctl);
    ++h->launches;
  }
  { int r = mg_zero_u32(h, &h->d_ctl->n_keys); if (r) return r; }
  KS_CUDA(h, cudaMemsetAsync(h->drank, 0, (size_t)(kMaxKeys + 1) * 4, h->stream));
  { int r = run_dict(h); if (r) return r; }
  { int r = read_ctl(h); if (r) return r; }
  { int r = mg_status(h, "ks_mg_global_keys"); if (r) return r; }
  h->mg_nk = h->h_ctl->n_keys;
  return (int64_t)h->mg_nk;
}

int64_t ks_mg_counts(ks_handle* h, uint64_t* launches, uint64_t* solo, int import) {
  if (!h || !launches || !solo) return -KS_ERR_ARG;
  KS_CUDA(h, cudaSetDevice(h->device));
  if (h->mg_nk) {
    k_counts_by_kid<<<(unsigned)((h->mg_nk + 255) / 256), 256, 0, h->stream>>>(h->slot_of_kid, h->dict_launches, h->dict_solo, (uint32_t)h->mg_nk,
                                                                               reinterpret_cast<unsigned long long*>(launches), reinterpret_cast<unsigned long long*>(solo), import);
    ++h->launches;
  }
  return (int64_t)h->mg_nk;
}

int64_t ks_mg_samples(ks_handle* h) {
  if (!h) return -KS_ERR_ARG;
  KS_CUDA(h, cudaSetDevice(h->device));
  const uint64_t n = h->mg_n_halo + h->mg_n_owned;
  uint64_t cap = sample_capacity(h);
  if (cap < std::max<uint64_t>(2 * n, 1u << 16)) { cap = std::max<uint64_t>(2 * n, 1u << 16); int r = ensure_samples(h, cap); if (r) return r; }
  for (int attempt = 0; attempt < 2; ++attempt) {
    SoloArgs s{};
    s.solo_stream = as<unsigned long long>(h->solo_stream);
    s.kid_of_slot = h->kid_of_slot;
    s.samples = as<uint4>(h->samples[0]);
    s.capacity = cap;
    s.ctl = h->d_ctl;
    k_solo_samples<<<h->sm_count * 4, 256, 0, h->stream>>>(s);
    ++h->launches;
    { int r = run_join(h, 0, n, cap, nullptr, nullptr, kHaloMax - h->mg_n_halo, h->mg_n_halo); if (r) return r; }
    { int r = read_ctl(h); if (r) return r; }
    { int r = mg_status(h, "ks_mg_samples"); if (r) return r; }
    h->mg_n_samples = h->h_ctl->n_pairs;
    if (h->mg_n_samples <= cap) break;
    if (h->mg_n_samples >= kSortMaxItems) return fail(h, KS_ERR_TOO_LARGE, "ks_mg_samples: 2^30 samples or more");
    if (attempt == 1) return fail(h, KS_ERR_CAPACITY, "ks_mg_samples: sample stream still too small");
    cap = h->mg_n_samples + h->mg_n_samples / 16;
    int r = ensure_samples(h, cap);
    if (r) return r;
  }
  return (int64_t)h->mg_n_samples;
}

int64_t ks_mg_key_histogram(ks_handle* h, uint64_t* hist, uint32_t* shift_out) {
  if (!h || !hist || !shift_out) return -KS_ERR_ARG;
  KS_CUDA(h, cudaSetDevice(h->device));
  const int bits = bit_length(h->mg_nk + h->mg_nk * h->mg_nk);
  const uint32_t shift = bits > 12 ? (uint32_t)(bits - 12) : 0u;
  *shift_out = shift;
  KS_CUDA(h, cudaMemsetAsync(hist, 0, (size_t)kKeyHistBins * 8, h->stream));
  if (h->mg_n_samples) {
    k_key_hist<<<h->sm_count * 2, 256, 0, h->stream>>>(as<uint4>(h->samples[0]), (uint32_t)h->mg_n_samples, shift, reinterpret_cast<unsigned long long*>(hist));
    ++h->launches;
  }
  return (int64_t)kKeyHistBins;
}

// splitters[r-1] = first histogram bin of rank r (n_ranks - 1 ascending values).  Writes the samples grouped by destination
// rank into send (capacity items); counts[r] = items for rank r.
int64_t ks_mg_partition(ks_handle* h, const uint32_t* splitters, uint32_t shift, uint32_t n_ranks, void* send, uint64_t capacity, uint64_t* counts) {
  if (!h || n_ranks == 0 || n_ranks > 16 || (n_ranks > 1 && !splitters) || (!send && capacity)) return -KS_ERR_ARG;
  KS_CUDA(h, cudaSetDevice(h->device));
  const uint64_t n = h->mg_n_samples;
  if (n > capacity) return fail(h, KS_ERR_CAPACITY, "ks_mg_partition: send buffer too small");
  constexpr int ITEMS = kSort16Items;
  constexpr int THREADS = kSort16Threads;
  constexpr int TILE = THREADS * ITEMS;
  const uint32_t ntiles = (uint32_t)((n + TILE - 1) / TILE);
  const size_t lb_bytes = ((size_t)ntiles * kSort16Bins + 64) * sizeof(uint32_t);
  KS_ENSURE(h, h->lookback, lb_bytes);
  KS_ENSURE(h, h->hist, 2 * 8 * 256 * sizeof(uint32_t));
  uint32_t* hist = as<uint32_t>(h->hist);
  uint32_t* gbase = hist + 8 * 256;
  KS_CUDA(h, cudaMemsetAsync(hist, 0, 256 * sizeof(uint32_t), h->stream));
  KS_CUDA(h, cudaMemsetAsync(h->lookback.p, 0, lb_bytes, h->stream));
  SortPass16Args a{};
  a.by_dest = 1;
  a.n_split = n_ranks - 1;
  a.split_shift = shift;
  for (uint32_t i = 0; i + 1 < n_ranks; ++i) a.split[i] = splitters[i];
  a.in = as<uint4>(h->samples[0]);
  a.out = reinterpret_cast<uint4*>(send);
  a.n = (uint32_t)n;
  a.shift = 0;
  a.bits = 8;
  a.gbase = gbase;
  a.lookback = as<uint32_t>(h->lookback);
  a.ticket = as<uint32_t>(h->lookback) + (size_t)ntiles * kSort16Bins;
  a.err = &h->d_ctl->err;
  if (counts) for (uint32_t r = 0; r < n_ranks; ++r) counts[r] = 0;
  if (n) {
    constexpr size_t smem = sort16_smem_bytes<ITEMS, THREADS>();
    KS_CUDA(h, cudaFuncSetAttribute(k_onesweep_pass16<ITEMS, THREADS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    k_dest_hist<<<h->sm_count * 2, 256, 0, h->stream>>>(a, hist);
    k_radix_scan_hist<<<1, 256, 0, h->stream>>>(hist, gbase, 1);
    k_onesweep_pass16<ITEMS, THREADS><<<(int)std::min<uint32_t>(ntiles, (uint32_t)h->sm_count * kSort16CtasPerSm), THREADS, smem, h->stream>>>(a);
    h->launches += 3;
    if (counts) {
      uint32_t hc[16];
      KS_CUDA(h, cudaMemcpyAsync(hc, hist, sizeof(hc), cudaMemcpyDeviceToHost, h->stream));
      { int r = read_ctl(h); if (r) return r; }
      { int r = mg_status(h, "ks_mg_partition"); if (r) return r; }
      for (uint32_t r = 0; r < n_ranks; ++r) counts[r] = hc[r];
    }
  }
  return (int64_t)n;
}

int64_t ks_mg_reduce(ks_handle* h, const void* samples, uint64_t n) {
  if (!h || (!samples && n)) return -KS_ERR_ARG;
  if (n >= kSortMaxItems) return fail(h, KS_ERR_TOO_LARGE, "ks_mg_reduce: 2^30 samples or more");
  KS_CUDA(h, cudaSetDevice(h->device));
  { int r = ensure_samples(h, std::max<uint64_t>(n, 16)); if (r) return r; }
  if (n) KS_CUDA(h, cudaMemcpyAsync(h->samples[0].p, samples, n * 16, cudaMemcpyDeviceToDevice, h->stream));
  { int r = mg_reduce_queue(h, n); if (r) return r; }
  { int r = read_ctl(h); if (r) return r; }
  { int r = mg_status(h, "ks_mg_reduce"); if (r) return r; }
  return (int64_t)h->h_ctl->n_rows;
}

int64_t ks_mg_row_count(ks_handle* h) {
  if (!h) return -KS_ERR_ARG;
  return (int64_t)h->h_ctl->n_rows - (int64_t)h->h_ctl->ticket2;  // as read back at the end of ks_mg_reduce
}

int64_t ks_mg_solo(ks_handle* h, double* solo, int import) {
  if (!h || !solo) return -KS_ERR_ARG;
  KS_CUDA(h, cudaSetDevice(h->device));
  if (h->mg_nk) {
    if (import) KS_CUDA(h, cudaMemcpyAsync(h->solo_ns, solo, h->mg_nk * 8, cudaMemcpyDeviceToDevice, h->stream));
    else KS_CUDA(h, cudaMemcpyAsync(solo, h->solo_ns, h->mg_nk * 8, cudaMemcpyDeviceToDevice, h->stream));
  }
  return (int64_t)h->mg_nk;
}

int64_t ks_mg_finalize(ks_handle* h) {
  if (!h) return -KS_ERR_ARG;
  KS_CUDA(h, cudaSetDevice(h->device));
  const uint64_t nk = h->mg_nk, n = h->mg_n_samples;
  const uint32_t max_rows = (uint32_t)std::min<uint64_t>(n, (uint64_t)h->cfg.max_pair_rows + nk) + 1;
  KS_ENSURE(h, h->pair_rows, (size_t)max_rows * sizeof(ks_pair_row));
  { int r = mg_finalize_queue(h, as<ks_pair_row>(h->pair_rows), max_rows); if (r) return r; }
  // no host round trip: the counts are known since ks_mg_reduce read them back
  h->n_key_rows = nk;
  h->n_pair_rows = h->h_ctl->n_rows - h->h_ctl->ticket2;
  h->pair_rows_src = h->pair_rows.p;
  return (int64_t)h->n_pair_rows;
}

}  // extern "C"

#include "ks_mg_native.cuh"
#include "ks_update_host.cuh"
#include "ks_stream_host.cuh"

// =========================================================================================================
// Agent timing log (TSV text) -> launch records on the device.  Three calls: parse (text in, counts out), dictionaries
// out (the distinct kernel symbols and models, for the host to canonicalise and number), finish (ids in, records out).
namespace {
TsvArgs tsv_args(ks_handle* h) {
  TsvArgs a{};
  a.text = h->tsv_dev_text;
  a.n_bytes = h->tsv_n_bytes;
  a.tile_cnt = as<uint32_t>(h->tsv_cnt);
  a.line_start = as<unsigned long long>(h->tsv_lines);
  a.max_lines = h->tsv_n_lines;
  a.parsed = as<ks_record>(h->tsv_parsed);
  a.valid = as<unsigned char>(h->tsv_valid);
  a.vtile_cnt = as<uint32_t>(h->tsv_vcnt);
  unsigned long long* d = as<unsigned long long>(h->tsv_dict);
  a.name_hash = d;
  a.name_where = d + kTsvNameSlots;
  a.model_hash = d + 2 * (size_t)kTsvNameSlots;
  a.model_where = a.model_hash + kTsvModelSlots;
  a.kernel_id = as<uint32_t>(h->tsv_kid);
  a.row_solo = h->tsv_labelled ? as<unsigned char>(h->tsv_rowsolo) : nullptr;
  a.ctl = h->d_ctl;
  return a;
}
}  // namespace

extern "C" {

int64_t ks_tsv_parse(ks_handle* h, const char* text, uint64_t n_bytes, uint32_t flags) {
  if (!h || (!text && n_bytes) || (flags & ~KS_ON_DEVICE)) return -KS_ERR_ARG;
  if (n_bytes >= (1ull << 40)) return fail(h, KS_ERR_TOO_LARGE, "ks_tsv_parse: text of 2^40 bytes or more");
  KS_CUDA(h, cudaSetDevice(h->device));
  { int r = reset_run(h); if (r) return r; }
  const unsigned char* d_text = nullptr;
  { int r = stage_in<unsigned char>(h, h->tsv_text, reinterpret_cast<const unsigned char*>(text), n_bytes, (flags & KS_ON_DEVICE) != 0, &d_text); if (r) return r; }
  h->tsv_dev_text = d_text;
  h->tsv_n_bytes = n_bytes;
  h->tsv_n_lines = h->tsv_n_valid = h->tsv_max_kid = 0;
  h->tsv_labelled = false;
  const uint64_t ntiles = (n_bytes + kTsvTile - 1) / kTsvTile;
  KS_ENSURE(h, h->tsv_cnt, (ntiles + 1) * 4);
  KS_ENSURE(h, h->tsv_dict, (2 * (size_t)kTsvNameSlots + 2 * kTsvModelSlots) * 8);
  {  // hashes start empty (0), first-occurrence words start at the maximum (they are lowered with atomicMin)
    unsigned long long* d = as<unsigned long long>(h->tsv_dict);
    KS_CUDA(h, cudaMemsetAsync(d, 0, (size_t)kTsvNameSlots * 8, h->stream));
    KS_CUDA(h, cudaMemsetAsync(d + kTsvNameSlots, 0xFF, (size_t)kTsvNameSlots * 8, h->stream));
    KS_CUDA(h, cudaMemsetAsync(d + 2 * (size_t)kTsvNameSlots, 0, (size_t)kTsvModelSlots * 8, h->stream));
    KS_CUDA(h, cudaMemsetAsync(d + 2 * (size_t)kTsvNameSlots + kTsvModelSlots, 0xFF, (size_t)kTsvModelSlots * 8, h->stream));
  }
  if (n_bytes == 0) return 0;
  TsvArgs a = tsv_args(h);
  const int grid = (int)std::min<uint64_t>(ntiles, (uint64_t)h->sm_count * 8);
  k_tsv_nl_count<<<grid, 256, 0, h->stream>>>(a);
  k_tsv_scan<<<1, 1024, 0, h->stream>>>(a.tile_cnt, ntiles, &h->d_ctl->scratch0, d_text, n_bytes);
  { int r = read_ctl(h); if (r) return r; }
  const uint64_t n_lines = h->h_ctl->scratch0;
  h->tsv_n_lines = n_lines;
  KS_ENSURE(h, h->tsv_lines, (n_lines + 2) * 8);
  KS_ENSURE(h, h->tsv_parsed, std::max<uint64_t>(n_lines, 1) * sizeof(ks_record));
  KS_ENSURE(h, h->tsv_valid, std::max<uint64_t>(n_lines, 1));
  KS_ENSURE(h, h->tsv_kid, std::max<uint64_t>(n_lines, 1) * 4);
  const uint64_t vtiles = (n_lines + 255) / 256;
  KS_ENSURE(h, h->tsv_vcnt, (vtiles + 1) * 4);
  a = tsv_args(h);
  k_tsv_nl_fill<<<grid, 256, 0, h->stream>>>(a);
  const int lgrid = (int)std::max<uint64_t>(1, std::min<uint64_t>((n_lines + 255) / 256, (uint64_t)h->sm_count * 16));
  k_tsv_parse<<<lgrid, 256, 0, h->stream>>>(a);
  k_tsv_valid_count<<<lgrid, 256, 0, h->stream>>>(a);
  k_tsv_scan<<<1, 1024, 0, h->stream>>>(a.vtile_cnt, vtiles, &h->d_ctl->n_pairs, nullptr, 0);
  h->launches += 6;
  KS_CUDA(h, cudaGetLastError());
  { int r = read_ctl(h); if (r) return r; }
  if (h->h_ctl->err & kErrTooManyKeys) return fail(h, KS_ERR_TOO_MANY_KEYS, "ks_tsv_parse: more than 65,536 distinct kernel symbols or 256 models in one file");
  h->tsv_n_valid = h->h_ctl->n_pairs;
  h->tsv_max_kid = h->h_ctl->max_start;
  return (int64_t)h->tsv_n_valid;
}

int64_t ks_tsv_extract(ks_handle* h, const char* text, uint64_t n_bytes, uint32_t n_cols, const uint32_t* cols, const uint32_t* kinds, uint64_t* out,
                       uint64_t capacity, uint32_t flags) {
  if (!h || (!text && n_bytes) || (flags & ~KS_ON_DEVICE) || !n_cols || n_cols > kTsvMaxCols || !cols || !kinds || (!out && capacity)) return -KS_ERR_ARG;
  for (uint32_t c = 0; c < n_cols; ++c) if (kinds[c] > KS_COL_SPAN) return fail(h, KS_ERR_ARG, "ks_tsv_extract: unknown column kind");
  if (n_bytes >= (1ull << 40)) return fail(h, KS_ERR_TOO_LARGE, "ks_tsv_extract: text of 2^40 bytes or more");
  KS_CUDA(h, cudaSetDevice(h->device));
  { int r = reset_run(h); if (r) return r; }
  const bool dev = (flags & KS_ON_DEVICE) != 0;
  const unsigned char* d_text = nullptr;
  { int r = stage_in<unsigned char>(h, h->tsv_text, reinterpret_cast<const unsigned char*>(text), n_bytes, dev, &d_text); if (r) return r; }
  h->tsv_dev_text = d_text;
  h->tsv_n_bytes = n_bytes;
  h->tsv_n_lines = h->tsv_n_valid = 0;
  if (n_bytes == 0) return 0;
  const uint64_t ntiles = (n_bytes + kTsvTile - 1) / kTsvTile;
  KS_ENSURE(h, h->tsv_cnt, (ntiles + 1) * 4);
  TsvArgs a = tsv_args(h);
  const int grid = (int)std::min<uint64_t>(ntiles, (uint64_t)h->sm_count * 8);
  k_tsv_nl_count<<<grid, 256, 0, h->stream>>>(a);
  k_tsv_scan<<<1, 1024, 0, h->stream>>>(a.tile_cnt, ntiles, &h->d_ctl->scratch0, d_text, n_bytes);
  { int r = read_ctl(h); if (r) return r; }
  const uint64_t n_lines = h->h_ctl->scratch0;
  h->tsv_n_lines = n_lines;
  KS_ENSURE(h, h->tsv_lines, (n_lines + 2) * 8);
  a = tsv_args(h);
  k_tsv_nl_fill<<<grid, 256, 0, h->stream>>>(a);
  h->launches += 3;
  const uint64_t rows = n_lines ? n_lines - 1 : 0, take = std::min(rows, capacity);
  if (take) {
    TsvExtractArgs x{};
    x.text = d_text;
    x.n_bytes = n_bytes;
    x.line_start = as<unsigned long long>(h->tsv_lines);
    x.n_lines = n_lines;
    x.n_cols = n_cols;
    for (uint32_t c = 0; c < n_cols; ++c) { x.col[c] = cols[c]; x.kind[c] = kinds[c]; }
    x.capacity = capacity;
    if (dev) {
      x.out = reinterpret_cast<unsigned long long*>(out);
    } else {
      KS_ENSURE(h, h->tsv_parsed, (size_t)n_cols * capacity * 8);
      x.out = as<unsigned long long>(h->tsv_parsed);
    }
    k_tsv_extract<<<(int)std::max<uint64_t>(1, std::min<uint64_t>((n_lines + 255) / 256, (uint64_t)h->sm_count * 16)), 256, 0, h->stream>>>(x);
    ++h->launches;
    KS_CUDA(h, cudaGetLastError());
    if (!dev) {
      for (uint32_t c = 0; c < n_cols; ++c) { int r = copy_out(h, out + (size_t)c * capacity, x.out + (size_t)c * capacity, take * 8, false); if (r) return r; }
    }
  }
  KS_CUDA(h, cudaStreamSynchronize(h->stream));
  return (int64_t)rows;
}

int64_t ks_segment_hist(ks_handle* h, const uint32_t* values, const uint64_t* offsets, uint64_t n_segments, uint32_t n_bins, uint32_t log2_bins, uint32_t flags,
                        uint32_t* out) {
  if (!h || !offsets || (n_segments && !out) || !n_bins || n_bins > 4096 || (flags & ~KS_ON_DEVICE)) return -KS_ERR_ARG;
  KS_CUDA(h, cudaSetDevice(h->device));
  if (n_segments == 0) return 0;
  const bool dev = (flags & KS_ON_DEVICE) != 0;
  uint64_t n_values;
  const unsigned long long* d_off = nullptr;
  { int r = stage_in<unsigned long long>(h, h->tmp[0], reinterpret_cast<const unsigned long long*>(offsets), n_segments + 1, dev, &d_off); if (r) return r; }
  if (dev) { KS_CUDA(h, cudaMemcpyAsync(&n_values, offsets + n_segments, 8, cudaMemcpyDeviceToHost, h->stream)); KS_CUDA(h, cudaStreamSynchronize(h->stream)); }
  else n_values = offsets[n_segments];
  if (!values && n_values) return -KS_ERR_ARG;
  const uint32_t* d_val = nullptr;
  { int r = stage_in<uint32_t>(h, h->tmp[1], values, n_values, dev, &d_val); if (r) return r; }
  const size_t bytes = (size_t)n_segments * n_bins * 4;
  uint32_t* d_out = out;
  if (!dev) { KS_ENSURE(h, h->tmp[2], bytes); d_out = as<uint32_t>(h->tmp[2]); }
  KS_CUDA(h, cudaMemsetAsync(d_out, 0, bytes, h->stream));
  k_segment_hist<<<(int)std::max<uint64_t>(1, std::min<uint64_t>((n_segments + 7) / 8, (uint64_t)h->sm_count * 8)), 256, 0, h->stream>>>(d_val, d_off, n_segments, n_bins,
                                                                                                                                  log2_bins, d_out);
  ++h->launches;
  KS_CUDA(h, cudaGetLastError());
  if (!dev) { int r = copy_out(h, out, d_out, bytes, false); if (r) return r; }
  KS_CUDA(h, cudaStreamSynchronize(h->stream));
  return (int64_t)n_segments;
}

// The profiling daemon's log of the same run: which launches of process `pid` ran alone (solo samples) and which in a
// gang.  Applies to the text parsed last; rows the log does not mention are dropped.  Returns the rows that remain.
int64_t ks_tsv_label(ks_handle* h, const char* log_text, uint64_t n_bytes, uint64_t pid, uint32_t flags) {
  if (!h || (!log_text && n_bytes) || (flags & ~KS_ON_DEVICE)) return -KS_ERR_ARG;
  if (n_bytes >= (1ull << 40)) return fail(h, KS_ERR_TOO_LARGE, "ks_tsv_label: text of 2^40 bytes or more");
  if (!h->tsv_dict.p) return fail(h, KS_ERR_ARG, "ks_tsv_label: no parsed text (ks_tsv_parse first)");
  KS_CUDA(h, cudaSetDevice(h->device));
  const uint64_t n_lines = h->tsv_n_lines;
  if (n_lines == 0) return 0;
  const unsigned char* d_text = nullptr;
  { int r = stage_in<unsigned char>(h, h->tsv_logtext, reinterpret_cast<const unsigned char*>(log_text), n_bytes, (flags & KS_ON_DEVICE) != 0, &d_text); if (r) return r; }
  const uint64_t label_cap = h->tsv_max_kid + 1;
  KS_ENSURE(h, h->tsv_label, label_cap);
  KS_ENSURE(h, h->tsv_rowsolo, n_lines);
  KS_CUDA(h, cudaMemsetAsync(h->tsv_label.p, 0, label_cap, h->stream));
  if (n_bytes) {
    // line starts of the log: the same three kernels, with buffers of their own and the line count in a free control word
    const uint64_t ntiles = (n_bytes + kTsvTile - 1) / kTsvTile;
    KS_ENSURE(h, h->tsv_logcnt, (ntiles + 1) * 4);
    TsvArgs la{};
    la.text = d_text;
    la.n_bytes = n_bytes;
    la.tile_cnt = as<uint32_t>(h->tsv_logcnt);
    la.ctl = h->d_ctl;
    const int grid = (int)std::min<uint64_t>(ntiles, (uint64_t)h->sm_count * 8);
    k_tsv_nl_count<<<grid, 256, 0, h->stream>>>(la);
    k_tsv_scan<<<1, 1024, 0, h->stream>>>(la.tile_cnt, ntiles, &h->d_ctl->batches_both, d_text, n_bytes);
    { int r = read_ctl(h); if (r) return r; }
    const uint64_t log_lines = h->h_ctl->batches_both;
    KS_ENSURE(h, h->tsv_loglines, (log_lines + 2) * 8);
    la.line_start = as<unsigned long long>(h->tsv_loglines);
    la.max_lines = log_lines;
    k_tsv_nl_fill<<<grid, 256, 0, h->stream>>>(la);
    TsvLabelArgs lb{};
    lb.text = d_text;
    lb.n_bytes = n_bytes;
    lb.line_start = la.line_start;
    lb.n_lines = log_lines;
    lb.pid = pid;
    lb.label = as<unsigned char>(h->tsv_label);
    lb.label_cap = label_cap;
    const int pgrid = (int)std::max<uint64_t>(1, std::min<uint64_t>((log_lines + 255) / 256, (uint64_t)h->sm_count * 16));
    k_pplog_parse<<<pgrid, 256, 0, h->stream>>>(lb);
    h->launches += 4;
  }
  TsvArgs a = tsv_args(h);
  const int lgrid = (int)std::max<uint64_t>(1, std::min<uint64_t>((n_lines + 255) / 256, (uint64_t)h->sm_count * 16));
  const uint64_t vtiles = (n_lines + 255) / 256;
  k_tsv_apply_labels<<<lgrid, 256, 0, h->stream>>>(a, as<unsigned char>(h->tsv_label), label_cap, as<unsigned char>(h->tsv_rowsolo));
  k_tsv_valid_count<<<lgrid, 256, 0, h->stream>>>(a);
  k_tsv_scan<<<1, 1024, 0, h->stream>>>(a.vtile_cnt, vtiles, &h->d_ctl->n_pairs, nullptr, 0);
  h->launches += 3;
  KS_CUDA(h, cudaGetLastError());
  { int r = read_ctl(h); if (r) return r; }
  h->tsv_n_valid = h->h_ctl->n_pairs;
  h->tsv_labelled = true;
  return (int64_t)h->tsv_n_valid;
}

// which = 0: kernel symbols (KS_TSV_NAME_SLOTS entries), 1: models (KS_TSV_MODEL_SLOTS).  hashes[i] != 0 marks a used slot;
// where[i] = offset << 20 | length of the string's first occurrence in the text.  HOST pointers.
int64_t ks_tsv_dictionary(ks_handle* h, int which, uint64_t* hashes, uint64_t* where) {
  if (!h || !hashes || !where || which < 0 || which > 1) return -KS_ERR_ARG;
  KS_CUDA(h, cudaSetDevice(h->device));
  if (!h->tsv_dict.p) return fail(h, KS_ERR_ARG, "ks_tsv_dictionary: no parsed text");
  const uint32_t slots = which ? kTsvModelSlots : kTsvNameSlots;
  const unsigned long long* base = as<unsigned long long>(h->tsv_dict) + (which ? 2 * (size_t)kTsvNameSlots : 0);
  KS_CUDA(h, cudaMemcpyAsync(hashes, base, (size_t)slots * 8, cudaMemcpyDeviceToHost, h->stream));
  KS_CUDA(h, cudaMemcpyAsync(where, base + slots, (size_t)slots * 8, cudaMemcpyDeviceToHost, h->stream));
  KS_CUDA(h, cudaStreamSynchronize(h->stream));
  return (int64_t)slots;
}

// name_ids[slot], tenants[slot]: HOST arrays over the dictionary slots; out: records (host, or device with KS_ON_DEVICE)
int64_t ks_tsv_finish(ks_handle* h, const uint32_t* name_ids, const uint32_t* tenants, uint32_t solo, ks_record* out, uint64_t capacity, uint32_t flags) {
  if (!h || !name_ids || !tenants || (!out && h->tsv_n_valid) || (flags & ~KS_ON_DEVICE)) return -KS_ERR_ARG;
  if (capacity < h->tsv_n_valid) return fail(h, KS_ERR_CAPACITY, "ks_tsv_finish: output buffer too small");
  KS_CUDA(h, cudaSetDevice(h->device));
  const uint64_t n = h->tsv_n_valid;
  if (n == 0) return 0;
  KS_ENSURE(h, h->tsv_maps, ((size_t)kTsvNameSlots + kTsvModelSlots) * 4);
  uint32_t* maps = as<uint32_t>(h->tsv_maps);
  KS_CUDA(h, cudaMemcpyAsync(maps, name_ids, (size_t)kTsvNameSlots * 4, cudaMemcpyHostToDevice, h->stream));
  KS_CUDA(h, cudaMemcpyAsync(maps + kTsvNameSlots, tenants, (size_t)kTsvModelSlots * 4, cudaMemcpyHostToDevice, h->stream));
  const bool dev = (flags & KS_ON_DEVICE) != 0;
  ks_record* d_out = out;
  if (!dev) { KS_ENSURE(h, h->records, n * sizeof(ks_record)); d_out = as<ks_record>(h->records); }
  TsvArgs a = tsv_args(h);
  a.out = d_out;
  a.out_capacity = n;
  a.name_map = maps;
  a.model_map = maps + kTsvNameSlots;
  a.solo = solo;
  const int lgrid = (int)std::max<uint64_t>(1, std::min<uint64_t>((h->tsv_n_lines + 255) / 256, (uint64_t)h->sm_count * 16));
  k_tsv_compact<<<lgrid, 256, 0, h->stream>>>(a);
  ++h->launches;
  KS_CUDA(h, cudaGetLastError());
  if (!dev) { int r = copy_out(h, out, d_out, n * sizeof(ks_record), false); if (r) return r; }
  KS_CUDA(h, cudaStreamSynchronize(h->stream));
  return (int64_t)n;
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------------------
// Sorting without allocating.  Callers that run inside somebody else's memory budget -- a plugin of a serving process
// whose allocator owns the whole device, a monitoring thread that must never take the device allocator's lock, code
// that runs while the application has allocation frozen -- cannot let this library call cudaMalloc.  For them the
// scratch of the radix sort (the second key/value buffer of the ping-pong, the per-tile look-back words, the digit
// histograms and the error word) lives in one file-scope device array of fixed size.  Every GPU that loads the library
// carries these 8,667,648 bytes until the process exits.
constexpr uint32_t kNoAllocMaxItems = 1u << 20;
constexpr int kNoAllocItems = 16;                                                   // keys per thread of the pass kernel
constexpr uint32_t kNoAllocTile = kSortThreads * kNoAllocItems;
constexpr uint32_t kNoAllocTiles = kNoAllocMaxItems / kNoAllocTile;
constexpr uint32_t kNaAltKeys = 0;                                                  // word offsets inside the array
constexpr uint32_t kNaAltVals = kNaAltKeys + kNoAllocMaxItems;
constexpr uint32_t kNaLookback = kNaAltVals + kNoAllocMaxItems;                     // [tiles][256] + ticket (+ padding)
constexpr uint32_t kNaHist = kNaLookback + kNoAllocTiles * 256 + 64;                // [8][256] counts, [8][256] offsets
constexpr uint32_t kNaErr = kNaHist + 2 * 8 * 256;
constexpr uint32_t kNaWords = kNaErr + 64;
static __device__ __align__(256) uint32_t g_noalloc_scratch[kNaWords];

namespace {
// Device address of g_noalloc_scratch per device.  In host code the array's name is only a handle for the runtime, not
// an address a kernel can use; the address comes from cudaGetSymbolAddress, asked once per device with it current.
uint32_t* g_noalloc_ptr[64] = {};
}  // namespace

extern "C" int64_t ks_sort_pairs_u32_noalloc(void* stream, uint32_t* keys, uint32_t* vals, uint64_t n, int begin_bit, int end_bit) {
  if ((!keys && n) || begin_bit < 0 || end_bit > 32 || begin_bit > end_bit) { g_null_error = "ks_sort_pairs_u32_noalloc: bad argument"; return -KS_ERR_ARG; }
  if (n > kNoAllocMaxItems) {
    g_null_error = "ks_sort_pairs_u32_noalloc: " + std::to_string(n) + " items, the fixed scratch holds at most " + std::to_string(kNoAllocMaxItems);
    return -KS_ERR_TOO_LARGE;
  }
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= 64) { g_null_error = std::string("ks_sort_pairs_u32_noalloc: cudaGetDevice: ") + cudaGetErrorString(e); return -KS_ERR_CUDA; }
  constexpr size_t smem = sort_smem_bytes<uint32_t, uint32_t, kNoAllocItems>();
  if (!g_noalloc_ptr[dev]) {  // set-up, first call on this device
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess || !p) { g_null_error = std::string("ks_sort_pairs_u32_noalloc: cudaGetSymbolAddress: ") + cudaGetErrorString(e); return -KS_ERR_CUDA; }
    e = cudaFuncSetAttribute(k_onesweep_pass<uint32_t, uint32_t, 1, kNoAllocItems>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(k_onesweep_pass<uint32_t, uint32_t, 0, kNoAllocItems>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) { g_null_error = std::string("ks_sort_pairs_u32_noalloc: cudaFuncSetAttribute: ") + cudaGetErrorString(e); return -KS_ERR_CUDA; }
    g_noalloc_ptr[dev] = static_cast<uint32_t*>(p);
  }
  const int passes = (end_bit - begin_bit + 7) / 8;
  if (n == 0 || passes == 0) return (int64_t)n;
  uint32_t* base = g_noalloc_ptr[dev];
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  uint32_t* kbuf[2] = {keys, base + kNaAltKeys};
  uint32_t* vbuf[2] = {vals, base + kNaAltVals};
  uint32_t* lookback = base + kNaLookback;
  uint32_t* hist = base + kNaHist;
  uint32_t* gbase = hist + 8 * 256;
  uint32_t* err = base + kNaErr;
  const uint32_t ntiles = (uint32_t)((n + kNoAllocTile - 1) / kNoAllocTile);
  const size_t lb_bytes = ((size_t)ntiles * 256 + 64) * sizeof(uint32_t);
#define KS_NA(call)                                                                                                       \
  do {                                                                                                                    \
    cudaError_t e__ = (call);                                                                                             \
    if (e__ != cudaSuccess) { g_null_error = std::string("ks_sort_pairs_u32_noalloc: " #call ": ") + cudaGetErrorString(e__); return -KS_ERR_CUDA; } \
  } while (0)
  // the array keeps whatever the last call left: counters and flags that must start at zero are cleared here
  KS_NA(cudaMemsetAsync(hist, 0, 8 * 256 * sizeof(uint32_t), st));
  KS_NA(cudaMemsetAsync(err, 0, 64 * sizeof(uint32_t), st));
  int sm_count = 148;
  cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
  const int hist_grid = (int)std::min<uint64_t>((n + 256 * 16 - 1) / (256 * 16), (uint64_t)sm_count * 6);
  k_radix_hist<uint32_t><<<hist_grid, 256, 0, st>>>(keys, 1u, nullptr, (uint32_t)n, begin_bit, end_bit, hist);
  k_radix_scan_hist<<<1, 256, 0, st>>>(hist, gbase, passes);
  int cur = 0;
  for (int p = 0; p < passes; ++p) {
    KS_NA(cudaMemsetAsync(lookback, 0, lb_bytes, st));
    SortPassArgs<uint32_t, uint32_t, 1> a1{};
    a1.kin = kbuf[cur]; a1.kout = kbuf[cur ^ 1];
    a1.vin[0] = vbuf[cur]; a1.vout[0] = vbuf[cur ^ 1];
    a1.n_dev = nullptr; a1.n = (uint32_t)n;
    a1.shift = begin_bit + 8 * p; a1.bits = std::min(8, end_bit - a1.shift);
    a1.gbase = gbase + p * 256; a1.lookback = lookback; a1.ticket = lookback + (size_t)ntiles * 256; a1.err = err;
    const int grid = (int)std::min<uint32_t>(ntiles, (uint32_t)sm_count * 4);
    if (vals) {
      k_onesweep_pass<uint32_t, uint32_t, 1, kNoAllocItems><<<grid, kSortThreads, smem, st>>>(a1);
    } else {
      SortPassArgs<uint32_t, uint32_t, 0> a0{};
      a0.kin = a1.kin; a0.kout = a1.kout; a0.n_dev = nullptr; a0.n = a1.n; a0.shift = a1.shift; a0.bits = a1.bits;
      a0.gbase = a1.gbase; a0.lookback = a1.lookback; a0.ticket = a1.ticket; a0.err = a1.err;
      k_onesweep_pass<uint32_t, uint32_t, 0, kNoAllocItems><<<grid, kSortThreads, smem, st>>>(a0);
    }
    cur ^= 1;
  }
  KS_NA(cudaGetLastError());
  if (cur == 1) {  // an odd number of passes ends in the scratch: bring the result home
    KS_NA(cudaMemcpyAsync(keys, kbuf[1], n * sizeof(uint32_t), cudaMemcpyDeviceToDevice, st));
    if (vals) KS_NA(cudaMemcpyAsync(vals, vbuf[1], n * sizeof(uint32_t), cudaMemcpyDeviceToDevice, st));
  }
  uint32_t h_err = 0;
  KS_NA(cudaMemcpyAsync(&h_err, err, sizeof(uint32_t), cudaMemcpyDeviceToHost, st));
  KS_NA(cudaStreamSynchronize(st));
#undef KS_NA
  if (h_err & kErrWait) { g_null_error = "ks_sort_pairs_u32_noalloc: a bounded device-side wait ran out"; return -KS_ERR_WAIT; }
  return (int64_t)n;
}
