// ks_mg_native.cuh -- the multi-GPU table build as ONE library call per rank: the phases of the ks_mg_* session with the
// collectives issued from C++ through NCCL on the handle's stream.  Part of ks_api.cu (included behind the handle and the
// phase functions); not a translation unit of its own.
//
// One process per GPU calls ks_mg_build with its window of the start-ordered trace.  The five exchanges:
//   1. all-gather  [header | tail launches | distinct keys + launch fields]      -> global key ids, halo
//   2. all-gather  [header | sample-key histogram]                               -> splitters, transfer sizes
//   3. all-to-all  samples to the rank that owns their key range                 (send/recv pairs, exact sizes)
//   4. all-gather  [header | solo times of the keys reduced here | launch counts] -> solo times, totals, shard sizes
//   5. all-gather  table shards, straight into place in the whole table          (send/recv pairs, exact sizes)
// Every block starts with a 256-byte header that carries the sender's control words, so after exchanges 2 and 4 every
// rank knows every rank's error bits and counts: an error on any rank makes ALL ranks return it from the same point, and
// decisions that change what is exchanged next (a larger key block, a larger sample stream, a larger peer buffer) are
// taken alike everywhere.  The host waits for the device behind exchanges 2 and 4 (it needs the histograms for the
// splitters and the shard sizes for the table); everything else is queued, and what exchange 1 feeds (key merge, halo)
// reads the other ranks' counts from the gathered headers on the device.
// With peer memory and a large table the build runs in two STAGES behind exchange 3: every rank owns two key ranges, and
// the table rows of the first are on their way into all GPUs' tables (a stream of their own) while the second range is
// sorted and reduced; exchange 4 is then made once per stage (see the stage rule in ks_mg_build).
//
// NCCL is bound at run time (dlopen of libnccl.so.2, or the library named by KS_NCCL_LIBRARY): the library has no link-time
// dependency on it, and a process that already loaded NCCL (PyTorch) shares that copy.
#pragma once

#include <dlfcn.h>

#include <algorithm>
#include <mutex>

namespace {

struct NcclId { char internal[128]; };  // ncclUniqueId

struct NcclApi {
  void* lib = nullptr;
  int (*GetUniqueId)(NcclId*) = nullptr;
  int (*CommInitRank)(void**, int, NcclId, int) = nullptr;
  int (*CommDestroy)(void*) = nullptr;
  int (*AllGather)(const void*, void*, size_t, int, void*, cudaStream_t) = nullptr;
  int (*Send)(const void*, size_t, int, int, void*, cudaStream_t) = nullptr;
  int (*Recv)(void*, size_t, int, int, void*, cudaStream_t) = nullptr;
  int (*GroupStart)() = nullptr;
  int (*GroupEnd)() = nullptr;
  const char* (*GetErrorString)(int) = nullptr;
  std::string error;
};
constexpr int kNcclUint8 = 1;  // ncclUint8

NcclApi* nccl_api() {
  static NcclApi api;
  static std::once_flag once;
  std::call_once(once, [] {
    const char* named = getenv("KS_NCCL_LIBRARY");
    const char* names[] = {named, "libnccl.so.2", "libnccl.so"};
    for (const char* name : names) {
      if (!name || !*name) continue;
      api.lib = dlopen(name, RTLD_NOW | RTLD_GLOBAL);
      if (api.lib) break;
    }
    if (!api.lib) { api.error = "NCCL not found (libnccl.so.2); name the library in KS_NCCL_LIBRARY"; return; }
    auto sym = [&](const char* name) {
      void* p = dlsym(api.lib, name);
      if (!p && api.error.empty()) api.error = std::string("NCCL symbol missing: ") + name;
      return p;
    };
    api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(sym("ncclGetUniqueId"));
    api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(sym("ncclCommInitRank"));
    api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(sym("ncclCommDestroy"));
    api.AllGather = reinterpret_cast<decltype(api.AllGather)>(sym("ncclAllGather"));
    api.Send = reinterpret_cast<decltype(api.Send)>(sym("ncclSend"));
    api.Recv = reinterpret_cast<decltype(api.Recv)>(sym("ncclRecv"));
    api.GroupStart = reinterpret_cast<decltype(api.GroupStart)>(sym("ncclGroupStart"));
    api.GroupEnd = reinterpret_cast<decltype(api.GroupEnd)>(sym("ncclGroupEnd"));
    api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(sym("ncclGetErrorString"));
  });
  return &api;
}

#define KS_NCCL(h, call)                                                                                              \
  do {                                                                                                                \
    int e__ = (call);                                                                                                 \
    if (e__ != 0) return fail((h), KS_ERR_COMM, std::string(#call) + ": " + nccl_api()->GetErrorString(e__));         \
  } while (0)

void mg_close_imports(ks_handle* h);
void mg_free_exports(ks_handle* h);

// ks_destroy calls this with orderly = false: it must never wait for another rank, so it closes its mappings of the other
// ranks' buffers and, in peer-memory mode, leaves its own exported buffers to the end of the process.
// ks_mg_comm_destroy is the orderly, collective way (all mappings closed everywhere, then every buffer freed).
void mg_native_release(ks_handle* h, bool orderly) {
  if (h->pair_rows_src && h->pair_rows_src != h->pair_rows.p) {  // the last table lives in an exported buffer
    h->pair_rows_src = nullptr;
    h->n_pair_rows = 0;
  }
  mg_close_imports(h);
  if (orderly || !h->mg_p2p) {
    mg_free_exports(h);
  } else {
    // Other ranks may still map these buffers and nobody told them to let go: exported memory must outlive its mappings,
    // so it is left to the end of the process instead of freed under them.
    h->mg_recv_x = ks_handle::Exported{};
    h->mg_table_x = ks_handle::Exported{};
    h->mg_retired.clear();
  }
  if (h->mg_bar) cudaFree(h->mg_bar);
  h->mg_bar = nullptr;
  h->mg_p2p = false;
  if (h->mg_comm) {
    nccl_api()->CommDestroy(h->mg_comm);
    h->mg_comm = nullptr;
  }
  for (DevBuf* b : {&h->mg_block, &h->mg_gathered, &h->mg_recv}) {
    if (b->p) cudaFree(b->p);
    b->p = nullptr;
    b->cap = 0;
  }
  if (h->mg_counts) cudaFree(h->mg_counts);
  h->mg_counts = nullptr;
  if (h->mg_host) cudaFreeHost(h->mg_host);
  h->mg_host = nullptr;
  h->mg_host_cap = 0;
}

// KS_MG_TRACE=1 in the environment: rank 0 prints the device time between the driver's steps of every call to stderr
// (KS_MG_TRACE=2: every rank)
struct MgTrace {
  bool on = false;
  int rank = 0;
  cudaStream_t stream = nullptr;
  std::vector<std::pair<const char*, cudaEvent_t>> marks;
  std::string note;  // appended to the line (the rows of this rank's parts)
  void mark(const char* name) {
    if (!on) return;
    cudaEvent_t e;
    cudaEventCreate(&e);
    cudaEventRecord(e, stream);
    marks.emplace_back(name, e);
  }
  void report() {
    if (!on) return;
    cudaStreamSynchronize(stream);
    std::string line = "ks_mg_build trace, rank " + std::to_string(rank) + " (ms):";
    for (size_t i = 1; i < marks.size(); ++i) {
      char buf[96];
      snprintf(buf, sizeof(buf), " %s=%.3f", marks[i].first, ev_ms(marks[i - 1].second, marks[i].second));
      line += buf;
    }
    fprintf(stderr, "%s%s\n", line.c_str(), note.c_str());
    note.clear();
    for (auto& m : marks) cudaEventDestroy(m.second);
    marks.clear();
  }
};

// An exported buffer of at least `bytes`.  A larger one REPLACES it; the old one is retired, not freed: other ranks may
// still have it mapped, and exported memory must outlive its mappings.  Retired buffers are freed when the session ends.
int mg_export_ensure(ks_handle* h, ks_handle::Exported& x, size_t bytes) {
  if (bytes <= x.cap) return 0;
  if (x.p) h->mg_retired.push_back(x.p);
  x.p = nullptr;
  x.cap = 0;
  const size_t want = (bytes + ((size_t)1 << 21) - 1) & ~(((size_t)1 << 21) - 1);
  cudaError_t e = cudaMalloc(&x.p, want);
  if (e != cudaSuccess) return fail(h, KS_ERR_CUDA, "cudaMalloc of " + std::to_string(want) + " bytes: " + cudaGetErrorString(e));
  x.cap = want;
  ++x.gen;
  if (h->mg_p2p) KS_CUDA(h, cudaIpcGetMemHandle(&x.handle, x.p));
  return 0;
}

MgIpc mg_ipc_of(const ks_handle::Exported& x) {
  MgIpc m{};
  static_assert(sizeof(cudaIpcMemHandle_t) == sizeof(m.handle), "IPC handle is 64 bytes");
  memcpy(m.handle, &x.handle, sizeof(m.handle));
  m.gen = x.gen;
  m.cap = x.cap;
  return m;
}

// maps the buffer a header advertises (again, if its sender replaced it since the last call)
int mg_import(ks_handle* h, ks_handle::Imported& im, const MgHeader& hd) {
  if (im.p && im.gen == hd.buf_gen) return 0;
  if (im.p) {
    KS_CUDA(h, cudaIpcCloseMemHandle(im.p));
    im.p = nullptr;
  }
  cudaIpcMemHandle_t handle;
  memcpy(&handle, hd.ipc, sizeof(handle));
  KS_CUDA(h, cudaIpcOpenMemHandle(&im.p, handle, cudaIpcMemLazyEnablePeerAccess));
  im.gen = hd.buf_gen;
  return 0;
}

// Stores into peer memory become visible to the peer's later kernels through this: every rank's collective kernel is
// ordered behind its own storing kernel on its stream, and completes only after every rank has entered it.
int mg_barrier(ks_handle* h) {
  KS_NCCL(h, nccl_api()->AllGather(h->mg_bar, h->mg_bar + 16, 16, kNcclUint8, h->mg_comm, h->stream));
  return 0;
}

void mg_close_imports(ks_handle* h) {
  for (auto* set : {h->mg_peer_recv, h->mg_peer_table})
    for (int q = 0; q < 16; ++q) {
      if (set[q].p) cudaIpcCloseMemHandle(set[q].p);
      set[q].p = nullptr;
      set[q].gen = 0;
    }
}

void mg_free_exports(ks_handle* h) {
  for (auto* x : {&h->mg_recv_x, &h->mg_table_x}) {
    if (x->p) cudaFree(x->p);
    x->p = nullptr;
    x->cap = 0;
  }
  for (void* p : h->mg_retired) cudaFree(p);
  h->mg_retired.clear();
}

constexpr size_t kMgTailBytes = (size_t)kHaloMax * 48;
constexpr size_t kMgHistBytes = (size_t)kKeyHistBins * 8;

// the first `width` bytes of every rank's gathered block -> pinned host memory, then wait for the device
int mg_fetch_heads(ks_handle* h, size_t stride, size_t width) {
  const size_t need = width * (size_t)h->mg_world;
  if (need > h->mg_host_cap) {
    if (h->mg_host) cudaFreeHost(h->mg_host);
    h->mg_host = nullptr;
    h->mg_host_cap = 0;
    KS_CUDA(h, cudaMallocHost(reinterpret_cast<void**>(&h->mg_host), need));
    h->mg_host_cap = need;
  }
  KS_CUDA(h, cudaMemcpy2DAsync(h->mg_host, width, h->mg_gathered.p, stride, width, (size_t)h->mg_world, cudaMemcpyDeviceToHost, h->stream));
  KS_CUDA(h, cudaStreamSynchronize(h->stream));
  return 0;
}

const MgHeader& mg_head(const ks_handle* h, size_t width, int q) { return *reinterpret_cast<const MgHeader*>(h->mg_host + width * (size_t)q); }

// the same verdict on every rank: the first rank (in rank order) whose control words carry an error decides
int mg_any_error(ks_handle* h, size_t width, const char* where) {
  for (int q = 0; q < h->mg_world; ++q) {
    const int st = status_of_err(mg_head(h, width, q).ctl.err, true);
    if (st) return fail(h, st, std::string("ks_mg_build (") + where + "), rank " + std::to_string(q) + ": " + ks_status_string(st));
  }
  return 0;
}

// the partition pass of ks_mg_partition with the destinations in peer memory: no separate count (the host knows every
// count from the exchanged histograms), one pass over the samples
int mg_partition_to_peers(ks_handle* h, const uint32_t* splitters, uint32_t shift, uint32_t n_ranks, uint4* const* dest) {
  const uint64_t n = h->mg_n_samples;
  if (!n) return 0;
  constexpr int ITEMS = kSort16Items;
  constexpr int THREADS = kSort16Threads;
  constexpr int TILE = THREADS * ITEMS;
  const uint32_t ntiles = (uint32_t)((n + TILE - 1) / TILE);
  const size_t lb_bytes = ((size_t)ntiles * kSort16Bins + 64) * sizeof(uint32_t);
  KS_ENSURE(h, h->lookback, lb_bytes);
  KS_CUDA(h, cudaMemsetAsync(h->lookback.p, 0, lb_bytes, h->stream));
  SortPass16Args a{};
  a.by_dest = 2;
  a.n_split = n_ranks - 1;
  a.split_shift = shift;
  for (uint32_t i = 0; i + 1 < n_ranks; ++i) a.split[i] = splitters[i];
  for (uint32_t d = 0; d < n_ranks; ++d) a.dest[d] = dest[d];
  a.in = as<uint4>(h->samples[0]);
  a.out = nullptr;
  a.n = (uint32_t)n;
  a.shift = 0;
  a.bits = 8;
  a.gbase = nullptr;
  a.lookback = as<uint32_t>(h->lookback);
  a.ticket = as<uint32_t>(h->lookback) + (size_t)ntiles * kSort16Bins;
  a.err = &h->d_ctl->err;
  constexpr size_t smem = sort16_smem_bytes<ITEMS, THREADS>();
  KS_CUDA(h, cudaFuncSetAttribute(k_onesweep_pass16<ITEMS, THREADS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  k_onesweep_pass16<ITEMS, THREADS><<<(int)std::min<uint32_t>(ntiles, (uint32_t)h->sm_count * kSort16CtasPerSm), THREADS, smem, h->stream>>>(a);
  ++h->launches;
  KS_CUDA(h, cudaGetLastError());
  return 0;
}

}  // namespace

extern "C" {

int ks_mg_unique_id(void* id128) {
  if (!id128) return -KS_ERR_ARG;
  NcclApi* api = nccl_api();
  if (!api->error.empty()) { g_null_error = api->error; return -KS_ERR_COMM; }
  NcclId id;
  const int e = api->GetUniqueId(&id);
  if (e != 0) { g_null_error = std::string("ncclGetUniqueId: ") + api->GetErrorString(e); return -KS_ERR_COMM; }
  memcpy(id128, id.internal, sizeof(id.internal));
  return KS_OK;
}

int ks_mg_comm_init(ks_handle* h, const void* id128, int rank, int world) {
  if (!h || !id128 || world < 1 || world > 16 || rank < 0 || rank >= world) return -KS_ERR_ARG;
  NcclApi* api = nccl_api();
  if (!api->error.empty()) return fail(h, KS_ERR_COMM, api->error);
  KS_CUDA(h, cudaSetDevice(h->device));
  if (h->mg_comm) { api->CommDestroy(h->mg_comm); h->mg_comm = nullptr; }
  NcclId id;
  memcpy(id.internal, id128, sizeof(id.internal));
  KS_NCCL(h, api->CommInitRank(&h->mg_comm, world, id, rank));
  h->mg_rank = rank;
  h->mg_world = world;
  h->mg_rows_hint = 0;
  if (!h->mg_counts) KS_CUDA(h, cudaMalloc(reinterpret_cast<void**>(&h->mg_counts), 16));
  if (!h->mg_bar) {
    KS_CUDA(h, cudaMalloc(reinterpret_cast<void**>(&h->mg_bar), 16 * 17));
    KS_CUDA(h, cudaMemset(h->mg_bar, 0, 16 * 17));
  }
  // Peer memory or NCCL for the two bulk exchanges?  Every rank exports a probe buffer and tries to map all the others;
  // the mode is peer memory only if every rank could (KS_MG_NO_P2P in the environment of ANY rank votes no).
  h->mg_p2p = false;
  if (world > 1) {
    constexpr size_t H = sizeof(MgHeader);
    KS_ENSURE(h, h->mg_block, H);
    KS_ENSURE(h, h->mg_gathered, H * (size_t)world);
    ks_handle::Exported probe;
    h->mg_p2p = true;  // so that the probe gets a handle
    int vote = getenv("KS_MG_NO_P2P") ? 0 : 1;
    if (mg_export_ensure(h, probe, 4096)) { vote = 0; cudaGetLastError(); }
    h->mg_p2p = false;
    auto exchange = [&](uint64_t word) -> int {
      k_mg_header<<<1, 32, 0, h->stream>>>(as<MgHeader>(h->mg_block), h->d_ctl, nullptr, nullptr, 0, word, mg_ipc_of(probe));
      KS_NCCL(h, api->AllGather(h->mg_block.p, h->mg_gathered.p, H, kNcclUint8, h->mg_comm, h->stream));
      return mg_fetch_heads(h, H, H);
    };
    { int r = exchange((uint64_t)vote); if (r) return r; }
    void* mapped[16] = {nullptr};
    for (int q = 0; q < world; ++q) {
      const MgHeader& hd = mg_head(h, H, q);
      if (hd.capacity != 1) vote = 0;
      if (q == rank || !vote || hd.capacity != 1) continue;
      cudaIpcMemHandle_t handle;
      memcpy(&handle, hd.ipc, sizeof(handle));
      if (cudaIpcOpenMemHandle(&mapped[q], handle, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
        mapped[q] = nullptr;
        vote = 0;
        cudaGetLastError();  // not an error of the handle: this pair of devices just stays on NCCL
      }
    }
    { int r = exchange((uint64_t)vote); if (r) return r; }
    bool all = true;
    for (int q = 0; q < world; ++q) all = all && mg_head(h, H, q).capacity == 1;
    for (int q = 0; q < world; ++q)
      if (mapped[q]) cudaIpcCloseMemHandle(mapped[q]);
    { int r = exchange(0); if (r) return r; }  // every rank has closed its mappings: the probes can go
    if (probe.p) cudaFree(probe.p);
    h->mg_p2p = all;
  }
  return KS_OK;
}

/* 1 if the two bulk exchanges of ks_mg_build go through peer memory (stores over NVLink from the producing kernels),
 * 0 if they go through NCCL send/recv */
int ks_mg_peer_memory(ks_handle* h) { return h && h->mg_p2p ? 1 : 0; }

int ks_mg_comm_destroy(ks_handle* h) {
  if (!h) return -KS_ERR_ARG;
  cudaSetDevice(h->device);
  if (h->stream) cudaStreamSynchronize(h->stream);
  bool orderly = true;
  if (h->mg_comm && h->mg_p2p && h->mg_world > 1) {  // collective: all mappings are closed before any exported buffer is freed
    mg_close_imports(h);
    orderly = mg_barrier(h) == 0 && cudaStreamSynchronize(h->stream) == cudaSuccess;
  }
  mg_native_release(h, orderly);
  return KS_OK;
}

int64_t ks_mg_build(ks_handle* h, const void* records, uint64_t n_owned, uint32_t flags, ks_table_info* info) {
  if (!h || (!records && n_owned) || (flags & ~(KS_KEY_TYPE | KS_TIMING))) return -KS_ERR_ARG;
  if (!h->mg_comm) return fail(h, KS_ERR_ARG, "ks_mg_build: no communicator (ks_mg_comm_init)");
  NcclApi* api = nccl_api();
  const int world = h->mg_world, rank = h->mg_rank;
  const unsigned char* rec = reinterpret_cast<const unsigned char*>(records);
  constexpr size_t H = sizeof(MgHeader);

  MgTrace tr;
  {
    const char* e = getenv("KS_MG_TRACE");
    tr.on = e && (rank == 0 || e[0] == '2');
    tr.rank = rank;
  }
  tr.stream = h->stream;
  tr.mark("start");
  cudaEvent_t* ev = h->ev;  // phase boundaries on the handle's stream (read only with KS_TIMING)
  // one rank with KS_MG_STAGES=2|4 in the environment: the staged build on the rank's own buffers (no peers to copy to),
  // so that the stage logic can be exercised on one GPU
  bool self_staged = false;
  if (world == 1)
    if (const char* e = getenv("KS_MG_STAGES")) self_staged = e[0] == '2' || e[0] == '4';
  const bool p2p = (h->mg_p2p && world > 1) || self_staged;
  const uint64_t n_tl = n_owned + kHaloMax;  // the join always sees all halo slots (unused ones are inert)
  const size_t width2 = H + kMgHistBytes, block2 = width2;
  // blocks 2 and 4 at their largest, so that the exchange buffers are sized once per key capacity
  const size_t block_other = std::max(width2, H + (size_t)kMaxKeys * 24);
  size_t block1 = 0;
  unsigned char* gathered = nullptr;
  uint64_t cap_s = 0;
  cudaEventRecord(ev[0], h->stream);
  for (int round = 0;; ++round) {
    // ---- phase 1: K1 over the window, its tail, its distinct keys; exchange 1                   (queued, no wait)
    { int64_t r = ks_mg_begin(h, records, n_owned, flags & KS_KEY_TYPE); if (r < 0) return r; }
    KS_ENSURE(h, h->tmp[0], (size_t)kHaloMax * 4 + 16);
    uint32_t* tail_idx = as<uint32_t>(h->tmp[0]);
    KS_CUDA(h, cudaMemsetAsync(h->mg_counts, 0, 16, h->stream));
    if (n_owned) {
      k_tail_select<<<1, 1024, 0, h->stream>>>(as<unsigned long long>(h->tl_start[0]) + kHaloMax, as<unsigned long long>(h->tl_dm[0]) + kHaloMax, (uint32_t)n_owned,
                                               tail_idx, kHaloMax, h->mg_counts, h->d_ctl);
      ++h->launches;
    }
    { int r = mg_zero_u32(h, &h->d_ctl->n_keys); if (r) return r; }
    DictArgs d{};
    d.dict_keys = h->dict_keys; d.dkeys = h->dkeys; d.dslot = h->dslot; d.drank = h->drank; d.kid_of_slot = h->kid_of_slot;
    d.slot_of_kid = h->slot_of_kid; d.keys_sorted = h->keys_sorted; d.ctl = h->d_ctl;
    k_dict_compact<<<kDictSlots / 256, 256, 0, h->stream>>>(d);
    ++h->launches;
    // the number of keys of the own window: the global count replaces it in the control words further down
    KS_CUDA(h, cudaMemcpyAsync(h->mg_counts + 2, &h->d_ctl->n_keys, 4, cudaMemcpyDeviceToDevice, h->stream));
    tr.mark("decode+tail+compact");

    const uint32_t cap = h->mg_key_cap;
    const size_t off_keys = H + kMgTailBytes, off_words = off_keys + (size_t)cap * 8;
    block1 = off_words + (size_t)cap * 32;
    KS_ENSURE(h, h->mg_block, std::max(block1, block_other));
    KS_ENSURE(h, h->mg_gathered, std::max(block1, block_other) * (size_t)world);
    gathered = as<unsigned char>(h->mg_gathered);
    unsigned char* blk = as<unsigned char>(h->mg_block);
    k_mg_header<<<1, 32, 0, h->stream>>>(reinterpret_cast<MgHeader*>(blk), h->d_ctl, h->mg_counts, rec, n_owned, 0, MgIpc{});
    if (n_owned)
      k_gather_records_dev<<<(kHaloMax * 3 + 255) / 256, 256, 0, h->stream>>>(reinterpret_cast<const uint4*>(rec), tail_idx, h->mg_counts, kHaloMax,
                                                                              reinterpret_cast<uint4*>(blk + H));
    k_export_keys_dev<<<(cap + 255) / 256, 256, 0, h->stream>>>(h->dkeys, h->dslot, h->dict_words, h->d_ctl, cap, reinterpret_cast<unsigned long long*>(blk + off_keys),
                                                                reinterpret_cast<uint4*>(blk + off_words));
    h->launches += n_owned ? 3 : 2;
    KS_CUDA(h, cudaGetLastError());
    tr.mark("pack1");
    KS_NCCL(h, api->AllGather(blk, h->mg_gathered.p, block1, kNcclUint8, h->mg_comm, h->stream));
    tr.mark("allgather1");

    // ---- phase 2: global key ids, halo, samples, histogram; exchange 2                          (queued, then wait 1)
    // Nothing here needs the host to have seen exchange 1: the kernels read the other ranks' counts from the gathered
    // headers.  What the host would have checked (tails and keys that fit) is checked behind exchange 2 instead.
    if (round == 0) cudaEventRecord(ev[1], h->stream);
    k_dict_insert_gathered<<<dim3((cap + 255) / 256, (unsigned)world), 256, 0, h->stream>>>(gathered, block1, off_keys, off_words, cap, h->dict_keys, h->dict_words,
                                                                                            h->d_ctl);
    ++h->launches;
    { int r = mg_zero_u32(h, &h->d_ctl->n_keys); if (r) return r; }
    KS_CUDA(h, cudaMemsetAsync(h->drank, 0, (size_t)(kMaxKeys + 1) * 4, h->stream));
    { int r = run_dict(h); if (r) return r; }
    {
      HaloArgs ha{};
      ha.gathered = gathered;
      ha.stride = block1;
      ha.rank = (uint32_t)rank;
      ha.own_records = rec;
      ha.n_owned = n_owned;
      ha.dict_keys = h->dict_keys;
      ha.type_mode = (flags & KS_KEY_TYPE) ? 1 : 0;
      ha.tl_start = as<unsigned long long>(h->tl_start[0]);
      ha.tl_dm = as<unsigned long long>(h->tl_dm[0]);
      ha.n_halo = h->mg_counts + 1;
      ha.ctl = h->d_ctl;
      k_halo_place<<<1, 1024, 0, h->stream>>>(ha);
      ++h->launches;
    }
    tr.mark("dict+halo");
    h->mg_n_halo = kHaloMax;
    cap_s = sample_capacity(h);
    if (cap_s < std::max<uint64_t>(2 * n_tl, 1u << 16)) {
      cap_s = std::max<uint64_t>(2 * n_tl, 1u << 16);
      int r = ensure_samples(h, cap_s);
      if (r) return r;
    }
    if (p2p) { int r = mg_export_ensure(h, h->mg_recv_x, cap_s * 16); if (r) return r; }
    bool keys_fit = true;
    for (int attempt = 0;; ++attempt) {
      KS_CUDA(h, cudaMemsetAsync(blk + H, 0, kMgHistBytes, h->stream));
      SoloArgs s{};
      s.solo_stream = as<unsigned long long>(h->solo_stream);
      s.kid_of_slot = h->kid_of_slot;
      s.samples = as<uint4>(h->samples[0]);
      s.capacity = cap_s;
      s.ctl = h->d_ctl;
      k_solo_samples<<<h->sm_count * 4, 256, 0, h->stream>>>(s);
      { int r = run_join(h, 0, n_tl, cap_s, nullptr, nullptr, 0, kHaloMax); if (r) return r; }
      tr.mark("samples+join");
      k_key_hist_dev<<<h->sm_count * 6, 256, 0, h->stream>>>(as<uint4>(h->samples[0]), h->d_ctl, cap_s, reinterpret_cast<unsigned long long*>(blk + H));
      k_mg_header<<<1, 32, 0, h->stream>>>(reinterpret_cast<MgHeader*>(blk), h->d_ctl, h->mg_counts, rec, n_owned, cap_s, mg_ipc_of(h->mg_recv_x));
      h->launches += 3;
      KS_CUDA(h, cudaGetLastError());
      tr.mark("hist+pack2");
      KS_NCCL(h, api->AllGather(blk, h->mg_gathered.p, block2, kNcclUint8, h->mg_comm, h->stream));
      tr.mark("allgather2");
      { int r = mg_fetch_heads(h, block2, width2); if (r) return r; }                                  // ---- wait 1
      // did every rank's keys fit exchange 1?  If not, nothing computed since means anything: grow (alike everywhere,
      // every rank sees the same headers) and start over
      uint32_t need = 0;
      for (int q = 0; q < world; ++q) need = std::max(need, mg_head(h, width2, q).n_local_keys);
      if (need > cap) {
        uint32_t grown = cap;
        while (grown < need) grown <<= 1;
        h->mg_key_cap = grown;
        keys_fit = false;
        break;
      }
      { int r = mg_any_error(h, width2, "decode and join"); if (r) return r; }
      bool any_over = false;
      for (int q = 0; q < world; ++q) {
        const MgHeader& hd = mg_head(h, width2, q);
        if (hd.n_tail > kHaloMax)
          return fail(h, KS_ERR_CAPACITY, "ks_mg_build: rank " + std::to_string(q) + " has more launches reaching into the next window than the halo can hold");
        if (hd.n_halo > kHaloMax)
          return fail(h, KS_ERR_CAPACITY, "ks_mg_build: " + std::to_string(hd.n_halo) + " launches of earlier windows reach into window " + std::to_string(q) +
                                              "; the halo holds " + std::to_string(kHaloMax));
        if (hd.ctl.n_keys != mg_head(h, width2, 0).ctl.n_keys) return fail(h, KS_ERR_COMM, "ks_mg_build: the ranks disagree on the number of keys");
        if (hd.ctl.n_pairs >= kSortMaxItems) return fail(h, KS_ERR_TOO_LARGE, "ks_mg_build: 2^30 samples or more on rank " + std::to_string(q));
        if (hd.ctl.n_pairs > hd.capacity) any_over = true;
      }
      if (!any_over) break;
      if (attempt == 1) return fail(h, KS_ERR_CAPACITY, "ks_mg_build: sample stream still too small");
      const uint64_t mine = mg_head(h, width2, rank).ctl.n_pairs;
      if (mine > cap_s) {  // only the ranks that ran over grow; all of them repeat the step
        cap_s = mine + mine / 16;
        int r = ensure_samples(h, cap_s);
        if (r) return r;
      }
    }
    if (keys_fit) break;
    if (round == 2) return fail(h, KS_ERR_COMM, "ks_mg_build: the key exchange keeps overflowing");
  }
  const Control ctl2 = mg_head(h, width2, rank).ctl;  // a copy: the pinned area is reused by the next exchange
  const uint64_t nk = ctl2.n_keys;
  h->mg_nk = nk;
  h->mg_n_samples = ctl2.n_pairs;
  const uint64_t n_solo = ctl2.n_solo, n_samples_local = ctl2.n_pairs;

  // ---- phase 3: splitters, partition, the samples travel                                        (queued, no wait)
  cudaEventRecord(ev[2], h->stream);
  std::vector<uint64_t> total(kKeyHistBins, 0);
  auto hist_of = [&](int q) { return reinterpret_cast<const uint64_t*>(h->mg_host + width2 * (size_t)q + H); };
  for (int q = 0; q < world; ++q)
    for (uint32_t b = 0; b < kKeyHistBins; ++b) total[b] += hist_of(q)[b];
  uint64_t all = 0;
  for (uint64_t v : total) all += v;
  const int key_bits = bit_length(nk + nk * nk);
  const uint32_t shift = key_bits > 12 ? (uint32_t)(key_bits - 12) : 0u;
  // One or several STAGES.  With peer memory every rank may own up to four key ranges ("parts"): part p belongs to rank
  // p % world and to stage p / world, and the table is the parts' rows in part order.  The rows of a stage are known (and
  // written into this GPU's table, from where the copy engines carry them to the peers on a stream of their own) while
  // the next stage is still being sorted and reduced, so the table's way over NVLink is hidden behind the statistics --
  // or, where the exchange is the longer of the two, the statistics behind the exchange.  Sorting halves costs about a
  // tenth more than sorting the whole, so stages are chosen when the last table of this session says that its exchange
  // takes longer than that (rows x 128 bytes, (world-1)/world of them over NVLink at about 600 GB/s; sort and statistics
  // about 64 ns per thousand samples) -- from numbers every rank has alike.  KS_MG_STAGES=1|2|4 (the same on every rank)
  // overrides the rule.
  int stages = 1;
  if (p2p) {
    const double exchange_ms = (double)h->mg_rows_hint * sizeof(ks_pair_row) * (double)(world - 1) / (double)world / 6.0e8;
    const double reduce_ms = (double)(all / (uint64_t)world) * 6.4e-8;
    if (exchange_ms > 0.1 * reduce_ms && exchange_ms > 0.2) stages = 2;
    if (exchange_ms > 0.4 * reduce_ms && exchange_ms > 2.0) stages = 4;
    if (const char* e = getenv("KS_MG_STAGES")) {
      if (e[0] == '1') stages = 1;
      else if (e[0] == '2') stages = 2;
      else if (e[0] == '4') stages = 4;
    }
    while (stages * world > kMaxDest) stages >>= 1;
  }
  const int parts = stages * world;
  // Part p owns the keys [edge[p], edge[p+1]) in units of FINE bins (key >> fshift).  First cut: the histogram bin in
  // which the share p/parts of the samples is reached.  A bin is 1/4,096 of the key space, and a hot kernel's pairs can put
  // a percent of all samples into one or two of them -- a third of a part when there are 32 parts.  With KS_MG_REFINE=1
  // (the same on every rank) the bins that hold a cut are counted once more in 256 sub-bins each (one more pass over the
  // sample keys, one more exchange and host wait) and the cut is placed inside them, so that all parts hold the same
  // number of samples; every count stays exact (whole bins from the first histogram, split bins from the second).
  // Off by default: on the 1 B-record trace it gained 1 ms of 57.5 on four GPUs and LOST 3.6 ms of 66.2 on eight -- the
  // ranks no longer wait for one another behind sort + statistics, but a part's ROWS (what the copy engines carry) then
  // differ more, and at eight GPUs the copies are what the build waits for.
  const uint32_t sub_bits = std::min<uint32_t>(8, shift);
  bool refine = false;
  if (const char* e = getenv("KS_MG_REFINE")) refine = e[0] == '1' && parts > 1 && sub_bits > 0 && all > 0;
  const uint32_t fshift = refine ? shift - sub_bits : shift;        // fine bin = key >> fshift
  const uint32_t fbits = refine ? sub_bits : 0;                     // fine bins per histogram bin = 1 << fbits
  std::vector<uint64_t> edge(parts + 1, (uint64_t)kKeyHistBins << fbits);
  edge[0] = 0;
  std::vector<uint64_t> coarse((size_t)world * kKeyHistBins);       // the pinned copies are overwritten by the next exchange
  for (int q = 0; q < world; ++q) memcpy(&coarse[(size_t)q * kKeyHistBins], hist_of(q), kMgHistBytes);
  KeySubHistArgs cut{};                                             // the bins that hold a cut, ascending
  std::vector<uint64_t> sub;                                        // [rank][cut bin][sub-bin]
  {
    // first cut, and for every part the samples of its cut bin that belong in front of the cut
    std::vector<uint32_t> cut_bin(parts, 0);
    std::vector<uint64_t> need(parts, 0);
    uint64_t before = 0;
    uint32_t b = 0;
    // (equal shares for all stages: a smaller first stage, so that the copies start earlier, was measured slower -- the
    // copy engines then fall behind and the last stage waits for them)
    for (int p = 1; p < parts; ++p) {
      const uint64_t target = (all * (uint64_t)p + (uint64_t)parts - 1) / (uint64_t)parts;
      while (b < kKeyHistBins && before < target) before += total[b++];
      edge[p] = (uint64_t)b << fbits;
      if (refine && b > 0 && before > target) {  // the cut lies inside bin b - 1
        cut_bin[p] = b;                          // + 1, 0 = none
        need[p] = target - (before - total[b - 1]);
        if (!cut.n_cut || cut.bin[cut.n_cut - 1] != b - 1) cut.bin[cut.n_cut++] = b - 1;
      }
    }
    if (cut.n_cut) {
      const size_t sub_words = (size_t)cut.n_cut << fbits, sub_bytes = sub_words * 8;
      unsigned char* blk = as<unsigned char>(h->mg_block);
      KS_CUDA(h, cudaMemsetAsync(blk, 0, sub_bytes, h->stream));
      cut.sub_bits = fbits;
      k_key_subhist_dev<<<h->sm_count * 6, 256, 0, h->stream>>>(as<uint4>(h->samples[0]), h->d_ctl, cap_s, cut, reinterpret_cast<unsigned long long*>(blk));
      ++h->launches;
      KS_CUDA(h, cudaGetLastError());
      KS_NCCL(h, api->AllGather(blk, h->mg_gathered.p, sub_bytes, kNcclUint8, h->mg_comm, h->stream));
      sub.resize(sub_words * (size_t)world);
      KS_CUDA(h, cudaMemcpyAsync(sub.data(), h->mg_gathered.p, sub_bytes * (size_t)world, cudaMemcpyDeviceToHost, h->stream));
      KS_CUDA(h, cudaStreamSynchronize(h->stream));                                                    // ---- wait 1b
      tr.mark("cut bins counted again");
      for (int p = 1; p < parts; ++p) {
        if (!cut_bin[p]) continue;
        const uint32_t cb = cut_bin[p] - 1;
        uint32_t ci = 0;
        while (cut.bin[ci] != cb) ++ci;
        uint64_t acc = 0;
        uint32_t j = 0;
        while (j < (1u << fbits) && acc < need[p]) {  // the first sub-bin boundary with at least `need` samples in front
          for (int q = 0; q < world; ++q) acc += sub[((size_t)q * cut.n_cut + ci) << fbits | j];
          ++j;
        }
        edge[p] = ((uint64_t)cb << fbits) + j;
      }
    }
    if (stages > 1 && nk) {  // every solo row in stage 0 (a bin boundary: no split bin needed): the table rows of every stage need all solo times
      const uint64_t solo_end = std::min<uint64_t>(kKeyHistBins, ((nk - 1) >> shift) + 1) << fbits;
      for (int p = world; p < parts; ++p) edge[p] = std::max(edge[p], solo_end);
    }
    for (int p = 1; p <= parts; ++p) edge[p] = std::max(edge[p], edge[p - 1]);
  }
  // cnt[q][p]: samples rank q holds for part p -- whole bins from its histogram, split bins from its sub-bin counts
  uint64_t cnt[16][kMaxDest] = {{0}};
  auto count_range = [&](int q, uint64_t lo, uint64_t hi) -> uint64_t {  // fine bins [lo, hi)
    const uint64_t* hq = &coarse[(size_t)q * kKeyHistBins];
    const uint64_t fmask = (1ull << fbits) - 1;
    uint64_t sum = 0;
    while (lo < hi) {
      const uint64_t bin = lo >> fbits, bin_end = (bin + 1) << fbits;
      if (!(lo & fmask) && hi >= bin_end) { sum += hq[bin]; lo = bin_end; continue; }
      uint32_t ci = 0;
      while (ci < cut.n_cut && cut.bin[ci] != bin) ++ci;
      if (ci == cut.n_cut) return ~0ull;  // a split bin that was not counted: cannot happen (checked below)
      const uint64_t stop = std::min(hi, bin_end);
      for (uint64_t f = lo; f < stop; ++f) sum += sub[(((size_t)q * cut.n_cut + ci) << fbits) | (f & fmask)];
      lo = stop;
    }
    return sum;
  };
  for (int q = 0; q < world; ++q)
    for (int p = 0; p < parts; ++p) {
      cnt[q][p] = count_range(q, edge[p], edge[p + 1]);
      if (cnt[q][p] == ~0ull) return fail(h, KS_ERR_COMM, "ks_mg_build: a key range ends inside a histogram bin that was not split");
    }
  std::vector<uint64_t> part_in(parts, 0);  // samples of part p over all ranks
  for (int p = 0; p < parts; ++p) {
    for (int q = 0; q < world; ++q) part_in[p] += cnt[q][p];
    if (part_in[p] >= kSortMaxItems)  // every rank sees the same counts, so all ranks refuse together
      return fail(h, KS_ERR_TOO_LARGE, "ks_mg_build: 2^30 samples or more in the key range of rank " + std::to_string(p % world));
  }
  auto recv_total = [&](int d) { uint64_t v = 0; for (int s = 0; s < stages; ++s) v += part_in[s * world + d]; return v; };
  const uint64_t n_recv = recv_total(rank);
  uint64_t n_stage[4] = {0, 0, 0, 0}, stage_off[5] = {0, 0, 0, 0, 0};  // my parts: their samples, where they begin in my receive buffer
  for (int s = 0; s < stages; ++s) { n_stage[s] = part_in[s * world + rank]; stage_off[s + 1] = stage_off[s] + n_stage[s]; }
  std::vector<uint64_t> send_cnt(world, 0), recv_cnt(world, 0);  // one stage: per peer (the send/recv exchange)
  for (int q = 0; q < world; ++q) { send_cnt[q] = cnt[rank][q]; recv_cnt[q] = cnt[q][rank]; }
  uint32_t splitters[kMaxDest] = {0};
  for (int p = 1; p < parts; ++p) splitters[p - 1] = (uint32_t)edge[p];
  std::vector<uint64_t> soff(world + 1, 0), roff(world + 1, 0);
  for (int q = 0; q < world; ++q) { soff[q + 1] = soff[q] + send_cnt[q]; roff[q + 1] = roff[q] + recv_cnt[q]; }
  {
    uint64_t mine = 0;
    for (int p = 0; p < parts; ++p) mine += cnt[rank][p];
    if (mine != n_samples_local) return fail(h, KS_ERR_COMM, "ks_mg_build: histogram and sample count disagree");
  }
  const uint4* sort_input = nullptr;  // null: sample set 0
  if (p2p) {
    // -- peer memory: the partition pass stores every item straight into its place in the destination's receive buffer:
    // rank d's buffer holds its parts stage after stage; inside a part the senders follow in rank order
    uint64_t my_off_at[kMaxDest] = {0};  // where my items of part p start in its owner's buffer
    bool grow = false;
    for (int d = 0; d < world; ++d) {
      uint64_t in = 0;
      for (int s = 0; s < stages; ++s) {
        const int p = s * world + d;
        for (int q = 0; q < world; ++q) {
          if (q == rank) my_off_at[p] = in;
          in += cnt[q][p];
        }
      }
      if (in * 16 > mg_head(h, width2, d).buf_cap) grow = true;  // rank d's buffer is too small: decided alike everywhere
    }
    if (grow) {
      if (n_recv * 16 > h->mg_recv_x.cap) { int r = mg_export_ensure(h, h->mg_recv_x, n_recv * 16 + n_recv * 4); if (r) return r; }
      unsigned char* blk = as<unsigned char>(h->mg_block);
      k_mg_header<<<1, 32, 0, h->stream>>>(reinterpret_cast<MgHeader*>(blk), h->d_ctl, h->mg_counts, rec, n_owned, cap_s, mg_ipc_of(h->mg_recv_x));
      ++h->launches;
      KS_NCCL(h, api->AllGather(blk, h->mg_gathered.p, H, kNcclUint8, h->mg_comm, h->stream));
      { int r = mg_fetch_heads(h, H, H); if (r) return r; }
    }
    const size_t wh = grow ? H : width2;  // layout of the pinned header copies
    uint4* dest[kMaxDest] = {nullptr};
    for (int p = 0; p < parts; ++p) {
      const int d = p % world;
      unsigned char* base = nullptr;
      if (d == rank) {
        base = reinterpret_cast<unsigned char*>(h->mg_recv_x.p);
      } else {
        { int r = mg_import(h, h->mg_peer_recv[d], mg_head(h, wh, d)); if (r) return r; }
        base = reinterpret_cast<unsigned char*>(h->mg_peer_recv[d].p);
      }
      dest[p] = reinterpret_cast<uint4*>(base + my_off_at[p] * 16);
    }
    { int r = mg_partition_to_peers(h, splitters, fshift, (uint32_t)parts, dest); if (r) return r; }
    tr.mark("wait1+partition to peers");
    { int r = mg_barrier(h); if (r) return r; }
    tr.mark("barrier");
    sort_input = reinterpret_cast<const uint4*>(h->mg_recv_x.p);
    const uint64_t largest = *std::max_element(n_stage, n_stage + 4);
    if (sample_capacity(h) < largest) { int r = ensure_samples(h, largest); if (r) return r; }  // the sort's two sets
  } else {
    // -- NCCL: partition into sample set 1, one send/recv pair per peer with exact sizes, own part by a local copy
    { int64_t r = ks_mg_partition(h, splitters, fshift, (uint32_t)world, h->samples[1].p, sample_capacity(h), nullptr); if (r < 0) return r; }
    tr.mark("wait1+partition");
    const bool in_place = n_recv <= sample_capacity(h);
    if (!in_place) KS_ENSURE(h, h->mg_recv, n_recv * 16);
    unsigned char* recv_base = in_place ? as<unsigned char>(h->samples[0]) : as<unsigned char>(h->mg_recv);
    const unsigned char* send_base = as<unsigned char>(h->samples[1]);
    if (send_cnt[rank])
      KS_CUDA(h, cudaMemcpyAsync(recv_base + roff[rank] * 16, send_base + soff[rank] * 16, send_cnt[rank] * 16, cudaMemcpyDeviceToDevice, h->stream));
    if (world > 1) {
      KS_NCCL(h, api->GroupStart());
      for (int q = 0; q < world; ++q) {
        if (q == rank) continue;
        if (send_cnt[q]) KS_NCCL(h, api->Send(send_base + soff[q] * 16, send_cnt[q] * 16, kNcclUint8, q, h->mg_comm, h->stream));
        if (recv_cnt[q]) KS_NCCL(h, api->Recv(recv_base + roff[q] * 16, recv_cnt[q] * 16, kNcclUint8, q, h->mg_comm, h->stream));
      }
      KS_NCCL(h, api->GroupEnd());
    }
    tr.mark("sample exchange");
    if (!in_place) {  // growing frees both sample sets; the free waits for the sends that still read set 1
      { int r = ensure_samples(h, n_recv); if (r) return r; }
      KS_CUDA(h, cudaMemcpyAsync(h->samples[0].p, h->mg_recv.p, n_recv * 16, cudaMemcpyDeviceToDevice, h->stream));
    }
  }

  // ---- phases 4 and 5, once per stage: K2 + K4 over the received part, exchange 4 (then a wait), the table rows
  // A returning call leaves nothing running on the side stream (the next call may free or overwrite what its copies read).
  struct SideGuard {
    ks_handle* h;
    bool armed = false;
    void drain() { if (armed) for (auto& st : h->mg_side) cudaStreamSynchronize(st); armed = false; }
    ~SideGuard() { drain(); }
  } side{h};
  std::vector<uint64_t> part_rows(parts, 0);  // table rows of every part, as the stages report them
  auto row_base = [&](int p) { uint64_t v = 0; for (int i = 0; i < p; ++i) v += part_rows[i]; return v; };
  uint64_t rows_total = 0;
  const size_t off_launches = H + (size_t)nk * 8, off_solo = off_launches + (size_t)nk * 8;
  const size_t block4 = (off_solo + (size_t)nk * 8 + 15) & ~(size_t)15;
  for (int s = 0; s < stages; ++s) {
    const bool last = s + 1 == stages;
    if (s == 0) cudaEventRecord(ev[3], h->stream);
    const uint4* in_s = sort_input ? sort_input + stage_off[s] : nullptr;
    // the part's keys lie in [edge << shift, next edge << shift): sorted over the bits of that width only
    const uint64_t key_end = nk + nk * nk + 1;
    const uint64_t key_lo = std::min<uint64_t>(edge[s * world + rank] << fshift, key_end);
    const uint64_t key_hi = s * world + rank + 1 == parts ? key_end : std::min<uint64_t>(edge[s * world + rank + 1] << fshift, key_end);
    { int r = mg_reduce_queue(h, p2p ? n_stage[s] : n_recv, in_s, s == 0, key_lo, key_hi); if (r) return r; }
    tr.mark("sort+stats");
    if (p2p && s == 0) { int r = mg_export_ensure(h, h->mg_table_x, std::max<size_t>(h->mg_table_x.cap, (size_t)8 << 20)); if (r) return r; }
    // block 4: [header | solo times | launches per key | solo launches per key], all by dense key id; later stages: the header
    const size_t width4 = s == 0 ? block4 : H;
    {
      unsigned char* blk = as<unsigned char>(h->mg_block);
      k_mg_header<<<1, 32, 0, h->stream>>>(reinterpret_cast<MgHeader*>(blk), h->d_ctl, nullptr, rec, n_owned, 0, mg_ipc_of(h->mg_table_x));
      ++h->launches;
      if (nk && s == 0) {
        KS_CUDA(h, cudaMemcpyAsync(blk + H, h->solo_ns, nk * 8, cudaMemcpyDeviceToDevice, h->stream));
        k_counts_export_dev<<<(unsigned)((nk + 255) / 256), 256, 0, h->stream>>>(h->slot_of_kid, h->dict_launches, h->dict_solo, h->d_ctl, (uint32_t)nk,
                                                                                 reinterpret_cast<unsigned long long*>(blk + off_launches),
                                                                                 reinterpret_cast<unsigned long long*>(blk + off_solo));
        ++h->launches;
      }
      KS_NCCL(h, api->AllGather(blk, h->mg_gathered.p, width4, kNcclUint8, h->mg_comm, h->stream));
    }
    tr.mark("allgather4");
    { int r = mg_fetch_heads(h, width4, H); if (r) return r; }                                         // ---- wait 2 (per stage)
    {
      // A key range with more rows than the row arrays were sized for (and no limit asked for): every rank sees it in the
      // gathered headers, sizes its arrays for the largest range and the whole build is made again, by all ranks alike.
      uint64_t most_rows = 0;
      for (int q = 0; q < world; ++q) {
        const Control& c = mg_head(h, H, q).ctl;
        if ((c.err & kErrTooLarge) && !(c.err & ~(kErrTooLarge | kErrUnordered))) most_rows = std::max<uint64_t>(most_rows, c.pad2[0]);
      }
      if (most_rows > h->cfg.max_pair_rows && most_rows < (1ull << 31) && h->rows_auto) {
        h->cfg.max_pair_rows = (uint32_t)std::min<uint64_t>(most_rows + most_rows / 8, 0x7FFFFFFFull);
        side.drain();
        return ks_mg_build(h, records, n_owned, flags, info);
      }
    }
    { int r = mg_any_error(h, H, "reduce"); if (r) return r; }
    for (int q = 0; q < world; ++q) {
      const Control& c = mg_head(h, H, q).ctl;
      part_rows[s * world + q] = c.n_rows > c.ticket2 ? c.n_rows - c.ticket2 : 0u;
    }
    const int p_mine = s * world + rank;
    const uint64_t rows_mine = part_rows[p_mine];
    if (tr.on) tr.note += " [stage " + std::to_string(s) + ": " + std::to_string(n_stage[s]) + " samples, " + std::to_string(rows_mine) + " rows]";
    const uint64_t rows_before = row_base(s * world);  // the rows of the stages before this one
    rows_total = row_base(parts);                      // the rows known so far; behind the last stage: the table
    if (s == 0) *h->h_ctl = mg_head(h, H, rank).ctl;

    // ---- phase 5: every key's solo time, this rank's rows straight into their place, the other ranks' rows around them
    if (last) cudaEventRecord(ev[4], h->stream);
    if (nk && s == 0) {
      k_solo_merge<<<(unsigned)((nk + 255) / 256), 256, 0, h->stream>>>(gathered, block4, (uint32_t)world, H, (uint32_t)nk, h->solo_ns);
      k_counts_sum_import<<<(unsigned)((nk + 255) / 256), 256, 0, h->stream>>>(gathered, block4, (uint32_t)world, off_launches, off_solo, h->slot_of_kid, (uint32_t)nk,
                                                                               h->dict_launches, h->dict_solo);
      h->launches += 2;
    }
    if (p2p) {
      // -- peer memory.  Behind the last stage the table's size is known; before, it is the last table's, or the rows seen
      // so far scaled to all stages and a quarter
      const uint64_t want_rows = last ? rows_total : std::max<uint64_t>(h->mg_rows_hint, rows_total * (uint64_t)stages / (uint64_t)(s + 1) * 5 / 4);
      const size_t table_bytes = std::max<uint64_t>(want_rows, 1) * sizeof(ks_pair_row);
      bool grow = false;
      for (int q = 0; q < world; ++q) grow = grow || table_bytes > mg_head(h, H, q).buf_cap;
      ks_pair_row* old_table = reinterpret_cast<ks_pair_row*>(h->mg_table_x.p);
      if (grow) {
        side.drain();  // the copies of the earlier stages went into the old tables: made again below
        if (table_bytes > h->mg_table_x.cap) { int r = mg_export_ensure(h, h->mg_table_x, table_bytes + table_bytes / 4); if (r) return r; }
        unsigned char* blk = as<unsigned char>(h->mg_block);
        k_mg_header<<<1, 32, 0, h->stream>>>(reinterpret_cast<MgHeader*>(blk), h->d_ctl, nullptr, rec, n_owned, 0, mg_ipc_of(h->mg_table_x));
        ++h->launches;
        KS_NCCL(h, api->AllGather(blk, h->mg_gathered.p, H, kNcclUint8, h->mg_comm, h->stream));  // behind k_solo_merge, which read the old blocks
        { int r = mg_fetch_heads(h, H, H); if (r) return r; }
      }
      ks_pair_row* peer_tab[16] = {nullptr};
      for (int q = 0; q < world; ++q) {
        if (q == rank) continue;
        { int r = mg_import(h, h->mg_peer_table[q], mg_head(h, H, q)); if (r) return r; }
        peer_tab[q] = reinterpret_cast<ks_pair_row*>(h->mg_peer_table[q].p);
      }
      ks_pair_row* table = reinterpret_cast<ks_pair_row*>(h->mg_table_x.p);
      const uint64_t base = row_base(p_mine);
      if (stages == 1) {
        // one stage: the table kernel stores its rows into every table itself (one pass, nothing to overlap with)
        ks_pair_row* peers[15];
        uint32_t n_peers = 0;
        for (int q = 0; q < world; ++q)
          if (q != rank) peers[n_peers++] = peer_tab[q] + base;
        { int r = mg_finalize_queue(h, table + base, (uint32_t)rows_mine, n_peers, peers); if (r) return r; }
      } else {
        // Stages: the kernel writes this GPU's table only and the copy engines carry the rows to the peers on the side
        // stream, one peer after the other -- they take no SM, register or shared memory from the sort and statistics
        // kernels of the next stage, which a storing kernel running beside them does (measured: the next stage a third
        // slower).  The peers are visited in a rotated order so that no GPU is everybody's target at the same time; two or
        // four streams side by side were measured no faster or slower than one.
        if (grow && s > 0 && table != old_table && rows_before)  // the earlier stages' rows (all ranks') move to the new table
          KS_CUDA(h, cudaMemcpyAsync(table, old_table, rows_before * sizeof(ks_pair_row), cudaMemcpyDeviceToDevice, h->stream));
        { int r = mg_finalize_queue(h, table + base, (uint32_t)rows_mine, 0, nullptr, s == 0); if (r) return r; }
        KS_CUDA(h, cudaEventRecord(h->mg_side_ev[0], h->stream));
        KS_CUDA(h, cudaStreamWaitEvent(h->mg_side[0], h->mg_side_ev[0], 0));
        side.armed = true;
        for (int k = 1; k < world; ++k) {
          const int q = (rank + k) % world;
          if (rows_mine)
            KS_CUDA(h, cudaMemcpyAsync(peer_tab[q] + base, table + base, rows_mine * sizeof(ks_pair_row), cudaMemcpyDeviceToDevice, h->mg_side[0]));
        }
        KS_CUDA(h, cudaEventRecord(h->mg_side_ev[1], h->mg_side[0]));
        if (last) {
          KS_CUDA(h, cudaStreamWaitEvent(h->stream, h->mg_side_ev[1], 0));
          side.armed = false;
        }
      }
      if (!last) {
        tr.mark("wait2+rows on their way");
      } else {
        tr.mark("wait2+finalize to peers");
        { int r = mg_barrier(h); if (r) return r; }
        tr.mark("barrier");
        h->pair_rows_src = table;
        h->mg_rows_hint = rows_total;
      }
    } else {
      KS_ENSURE(h, h->pair_rows, std::max<size_t>(rows_total, 1) * sizeof(ks_pair_row));
      ks_pair_row* table = as<ks_pair_row>(h->pair_rows);
      { int r = mg_finalize_queue(h, table + row_base(rank), (uint32_t)rows_mine); if (r) return r; }
      tr.mark("wait2+finalize");
      if (world > 1) {
        KS_NCCL(h, api->GroupStart());
        for (int q = 0; q < world; ++q) {
          if (q == rank) continue;
          const uint64_t rows_q = part_rows[q];
          if (rows_mine) KS_NCCL(h, api->Send(table + row_base(rank), rows_mine * sizeof(ks_pair_row), kNcclUint8, q, h->mg_comm, h->stream));
          if (rows_q) KS_NCCL(h, api->Recv(table + row_base(q), rows_q * sizeof(ks_pair_row), kNcclUint8, q, h->mg_comm, h->stream));
        }
        KS_NCCL(h, api->GroupEnd());
      }
      tr.mark("shard exchange");
      h->pair_rows_src = table;
    }
  }
  tr.report();
  h->n_key_rows = nk;
  h->n_pair_rows = rows_total;
  if (info) {
    memset(info, 0, sizeof(*info));
    info->n_records = n_owned;
    info->n_keys = nk;
    info->n_solo = n_solo;
    info->n_pairs = n_samples_local - n_solo;
    info->n_rows = rows_total;
    info->max_duration_ns = ctl2.max_dur;
    info->min_start_ns = ctl2.min_start;
    info->max_start_ns = ctl2.max_start;
    info->was_time_ordered = 1;
    if (flags & KS_TIMING) {  // device time of the five phases, each up to and including its exchange: one more host wait
      cudaEventRecord(ev[5], h->stream);
      KS_CUDA(h, cudaStreamSynchronize(h->stream));
      info->ms_decode = ev_ms(ev[0], ev[1]);
      info->ms_join = ev_ms(ev[1], ev[2]);
      info->ms_order = ev_ms(ev[2], ev[3]);   // partition by key range + the sample exchange
      info->ms_reduce = ev_ms(ev[3], ev[4]);  // K2 + K4
      info->ms_finalize = ev_ms(ev[4], ev[5]);
      info->ms_total = ev_ms(ev[0], ev[5]);
    }
  }
  return (int64_t)rows_total;
}

}  // extern "C"
