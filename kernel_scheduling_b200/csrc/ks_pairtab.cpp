// ks_pairtab.cpp -- writer of the shared-memory pair table (include/ks_pairtab_shm.h).  Host code only: it takes the
// key rows and pair rows of finished tables (SHAPE and TYPE) from host memory, builds the sorted-keys + CSR image and
// makes it visible under the segment's name with tmp + rename, so a reader never sees a half-written table.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cerrno>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "../../include/ks_b200.h"
#include "../../include/ks_pairtab_shm.h"

namespace {

thread_local std::string g_pairtab_error;

uint64_t align8(uint64_t v) { return (v + 7u) & ~(uint64_t)7u; }

struct TableImage {
  std::vector<ks_pairtab_key> keys;
  std::vector<uint32_t> row_ptr, cols;
  std::vector<ks_pairtab_val> vals;
};

int64_t find_key(const std::vector<ks_pairtab_key>& keys, uint64_t key) {
  size_t lo = 0, hi = keys.size();
  while (lo < hi) {
    const size_t mid = (lo + hi) >> 1;
    if (keys[mid].key < key) lo = mid + 1; else hi = mid;
  }
  return lo < keys.size() && keys[lo].key == key ? (int64_t)lo : -1;
}

bool build_table(const ks_key_row* key_rows, uint64_t n_keys, const ks_pair_row* pair_rows, uint64_t n_rows, TableImage* out, std::string* err) {
  out->keys.resize(n_keys);
  for (uint64_t i = 0; i < n_keys; ++i) {
    const ks_key_row& r = key_rows[i];
    if (i && key_rows[i - 1].key >= r.key) { *err = "key rows are not sorted by key"; return false; }
    ks_pairtab_key& k = out->keys[i];
    k.key = r.key;
    k.name_id = r.name_id;
    k.tenant = r.tenant;
    for (int d = 0; d < 3; ++d) { k.grid[d] = r.grid[d]; k.block[d] = r.block[d]; }
    k.solo_us = r.solo_ns / 1000.0;  // NaN stays NaN
    k.launches = r.launches;
  }
  out->row_ptr.assign(n_keys + 1, 0);
  out->cols.resize(n_rows);
  out->vals.resize(n_rows);
  int64_t prev_a = -1, prev_b = -1;
  for (uint64_t i = 0; i < n_rows; ++i) {
    const ks_pair_row& p = pair_rows[i];
    const int64_t ia = find_key(out->keys, p.key_a), ib = find_key(out->keys, p.key_b);
    if (ia < 0 || ib < 0) { *err = "a pair row names a key that has no key row"; return false; }
    if (ia < prev_a || (ia == prev_a && ib <= prev_b)) { *err = "pair rows are not sorted by (key_a, key_b)"; return false; }
    prev_a = ia; prev_b = ib;
    ++out->row_ptr[ia + 1];
    out->cols[i] = (uint32_t)ib;
    out->vals[i].efficiency = (float)p.efficiency;
    out->vals[i].gangs = p.count > 0xFFFFFFFFull ? 0xFFFFFFFFu : (uint32_t)p.count;
  }
  for (uint64_t i = 0; i < n_keys; ++i) out->row_ptr[i + 1] += out->row_ptr[i];
  return true;
}

uint64_t strings_bytes(const char* const* s, uint64_t n) {
  uint64_t b = (n + 1) * 8;
  for (uint64_t i = 0; i < n; ++i) b += strlen(s[i]);
  return align8(b);
}

void write_strings(char* base, uint64_t table_off, const char* const* s, uint64_t n) {
  uint64_t* off = reinterpret_cast<uint64_t*>(base + table_off);
  uint64_t at = table_off + (n + 1) * 8;
  for (uint64_t i = 0; i < n; ++i) {
    off[i] = at;
    const size_t len = strlen(s[i]);
    memcpy(base + at, s[i], len);
    at += len;
  }
  off[n] = at;
}

uint64_t place_table(char* base, uint64_t at, const TableImage& t, ks_pairtab_table* d) {
  d->n_keys = t.keys.size();
  d->n_rows = t.cols.size();
  d->keys_off = at;
  if (base && d->n_keys) memcpy(base + at, t.keys.data(), t.keys.size() * sizeof(ks_pairtab_key));
  at = align8(at + t.keys.size() * sizeof(ks_pairtab_key));
  d->row_ptr_off = at;
  if (base) memcpy(base + at, t.row_ptr.data(), t.row_ptr.size() * 4);
  at = align8(at + t.row_ptr.size() * 4);
  d->cols_off = at;
  if (base && d->n_rows) memcpy(base + at, t.cols.data(), t.cols.size() * 4);
  at = align8(at + t.cols.size() * 4);
  d->vals_off = at;
  if (base && d->n_rows) memcpy(base + at, t.vals.data(), t.vals.size() * sizeof(ks_pairtab_val));
  return align8(at + t.vals.size() * sizeof(ks_pairtab_val));
}

int fail_pairtab(const std::string& msg) {
  g_pairtab_error = msg;
  return -KS_ERR_ARG;
}

}  // namespace

extern "C" {

const char* ks_pairtab_last_error(void) { return g_pairtab_error.c_str(); }

int64_t ks_pairtab_publish(const char* shm_name, const ks_key_row* shape_keys, uint64_t n_shape_keys, const ks_pair_row* shape_pairs, uint64_t n_shape_rows,
                           const ks_key_row* type_keys, uint64_t n_type_keys, const ks_pair_row* type_pairs, uint64_t n_type_rows, const char* const* names,
                           uint64_t n_names, const char* const* models, uint64_t n_models, uint64_t generation) {
  if (!shm_name || shm_name[0] != '/' || strchr(shm_name + 1, '/')) return fail_pairtab("ks_pairtab_publish: the name must look like \"/segment\"");
  if ((!shape_keys && n_shape_keys) || (!shape_pairs && n_shape_rows) || (!type_keys && n_type_keys) || (!type_pairs && n_type_rows) || (!names && n_names) ||
      (!models && n_models))
    return fail_pairtab("ks_pairtab_publish: null array");
  if (n_shape_rows >= (1ull << 32) || n_type_rows >= (1ull << 32) || n_shape_keys >= (1ull << 32) || n_type_keys >= (1ull << 32))
    return fail_pairtab("ks_pairtab_publish: 2^32 rows or more");
  TableImage shape, type;
  std::string err;
  if (!build_table(shape_keys, n_shape_keys, shape_pairs, n_shape_rows, &shape, &err)) return fail_pairtab("ks_pairtab_publish (SHAPE table): " + err);
  if (!build_table(type_keys, n_type_keys, type_pairs, n_type_rows, &type, &err)) return fail_pairtab("ks_pairtab_publish (TYPE table): " + err);

  ks_pairtab_header hd;
  memset(&hd, 0, sizeof(hd));
  hd.magic = KS_PAIRTAB_MAGIC;
  hd.version = 1;
  hd.generation = generation;
  uint64_t at = align8(sizeof(hd));
  hd.n_names = n_names;
  hd.names_off = at;
  at += strings_bytes(names, n_names);
  hd.n_models = n_models;
  hd.models_off = at;
  at += strings_bytes(models, n_models);
  const uint64_t tables_at = at;
  at = place_table(nullptr, at, shape, &hd.shape);
  at = place_table(nullptr, at, type, &hd.type);
  hd.total_bytes = at;

  const std::string tmp = std::string(shm_name) + ".tmp";
  const int fd = shm_open(tmp.c_str(), O_CREAT | O_RDWR | O_TRUNC, 0644);
  if (fd < 0) return fail_pairtab(std::string("ks_pairtab_publish: shm_open: ") + strerror(errno));
  if (ftruncate(fd, (off_t)hd.total_bytes) != 0) {
    const std::string e = strerror(errno);
    close(fd);
    shm_unlink(tmp.c_str());
    return fail_pairtab("ks_pairtab_publish: ftruncate: " + e);
  }
  void* map = mmap(nullptr, hd.total_bytes, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  close(fd);
  if (map == MAP_FAILED) {
    const std::string e = strerror(errno);
    shm_unlink(tmp.c_str());
    return fail_pairtab("ks_pairtab_publish: mmap: " + e);
  }
  char* base = static_cast<char*>(map);
  memcpy(base, &hd, sizeof(hd));
  write_strings(base, hd.names_off, names, n_names);
  write_strings(base, hd.models_off, models, n_models);
  ks_pairtab_table scratch;
  uint64_t w = place_table(base, tables_at, shape, &scratch);
  place_table(base, w, type, &scratch);
  msync(map, hd.total_bytes, MS_SYNC);
  munmap(map, hd.total_bytes);
  // POSIX shared memory lives under /dev/shm on Linux (the reference is Linux-only: shm_open + CUPTI); rename is atomic there
  const std::string from = "/dev/shm" + tmp, to = std::string("/dev/shm") + shm_name;
  if (rename(from.c_str(), to.c_str()) != 0) {
    const std::string e = strerror(errno);
    shm_unlink(tmp.c_str());
    return fail_pairtab("ks_pairtab_publish: rename: " + e);
  }
  return (int64_t)hd.total_bytes;
}

int ks_pairtab_unlink(const char* shm_name) {
  if (!shm_name) return -KS_ERR_ARG;
  return shm_unlink(shm_name) == 0 || errno == ENOENT ? KS_OK : -KS_ERR_ARG;
}

}  // extern "C"
