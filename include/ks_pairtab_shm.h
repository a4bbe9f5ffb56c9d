/* ks_pairtab_shm.h -- the pair table in a POSIX shared-memory segment, for a scheduler that wants the lookup of
 * scheduler/scheduler_daemon.cpp:269-274 (lookup_eff) as a binary search over arrays instead of a string-keyed hash map
 * filled from pair_eff.tsv (:230-249).  No counterpart in the reference: its shared memory (scheduler/shared_state.hpp)
 * carries the launch queue only; this is a segment of its own, and a new layout gets a new name, as there (:11-14).
 *
 * Writer: ks_pairtab_publish (libks_b200.so, host code).  It writes a complete image to "<name>.tmp" and renames it over
 * "<name>" (the tmp + rename of scheduler_daemon.cpp:766-789): a segment never changes once visible, so readers need no
 * lock; a reader that wants a newer table opens the name again.
 *
 * Reader: this header alone (C99 or C++), no library.
 *
 * Image: header | names | models | SHAPE table | TYPE table.  A table = keys sorted by kernel key + CSR over the pair rows
 * (row i of the CSR = pairs whose lower-tenant key is keys[i]; cols = index of the other key, ascending).  Kernel key =
 * ks_kernel_key (the 64-bit key of include/ks_b200.h) of (name id, grid, block, smem = 0, tenant); TYPE keys have grid 0. */
#ifndef KS_PAIRTAB_SHM_H
#define KS_PAIRTAB_SHM_H

#include <stdint.h>
#include <string.h>

#ifdef __cplusplus
extern "C" {
#endif

#define KS_PAIRTAB_SHM_NAME "/kernel_sched_pairtab_v1"
#define KS_PAIRTAB_MAGIC 0x3154524941505348ull /* "HSPAIRT1" little endian */

typedef struct ks_pairtab_key {
  uint64_t key;
  uint32_t name_id, tenant;
  uint32_t grid[3], block[3];
  double solo_us;    /* median solo time; NaN if the key has no solo launch (kernel_us.tsv leaves such rows out) */
  uint64_t launches;
} ks_pairtab_key; /* 56 bytes */

typedef struct ks_pairtab_val {
  float efficiency;  /* NaN if one of the keys has no solo time */
  uint32_t gangs;    /* how often the two kernels overlapped (saturates at 2^32 - 1) */
} ks_pairtab_val;

typedef struct ks_pairtab_table {
  uint64_t n_keys, n_rows;
  uint64_t keys_off;     /* ks_pairtab_key[n_keys] */
  uint64_t row_ptr_off;  /* uint32_t[n_keys + 1] */
  uint64_t cols_off;     /* uint32_t[n_rows] */
  uint64_t vals_off;     /* ks_pairtab_val[n_rows] */
} ks_pairtab_table;

typedef struct ks_pairtab_header {
  uint64_t magic;
  uint32_t version;      /* 1 */
  uint32_t reserved;
  uint64_t total_bytes;
  uint64_t generation;   /* the writer's count of published tables */
  uint64_t n_names, names_off;    /* names_off: uint64_t[n_names + 1] offsets into the blob behind them */
  uint64_t n_models, models_off;  /* the same for model (tenant) strings */
  ks_pairtab_table shape, type;
} ks_pairtab_header;

static inline const ks_pairtab_header* ks_pairtab_check(const void* seg, uint64_t mapped_bytes) {
  const ks_pairtab_header* h = (const ks_pairtab_header*)seg;
  if (!seg || mapped_bytes < sizeof(*h) || h->magic != KS_PAIRTAB_MAGIC || h->version != 1 || h->total_bytes > mapped_bytes) return 0;
  return h;
}

/* string i of a string table (names or models): pointer and length (not NUL terminated) */
static inline const char* ks_pairtab_string(const void* seg, uint64_t table_off, uint64_t i, uint64_t* len) {
  const uint64_t* off = (const uint64_t*)((const char*)seg + table_off);
  *len = off[i + 1] - off[i];
  return (const char*)seg + off[i];
}

/* index of `key` in the table's keys, or -1 */
static inline int64_t ks_pairtab_find_key(const void* seg, const ks_pairtab_table* t, uint64_t key) {
  const ks_pairtab_key* keys = (const ks_pairtab_key*)((const char*)seg + t->keys_off);
  uint64_t lo = 0, hi = t->n_keys;
  while (lo < hi) {
    const uint64_t mid = (lo + hi) >> 1;
    if (keys[mid].key < key) lo = mid + 1; else hi = mid;
  }
  return lo < t->n_keys && keys[lo].key == key ? (int64_t)lo : -1;
}

/* the pair row of two kernels of one table (either order), or NULL */
static inline const ks_pairtab_val* ks_pairtab_find_pair(const void* seg, const ks_pairtab_table* t, uint64_t key_x, uint64_t key_y) {
  const ks_pairtab_key* keys = (const ks_pairtab_key*)((const char*)seg + t->keys_off);
  int64_t ix = ks_pairtab_find_key(seg, t, key_x), iy = ks_pairtab_find_key(seg, t, key_y);
  if (ix < 0 || iy < 0) return 0;
  if (keys[ix].tenant > keys[iy].tenant) { const int64_t s = ix; ix = iy; iy = s; }  /* rows are stored under the lower tenant */
  const uint32_t* row_ptr = (const uint32_t*)((const char*)seg + t->row_ptr_off);
  const uint32_t* cols = (const uint32_t*)((const char*)seg + t->cols_off);
  uint32_t lo = row_ptr[ix], hi = row_ptr[ix + 1];
  while (lo < hi) {
    const uint32_t mid = (lo + hi) >> 1;
    if (cols[mid] < (uint32_t)iy) lo = mid + 1; else hi = mid;
  }
  if (lo == row_ptr[ix + 1] || cols[lo] != (uint32_t)iy) return 0;
  return (const ks_pairtab_val*)((const char*)seg + t->vals_off) + lo;
}

/* scheduler_daemon.cpp:269-274: the shape-pair row if at least min_gangs gangs measured it, else the type-pair row, else NULL */
static inline const ks_pairtab_val* ks_pairtab_lookup_eff(const void* seg, uint64_t shape_a, uint64_t shape_b, uint64_t type_a, uint64_t type_b, uint32_t min_gangs) {
  const ks_pairtab_header* h = (const ks_pairtab_header*)seg;
  const ks_pairtab_val* s = ks_pairtab_find_pair(seg, &h->shape, shape_a, shape_b);
  if (s && s->gangs >= min_gangs) return s;
  return ks_pairtab_find_pair(seg, &h->type, type_a, type_b);
}

/* scheduler_daemon.cpp:250-264 / :265-268: a kernel's median solo time, the exact shape first, then its type; NaN if unknown */
static inline double ks_pairtab_kernel_us(const void* seg, uint64_t shape_key, uint64_t type_key) {
  const ks_pairtab_header* h = (const ks_pairtab_header*)seg;
  int64_t i = ks_pairtab_find_key(seg, &h->shape, shape_key);
  if (i >= 0) {
    const double v = ((const ks_pairtab_key*)((const char*)seg + h->shape.keys_off))[i].solo_us;
    if (v == v) return v;
  }
  i = ks_pairtab_find_key(seg, &h->type, type_key);
  if (i >= 0) return ((const ks_pairtab_key*)((const char*)seg + h->type.keys_off))[i].solo_us;
  { union { uint64_t u; double d; } nan; nan.u = 0x7FF8000000000000ull; return nan.d; }
}

#ifdef __cplusplus
}
#endif
#endif
