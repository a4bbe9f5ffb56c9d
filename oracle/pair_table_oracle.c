/* pair_table_oracle.c -- CPU oracle for the trace -> interference-table path, in plain C with OpenMP.
 *
 * TEST INFRASTRUCTURE, NOT A PRODUCT PATH.  Only the tests, the smoke check and the CPU-baseline / reference legs of
 * the benchmark may load this library; the product library never does.
 *
 * It restates the same definitions as oracle/pair_table_oracle.py (whose header lists the reference lines they come
 * from: key composition scheduler/scheduler_daemon.cpp:196-197, :210-213; TYPE key :213 and
 * profiling/pairprof_daemon.cpp:122-123; solo time = median, scheduler_daemon.cpp:207; pair orientation
 * pairprof_daemon.cpp:127; NaN convention postprocess/profile_postprocess.py:14; efficiency scheduler_daemon.cpp:6,
 * :319-320) at a speed that lets the parity tests run at the benchmark's full sizes.  It is kept equal to the numpy
 * oracle column by column (tests/test_oracle_golden.py) and deliberately works differently from the CUDA path:
 * per-tenant timelines joined pairwise with binary searches, every slowdown sample divided in floating point first
 * and the order statistics then selected on the doubles.
 *
 * PARITY PINNING: like the numpy oracle, the join and the statistics are "parity unpinned" (the reference has no
 * implementation or test of them); the parts the reference defines are pinned elsewhere (tests/golden/).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <stdio.h>
#include <time.h>
#ifdef _OPENMP
#include <omp.h>
#endif

typedef struct {
  uint32_t name_id, grid[3], block[3], smem_word;
  uint64_t start_ns, end_ns;
} kso_record;

typedef struct {
  uint64_t n_keys, n_rows, n_pairs;
  /* per key, sorted by key */
  uint64_t* key;
  uint32_t *name_id, *grid, *block, *smem, *tenant; /* grid, block: 3 per key */
  uint64_t *launches, *solo_launches;
  double* solo_ns;
  /* per pair row, sorted by (key_a, key_b) */
  uint64_t *key_a, *key_b, *count, *flags, *span_sum_ns;
  double *sum_a, *mean_a, *min_a, *max_a, *median_a;
  double *sum_b, *mean_b, *min_b, *max_b, *median_b;
  double* efficiency;
} kso_table;

static double now_s(void) { struct timespec t; clock_gettime(CLOCK_MONOTONIC, &t); return t.tv_sec + 1e-9 * t.tv_nsec; }
#define TICK(name) do { if (timing) { double t_ = now_s(); fprintf(stderr, "  kso %-10s %.3f s\n", name, t_ - t_last); t_last = t_; } } while (0)

enum { KSO_OK = 0, KSO_ERR_RECORD = -1, KSO_ERR_DURATION = -2, KSO_ERR_MEMORY = -3, KSO_ERR_KEYS = -4 };

#define SOLO_BIT 0x00800000u
#define SMEM_MASK 0x007FFFFFu

static uint64_t mix64(uint64_t x) { /* splitmix64's output function */
  x ^= x >> 30;
  x *= 0xBF58476D1CE4E5B9ull;
  x ^= x >> 27;
  x *= 0x94D049BB133111EBull;
  x ^= x >> 31;
  return x;
}

static uint64_t key_of(const kso_record* r, int type_mode) {
  const uint64_t G = 0x9E3779B97F4A7C15ull;
  uint64_t g0 = r->grid[0], g1 = r->grid[1], g2 = r->grid[2];
  uint64_t w = r->smem_word & ~SOLO_BIT;
  if (type_mode) { g0 = g1 = g2 = 0; w &= 0xFF000000u; }
  uint64_t h = mix64(((uint64_t)r->name_id | (g0 << 32)) + G);
  h = mix64((h ^ (g1 | (g2 << 32))) + G);
  h = mix64((h ^ ((uint64_t)r->block[0] | ((uint64_t)r->block[1] << 32))) + G);
  h = mix64((h ^ ((uint64_t)r->block[2] | (w << 32))) + G);
  return h ? h : 1ull;
}

void kso_kernel_keys(const void* records, uint64_t n, int type_mode, uint64_t* out) {
  const kso_record* rec = (const kso_record*)records;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < (int64_t)n; ++i) out[i] = key_of(rec + i, type_mode);
}

/* ---- distinct keys: an open-addressing set that remembers the first record of every key ------------------ */
typedef struct {
  uint64_t* key;
  uint64_t* first;
  uint32_t* kid;
  uint64_t mask, used;
} keyset;

static int keyset_init(keyset* s, uint64_t slots) {
  s->key = (uint64_t*)calloc(slots, 8);
  s->first = (uint64_t*)malloc(slots * 8);
  s->kid = (uint32_t*)malloc(slots * 4);
  s->mask = slots - 1;
  s->used = 0;
  return s->key && s->first && s->kid;
}
static void keyset_free(keyset* s) { free(s->key); free(s->first); free(s->kid); }
static uint64_t keyset_slot(const keyset* s, uint64_t k) {
  uint64_t i = (k * 0x9E3779B97F4A7C15ull) >> 20 & s->mask;
  while (s->key[i] && s->key[i] != k) i = (i + 1) & s->mask;
  return i;
}
static int keyset_add(keyset* s, uint64_t k, uint64_t idx) {
  const uint64_t i = keyset_slot(s, k);
  if (!s->key[i]) {
    if (s->used * 2 > s->mask) return 0; /* too many distinct keys for the table */
    s->key[i] = k;
    s->first[i] = idx;
    ++s->used;
  } else if (idx < s->first[i]) {
    s->first[i] = idx;
  }
  return 1;
}

static int cmp_u64(const void* a, const void* b) {
  const uint64_t x = *(const uint64_t*)a, y = *(const uint64_t*)b;
  return x < y ? -1 : x > y;
}
static int cmp_u32(const void* a, const void* b) {
  const uint32_t x = *(const uint32_t*)a, y = *(const uint32_t*)b;
  return x < y ? -1 : x > y;
}

/* ---- order statistics on doubles: x[k] of the sorted array, by quickselect (in place) -------------------- */
static double select_k(double* x, uint64_t n, uint64_t k_) {
  int64_t lo = 0, hi = (int64_t)n - 1;
  const int64_t k = (int64_t)k_;
  while (lo < hi) {
    const int64_t mid = lo + (hi - lo) / 2;
    const double a = x[lo], b = x[mid], c = x[hi]; /* median of three as the pivot */
    const double p = a < b ? (b < c ? b : (a < c ? c : a)) : (a < c ? a : (b < c ? c : b));
    int64_t i = lo, j = hi;
    do {
      while (x[i] < p) ++i;
      while (x[j] > p) --j;
      if (i <= j) {
        const double t = x[i]; x[i] = x[j]; x[j] = t;
        ++i;
        --j;
      }
    } while (i <= j);
    /* x[lo..j] <= p <= x[i..hi], everything between j and i equals p */
    if (k <= j) hi = j;
    else if (k >= i) lo = i;
    else break;
  }
  return x[k];
}
/* (x[(n-1)/2] + x[n/2]) * 0.5 */
static double median_of(double* x, uint64_t n) {
  const double hi = select_k(x, n, n / 2);
  double lo = hi;
  if ((n & 1) == 0) { /* the largest value in front of position n/2 */
    lo = x[0];
    for (uint64_t i = 1; i < n / 2; ++i) if (x[i] > lo) lo = x[i];
  }
  return (lo + hi) * 0.5;
}

/* ---- samples: one per overlapping pair of launches --------------------------------------------------------- */
typedef struct {
  uint32_t pid, da, db, pad;
  uint64_t span;
} sample_t;

/* stable parallel LSD radix sort of samples by pid, 16 bits per pass */
static int sort_samples(sample_t** pa, uint64_t n, uint64_t max_pid) {
  sample_t* a = *pa;
  sample_t* b = (sample_t*)malloc((n ? n : 1) * sizeof(sample_t));
  if (!b) return 0;
  int nt = 1;
#ifdef _OPENMP
  nt = omp_get_max_threads();
#endif
  uint64_t* hist = (uint64_t*)malloc((size_t)nt * 65536 * 8);
  if (!hist) { free(b); return 0; }
  for (int shift = 0; shift < 32 && (max_pid >> shift); shift += 16) {
    memset(hist, 0, (size_t)nt * 65536 * 8);
#pragma omp parallel num_threads(nt)
    {
      int t = 0, team = 1; /* the team may be smaller than asked for */
#ifdef _OPENMP
      t = omp_get_thread_num();
      team = omp_get_num_threads();
#endif
      const uint64_t c0 = n / team * (uint64_t)t, c1 = t + 1 == team ? n : n / team * (uint64_t)(t + 1);
      uint64_t* h = hist + (size_t)t * 65536;
      for (uint64_t i = c0; i < c1; ++i) ++h[(a[i].pid >> shift) & 0xFFFFu];
#pragma omp barrier
#pragma omp single
      {
        uint64_t acc = 0;
        for (uint32_t d = 0; d < 65536; ++d)
          for (int u = 0; u < team; ++u) {
            const uint64_t c = hist[(size_t)u * 65536 + d];
            hist[(size_t)u * 65536 + d] = acc;
            acc += c;
          }
      }
      for (uint64_t i = c0; i < c1; ++i) b[h[(a[i].pid >> shift) & 0xFFFFu]++] = a[i];
    }
    sample_t* t2 = a; a = b; b = t2;
  }
  free(hist);
  free(b);
  *pa = a;
  return 1;
}

typedef struct {
  uint64_t n;
  uint64_t* idx;     /* record index, ordered by (start, index) */
  uint64_t* start;
  uint64_t* end;
  uint64_t* endmax;  /* running maximum of end */
} timeline;

typedef struct { uint64_t start, idx; } start_idx;
static int cmp_start_idx(const void* a, const void* b) {
  const start_idx *x = (const start_idx*)a, *y = (const start_idx*)b;
  if (x->start != y->start) return x->start < y->start ? -1 : 1;
  return x->idx < y->idx ? -1 : x->idx > y->idx;
}

/* first position with v[pos] >= x */
static uint64_t lower_bound(const uint64_t* v, uint64_t n, uint64_t x) {
  uint64_t lo = 0, hi = n;
  while (lo < hi) { const uint64_t m = lo + (hi - lo) / 2; if (v[m] < x) lo = m + 1; else hi = m; }
  return lo;
}
/* first position with v[pos] > x */
static uint64_t upper_bound(const uint64_t* v, uint64_t n, uint64_t x) {
  uint64_t lo = 0, hi = n;
  while (lo < hi) { const uint64_t m = lo + (hi - lo) / 2; if (v[m] <= x) lo = m + 1; else hi = m; }
  return lo;
}

void kso_free(kso_table* t) {
  if (!t) return;
  void* p[] = {t->key, t->name_id, t->grid, t->block, t->smem, t->tenant, t->launches, t->solo_launches, t->solo_ns,
               t->key_a, t->key_b, t->count, t->flags, t->span_sum_ns, t->sum_a, t->mean_a, t->min_a, t->max_a, t->median_a,
               t->sum_b, t->mean_b, t->min_b, t->max_b, t->median_b, t->efficiency};
  for (size_t i = 0; i < sizeof(p) / sizeof(p[0]); ++i) free(p[i]);
  memset(t, 0, sizeof(*t));
}

#define ALLOC(ptr, count, type)                                   \
  do {                                                            \
    (ptr) = (type*)malloc(((count) != 0 ? (size_t)(count) : (size_t)1) * sizeof(type)); \
    if (!(ptr)) { status = KSO_ERR_MEMORY; goto done; }           \
  } while (0)

int kso_build_pair_table(const void* records, uint64_t n, int type_mode, int threads, kso_table* out) {
  const kso_record* rec = (const kso_record*)records;
  int status = KSO_OK;
  const int timing = getenv("KSO_TIMING") != NULL;
  double t_last = now_s();
  memset(out, 0, sizeof(*out));
#ifdef _OPENMP
  if (threads > 0) omp_set_num_threads(threads);
#else
  (void)threads;
#endif
  uint64_t* keys = NULL;
  uint32_t* kid = NULL;
  uint32_t* solo_sorted = NULL;
  uint64_t* solo_off = NULL;
  sample_t* smp = NULL;
  uint64_t* row_start = NULL;
  timeline tl[256];
  memset(tl, 0, sizeof(tl));
  keyset set;
  memset(&set, 0, sizeof(set));

  /* ---- checks */
  {
    int bad = 0, toolong = 0;
#pragma omp parallel for schedule(static) reduction(| : bad, toolong)
    for (int64_t i = 0; i < (int64_t)n; ++i) {
      if (rec[i].end_ns < rec[i].start_ns) bad |= 1;
      else if (rec[i].end_ns - rec[i].start_ns >= (1ull << 31)) toolong |= 1;
    }
    if (bad) return KSO_ERR_RECORD;
    if (toolong) return KSO_ERR_DURATION;
  }

  /* ---- keys, distinct keys, dense ids = rank of the key */
  ALLOC(keys, n, uint64_t);
  ALLOC(kid, n, uint32_t);
  kso_kernel_keys(records, n, type_mode, keys);
  if (!keyset_init(&set, 1u << 18)) { status = KSO_ERR_MEMORY; goto done; }
  for (uint64_t i = 0; i < n; ++i)
    if (!keyset_add(&set, keys[i], i)) { status = KSO_ERR_KEYS; goto done; }
  const uint64_t nk = set.used;
  if (nk > 65535) { status = KSO_ERR_KEYS; goto done; }
  out->n_keys = nk;
  ALLOC(out->key, nk, uint64_t);
  {
    uint64_t j = 0;
    for (uint64_t s = 0; s <= set.mask; ++s) if (set.key[s]) out->key[j++] = set.key[s];
    qsort(out->key, nk, 8, cmp_u64);
    for (uint64_t r = 0; r < nk; ++r) set.kid[keyset_slot(&set, out->key[r])] = (uint32_t)r;
  }
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < (int64_t)n; ++i) kid[i] = set.kid[keyset_slot(&set, keys[i])];

  ALLOC(out->name_id, nk, uint32_t); ALLOC(out->grid, nk * 3, uint32_t); ALLOC(out->block, nk * 3, uint32_t);
  ALLOC(out->smem, nk, uint32_t); ALLOC(out->tenant, nk, uint32_t);
  ALLOC(out->launches, nk, uint64_t); ALLOC(out->solo_launches, nk, uint64_t); ALLOC(out->solo_ns, nk, double);
  for (uint64_t r = 0; r < nk; ++r) {
    const kso_record* f = rec + set.first[keyset_slot(&set, out->key[r])];
    out->name_id[r] = f->name_id;
    for (int d = 0; d < 3; ++d) { out->grid[3 * r + d] = type_mode ? 0 : f->grid[d]; out->block[3 * r + d] = f->block[d]; }
    out->smem[r] = type_mode ? 0 : (f->smem_word & SMEM_MASK);
    out->tenant[r] = f->smem_word >> 24;
    out->launches[r] = out->solo_launches[r] = 0;
    out->solo_ns[r] = NAN;
  }
  for (uint64_t i = 0; i < n; ++i) {
    ++out->launches[kid[i]];
    if (rec[i].smem_word & SOLO_BIT) ++out->solo_launches[kid[i]];
  }

  TICK("keys");
  /* ---- solo time per key: median of the integer durations of its solo launches */
  ALLOC(solo_off, nk + 1, uint64_t);
  {
    uint64_t acc = 0;
    for (uint64_t r = 0; r < nk; ++r) { solo_off[r] = acc; acc += out->solo_launches[r]; }
    solo_off[nk] = acc;
    ALLOC(solo_sorted, acc, uint32_t);
    uint64_t* cur = (uint64_t*)malloc((nk ? nk : 1) * 8);
    if (!cur) { status = KSO_ERR_MEMORY; goto done; }
    memcpy(cur, solo_off, nk * 8);
    for (uint64_t i = 0; i < n; ++i)
      if (rec[i].smem_word & SOLO_BIT) solo_sorted[cur[kid[i]]++] = (uint32_t)(rec[i].end_ns - rec[i].start_ns);
    free(cur);
#pragma omp parallel for schedule(dynamic, 16)
    for (int64_t r = 0; r < (int64_t)nk; ++r) {
      const uint64_t c = solo_off[r + 1] - solo_off[r];
      if (!c) continue;
      uint32_t* v = solo_sorted + solo_off[r];
      qsort(v, c, 4, cmp_u32);
      out->solo_ns[r] = ((double)v[(c - 1) / 2] + (double)v[c / 2]) * 0.5;
    }
  }

  TICK("solo");
  /* ---- per-tenant timelines of the co-run launches, ordered by start */
  {
    uint64_t cnt[256];
    memset(cnt, 0, sizeof(cnt));
    for (uint64_t i = 0; i < n; ++i) if (!(rec[i].smem_word & SOLO_BIT)) ++cnt[rec[i].smem_word >> 24];
    for (int t = 0; t < 256; ++t) {
      if (!cnt[t]) continue;
      ALLOC(tl[t].idx, cnt[t], uint64_t); ALLOC(tl[t].start, cnt[t], uint64_t);
      ALLOC(tl[t].end, cnt[t], uint64_t); ALLOC(tl[t].endmax, cnt[t], uint64_t);
    }
    for (uint64_t i = 0; i < n; ++i) {
      if (rec[i].smem_word & SOLO_BIT) continue;
      timeline* L = tl + (rec[i].smem_word >> 24);
      L->idx[L->n++] = i;
    }
#pragma omp parallel for schedule(dynamic, 1)
    for (int t = 0; t < 256; ++t) {
      timeline* L = tl + t;
      if (!L->n) continue;
      int ordered = 1;
      for (uint64_t j = 1; j < L->n && ordered; ++j) ordered = rec[L->idx[j - 1]].start_ns <= rec[L->idx[j]].start_ns;
      if (!ordered) {
        start_idx* tmp = (start_idx*)malloc(L->n * sizeof(start_idx));
        if (tmp) {
          for (uint64_t j = 0; j < L->n; ++j) { tmp[j].start = rec[L->idx[j]].start_ns; tmp[j].idx = L->idx[j]; }
          qsort(tmp, L->n, sizeof(start_idx), cmp_start_idx);
          for (uint64_t j = 0; j < L->n; ++j) L->idx[j] = tmp[j].idx;
          free(tmp);
        } else {
          L->n = ~0ull; /* reported below */
        }
      }
      if (L->n == ~0ull) continue;
      uint64_t m = 0;
      for (uint64_t j = 0; j < L->n; ++j) {
        const kso_record* r = rec + L->idx[j];
        L->start[j] = r->start_ns;
        L->end[j] = r->end_ns;
        if (r->end_ns > m) m = r->end_ns;
        L->endmax[j] = m;
      }
    }
    for (int t = 0; t < 256; ++t) if (tl[t].n == ~0ull) { tl[t].n = 0; status = KSO_ERR_MEMORY; goto done; }
  }

  TICK("timelines");
  /* ---- interval join of every two tenants: a.start < b.end and b.start < a.end; count, then emit */
  uint64_t n_pairs = 0;
  {
    /* pass 0 counts per (tenant pair, a), pass 1 writes; offsets per tenant pair come from the counts */
    for (int pass = 0; pass < 2; ++pass) {
      uint64_t base = 0;
      for (int ta = 0; ta < 256; ++ta) {
        if (!tl[ta].n) continue;
        for (int tb = ta + 1; tb < 256; ++tb) {
          if (!tl[tb].n) continue;
          const timeline *A = tl + ta, *B = tl + tb;
          uint64_t* off = (uint64_t*)malloc((A->n + 1) * 8);
          if (!off) { status = KSO_ERR_MEMORY; goto done; }
#pragma omp parallel for schedule(static)
          for (int64_t i = 0; i < (int64_t)A->n; ++i) {
            const uint64_t hi = lower_bound(B->start, B->n, A->end[i]);      /* b.start < a.end  <=> position < hi */
            const uint64_t lo = upper_bound(B->endmax, B->n, A->start[i]);   /* nothing in front of lo ends after a.start */
            uint64_t c = 0;
            for (uint64_t j = lo; j < hi; ++j) c += A->start[i] < B->end[j] && B->start[j] < A->end[i];
            off[i + 1] = c;
          }
          off[0] = 0;
          for (uint64_t i = 0; i < A->n; ++i) off[i + 1] += off[i];
          if (pass == 1) {
#pragma omp parallel for schedule(static)
            for (int64_t i = 0; i < (int64_t)A->n; ++i) {
              if (off[i + 1] == off[i]) continue;
              const uint64_t hi = lower_bound(B->start, B->n, A->end[i]);
              const uint64_t lo = upper_bound(B->endmax, B->n, A->start[i]);
              sample_t* o = smp + base + off[i];
              const uint64_t ia = A->idx[i];
              for (uint64_t j = lo; j < hi; ++j) {
                if (!(A->start[i] < B->end[j] && B->start[j] < A->end[i])) continue;
                const uint64_t ib = B->idx[j];
                o->pid = kid[ia] * (uint32_t)nk + kid[ib];
                o->da = (uint32_t)(A->end[i] - A->start[i]);
                o->db = (uint32_t)(B->end[j] - B->start[j]);
                o->pad = 0;
                o->span = (A->end[i] > B->end[j] ? A->end[i] : B->end[j]) - (A->start[i] < B->start[j] ? A->start[i] : B->start[j]);
                ++o;
              }
            }
          }
          base += off[A->n];
          free(off);
        }
      }
      if (pass == 0) {
        n_pairs = base;
        ALLOC(smp, n_pairs, sample_t);
      }
    }
  }
  out->n_pairs = n_pairs;

  TICK("join");
  /* ---- group by (key_a, key_b) */
  if (!sort_samples(&smp, n_pairs, nk * nk)) { status = KSO_ERR_MEMORY; goto done; }
  TICK("sort");
  uint64_t n_rows = 0;
  for (uint64_t i = 0; i < n_pairs; ++i) n_rows += i == 0 || smp[i].pid != smp[i - 1].pid;
  ALLOC(row_start, n_rows + 1, uint64_t);
  {
    uint64_t r = 0;
    for (uint64_t i = 0; i < n_pairs; ++i) if (i == 0 || smp[i].pid != smp[i - 1].pid) row_start[r++] = i;
    row_start[n_rows] = n_pairs;
  }
  out->n_rows = n_rows;
  ALLOC(out->key_a, n_rows, uint64_t); ALLOC(out->key_b, n_rows, uint64_t); ALLOC(out->count, n_rows, uint64_t);
  ALLOC(out->flags, n_rows, uint64_t); ALLOC(out->span_sum_ns, n_rows, uint64_t);
  ALLOC(out->sum_a, n_rows, double); ALLOC(out->mean_a, n_rows, double); ALLOC(out->min_a, n_rows, double);
  ALLOC(out->max_a, n_rows, double); ALLOC(out->median_a, n_rows, double);
  ALLOC(out->sum_b, n_rows, double); ALLOC(out->mean_b, n_rows, double); ALLOC(out->min_b, n_rows, double);
  ALLOC(out->max_b, n_rows, double); ALLOC(out->median_b, n_rows, double);
  ALLOC(out->efficiency, n_rows, double);

  TICK("rows");
  int oom = 0;
#pragma omp parallel
  {
    double* buf = NULL;
    uint64_t cap = 0;
#pragma omp for schedule(dynamic, 64)
    for (int64_t r = 0; r < (int64_t)n_rows; ++r) {
      const uint64_t s = row_start[r], c = row_start[r + 1] - s;
      const uint32_t ka = smp[s].pid / (uint32_t)nk, kb = smp[s].pid % (uint32_t)nk;
      const double sa = out->solo_ns[ka], sb = out->solo_ns[kb];
      const int va = sa > 0.0, vb = sb > 0.0; /* false for NaN: no baseline */
      out->key_a[r] = out->key[ka];
      out->key_b[r] = out->key[kb];
      out->count[r] = c;
      out->flags[r] = (uint64_t)va | ((uint64_t)vb << 1);
      if (c > cap) {
        free(buf);
        cap = c + c / 2 + 64;
        buf = (double*)malloc(cap * sizeof(double));
        if (!buf) { cap = 0; oom = 1; continue; }
      }
      uint64_t span_sum = 0;
      for (uint64_t i = 0; i < c; ++i) span_sum += smp[s + i].span;
      out->span_sum_ns[r] = span_sum;
      for (int side = 0; side < 2; ++side) {
        double *sum = side ? out->sum_b : out->sum_a, *mean = side ? out->mean_b : out->mean_a, *mn = side ? out->min_b : out->min_a;
        double *mx = side ? out->max_b : out->max_a, *med = side ? out->median_b : out->median_a;
        if (!(side ? vb : va)) { sum[r] = mean[r] = mn[r] = mx[r] = med[r] = NAN; continue; }
        const double base = side ? sb : sa;
        double acc = 0.0, lo = INFINITY, hi = -INFINITY;
        for (uint64_t i = 0; i < c; ++i) {
          const double x = (double)(side ? smp[s + i].db : smp[s + i].da) / base; /* one IEEE division per sample */
          buf[i] = x;
          acc += x;
          if (x < lo) lo = x;
          if (x > hi) hi = x;
        }
        sum[r] = acc;
        mean[r] = acc / (double)c;
        mn[r] = lo;
        mx[r] = hi;
        med[r] = median_of(buf, c);
      }
      if (va && vb) {
        for (uint64_t i = 0; i < c; ++i) buf[i] = (sa + sb) / (double)smp[s + i].span;
        out->efficiency[r] = median_of(buf, c);
      } else {
        out->efficiency[r] = NAN;
      }
    }
    free(buf);
  }
  if (oom) status = KSO_ERR_MEMORY;
  TICK("stats");

done:
  free(keys); free(kid); free(solo_sorted); free(solo_off); free(smp); free(row_start);
  for (int t = 0; t < 256; ++t) { free(tl[t].idx); free(tl[t].start); free(tl[t].end); free(tl[t].endmax); }
  keyset_free(&set);
  if (status != KSO_OK) kso_free(out);
  return status;
}
