/* ks_b200.h -- C ABI of the B200 trace -> interference-table library (libks_b200.so).
 *
 * Calling convention, copied from the reference's own ctypes exports (scheduler/agent.cpp:39,71,75,643,788,805 and
 * the binding table scheduler/sched_hooks.py:36-59): plain C scalars and pointers, no exceptions, no exit(); an
 * integer comes back, negative = error (sched_prefetch returns -1 on a null tag, agent.cpp:788-790), zero or
 * positive = rows / items produced.  The text of the last error of a handle is ks_last_error().
 *
 * Threading: one handle = one CUDA stream = not re-entrant.  A call may arrive on a thread with no current CUDA
 * context (ctypes releases the GIL and the reference guards against exactly that, agent.cpp:653-656), so every
 * entry point selects the handle's device itself.
 *
 * Memory: the caller owns inputs and outputs; the handle owns its scratch.  Unless a flag says otherwise pointers
 * are HOST pointers; KS_ON_DEVICE marks them as device pointers on the handle's device (all pointer arguments of
 * that call).  There is no CPU fallback anywhere: without a CUDA device every call fails with KS_ERR_CUDA.
 */
#ifndef KS_B200_H
#define KS_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define KS_VERSION 1

/* ---- status codes (returned negated: -KS_ERR_x) */
#define KS_OK 0
#define KS_ERR_ARG 1          /* null pointer, bad flag, size out of range */
#define KS_ERR_CUDA 2         /* a CUDA call failed; see ks_last_error */
#define KS_ERR_RECORD 3       /* a record has end_ns < start_ns or a duration >= 2^31 ns */
#define KS_ERR_NOT_ORDERED 4  /* KS_ASSUME_TIME_ORDERED was given but start_ns decreases somewhere */
#define KS_ERR_TOO_MANY_KEYS 5 /* more than 65,535 distinct kernel keys */
#define KS_ERR_TABLE_FULL 6   /* the pair dictionary is full: create the handle with a larger max_pair_rows */
#define KS_ERR_CAPACITY 7     /* an output buffer is too small */
#define KS_ERR_WAIT 8         /* a bounded device-side wait ran out (the result is not valid) */
#define KS_ERR_DUPLICATE 9    /* ks_count_batches: a start_ns occurs twice in one file (the reference asserts) */
#define KS_ERR_TOO_LARGE 10   /* more items than one call supports (2^30 per sort, 2^32 overlapping pairs) */
#define KS_ERR_COMM 11        /* NCCL is missing or one of its calls failed (ks_mg_build and its communicator) */
#define KS_ERR_REBUILD 12     /* ks_update: the resident statistics are no longer exact (or an earlier window failed): begin again, replay */

/* ---- flags */
#define KS_ON_DEVICE 1u            /* pointer arguments are device pointers */
#define KS_ASSUME_TIME_ORDERED 2u  /* records are ordered by start_ns: verified, not sorted */
#define KS_KEY_TYPE 4u             /* key = tenant + name + block (a TYPE row); default is the SHAPE key */
#define KS_TIMING 8u               /* ks_mg_build: wait for the call to finish and fill the ms_ fields of info */

/* 48-byte launch record.  Replaces one row of the agent's timing log: scheduler/agent.cpp:500-508 (TimingResult)
 * as written at :692-705, with the kernel name (kernel_key.hpp:13-55 short form) replaced by a dictionary id. */
typedef struct ks_record {
  uint32_t name_id;
  uint32_t grid[3];
  uint32_t block[3];
  uint32_t smem_word; /* bits 0..22 dynamic smem bytes, bit 23 solo run, bits 24..31 tenant */
  uint64_t start_ns;
  uint64_t end_ns;
} ks_record;

/* One row of the pair table, sorted by (key_a, key_b); side a is the lower tenant.  Carries what the daemon's
 * pair_eff.tsv row needs (scheduler/scheduler_daemon.cpp:193-202: efficiency, gangs = count) plus the slowdown
 * statistics of both sides.  A side whose key has no solo baseline has NaN statistics and its flag bit clear. */
typedef struct ks_pair_row {
  uint64_t key_a, key_b;
  uint64_t count;
  uint64_t flags; /* bit 0: side a has a baseline; bit 1: side b has one */
  double sum_a, mean_a, min_a, max_a, median_a;
  double sum_b, mean_b, min_b, max_b, median_b;
  double efficiency;    /* median over occurrences of (solo_a + solo_b) / (max(end) - min(start)) */
  uint64_t span_sum_ns; /* sum over occurrences of max(end) - min(start) */
} ks_pair_row;

/* One row of the per-key table, sorted by key: what kernel_us.tsv needs (scheduler_daemon.cpp:195, :250-264). */
typedef struct ks_key_row {
  uint64_t key;
  uint32_t name_id;
  uint32_t grid[3];
  uint32_t block[3];
  uint32_t smem;
  uint32_t tenant;
  uint32_t reserved;
  uint64_t launches;
  uint64_t solo_launches;
  double solo_ns; /* exact median duration of the solo launches; NaN if there are none */
} ks_key_row;

typedef struct ks_config {
  uint64_t max_records;   /* scratch is sized for this many records up front (it grows on demand) */
  uint64_t max_pairs;     /* ... and this many overlapping launch pairs */
  uint32_t max_pair_rows; /* limit on the rows of the pair table (KS_ERR_TOO_LARGE beyond); 0 = no limit, the arrays grow */
  uint32_t reserved;
} ks_config;

typedef struct ks_table_info {
  uint64_t n_records, n_keys, n_solo, n_pairs, n_rows;
  uint64_t max_duration_ns;
  uint64_t min_start_ns, max_start_ns;
  uint32_t was_time_ordered; /* 1 if the input needed no sort */
  uint32_t sort_passes;      /* passes of the sample sort (one launch of the pass kernel each) */
  /* device time of the stages of the last call, CUDA events on the handle's stream */
  float ms_stage_in, ms_decode, ms_order, ms_dict, ms_join, ms_sort, ms_reduce, ms_finalize, ms_total;
  float ms_sort_pass;        /* average device time of one pass of the sample sort (one launch of the pass kernel) */
} ks_table_info;

typedef struct ks_handle ks_handle;

int ks_version(void);
const char* ks_status_string(int status);

/* stream: a cudaStream_t to launch on, or NULL for a stream of the handle's own.  cfg may be NULL. */
ks_handle* ks_create(int device, void* stream, const ks_config* cfg);
void ks_destroy(ks_handle* h);
const char* ks_last_error(ks_handle* h);
/* the stream the handle launches on (for timing with events) */
void* ks_stream(ks_handle* h);
/* kernels of this library launched through the handle so far (cumulative) */
uint64_t ks_launch_count(ks_handle* h);
/* page-locked host buffers for records and tables that cross PCIe on every call */
void* ks_pinned_alloc(uint64_t bytes);
void ks_pinned_free(void* p);

/* ---- the whole path.  Stands where the reference runs its offline post-processing over the agents' logs
 * (scheduler/postprocess.py:8-41 and the absent make_pair_eff.py named at scheduler_daemon.cpp:5,193,848).
 * Returns the number of pair rows; the tables stay in the handle until the next call. info may be NULL. */
int64_t ks_build_table(ks_handle* h, const void* records, uint64_t n, uint32_t flags, ks_table_info* info);
/* The same table for a trace whose overlapping pairs do not fit one call (2^30 samples, twice in memory): decoded once,
 * joined in windows of window_records launches (0 = 2^26), the samples kept in n_parts key ranges (0 = 16, at most 16) that
 * are sorted and reduced one after the other.  No counterpart in the reference, whose script gives up on long logs by cutting
 * them to 200,000 rows (scheduler/postprocess.py:12).  records: fewer than 2^30, ordered by start_ns (KS_ERR_NOT_ORDERED
 * otherwise); flags: KS_ON_DEVICE, KS_KEY_TYPE.  info: ms_join = the windows (join + partition), ms_reduce = the key ranges. */
int64_t ks_build_table_streamed(ks_handle* h, const void* records, uint64_t n, uint32_t flags, uint64_t window_records, uint32_t n_parts,
                                ks_table_info* info);
/* Runs one sort pass in which a tile waits for a predecessor that was never started, with a wait limit of a few thousand
 * polls: the wait must run out, the kernel must end and the call must return -KS_ERR_WAIT (0 would mean the bound is gone).
 * The handle stays usable.  A check of the library's hang protection; no counterpart in the reference. */
int64_t ks_selftest_bounded_wait(ks_handle* h);
int64_t ks_copy_pair_rows(ks_handle* h, ks_pair_row* dst, uint64_t capacity_rows, uint32_t flags);
int64_t ks_copy_key_rows(ks_handle* h, ks_key_row* dst, uint64_t capacity_rows, uint32_t flags);

/* ---- stage entry points (each is what one kernel family computes; used by the parity tests) */

/* K1: 64-bit kernel key of every record.  Key composition: scheduler_daemon.cpp:196-197, :210-213 (shape
 * signature model|kernel|block|grid) and :213 / pairprof_daemon.cpp:122-123 (type: no grid). */
int64_t ks_hash_keys(ks_handle* h, const void* records, uint64_t n, uint32_t flags, uint64_t* keys_out);

/* K2: stable LSD radix sort of (key, value) pairs on key bits [begin_bit, end_bit), in place.  The grouping
 * primitive behind pandas' sort-based groupby in postprocess/profile_postprocess.py:10-25. */
int64_t ks_sort_pairs_u64(ks_handle* h, uint64_t* keys, uint64_t* vals, uint64_t n, int begin_bit, int end_bit, uint32_t flags);
int64_t ks_sort_pairs_u32(ks_handle* h, uint32_t* keys, uint32_t* vals, uint64_t n, int begin_bit, int end_bit, uint32_t flags);

/* The same sort for callers that must not allocate device memory (no counterpart in the reference: its post-processing
 * is host-side pandas).  Meant for code living inside another program's memory budget -- a plugin of a serving process
 * whose caching allocator owns the device, a watchdog thread that may not wait on the allocator's lock.  keys and vals
 * are DEVICE pointers on the current device (vals may be NULL), sorted in place on `stream`; no handle is needed.
 * All scratch is a fixed device array inside the library (8,667,648 bytes per GPU, held until the process exits), so:
 *   - at most KS_NOALLOC_MAX_ITEMS items; more is refused with -KS_ERR_TOO_LARGE;
 *   - the call never calls cudaMalloc / cudaFree or anything that allocates;
 *   - every call on a device shares that array: two calls whose GPU work overlaps (different streams or threads) race;
 *   - the first call on a device looks up the array's device address and sets kernel attributes; make that first call
 *     before any stream capture starts.
 * Returns n, or a negative status (text in ks_last_error(NULL)).  The call synchronises `stream` before returning. */
#define KS_NOALLOC_MAX_ITEMS (1u << 20)
int64_t ks_sort_pairs_u32_noalloc(void* stream, uint32_t* keys, uint32_t* vals, uint64_t n, int begin_bit, int end_bit);

/* K1+K2: the launches grouped by key: (key, start_ns) of every record in (key, start_ns) order. */
int64_t ks_sort_launches(ks_handle* h, const void* records, uint64_t n, uint32_t flags, uint64_t* keys_out, uint64_t* start_out);

/* K3: the interval join.  Writes the overlapping launch pairs as positions in the start_ns-ordered trace
 * (idx_a: the launch of the lower tenant).  Replaces the quadratic scans of postprocess.py:19-39 with the interval
 * rule a.start < b.end && b.start < a.end.  The order of the pairs is unspecified.  Returns the pair count; if it
 * exceeds capacity only the count is valid (-KS_ERR_CAPACITY is NOT returned, so a first call with capacity 0
 * sizes the buffers). */
int64_t ks_join_overlaps(ks_handle* h, const void* records, uint64_t n, uint32_t flags, uint32_t* idx_a, uint32_t* idx_b, uint64_t capacity);

/* K4: per segment of `values` (segment s = [offsets[s], offsets[s+1])): sum, min, max and the two middle order
 * statistics x[(n-1)/2], x[n/2] -- exact, by selection.  out: 6 uint64 per segment {count, sum, min, max, lo, hi}. */
int64_t ks_segment_stats(ks_handle* h, const uint32_t* values, const uint64_t* offsets, uint64_t n_segments, uint32_t flags, uint64_t* out);

/* The reference's batch counter verbatim: scheduler/postprocess.py:17-41 prints [n_alone, n_pairs] where a pair is
 * two launches, one per file, with the same start_ns.  The caller applies the [-200000:] slice of :12. */
int64_t ks_count_batches(ks_handle* h, const uint64_t* start1, uint64_t n1, const uint64_t* start2, uint64_t n2, uint32_t flags, uint64_t out[2]);

/* postprocess/profile_postprocess.py:5-27 combine_duplicates: launches-weighted mean per group, NaN cells skipped
 * in numerator and weight (min_count=1 semantics, :14,:21), plus the group's total launches (:25).
 * group: dense group id per row (the host maps (Kernel, Block) to ids); values: rows x cols, row major. */
int64_t ks_combine_duplicates(ks_handle* h, const uint32_t* group, const double* launches, const double* values, uint64_t rows, uint32_t cols,
                              uint32_t n_groups, uint32_t flags, double* out_total, double* out_means);

/* profiling/ncu-bench/ncu_summary.py:185-245, the pooling of per-launch profiler metrics: per group (the host maps
 * (kernel name, block) to dense ids) the number of launches, and per column the mean and the SAMPLE standard deviation
 * (:239-240: statistics.mean, statistics.stdev, 0 for a single value) over the launches that have the metric (NaN =
 * absent; a column no launch of the group has gives NaN, the script's None).  values: rows x cols, row major. */
int64_t ks_pool_launches(ks_handle* h, const uint32_t* group, const double* values, uint64_t rows, uint32_t cols, uint32_t n_groups, uint32_t flags,
                         uint64_t* out_launches, double* out_mean, double* out_std);

/* ---- multi-GPU session: one process and one handle per GPU, each owning one window of the start-ordered trace.
 * The reference has no multi-GPU path; these phases are what kernel_scheduling_b200/parallel.py runs between its
 * collectives (all-gather of keys, sum of counts, all-to-all of samples, all-gather of solo times and table shards).
 * All pointers are DEVICE pointers.  A pair of overlapping launches is reduced by the rank whose key range holds its
 * (key_a, key_b); it is produced by the rank that owns its LATER launch. */
#define KS_MG_HALO_MAX 4096    /* launches of the previous window that may still run when this one begins */
#define KS_MG_HIST_BINS 4096   /* bins of the sample-key histogram the splitters are chosen from */
int64_t ks_mg_begin(ks_handle* h, const void* records, uint64_t n_owned, uint32_t flags);      /* K1 over the window */
int64_t ks_mg_tail(ks_handle* h, void* out_records, uint64_t capacity);                         /* launches reaching into the next window, start order */
int64_t ks_mg_halo(ks_handle* h, const void* halo_records, uint64_t n_halo);                    /* the previous rank's tail */
int64_t ks_mg_local_keys(ks_handle* h, uint64_t* keys_out, void* words_out, uint64_t capacity); /* distinct keys + 32 bytes of launch fields each */
int64_t ks_mg_global_keys(ks_handle* h, const uint64_t* keys, const void* words, uint64_t n);   /* every rank's keys -> same dense ids everywhere; returns K */
int64_t ks_mg_counts(ks_handle* h, uint64_t* launches, uint64_t* solo, int import);             /* per-key launch counts by dense id, out (0) or in (1) */
int64_t ks_mg_samples(ks_handle* h);                                                            /* solo samples + K3; returns the local sample count */
int64_t ks_mg_key_histogram(ks_handle* h, uint64_t* hist, uint32_t* shift_out);                 /* hist[KS_MG_HIST_BINS] of sort key >> shift */
int64_t ks_mg_partition(ks_handle* h, const uint32_t* splitters, uint32_t shift, uint32_t n_ranks, void* send, uint64_t capacity, uint64_t* counts);
int64_t ks_mg_reduce(ks_handle* h, const void* samples, uint64_t n);                            /* K2 + K4 over the received samples */
int64_t ks_mg_row_count(ks_handle* h);                                                          /* pair rows of this rank's range (after ks_mg_reduce) */
int64_t ks_mg_solo(ks_handle* h, double* solo, int import);                                     /* solo times by dense id, out (0) or in (1) */
int64_t ks_mg_finalize(ks_handle* h);                                                           /* tables of this rank's key range; then ks_copy_*_rows */

/* The same build as ONE call per rank: the phases above with the five exchanges issued by the library itself through NCCL
 * on the handle's stream (NCCL is bound at run time: libnccl.so.2, or the file named by the environment variable
 * KS_NCCL_LIBRARY).  No counterpart in the reference.
 *   ks_mg_unique_id     rank 0 makes the 128-byte NCCL id; the caller hands it to every rank (any transport)
 *   ks_mg_comm_init     collective over the ranks: the handle's communicator (world <= 16)
 *   ks_mg_build         collective: records = this rank's window (DEVICE pointer, start order, 16-byte aligned).  Returns
 *                       the rows of the WHOLE table, which every rank then holds (ks_copy_pair_rows / ks_copy_key_rows);
 *                       queued on the handle's stream, the copies are ordered behind it.  flags: KS_KEY_TYPE, KS_TIMING.
 *                       info (optional): this rank's counts; with KS_TIMING (one more host wait) also the device time
 *                       of the five phases, each with its exchange: ms_decode, ms_join, ms_order (partition + sample
 *                       exchange), ms_reduce (K2 + K4), ms_finalize.
 *                       Errors found on the device (bad record, order, capacity) are returned by ALL ranks alike; an
 *                       argument, CUDA or NCCL failure is local to its rank and fatal for the job.
 *   ks_mg_comm_destroy  releases the communicator and the exchange buffers (ks_destroy does it too) */
int ks_mg_unique_id(void* id128);
int ks_mg_comm_init(ks_handle* h, const void* id128, int rank, int world);
int64_t ks_mg_build(ks_handle* h, const void* records, uint64_t n_owned, uint32_t flags, ks_table_info* info);
int ks_mg_comm_destroy(ks_handle* h);
/* The two bulk exchanges of ks_mg_build (samples to their key range's owner; table shards to everyone) go through PEER
 * MEMORY when every rank can map every other rank's buffers (CUDA IPC, decided once in ks_mg_comm_init; KS_MG_NO_P2P in
 * the environment of any rank turns it off): the partition kernel and the finalize kernel store straight into the other
 * GPUs' buffers over NVLink, and a 16-byte all-gather orders the stores before the readers.  Otherwise they are NCCL
 * send/recv pairs.  Returns 1 for peer memory, 0 for NCCL.  ks_mg_comm_destroy is collective in peer-memory mode (every
 * rank unmaps before any rank frees).
 * In peer-memory mode a large table (its size is known from the session's previous build) is built in two or four
 * STAGES: every rank owns several key ranges, and while one range is sorted and reduced the copy engines carry the rows
 * of the range before it into the other GPUs' tables.  Environment (the same on every rank): KS_MG_STAGES=1|2|4 forces the
 * stage count (with one rank: the staged build on the rank's own buffers), KS_MG_REFINE=1 places the cuts between key
 * ranges inside histogram bins so that the ranges hold equal sample counts, KS_MG_TRACE=1|2 prints the device time
 * between the driver's steps (rank 0 | every rank). */
int ks_mg_peer_memory(ks_handle* h);

/* ---- the agent's timing log (text) -> launch records, on the device.  Replaces the pandas read of the 17-column TSV the
 * agent writes (scheduler/agent.cpp:692-705; read at scheduler/postprocess.py:12-13).  Rows without end_ns (no completion
 * callback, agent.cpp:702) are dropped.  Three steps because names are canonicalised on the host (ks_function_base), once
 * per DISTINCT symbol:
 *   ks_tsv_parse       text in; returns the number of valid launch rows
 *   ks_tsv_dictionary  the distinct kernel symbols (which = 0) or models (1): hashes[slot] != 0 marks a used slot,
 *                      where[slot] = offset << 20 | length of the string's first occurrence in the text (HOST arrays)
 *   ks_tsv_finish      name id and tenant per dictionary slot in (HOST arrays over all slots), records out, file order */
#define KS_TSV_NAME_SLOTS 65536
#define KS_TSV_MODEL_SLOTS 256
int64_t ks_tsv_parse(ks_handle* h, const char* text, uint64_t n_bytes, uint32_t flags);
int64_t ks_tsv_dictionary(ks_handle* h, int which, uint64_t* hashes, uint64_t* where);
/* Optional, between ks_tsv_parse and ks_tsv_finish: the profiling daemon's log of the same run (one row per released
 * kernel: batch_id, kind, pid, kernel_id, ...; profiling/pairprof_daemon.cpp:266, :317-318), parsed on the device.  The
 * rows of process `pid` label the parsed launches by kernel_id (column 0 of the agent log): kind alone* -> a solo sample,
 * gang* -> a co-run launch; launches the log does not mention (warm-up) are dropped.  ks_tsv_finish then ignores its
 * `solo` argument.  Returns the rows that remain. */
int64_t ks_tsv_label(ks_handle* h, const char* log_text, uint64_t n_bytes, uint64_t pid, uint32_t flags);
int64_t ks_tsv_finish(ks_handle* h, const uint32_t* name_ids, const uint32_t* tenants, uint32_t solo, ks_record* out, uint64_t capacity, uint32_t flags);

/* Column extraction from any tab-separated log with a header line, on the device: the daemon's decision log
 * (scheduler/scheduler_daemon.cpp:674-676, one row per finished kernel; fields :585-605) and the agent's timing log
 * (scheduler/agent.cpp:692-705).  Per data line and requested column (at most 16) one 64-bit word, out[c * capacity + row]:
 *   KS_COL_U64    decimal integer; blank or malformed = UINT64_MAX
 *   KS_COL_MILLI  decimal with up to three fraction digits (printf "%.3f") -> value x 1000; blank = UINT64_MAX
 *   KS_COL_DIMS   "(x, y, z)" or "x,y,z" -> x | y << 21 | z << 42 (each below 2^21); malformed = UINT64_MAX
 *   KS_COL_HASH   64-bit FNV-1a of the field
 *   KS_COL_SPAN   offset of the field in the text << 20 | its length
 * Returns the number of data lines (only the first `capacity` are written).  KS_ON_DEVICE: text and out are device pointers. */
#define KS_COL_U64 0u
#define KS_COL_MILLI 1u
#define KS_COL_DIMS 2u
#define KS_COL_HASH 3u
#define KS_COL_SPAN 4u
int64_t ks_tsv_extract(ks_handle* h, const char* text, uint64_t n_bytes, uint32_t n_cols, const uint32_t* cols, const uint32_t* kinds, uint64_t* out,
                       uint64_t capacity, uint32_t flags);
/* Per segment of `values` (segment s = [offsets[s], offsets[s+1])) a histogram of n_bins counters: bin = the value itself
 * (log2_bins = 0) or its bit length, 0 for 0 (log2_bins = 1), clamped to the last bin.  out: n_segments x n_bins uint32.
 * The queue-wait and batch-size histograms per kernel of the decision-log analytics. */
int64_t ks_segment_hist(ks_handle* h, const uint32_t* values, const uint64_t* offsets, uint64_t n_segments, uint32_t n_bins, uint32_t log2_bins,
                        uint32_t flags, uint32_t* out);

/* ---- the resident table: windows of new launches merged into statistics that stay in HBM (benchmark configuration 5: "online
 * incremental mode"; the reference has no such path, its tables are rebuilt offline).  At any time the table read out is
 * exactly the one ks_build_table gives for all launches so far: counts, sums, minima and maxima are accumulators, and
 * for the medians every row keeps the 64 values around its median in sorted order plus how many lie below (ks_update.cuh).
 *   ks_update_begin  an empty table (flags: KS_KEY_TYPE or 0).  At most 2,048 distinct keys; 3.5 GB of HBM for the rows.
 *                    The handle belongs to the session until ks_update_end (other calls on it clear the dictionary).
 *   ks_update        one window of launches in start order, not earlier than the previous window (HOST records, or DEVICE
 *                    with KS_ON_DEVICE).  Launches still running when a window ends are carried into the next (at most
 *                    4,096).  Returns the samples merged.  If the distribution of a row jumps so far in one window that
 *                    its median leaves the kept values: -KS_ERR_REBUILD (never a wrong table); after any error the
 *                    session is over.  info: counts of this window, ms_total = device time of the update.
 *   ks_update_table  reads the table out (key rows by key, pair rows by (key_a, key_b)); then ks_copy_*_rows.
 *   ks_update_end    frees the resident rows. */
int64_t ks_update_begin(ks_handle* h, uint32_t flags);
int64_t ks_update(ks_handle* h, const void* records, uint64_t n, uint32_t flags, ks_table_info* info);
int64_t ks_update_table(ks_handle* h);
int64_t ks_update_end(ks_handle* h);

/* The kernel key of one launch shape, on the host: bit for bit what the device computes for a record with these fields
 * (flags: KS_KEY_TYPE or 0).  For programs that look keys up in a finished table (include/ks_pairtab_shm.h). */
uint64_t ks_kernel_key(uint32_t name_id, const uint32_t grid[3], const uint32_t block[3], uint32_t smem, uint32_t tenant, uint32_t flags);

/* The pair table in a POSIX shared-memory segment (layout and reader: include/ks_pairtab_shm.h; the reference keeps its
 * table in a string-keyed map filled from pair_eff.tsv, scheduler_daemon.cpp:230-274).  Host code, HOST arrays: the key
 * rows and pair rows of a SHAPE table and of a TYPE table as ks_copy_key_rows / ks_copy_pair_rows return them, and the
 * strings behind name ids and tenants.  Written to "<name>.tmp", then renamed over "<name>".  Returns the bytes of the
 * image, or -KS_ERR_ARG (ks_pairtab_last_error says why). */
int64_t ks_pairtab_publish(const char* shm_name, const ks_key_row* shape_keys, uint64_t n_shape_keys, const ks_pair_row* shape_pairs, uint64_t n_shape_rows,
                           const ks_key_row* type_keys, uint64_t n_type_keys, const ks_pair_row* type_pairs, uint64_t n_type_rows, const char* const* names,
                           uint64_t n_names, const char* const* models, uint64_t n_models, uint64_t generation);
int ks_pairtab_unlink(const char* shm_name);
const char* ks_pairtab_last_error(void);

/* Seeded synthetic launch traces with the shapes of the benchmark configurations, generated on the host's cores (no
 * counterpart in the reference: its traces come from live model servers, scheduler/agent.cpp:643-709).  A tenant is one
 * process with at most one launch in flight: per launch a key drawn from the Zipf table `cdf`, a duration = the key's
 * typical duration x lognormal jitter (x 1 + |N(0, corun_slowdown)| when co-running), an exponential idle gap in front.
 * Solo launches (probability solo_fraction) run one at a time in a phase of their own before the co-run phase.  Writes
 * sum(n_launches) records ordered by start_ns into `out` (HOST memory) and returns their number.  The trace is a pure
 * function of the arguments: it does not depend on `threads` (0 = every core). */
typedef struct ks_synth_tenant {
  uint32_t n_keys;
  uint32_t tenant;         /* tenant id written into the records (0..255) */
  const uint32_t* name_id; /* [n_keys] */
  const uint32_t* grid;    /* [n_keys][3] */
  const uint32_t* block;   /* [n_keys][3] */
  const uint32_t* smem;    /* [n_keys] dynamic shared memory in bytes */
  const double* dur_ns;    /* [n_keys] typical duration of the key */
  const double* cdf;       /* [n_keys] cumulative launch probability of the keys, cdf[n_keys-1] = 1 */
  uint64_t n_launches;
  double gap_mean_ns;      /* mean idle gap in front of a co-run launch */
} ks_synth_tenant;
#define KS_SYNTH_INTERLEAVE_SOLO 1u /* solo launches take their turn on their tenant's timeline instead of a phase of their own */
int64_t ks_synth_trace(const ks_synth_tenant* tenants, uint32_t n_tenants, double solo_fraction, double jitter_sigma, double corun_slowdown,
                       uint64_t seed, uint64_t t0_ns, ks_record* out, uint64_t capacity, uint32_t threads, uint32_t flags);

/* scheduler/kernel_key.hpp:13-55 ncu_function_base: symbol -> short kernel name.  Host-side (strings).
 * Writes a NUL-terminated string; returns its length, or -KS_ERR_CAPACITY. */
int64_t ks_function_base(const char* symbol, char* out, uint64_t capacity);

#ifdef __cplusplus
}
#endif
#endif
