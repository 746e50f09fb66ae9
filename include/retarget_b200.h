/*
 * retarget_b200 -- C ABI of the B200-native KV-cache placement planner.
 *
 * Plain C, no CUDA or framework types in any signature: device pointers are
 * `const void *` / typed pointers to device memory, streams are passed as
 * `void *` (a cudaStream_t / CUstream).  NULL selects the plan's own
 * non-blocking stream, NOT the legacy default stream; pass cudaStreamLegacy or
 * cudaStreamPerThread to name those.
 *
 * Every function returns an `int` status: 0 (RT_OK) on success, a negative
 * `rt_status` otherwise; `rt_strerror()` turns it into text.  Where the
 * reference reports a specific message or socket error string the same text is
 * returned.  Nothing throws, nothing calls back, the caller owns every buffer
 * it passes in.  A plan handle may be used from one thread at a time.
 *
 * Each entry point names the reference code it stands in for (paths relative
 * to the reference project root).
 */
#ifndef RETARGET_B200_H
#define RETARGET_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define RT_ABI_VERSION 1
#define RT_MAX_GROUPS 128u      /* bitmaps per plan (one per layer at most)          */
#define RT_MAX_BLOCKS 1024u     /* bits per bitmap: the 256-hex-digit mask limit,    */
                                /* select.cpp:24155                                  */
#define RT_MAX_BUFFERS 1024u    /* cache allocations per plan                        */
#define RT_BITMAP_WORDS 32u     /* RT_MAX_BLOCKS / 32                                */
#define RT_DST_CPU (-1)         /* CU_DEVICE_CPU                                     */
#define RT_INITIAL UINT64_MAX   /* "no previous window", experiments/cache_window.py:16 */

typedef enum rt_status {
    RT_OK = 0,
    RT_ERR_INVALID_ARGUMENT = -1,
    RT_ERR_NO_DEVICE = -2,          /* CUDA runtime/driver unusable: there is no CPU fallback */
    RT_ERR_CUDA = -3,               /* a CUDA call failed; rt_last_cuda_error() has the code  */
    RT_ERR_OUT_OF_MEMORY = -4,
    RT_ERR_CAPACITY = -5,           /* more indices / ranges than the plan was created for    */
    RT_ERR_ALIGNMENT = -6,          /* slot array not 16-byte aligned                         */
    RT_ERR_SLOT_RANGE = -7,         /* a slot id above capacity (the reference asserts)       */
    RT_ERR_BUSY = -8,
    RT_ERR_NOT_RUNNING = -9,
    RT_ERR_IO = -10,
    RT_ERR_PLAN = -11,              /* plan command rejected; text from rt_uvm_command reply  */
    RT_ERR_TIMEOUT = -12,           /* a bounded device-side wait gave up; nothing was planned */
    /* experiments/cache_window.py:31-50, one code per message, in check order */
    RT_ERR_SPEC_POSITIVE = -20,
    RT_ERR_SPEC_TRAILING = -21,
    RT_ERR_SPEC_PAGE = -22,
    RT_ERR_SPEC_MULTIPLE = -23,
    RT_ERR_SPEC_EXCEEDS = -24,
    RT_ERR_SPEC_INTERVAL = -25,
    RT_ERR_SPEC_MODE = -26,
    RT_ERR_COMPLETED_COUNT = -27,   /* experiments/cache_window.py:53-54 */
    /* experiments/slot_placement.py:60-64 */
    RT_ERR_BUDGET_DIVISIBLE = -28,
    RT_ERR_BLOCK_PAGE = -29,
    /* controllers: experiments/cache_window.py:79-87,105-107 and slot_placement.py:28-34,74-75 */
    RT_ERR_METRICS_MISSING = -30,      /* a completed-token counter is not in the scrape          */
    RT_ERR_METRICS_INVALID = -31,      /* a completed-token counter is negative or not finite     */
    RT_ERR_METRICS_KEY_RUNNING = -32,  /* sglang:num_running_reqs was needed and is not there     */
    RT_ERR_METRICS_KEY_QUEUE = -33,    /* sglang:num_queue_reqs was needed and is not there       */
    RT_ERR_LAYOUT_MISMATCH = -34,      /* not allocation_count allocations of allocation_bytes    */
    RT_ERR_SLOT_SPEC = -35,            /* a SlotPlacementSpec field is out of range               */
    RT_ERR_FEEDBACK_IDENTITY = -36     /* snapshot of another process or another block size       */
} rt_status;

const char *rt_strerror(int status);
int rt_abi_version(void);
/* Last cudaError_t / CUresult seen by the calling thread (0 if none). */
int rt_last_cuda_error(void);

/* ------------------------------------------------------------------ */
/* Window policy: host arithmetic                                      */
/* ------------------------------------------------------------------ */

/* experiments/cache_window.py:19-29 (CacheWindowSpec fields) */
typedef struct rt_window_spec {
    uint64_t allocation_bytes;
    uint64_t allocation_count;
    uint64_t bytes_per_token;
    uint64_t width_tokens;
    uint64_t lookahead_tokens;
    uint64_t quantum_tokens;
    double min_update_seconds;
    int32_t idle_only;       /* 0 / 1 */
    int32_t update_mode;     /* 0 incremental, 1 initial_only, 2 full_cache */
} rt_window_spec;

/* CacheWindowSpec.__post_init__, experiments/cache_window.py:31-50.
 * On RT_ERR_SPEC_POSITIVE *bad_field (optional) gets the index of the
 * offending field in declaration order. */
int rt_window_spec_check(const rt_window_spec *spec, int *bad_field);

/* CacheWindowSpec.window, experiments/cache_window.py:52-63. */
int rt_window(const rt_window_spec *spec, double completed_tokens, uint64_t out[2]);

/* interval_difference, experiments/cache_window.py:66-68.
 * Writes up to two (lo, hi) pairs to out[4]; returns the pair count. */
int rt_interval_difference(const uint64_t a[2], const uint64_t b[2], uint64_t out[4]);

/* requested_gpu_bytes / requested_cpu_bytes of a window plan,
 * experiments/cache_window.py:122-131.  `other_bytes` is the total size of the
 * non-cache allocations (only counted for a full plan). */
int rt_window_accounting(const rt_window_spec *spec, uint64_t n_cache, uint64_t other_bytes,
                         const uint64_t old_window[2], const uint64_t new_window[2],
                         int full, int refresh, uint64_t *gpu_bytes, uint64_t *cpu_bytes);

/* aligned_uvm_target, experiments/control.py:379-400: a global residency target
 * of `desired` bytes over the allocations in registry order, rounded down so
 * that the one partly resident allocation is cut at a page boundary (the
 * prefix walk of target/targetv/retarget, select.cpp:24257-24263, rejects
 * anything else as unaligned_target).  A target beyond the total is the total. */
int rt_aligned_target(const uint64_t *allocation_bytes, size_t n, uint64_t desired, uint64_t page,
                      uint64_t *target);

/* SlotPlacementController.__init__ budget rule, experiments/slot_placement.py:60-64. */
int rt_slot_budget(const rt_window_spec *spec, uint64_t block_tokens, uint64_t *budget_blocks);

/* encode_mask, experiments/slot_placement.py:47-51: lower-case hex of the OR of
 * (1 << block), no leading zeros, "0" when empty.  Returns the string length. */
int rt_encode_mask(const uint32_t *blocks, size_t n, char *out, size_t cap);

/* encode_runs, experiments/kv_audit/kv_audit_probe.py:23-32: half-open runs of
 * consecutive values, order and repeats preserved.  runs_out holds
 * (begin, end) pairs; *n_runs gets the count even when cap_runs is too small
 * (then RT_ERR_CAPACITY is returned). */
int rt_encode_runs(const int64_t *values, size_t n, int64_t *runs_out, size_t cap_runs,
                   size_t *n_runs);

/* ------------------------------------------------------------------ */
/* The two scheduler-facing controllers: host state machines            */
/* ------------------------------------------------------------------ */

/* One registry entry, select.cpp:23770-23778 (ctx and pointer omitted). */
typedef struct rt_alloc_info {
    uint64_t id;
    uint64_t bytes;
    int32_t device;
    int32_t concurrent;
} rt_alloc_info;

/* The serving engine's counters and gauges the window policy reads
 * (experiments/cache_window.py:80,98-99).  Bit k of `present` says that field k
 * (in declaration order) was in the scrape: the reference fails differently on
 * a missing name than on a bad value. */
typedef struct rt_metrics {
    double prompt_tokens_total;        /* sglang:prompt_tokens_total      */
    double generation_tokens_total;    /* sglang:generation_tokens_total  */
    double num_running_reqs;           /* sglang:num_running_reqs         */
    double num_queue_reqs;             /* sglang:num_queue_reqs           */
    uint32_t present;
    uint32_t reserved;
} rt_metrics;

/* What one window update decided; the fields of the result dictionary of
 * CacheWindowController.update, experiments/cache_window.py:133-140. */
typedef struct rt_window_update {
    int32_t full;                      /* "initial"                                   */
    int32_t refresh;                   /* "full_cache_refresh"                        */
    uint64_t old_window[2];            /* RT_INITIAL twice when full                  */
    uint64_t new_window[2];
    uint64_t generation;
    uint64_t cache_count;              /* also set when RT_ERR_LAYOUT_MISMATCH        */
    uint64_t gpu_bytes;                /* requested_gpu_bytes                         */
    uint64_t cpu_bytes;                /* requested_cpu_bytes                         */
    double completed_highwater;
} rt_window_update;

typedef struct rt_window_state {
    int32_t has_current;
    int32_t has_signature;
    uint64_t current[2];
    double last_update;
    double completed_highwater;
    uint64_t signature_count;
} rt_window_state;

/* CacheWindowController, experiments/cache_window.py:71-148, as a state machine.
 * An update is cut where the reference talks to the control socket:
 *
 *   rt_window_controller_begin   counters, window, gates (:90-100); 1 = go on
 *   (caller: wait_idle, list)
 *   rt_window_controller_plan    cache filter, signature, full / incremental /
 *                                refresh, the command line, byte accounting
 *                                (:102-113,122-131)
 *   (caller: send the command, wait for the job)
 *   rt_window_controller_commit  (:132)   or   rt_window_controller_fail (:115-118)
 *
 * rt_window_controller_due is `due` (:142-148): 1, 0 or a negative status. */
typedef struct rt_window_controller rt_window_controller;
int rt_window_controller_create(const rt_window_spec *spec, rt_window_controller **out);
int rt_window_controller_destroy(rt_window_controller *c);
int rt_window_controller_due(rt_window_controller *c, const rt_metrics *metrics, double now);
int rt_window_controller_begin(rt_window_controller *c, const rt_metrics *metrics, double now, int initial);
int rt_window_controller_plan(rt_window_controller *c, const rt_alloc_info *allocations, size_t n,
                              uint64_t generation, char *command, size_t cap, rt_window_update *out);
int rt_window_controller_commit(rt_window_controller *c, double now);
int rt_window_controller_fail(rt_window_controller *c);
/* State access for bindings that expose `current`, `signature`, `last_update`
 * and `completed_highwater` like the reference's attributes.
 * rt_window_controller_get_signature returns 1 when no signature is on record. */
int rt_window_controller_get(const rt_window_controller *c, rt_window_state *out);
int rt_window_controller_set(rt_window_controller *c, const rt_window_state *in);
int rt_window_controller_get_signature(const rt_window_controller *c, rt_alloc_info *out, size_t cap, size_t *n);
int rt_window_controller_set_signature(rt_window_controller *c, const rt_alloc_info *sig, size_t n, int known);

/* SlotPlacementSpec, experiments/slot_placement.py:18-26. */
typedef struct rt_slot_spec {
    uint64_t block_tokens;
    uint64_t lookahead_tokens;
    double min_update_seconds;
    uint64_t max_blocks_per_update;
    double active_seconds;
    double refresh_seconds;
    double max_feedback_lag_seconds;
} rt_slot_spec;

/* SlotPlacementSpec.__post_init__, experiments/slot_placement.py:28-34; on
 * RT_ERR_SLOT_SPEC *bad_field gets the field's index in declaration order. */
int rt_slot_spec_check(const rt_slot_spec *spec, int *bad_field);

typedef struct rt_block_stamp {
    uint32_t block;
    uint32_t reserved;
    double t;
} rt_block_stamp;

/* The fields of a feedback snapshot document (experiments/slot_feedback.py:86-91)
 * that the controller reads.  Lists keep the document's order. */
typedef struct rt_snapshot_doc {
    uint64_t pid;
    uint64_t epoch;
    uint64_t block_tokens;
    int64_t sequence;
    double observed_monotonic_s;
    double published_monotonic_s;
    const int32_t *block_versions;
    size_t n_versions;
    const rt_block_stamp *recent_reads;
    size_t n_reads;
    const rt_block_stamp *recent_writes;
    size_t n_writes;
    const uint32_t *free_head_blocks;
    size_t n_free;
} rt_snapshot_doc;

/* target_blocks, experiments/slot_placement.py:37-44. */
int rt_target_blocks(const rt_snapshot_doc *snapshot, const rt_slot_spec *spec, uint64_t budget,
                     double now, uint32_t *out, size_t cap, size_t *n);

typedef struct rt_slot_update {
    uint64_t generation;
    uint64_t epoch;                    /* feedback_epoch                 */
    int64_t sequence;                  /* feedback_sequence              */
    double observed_monotonic_s;       /* feedback_observed_monotonic_s  */
    uint64_t cache_count;              /* also set when RT_ERR_LAYOUT_MISMATCH */
    uint64_t gpu_bytes;                /* requested_gpu_bytes            */
    uint64_t n_desired;
    uint64_t n_selected;
} rt_slot_update;

typedef struct rt_slot_state {
    int32_t has_epoch;
    int32_t reserved;
    uint64_t epoch;
    double last_attempt;
    uint64_t committed_count;
} rt_slot_state;

typedef struct rt_block_commit {
    uint32_t block;
    int32_t version;
    double at;
} rt_block_commit;

/* SlotPlacementController, experiments/slot_placement.py:55-162.  It extends the
 * window controller: rt_slot_controller_window() is the window controller
 * inside it (borrowed; it shares the cache signature).
 *
 *   rt_slot_controller_accept   the checks of snapshot() (:74-78): 1 usable,
 *                               0 too old, RT_ERR_FEEDBACK_IDENTITY
 *   rt_slot_controller_choose   choose (:83-94)
 *   rt_slot_controller_due      due (:96-104); snapshot NULL = none to act on
 *   rt_slot_controller_begin    update (:119-132): stamps the attempt, a new
 *                               epoch empties the record, chooses; 1 = send
 *   rt_slot_controller_plan     (:133-139,154): cache filter, a new signature
 *                               empties the record and chooses again, command
 *   rt_slot_controller_pending  desired / selected of the update in progress
 *   rt_slot_controller_commit   (:148-153)   or   rt_slot_controller_fail (:140-147)
 *   rt_slot_controller_seed     after the initial window plan (:107-118) */
typedef struct rt_slot_controller rt_slot_controller;
int rt_slot_controller_create(const rt_window_spec *cache_spec, const rt_slot_spec *slot_spec, uint64_t pid,
                              rt_slot_controller **out);
int rt_slot_controller_destroy(rt_slot_controller *c);
rt_window_controller *rt_slot_controller_window(rt_slot_controller *c);
uint64_t rt_slot_controller_budget(const rt_slot_controller *c);
int rt_slot_controller_accept(const rt_slot_controller *c, const rt_snapshot_doc *snapshot);
int rt_slot_controller_choose(const rt_slot_controller *c, const rt_snapshot_doc *snapshot, double now,
                              uint32_t *desired, size_t cap_desired, size_t *n_desired, uint32_t *selected,
                              size_t cap_selected, size_t *n_selected);
int rt_slot_controller_due(const rt_slot_controller *c, const rt_snapshot_doc *snapshot, double now);
int rt_slot_controller_attempt_allowed(const rt_slot_controller *c, double now);
int rt_slot_controller_begin(rt_slot_controller *c, const rt_snapshot_doc *snapshot, double now);
int rt_slot_controller_plan(rt_slot_controller *c, const rt_alloc_info *allocations, size_t n,
                            uint64_t generation, char *command, size_t cap, rt_slot_update *out);
int rt_slot_controller_pending(const rt_slot_controller *c, uint32_t *desired, size_t cap_desired,
                               uint32_t *selected, size_t cap_selected);
int rt_slot_controller_commit(rt_slot_controller *c, double commit_time);
int rt_slot_controller_fail(rt_slot_controller *c);
int rt_slot_controller_seed(rt_slot_controller *c, const rt_snapshot_doc *snapshot, double commit_time);
int rt_slot_controller_get(const rt_slot_controller *c, rt_slot_state *out);
int rt_slot_controller_set(rt_slot_controller *c, const rt_slot_state *in);
int rt_slot_controller_get_committed(const rt_slot_controller *c, rt_block_commit *out, size_t cap, size_t *n);
int rt_slot_controller_set_committed(rt_slot_controller *c, const rt_block_commit *in, size_t n);

/* ------------------------------------------------------------------ */
/* Plan-command expansion: host, no GPU                                 */
/* ------------------------------------------------------------------ */

/* One migration request, select.cpp:23779-23784. */
typedef struct rt_id_range {
    uint64_t id;
    uint64_t offset;
    uint64_t bytes;
    int32_t dst;          /* device ordinal or RT_DST_CPU */
    int32_t reserved;
} rt_id_range;

/* The plan half of uvm_command, select.cpp:24099-24309: parses one command line
 * (prefetch / target / targetv / retarget / windowv / windowfullv / blocksv)
 * against a registry snapshot and writes the ranges it would queue, in queue
 * order.  On rejection returns RT_ERR_PLAN and *error points at the socket's
 * error string (static storage).  `page` is the host page size (0 = ask the OS). */
int rt_expand_command(const rt_alloc_info *registry, size_t n_alloc, uint64_t generation,
                      const char *line, uint64_t page, rt_id_range *out, size_t cap,
                      size_t *n_out, const char **error);

/* ------------------------------------------------------------------ */
/* Device planner                                                       */
/* ------------------------------------------------------------------ */

/* One emitted range: buffer = index of the cache allocation in registry order. */
typedef struct rt_range {
    uint32_t buffer;
    int32_t dst;          /* device ordinal or RT_DST_CPU */
    uint64_t offset;
    uint64_t bytes;
} rt_range;

/* KV geometry the planner works on.  All cache allocations have alloc_bytes;
 * bitmap g covers the buffers whose buffer_group entry is g (NULL: one bitmap
 * for all buffers).  Valid slot ids are 1..capacity_slots
 * (experiments/slot_feedback.py:27-28,39-43). */
typedef struct rt_layout {
    uint32_t n_buffers;
    uint32_t n_groups;
    uint64_t alloc_bytes;
    uint32_t bytes_per_slot;
    uint32_t block_bytes;
    uint64_t capacity_slots;
    const uint32_t *buffer_group;
    int32_t dst_device;   /* ordinal written into GPU-bound ranges */
    int32_t reserved;
} rt_layout;

#define RT_PLAN_EVICT   1u   /* also emit resident-but-not-wanted blocks, CPU-bound, first */
#define RT_PLAN_DRY_RUN 2u   /* do not commit the wanted set as the new resident set       */
#define RT_PLAN_TMA     4u   /* stage ids through shared memory with bulk async copies     */
                             /* (default: register-staged 128-bit loads, which measured    */
                             /* faster at the sizes a decode step produces)                */
#define RT_PLAN_CHAINED 8u   /* device-side step calls only: this step may start scanning  */
                             /* while the kernel before it in `stream` is still finishing. */
                             /* Meant for steps of one plan issued back to back (or        */
                             /* captured into one CUDA graph): the slot scan of step i+1   */
                             /* then runs over the range-emitting tail of step i; results  */
                             /* are identical.  The caller promises that the slot ids and  */
                             /* offsets of this step are complete before the PREVIOUS      */
                             /* operation in `stream` starts -- true when that operation   */
                             /* is another step, false when it is the kernel that writes   */
                             /* this step's ids and that kernel itself releases its        */
                             /* dependents early (programmatic dependent launch).  After   */
                             /* any other kind of operation the flag changes nothing.      */
#define RT_PLAN_WIDE_COPY 16u /* host-buffer call only: copy the 64-bit ids as they are.     */
                             /* Without it rt_plan_step narrows the ids of a pool with      */
                             /* fewer than 2^31 - 1 slots to 32 bits on the host cores      */
                             /* before they cross the host link (same results; ids outside  */
                             /* 0 .. 2^31 keep their class: negative stays "ignored", large */
                             /* stays "out of range"), when there are at least 2^20 of them.*/
                             /* RETARGET_B200_PACK_THREADS sets the number of host threads  */
                             /* (0: never narrow).  Default: 3/4 of the process's CPUs, at  */
                             /* most 16, when ONE GPU is visible; with more GPUs visible,   */
                             /* or fewer than 8 threads, the call copies the ids as they    */
                             /* are (narrowing costs host memory traffic, which is what is  */
                             /* short when several planners share a host).                  */

/* A step whose result carries any of these flags has NOT changed the resident
 * bitmaps: a plan that cannot be delivered in full is not committed (the
 * reference drops its record on any failure, experiments/slot_placement.py:140-147,
 * and checks the slot range before it stamps anything, experiments/slot_feedback.py:42).
 * The host-buffer calls turn them into RT_ERR_CAPACITY, RT_ERR_SLOT_RANGE and
 * RT_ERR_TIMEOUT; callers of the device-side calls read them from the result. */
#define RT_RESULT_OVERFLOW   1u   /* more ranges than `cap`: n_ranges says how many the   */
                                  /* plan needs, the first cap were written               */
#define RT_RESULT_SLOT_RANGE 2u   /* some slot id was above capacity; no range reported   */
#define RT_RESULT_TIMEOUT    4u   /* a bounded device-side wait gave up (bulk-copy        */
                                  /* staging only); no range reported                     */

typedef struct rt_plan_result {
    uint32_t n_ranges;        /* total emitted (may exceed cap, see flags)  */
    uint32_t n_cpu_ranges;    /* the first n_cpu_ranges move to the CPU      */
    uint32_t flags;
    uint32_t blocks_touched;  /* distinct blocks seen, summed over bitmaps   */
    uint32_t blocks_desired;  /* after the budget cut                        */
    uint32_t blocks_added;
    uint32_t blocks_evicted;
    uint32_t reserved;
    uint64_t invalid_slots;   /* ids above capacity                          */
    uint64_t ignored_slots;   /* ids below 1 (dropped, as the reference does)*/
    uint64_t gpu_bytes;       /* requested_gpu_bytes, experiments/slot_placement.py:154 */
    uint64_t cpu_bytes;
} rt_plan_result;

typedef struct rt_plan rt_plan;

/* Creates the planner state on `device`: resident bitmaps (all clear), scratch,
 * a side stream, a device staging buffer for max_indices slot ids and a pinned
 * host buffer for max_ranges ranges (both only used by the host-buffer call).
 * Fails with RT_ERR_NO_DEVICE when no usable GPU is present. */
int rt_plan_create(const rt_layout *layout, int device, uint64_t max_indices,
                   uint32_t max_ranges, rt_plan **out);
int rt_plan_destroy(rt_plan *plan);

/* Resident ("committed") bitmaps, n_groups x RT_BITMAP_WORDS uint32 words, bit b
 * of a bitmap = block b.  Stands in for SlotPlacementController.committed,
 * experiments/slot_placement.py:65,150-153. */
int rt_plan_set_resident(rt_plan *plan, const uint32_t *words);
int rt_plan_get_resident(rt_plan *plan, uint32_t *words);

/* One planning step over slot ids that are already in device memory.
 *
 *   d_slots      int64 slot ids, 16-byte aligned; group g owns
 *                d_slots[group_off[g] .. group_off[g+1])
 *   group_off    HOST array of n_groups+1 ascending offsets
 *   budget       keep at most this many blocks per bitmap
 *   out/result   device or mapped-pinned memory; written by the kernel
 *
 * Replaces, per bitmap: encode_runs (kv_audit_probe.py:23-32) ->
 * SlotFeedback.blocks (slot_feedback.py:35-46) -> read stamps (:72-74) ->
 * publish/target_blocks (slot_feedback.py:81-85, slot_placement.py:37-44) ->
 * choose (slot_placement.py:83-94) -> encode_mask + blocksv expansion
 * (slot_placement.py:47-51, select.cpp:24147-24195).
 * Asynchronous on `stream`. */
int rt_plan_step_device(rt_plan *plan, const int64_t *d_slots, const int64_t *group_off,
                        uint32_t budget, uint32_t flags, rt_range *out, uint32_t cap,
                        rt_plan_result *result, void *stream);

/* Same step from HOST memory: copies the slot ids to the device, plans, copies
 * the ranges back and waits.  This is the call a scheduler makes when the slot
 * table lives on the host, as in kv_audit_probe.py:54-105.  The copy is what
 * bounds it, so large lists of 64-bit ids cross the link as 32-bit ids (see
 * RT_PLAN_WIDE_COPY); h_slots may be pageable or pinned memory. */
int rt_plan_step(rt_plan *plan, const int64_t *h_slots, const int64_t *group_off,
                 uint32_t budget, uint32_t flags, rt_range *out, uint32_t cap,
                 rt_plan_result *result);

/* Host threads rt_plan_step narrows with for this plan; 0: it copies 64-bit
 * ids as they are (see RT_PLAN_WIDE_COPY for the rule). */
int rt_plan_narrow_threads(rt_plan *plan, uint32_t *threads);

/* What rt_plan_step does to 64-bit ids before they cross the host link, as a
 * host utility: dst[i] = src[i] for ids in [0, 2^31), -1 for ids below zero,
 * INT32_MAX for ids of 2^31 and above.  `threads` host threads share the work
 * (0: as many as rt_plan_step would use). */
int rt_narrow_ids(const int64_t *src, int32_t *dst, uint64_t n, uint32_t threads);

/* Padded request table (the serving engine's req_to_token layout): row r holds
 * lens[r] valid ids in d_table[r*stride ..]; one bitmap for all buffers
 * (n_groups must be 1).  d_lens is a DEVICE int32 array. */
int rt_plan_step_table(rt_plan *plan, const int64_t *d_table, const int32_t *d_lens,
                       uint32_t n_rows, uint64_t stride, uint32_t budget, uint32_t flags,
                       rt_range *out, uint32_t cap, rt_plan_result *result, void *stream);

/* Scan only: OR of touched blocks per bitmap into d_bitmaps
 * (n_groups x RT_BITMAP_WORDS words, overwritten).  slot_feedback.py:35-46. */
int rt_scan_slots(rt_plan *plan, const int64_t *d_slots, const int64_t *group_off,
                  uint32_t *d_bitmaps, rt_plan_result *result, void *stream);

/* The same four calls for 32-bit slot ids, the width the serving engine itself
 * keeps them in (its kv_indices and req_to_token tensors are int32; the probe
 * copies whatever dtype it is handed, kv_audit_probe.py:66-71, and widens the
 * ids to Python ints with tolist() at :92).  Reading the engine's tensors in
 * place halves the bytes per id.  Results are identical to the int64 calls on
 * the same ids.  A negative id is ignored like any id below 1
 * (slot_feedback.py:39); capacity_slots must not exceed 2^31 - 1
 * (RT_ERR_INVALID_ARGUMENT).  RT_PLAN_TMA has no effect here: the bulk-copy
 * kernel reads int64 ids only.  Pointers are 16-byte aligned as above. */
int rt_plan_step_device_i32(rt_plan *plan, const int32_t *d_slots, const int64_t *group_off,
                            uint32_t budget, uint32_t flags, rt_range *out, uint32_t cap,
                            rt_plan_result *result, void *stream);
int rt_plan_step_i32(rt_plan *plan, const int32_t *h_slots, const int64_t *group_off,
                     uint32_t budget, uint32_t flags, rt_range *out, uint32_t cap,
                     rt_plan_result *result);
int rt_plan_step_table_i32(rt_plan *plan, const int32_t *d_table, const int32_t *d_lens,
                           uint32_t n_rows, uint64_t stride, uint32_t budget, uint32_t flags,
                           rt_range *out, uint32_t cap, rt_plan_result *result, void *stream);
int rt_scan_slots_i32(rt_plan *plan, const int32_t *d_slots, const int64_t *group_off,
                      uint32_t *d_bitmaps, rt_plan_result *result, void *stream);

/* Diff + budget + coalesce only, from wanted bitmaps already on the device.
 * With the resident set holding the old window and d_want the new one this
 * yields the windowv symmetric difference (select.cpp:24231-24240) for
 * block-aligned windows. */
int rt_plan_from_bitmaps(rt_plan *plan, const uint32_t *d_want, uint32_t budget, uint32_t flags,
                         rt_range *out, uint32_t cap, rt_plan_result *result, void *stream);

/* Waits for everything queued on the plan's own stream. */
int rt_plan_sync(rt_plan *plan);

/* Scan for callers that must not allocate: no plan handle, no cudaMalloc /
 * cudaFree or any other allocating call.  (No counterpart in the reference; it
 * exists for this library's own use inside a serving process, see below.)
 *
 * Code that runs inside the preload library cannot allocate device memory
 * without disturbing what it manages -- the allocation would go through the
 * library's own cuMemAlloc hook, become a registered managed allocation and
 * bump the generation that plans are validated against -- and a process whose
 * device memory belongs entirely to the serving engine's pool has nothing left
 * to allocate from.  For them the scan's working memory is a static device
 * array of 8.25 KiB inside the library (held by every GPU that loads it), which
 * limits a call to RT_STATIC_MAX_GROUPS bitmaps; more is refused with
 * RT_ERR_CAPACITY.  The number of slot ids is not limited.
 *
 * Same result as rt_scan_slots: d_bitmaps gets n_groups x RT_BITMAP_WORDS words,
 * d_result the counters (blocks_touched, invalid_slots, ignored_slots, flags).
 * Runs on the calling thread's current device, asynchronously on `stream`
 * (NULL here is the legacy default stream).  The first call on a device also
 * looks up the array's device address; make that first call before any stream
 * capture.  All calls on a device share the array: calls that overlap on the GPU
 * race, so keep them on one stream or otherwise serialised.  The address is kept
 * for the life of the process: after cudaDeviceReset (or any other destruction
 * of the device's primary context) it is stale and this entry point must not be
 * called again in that process. */
#define RT_STATIC_MAX_GROUPS 64u
int rt_scan_slots_static(const int64_t *d_slots, const int64_t *group_off, uint32_t n_groups,
                         uint64_t capacity_slots, uint32_t block_tokens, uint32_t n_blocks,
                         uint32_t *d_bitmaps, rt_plan_result *d_result, void *stream);

/* ------------------------------------------------------------------ */
/* Slot-feedback state in GPU memory                                    */
/* ------------------------------------------------------------------ */

/* Device-resident twin of SlotFeedback (experiments/slot_feedback.py:10-96):
 * per-slot generation counters, per-block version / last-read / last-write
 * stamps and the sampled free-list head, updated straight from the serving
 * engine's device tensors -- no pinned copy, no run encoding on the host, no
 * JSON file.  Bound to a plan with ONE bitmap (the reference plans one mask for
 * all allocations); the plan's resident words are the committed set. */
typedef struct rt_feedback rt_feedback;

int rt_feedback_create(rt_plan *plan, rt_feedback **out);
int rt_feedback_destroy(rt_feedback *fb);

/* allocator_clear: SlotFeedback.reset, slot_feedback.py:25-33 (also forgets the
 * committed set, as the controller does on a new epoch, slot_placement.py:123-124). */
int rt_feedback_reset(rt_feedback *fb, void *stream);

/* alloc event, slot_feedback.py:52-70: generations += 1 per allocated slot,
 * version = max generation and write stamp for every touched block; the free
 * head is replaced by d_free_head (first n_free <= 4096 free slots) or, when
 * d_free_head is NULL, loses the slots just allocated. */
int rt_feedback_alloc(rt_feedback *fb, const int64_t *d_slots, uint64_t n, const int64_t *d_free_head,
                      uint32_t n_free, double t, void *stream);

/* attention event, slot_feedback.py:71-75: read stamps, then write stamps. */
int rt_feedback_attention(rt_feedback *fb, const int64_t *d_read, uint64_t n_read,
                          const int64_t *d_write, uint64_t n_write, double t, void *stream);

/* The two event calls for 32-bit ids (the serving engine's kv_indices are
 * int32); all lists of one call have the same width.  Same state, same plans.
 * capacity_slots must not exceed 2^31 - 1 (RT_ERR_INVALID_ARGUMENT). */
int rt_feedback_alloc_i32(rt_feedback *fb, const int32_t *d_slots, uint64_t n,
                          const int32_t *d_free_head, uint32_t n_free, double t, void *stream);
int rt_feedback_attention_i32(rt_feedback *fb, const int32_t *d_read, uint64_t n_read,
                              const int32_t *d_write, uint64_t n_write, double t, void *stream);

/* Copies the state to the host (any pointer may be NULL): n_blocks versions and
 * stamps (-inf = never), up to 4096 free-head slot ids.  This is the content of
 * the snapshot file of slot_feedback.py:86-91 before ranking.  Synchronous. */
int rt_feedback_snapshot(rt_feedback *fb, int32_t *versions, double *read_seen, double *write_seen,
                         int64_t *free_head, uint32_t *n_free, uint64_t *epoch,
                         uint64_t *invalid_slots);

/* experiments/slot_placement.py:18-26, the fields the plan uses. */
typedef struct rt_feedback_policy {
    uint32_t budget;                 /* width_tokens / block_tokens, slot_placement.py:60 */
    uint32_t max_blocks_per_update;
    uint32_t flags;                  /* RT_PLAN_EVICT */
    uint32_t reserved;
    double active_seconds;
    double refresh_seconds;
} rt_feedback_policy;

/* Ranks the blocks on the device (active reads, active writes, free-list head,
 * history by recency; ties by ascending block id), cuts at the budget, keeps
 * the blocks that are new / re-versioned / due for refresh up to
 * max_blocks_per_update, commits them and emits their ranges:
 * publish + target_blocks + choose + encode_mask + blocksv expansion,
 * slot_feedback.py:81-85, slot_placement.py:37-51,83-94,150-153,
 * select.cpp:24147-24195.  `at` is the time of the last event (30 s horizon),
 * `now` the planning time.  Asynchronous on `stream`. */
int rt_feedback_plan(rt_feedback *fb, const rt_feedback_policy *policy, double at, double now,
                     rt_range *out, uint32_t cap, rt_plan_result *result, void *stream);

/* One decode step's events, as the serving engine produces them: the slots
 * the allocator handed out (with the new free-list head, or null), then the
 * slots attention read and wrote.  All pointers are DEVICE pointers, int64 for
 * rt_feedback_step, int32 for rt_feedback_step_i32. */
typedef struct rt_feedback_step_ids {
    const void *d_allocated;         /* may be null with n_allocated == 0: no allocation this step */
    uint64_t n_allocated;
    const void *d_free_head;         /* null: derive the head from the known one */
    uint32_t n_free;
    uint32_t reserved;
    double t_allocated;
    const void *d_read;
    uint64_t n_read;
    const void *d_written;
    uint64_t n_written;
    double t_attention;
} rt_feedback_step_ids;

/* rt_feedback_alloc + rt_feedback_attention + rt_feedback_plan (at =
 * t_attention) as ONE kernel launch, with the same results as the three calls
 * in that order: the hooks of one decode step (slot_feedback.py:49-79) and the
 * controller's update that follows them (slot_placement.py:83-94,150-153). */
int rt_feedback_step(rt_feedback *fb, const rt_feedback_step_ids *ids, const rt_feedback_policy *policy,
                     double now, rt_range *out, uint32_t cap, rt_plan_result *result, void *stream);
int rt_feedback_step_i32(rt_feedback *fb, const rt_feedback_step_ids *ids, const rt_feedback_policy *policy,
                         double now, rt_range *out, uint32_t cap, rt_plan_result *result, void *stream);

/* ------------------------------------------------------------------ */
/* Synthetic paged KV reader                                            */
/* ------------------------------------------------------------------ */

/* Reads, for every valid slot id in d_slots, the bytes_per_slot-byte row of
 * that slot in each of the n_buffers KV buffers (d_buffers: DEVICE array of
 * n_buffers base pointers) and writes one checksum per buffer (sum of the rows'
 * 16-bit words) to d_sums.  No reference counterpart: it plays the serving
 * engine's paged decode attention in the prefetch experiments, so that the same
 * reads can be timed with the pages on the CPU, on the GPU, or moved there by a
 * plan.  Runs on the current device, asynchronously on `stream` (NULL: legacy
 * default stream). */
int rt_paged_read(const void *const *d_buffers, uint32_t n_buffers, uint32_t bytes_per_slot,
                  const int64_t *d_slots, uint64_t n_slots, uint64_t capacity_slots,
                  uint64_t *d_sums, void *stream);

/* Read-only bandwidth yardstick: reads `bytes` (a multiple of 16, 16-byte
 * aligned) of device memory once, with the slot scan's access pattern, and
 * folds them into *d_sink (xor of the 64-bit words, folded; the caller zeroes
 * it).  No reference counterpart: the bench quotes its GB/s beside the scan's.
 * Asynchronous on `stream`. */
int rt_read_probe(const void *d_data, uint64_t bytes, uint64_t *d_sink, void *stream);

/* Synthetic paged bf16 decode attention: for every request r and every layer,
 * out = softmax(q . K^T / sqrt(128)) . V over the K and V rows of the request's
 * slots d_slots[d_req_off[r] .. d_req_off[r+1]) (slot 0 and ids outside
 * 1..capacity_slots are skipped).  A layer's K and V buffers are
 * [pool_slots][n_kv_heads][128] bf16 (n_kv_heads <= 8); d_q is
 * [n_requests][n_layers][n_kv_heads][128] bf16, d_out the same shape in fp32
 * (bf16 inputs, fp32 accumulation).  d_k_buffers / d_v_buffers are DEVICE arrays
 * of n_layers base pointers; d_slots and d_req_off are device arrays.
 * No reference counterpart: it stands in for the serving engine's decode
 * attention in the end-to-end prefetch experiment, where the point is that real
 * arithmetic waits for the KV pages a plan did or did not bring in.  Runs on
 * the current device, asynchronously on `stream` (NULL: legacy default stream). */
int rt_paged_attention(const void *const *d_k_buffers, const void *const *d_v_buffers, uint32_t n_layers,
                       uint32_t n_kv_heads, const void *d_q, const int64_t *d_slots,
                       const int64_t *d_req_off, uint32_t n_requests, uint64_t capacity_slots,
                       float *d_out, void *stream);

/* ------------------------------------------------------------------ */
/* UVM control server + prefetch executor (process-wide singleton)      */
/* ------------------------------------------------------------------ */

/* Stands in for the UVM block of the reference preload library,
 * select.cpp:23750-24446: allocation registry, the text protocol of the control
 * socket (same commands, replies and error strings), one migration job at a
 * time executed by a worker thread.  Differences are confined to HOW the job
 * runs: persistent side streams instead of a stream created and destroyed per
 * chunk, several chunks in flight, one wait per batch. */
typedef struct rt_uvm_config {
    const char *socket_path;   /* NULL: /tmp/select-uvm-<uid>-<pid>.sock, select.cpp:24416 */
    uint64_t chunk_bytes;      /* 0: SELECT_UVM_CHUNK_MB (1..256) or 16 MiB, select.cpp:23853 */
    uint64_t batch_bytes;      /* bytes issued between two waits; 0: 256 MiB             */
    uint32_t streams;          /* side streams per context; 0: 4                         */
    int32_t listen;            /* 0: no socket, commands only through rt_uvm_command     */
    uint32_t overlap_phases;   /* 0: every CPU-bound range has landed before the first   */
                               /* GPU-bound one is issued (the reference's order).  1:   */
                               /* the two stretches of a plan move at the same time, one */
                               /* direction of the host link each; for callers whose     */
                               /* evictions are not what makes room for the additions    */
    uint32_t reserved;
} rt_uvm_config;

int rt_uvm_start(const rt_uvm_config *config);
int rt_uvm_stop(void);

/* Registry, select.cpp:24724-24761 (insert) and 23871-23913 (remove).  Every
 * change bumps the allocation generation.  ctx may be NULL (current context). */
int rt_uvm_register(uint64_t ptr, uint64_t bytes, void *ctx, int device, int concurrent,
                    uint64_t *id);
int rt_uvm_unregister_ptr(uint64_t ptr);
int rt_uvm_unregister_ctx(void *ctx);
int rt_uvm_unregister_device(int device);

/* One protocol line in, one JSON reply line out (without the newline); exactly
 * what a socket client would get, select.cpp:24045-24327.  Returns the reply
 * length, or RT_ERR_CAPACITY. */
int rt_uvm_command(const char *line, char *reply, size_t cap);

/* Queues ranges produced by the device planner as one job: ranges[i].buffer
 * indexes buffer_ids (allocation ids in registry order).  No reference
 * counterpart: it skips the text round trip of blocksv/windowv, the job itself
 * is what select.cpp:23990-24024 runs.  RT_ERR_BUSY while a job is in flight. */
int rt_uvm_submit_ranges(const rt_range *ranges, size_t n, const uint64_t *buffer_ids,
                         size_t n_ids, uint64_t *job_id);

/* Blocks until job_id has completed (or timeout_s passed: RT_ERR_BUSY).
 * *cuda_error gets the job's CUresult. */
int rt_uvm_wait(uint64_t job_id, double timeout_s, int *cuda_error);

/* Path the listener is bound to ("" when not listening).  Returns its length. */
int rt_uvm_socket_path(char *out, size_t cap);

/* ------------------------------------------------------------------ */
/* Client side of the control socket                                    */
/* ------------------------------------------------------------------ */

/* One command over the control socket of another process
 * (UvmController.command, experiments/control.py:427-460): connects to
 * `socket_path`, sends `line` (no terminator; at most 510 bytes, no CR / LF) and
 * collects the reply up to its newline into `reply`.  One deadline of
 * `timeout_s` covers connect, send and receive.  Returns the reply's length;
 * RT_ERR_IO with the errno in *os_error (ETIMEDOUT when the deadline passed);
 * RT_ERR_CAPACITY for a reply beyond `cap` or 1 MiB. */
int rt_uvm_client_command(const char *socket_path, const char *line, double timeout_s, char *reply,
                          size_t cap, int *os_error);

/* The fields of a `status` reply, select.cpp:24058-24068
 * (UvmStatus, experiments/control.py:53-83). */
typedef struct rt_uvm_status {
    uint64_t pid;
    uint64_t managed_bytes;
    uint64_t allocation_count;
    uint64_t allocation_generation;
    int32_t busy;
    int32_t last_error;
    uint64_t job_id;
    uint64_t completed_job;
    uint64_t completed_cpu_bytes;
    uint64_t completed_gpu_bytes;
    uint64_t job_completed_bytes;
} rt_uvm_status;

/* Parses a status reply.  RT_ERR_PLAN when the reply says ok:false,
 * RT_ERR_INVALID_ARGUMENT when a field is missing. */
int rt_uvm_parse_status(const char *reply, rt_uvm_status *out);

/* What a client checks before it trusts a PID (experiments/control.py:403-425):
 * the start time of the process (clock ticks since boot; another value later
 * means the PID was reused) and the uid that owns it. */
int rt_process_start_time(uint64_t pid, uint64_t *ticks, int *os_error);
int rt_process_owner(uint64_t pid, uint32_t *uid, int *os_error);

#ifdef __cplusplus
}
#endif
#endif /* RETARGET_B200_H */
