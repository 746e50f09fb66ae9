/*
 * Oracle (C): one planning step on the CPU, restating the reference chain
 *   encode_runs            experiments/kv_audit/kv_audit_probe.py:23-32
 *   SlotFeedback.blocks    experiments/slot_feedback.py:35-46
 *   target_blocks (one event, ties by ascending block id)
 *                          experiments/slot_placement.py:37-44
 *   choose                 experiments/slot_placement.py:83-94
 *   blocksv run walk       select.cpp:24177-24194
 * plus the eviction glue described in oracle/compose.py.
 *
 * TEST INFRASTRUCTURE ONLY: used as a checker and as the timed CPU baseline,
 * never by the shipped library.  Pinned by tests/test_oracle_compose.py against
 * the Python oracle, which is itself pinned to reference-generated fixtures.
 *
 * Build: make -C oracle   (gcc -O2 -fopenmp -shared -fPIC)
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

typedef struct {
    uint32_t buffer;
    int32_t dst;
    uint64_t offset;
    uint64_t bytes;
} orc_range;

#define ORC_MAX_BLOCKS 1024

/* Marks the blocks touched by slots[lo..hi): consecutive ids are first merged
 * into half-open runs, then each run marks begin/T .. (end-1)/T with slot 0
 * clipped away, exactly like the reference's two functions. */
static void mark_span(const int64_t *slots, int64_t lo, int64_t hi, uint32_t T, uint64_t capacity,
                      uint8_t *touched, uint64_t *invalid)
{
    int64_t i = lo;
    while (i < hi) {
        int64_t begin = slots[i], end = begin + 1;
        ++i;
        while (i < hi && slots[i] == end) { ++end; ++i; }
        if (begin < 1) begin = 1;
        if (begin >= end) continue;
        if ((uint64_t)end > capacity + 1) {          /* the reference asserts here */
            int64_t over = end - (int64_t)(capacity + 1);
            if (over > end - begin) over = end - begin;
            *invalid += (uint64_t)over;
            end = (int64_t)capacity + 1;
            if (begin >= end) continue;
        }
        for (int64_t b = begin / T; b <= (end - 1) / T; ++b) touched[b] = 1;
    }
}

static int64_t emit_runs(const uint8_t *bits, uint32_t n_blocks, uint32_t buffer, int32_t dst,
                         uint64_t alloc_bytes, uint64_t block_bytes, orc_range *out, int64_t pos,
                         int64_t cap)
{
    uint64_t whole = alloc_bytes / block_bytes;
    uint32_t b = 0;
    while (b < n_blocks) {
        if (!bits[b]) { ++b; continue; }
        uint32_t e = b;
        while (e < n_blocks && bits[e]) ++e;
        uint64_t end = e > whole ? alloc_bytes : (uint64_t)e * block_bytes;
        if (pos < cap) {
            out[pos].buffer = buffer;
            out[pos].dst = dst;
            out[pos].offset = (uint64_t)b * block_bytes;
            out[pos].bytes = end - (uint64_t)b * block_bytes;
        }
        ++pos;
        b = e;
    }
    return pos;
}

int orc_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* resident: n_groups x ORC_MAX_BLOCKS bytes (0/1), updated in place.
 * Returns the number of ranges (may exceed cap). */
int64_t orc_plan_step(const int64_t *slots, const int64_t *group_off, int n_groups,
                      const uint32_t *buffer_group, int n_buffers, uint64_t alloc_bytes,
                      uint64_t block_bytes, uint32_t block_tokens, uint64_t capacity, uint32_t budget,
                      int evict, int32_t dst_device, uint8_t *resident, orc_range *out, int64_t cap,
                      uint64_t *invalid_out, int threads)
{
    uint32_t n_blocks = (uint32_t)(alloc_bytes / block_bytes + (alloc_bytes % block_bytes != 0));
    uint8_t *add = calloc((size_t)n_groups * ORC_MAX_BLOCKS, 1);
    uint8_t *ev = calloc((size_t)n_groups * ORC_MAX_BLOCKS, 1);
    uint64_t invalid = 0;
    if (threads < 1) threads = 1;
    if (n_groups > 1) {
#pragma omp parallel for schedule(dynamic, 1) num_threads(threads) reduction(+ : invalid)
        for (int g = 0; g < n_groups; ++g) {
            uint8_t touched[ORC_MAX_BLOCKS + 1];
            memset(touched, 0, sizeof(touched));
            uint64_t bad = 0;
            mark_span(slots, group_off[g], group_off[g + 1], block_tokens, capacity, touched, &bad);
            invalid += bad;
            memcpy(add + (size_t)g * ORC_MAX_BLOCKS, touched, ORC_MAX_BLOCKS);
        }
    } else {
        /* one bitmap: split the span at run boundaries is not needed, because a
         * run cut in two marks the same blocks */
        int64_t lo = group_off[0], hi = group_off[1];
        int parts = threads;
        uint8_t *part_bits = calloc((size_t)parts * (ORC_MAX_BLOCKS + 1), 1);
#pragma omp parallel for schedule(static) num_threads(threads) reduction(+ : invalid)
        for (int p = 0; p < parts; ++p) {
            int64_t a = lo + (hi - lo) * p / parts, b = lo + (hi - lo) * (p + 1) / parts;
            uint64_t bad = 0;
            mark_span(slots, a, b, block_tokens, capacity, part_bits + (size_t)p * (ORC_MAX_BLOCKS + 1), &bad);
            invalid += bad;
        }
        for (int p = 0; p < parts; ++p)
            for (uint32_t b = 0; b < n_blocks; ++b) add[b] |= part_bits[(size_t)p * (ORC_MAX_BLOCKS + 1) + b];
        free(part_bits);
    }
    /* budget cut (lowest ids first), then diff against the resident set */
    for (int g = 0; g < n_groups; ++g) {
        uint8_t *want = add + (size_t)g * ORC_MAX_BLOCKS, *res = resident + (size_t)g * ORC_MAX_BLOCKS;
        uint8_t *out_ev = ev + (size_t)g * ORC_MAX_BLOCKS;
        uint8_t desired[ORC_MAX_BLOCKS];
        uint32_t kept = 0, moved = 0;
        for (uint32_t b = 0; b < ORC_MAX_BLOCKS; ++b) {
            desired[b] = 0;
            if (b < n_blocks && want[b] && kept < budget) { desired[b] = 1; ++kept; }
            out_ev[b] = (uint8_t)(evict && res[b] && !desired[b]);
            want[b] = (uint8_t)(desired[b] && !res[b]);
            moved += out_ev[b] + want[b];
        }
        /* nothing selected: the controller returns before it touches `committed`
         * (experiments/slot_placement.py:131-132); otherwise committed = the part
         * of it that is still desired + what was sent (:150-153) */
        if (moved) memcpy(res, desired, ORC_MAX_BLOCKS);
    }
    int64_t pos = 0;
    for (int j = 0; j < n_buffers; ++j)
        pos = emit_runs(ev + (size_t)buffer_group[j] * ORC_MAX_BLOCKS, n_blocks, (uint32_t)j, -1, alloc_bytes,
                        block_bytes, out, pos, cap);
    for (int j = 0; j < n_buffers; ++j)
        pos = emit_runs(add + (size_t)buffer_group[j] * ORC_MAX_BLOCKS, n_blocks, (uint32_t)j, dst_device,
                        alloc_bytes, block_bytes, out, pos, cap);
    free(add);
    free(ev);
    if (invalid_out) *invalid_out = invalid;
    return pos;
}
