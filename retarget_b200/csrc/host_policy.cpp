// Host arithmetic of the placement policy and the plan-command expander.
// No CUDA in this file: it is the part of the path that is O(1) or
// O(#allocations) per plan and runs inside the preload library's socket thread.
#include <unistd.h>

#include <cmath>
#include <cstdint>
#include <cstring>
#include <string>
#include <vector>

#include "rt_internal.h"
#include "uvm_plan.h"

namespace {

const char *kPositiveNames[] = {"allocation_bytes", "allocation_count", "bytes_per_token",
                                "width_tokens", "lookahead_tokens", "quantum_tokens"};

}  // namespace

extern "C" {

int rt_abi_version(void) { return RT_ABI_VERSION; }

int rt_last_cuda_error(void) { return rt::last_cuda_error_get(); }

const char *rt_strerror(int status) {
    switch (status) {
        case RT_OK: return "ok";
        case RT_ERR_INVALID_ARGUMENT: return "invalid argument";
        case RT_ERR_NO_DEVICE: return "no usable CUDA device (this library has no CPU fallback)";
        case RT_ERR_CUDA: return "CUDA call failed";
        case RT_ERR_OUT_OF_MEMORY: return "out of memory";
        case RT_ERR_CAPACITY: return "more slot ids, ranges or bitmaps than the plan (or the static scratch) can hold";
        case RT_ERR_ALIGNMENT: return "slot array must be 16-byte aligned";
        case RT_ERR_SLOT_RANGE: return "slot beyond capacity";
        case RT_ERR_BUSY: return "busy";
        case RT_ERR_NOT_RUNNING: return "UVM server not running";
        case RT_ERR_IO: return "I/O error";
        case RT_ERR_PLAN: return "plan command rejected";
        case RT_ERR_TIMEOUT: return "a bounded device-side wait gave up; nothing was planned";
        // messages of experiments/cache_window.py:31-54
        case RT_ERR_SPEC_POSITIVE: return "cache_window field must be a positive integer";
        case RT_ERR_SPEC_TRAILING: return "cache window must retain a trailing region";
        case RT_ERR_SPEC_PAGE: return "cache window quantum must be page aligned";
        case RT_ERR_SPEC_MULTIPLE: return "cache window dimensions must be multiples of the quantum";
        case RT_ERR_SPEC_EXCEEDS: return "cache window exceeds each allocation";
        case RT_ERR_SPEC_INTERVAL: return "invalid cache window update interval";
        case RT_ERR_SPEC_MODE: return "invalid cache_window.update_mode";
        case RT_ERR_COMPLETED_COUNT: return "invalid completed-token count";
        // messages of experiments/slot_placement.py:60-64
        case RT_ERR_BUDGET_DIVISIBLE: return "KV budget must be divisible by block_tokens";
        case RT_ERR_BLOCK_PAGE: return "slot blocks must be page aligned";
        // messages of experiments/cache_window.py:82-85,105-107 and slot_placement.py:75
        case RT_ERR_METRICS_MISSING: return "cache-window policy requires SGLang completed-token counters";
        case RT_ERR_METRICS_INVALID: return "invalid SGLang completed-token counters";
        case RT_ERR_METRICS_KEY_RUNNING: return "sglang:num_running_reqs";
        case RT_ERR_METRICS_KEY_QUEUE: return "sglang:num_queue_reqs";
        case RT_ERR_LAYOUT_MISMATCH: return "cache layout mismatch";
        case RT_ERR_SLOT_SPEC: return "slot placement field out of range";
        case RT_ERR_FEEDBACK_IDENTITY: return "slot feedback identity or geometry mismatch";
        default: return "unknown status";
    }
}

int rt_window_spec_check(const rt_window_spec *s, int *bad_field) {
    if (!s) return RT_ERR_INVALID_ARGUMENT;
    const uint64_t fields[6] = {s->allocation_bytes, s->allocation_count, s->bytes_per_token,
                                s->width_tokens, s->lookahead_tokens, s->quantum_tokens};
    (void)kPositiveNames;
    for (int i = 0; i < 6; ++i)
        if (fields[i] == 0 || fields[i] > (uint64_t)INT64_MAX) {
            if (bad_field) *bad_field = i;
            return RT_ERR_SPEC_POSITIVE;
        }
    if (s->lookahead_tokens >= s->width_tokens) return RT_ERR_SPEC_TRAILING;
    // products are taken in 128 bits: Python integers do not wrap
    unsigned __int128 qb = (unsigned __int128)s->quantum_tokens * s->bytes_per_token;
    if (qb % 4096) return RT_ERR_SPEC_PAGE;
    if (s->width_tokens % s->quantum_tokens || s->lookahead_tokens % s->quantum_tokens)
        return RT_ERR_SPEC_MULTIPLE;
    if ((unsigned __int128)s->width_tokens * s->bytes_per_token > s->allocation_bytes)
        return RT_ERR_SPEC_EXCEEDS;
    if (!std::isfinite(s->min_update_seconds) || s->min_update_seconds < 0) return RT_ERR_SPEC_INTERVAL;
    if (s->idle_only != 0 && s->idle_only != 1) return RT_ERR_INVALID_ARGUMENT;
    if (s->update_mode < 0 || s->update_mode > 2) return RT_ERR_SPEC_MODE;
    return RT_OK;
}

int rt_window(const rt_window_spec *s, double completed, uint64_t out[2]) {
    if (!s || !out) return RT_ERR_INVALID_ARGUMENT;
    if (!std::isfinite(completed) || completed < 0) return RT_ERR_COMPLETED_COUNT;
    if (!s->quantum_tokens || !s->bytes_per_token) return RT_ERR_INVALID_ARGUMENT;
    const uint64_t q = s->quantum_tokens;
    // The division and the round-up are done in binary64, like the Python
    // expression math.ceil((completed + lookahead) / q); the product with q is
    // exact integer arithmetic, saturated far above any reachable end.
    double steps = std::ceil((completed + (double)s->lookahead_tokens) / (double)q);
    const uint64_t max_end = s->allocation_bytes / (q * s->bytes_per_token) * q;
    uint64_t desired_end;
    if (steps >= 18446744073709551615.0 / (double)q) {
        desired_end = UINT64_MAX;
    } else {
        desired_end = (uint64_t)steps * q;
    }
    if (desired_end < s->width_tokens) desired_end = s->width_tokens;
    uint64_t end = desired_end < max_end ? desired_end : max_end;
    if (end < s->width_tokens) return RT_ERR_SPEC_EXCEEDS;
    out[0] = (end - s->width_tokens) * s->bytes_per_token;
    out[1] = end * s->bytes_per_token;
    return RT_OK;
}

int rt_interval_difference(const uint64_t a[2], const uint64_t b[2], uint64_t out[4]) {
    if (!a || !b || !out) return RT_ERR_INVALID_ARGUMENT;
    int n = 0;
    uint64_t lo = a[0], hi = a[1] < b[0] ? a[1] : b[0];
    if (hi > lo) { out[0] = lo; out[1] = hi; n = 1; }
    lo = a[0] > b[1] ? a[0] : b[1];
    hi = a[1];
    if (hi > lo) { out[2 * n] = lo; out[2 * n + 1] = hi; ++n; }
    return n;
}

int rt_window_accounting(const rt_window_spec *s, uint64_t n_cache, uint64_t other_bytes,
                         const uint64_t old_window[2], const uint64_t new_window[2], int full,
                         int refresh, uint64_t *gpu_bytes, uint64_t *cpu_bytes) {
    if (!s || !new_window || !gpu_bytes || !cpu_bytes) return RT_ERR_INVALID_ARGUMENT;
    const uint64_t width = new_window[1] - new_window[0];
    if (full || refresh) {
        *gpu_bytes = (full ? other_bytes : 0) + n_cache * width;
        *cpu_bytes = n_cache * (s->allocation_bytes - new_window[1] + new_window[0]);
        return RT_OK;
    }
    if (!old_window) return RT_ERR_INVALID_ARGUMENT;
    uint64_t pieces[4];
    int n = rt_interval_difference(new_window, old_window, pieces);
    uint64_t grow = 0, shrink = 0;
    for (int i = 0; i < n; ++i) grow += pieces[2 * i + 1] - pieces[2 * i];
    n = rt_interval_difference(old_window, new_window, pieces);
    for (int i = 0; i < n; ++i) shrink += pieces[2 * i + 1] - pieces[2 * i];
    *gpu_bytes = n_cache * grow;
    *cpu_bytes = n_cache * shrink;
    return RT_OK;
}

int rt_aligned_target(const uint64_t *allocation_bytes, size_t n, uint64_t desired, uint64_t page,
                      uint64_t *target) {
    if ((!allocation_bytes && n) || !page || !target) return RT_ERR_INVALID_ARGUMENT;
    uint64_t covered = 0;                 // bytes of the allocations that are resident in full
    for (size_t i = 0; i < n; ++i) {
        const uint64_t size = allocation_bytes[i];
        if (size > UINT64_MAX - covered) return RT_ERR_INVALID_ARGUMENT;
        if (desired - covered >= size) {  // desired >= covered holds throughout
            covered += size;
            continue;
        }
        const uint64_t inside = desired - covered;
        *target = covered + inside / page * page;
        return RT_OK;
    }
    *target = covered;
    return RT_OK;
}

int rt_slot_budget(const rt_window_spec *s, uint64_t block_tokens, uint64_t *budget_blocks) {
    if (!s || !block_tokens || !budget_blocks) return RT_ERR_INVALID_ARGUMENT;
    uint64_t budget = s->width_tokens / block_tokens;
    if (!budget || s->width_tokens % block_tokens) return RT_ERR_BUDGET_DIVISIBLE;
    if (((unsigned __int128)block_tokens * s->bytes_per_token) % 4096) return RT_ERR_BLOCK_PAGE;
    *budget_blocks = budget;
    return RT_OK;
}

int rt_encode_mask(const uint32_t *blocks, size_t n, char *out, size_t cap) {
    if ((!blocks && n) || !out || !cap) return RT_ERR_INVALID_ARGUMENT;
    uint32_t top = 0;
    for (size_t i = 0; i < n; ++i)
        if (blocks[i] > top) top = blocks[i];
    std::vector<uint8_t> nibbles(top / 4 + 1, 0);
    for (size_t i = 0; i < n; ++i) nibbles[blocks[i] / 4] |= (uint8_t)(1u << (blocks[i] % 4));
    size_t digits = nibbles.size();
    while (digits > 1 && !nibbles[digits - 1]) --digits;
    if (digits + 1 > cap) return RT_ERR_CAPACITY;
    for (size_t d = 0; d < digits; ++d) out[d] = "0123456789abcdef"[nibbles[digits - 1 - d]];
    out[digits] = 0;
    return (int)digits;
}

int rt_encode_runs(const int64_t *values, size_t n, int64_t *runs_out, size_t cap_runs,
                   size_t *n_runs) {
    if ((!values && n) || !n_runs || (!runs_out && cap_runs)) return RT_ERR_INVALID_ARGUMENT;
    size_t count = 0;
    int64_t run_begin = 0, run_end = 0;
    bool open = false;
    auto close = [&] {
        if (count < cap_runs) { runs_out[2 * count] = run_begin; runs_out[2 * count + 1] = run_end; }
        ++count;
    };
    for (size_t i = 0; i < n; ++i) {
        int64_t v = values[i];
        if (open && run_end == v) {
            run_end = v + 1;
        } else {
            if (open) close();
            run_begin = v;
            run_end = v + 1;
            open = true;
        }
    }
    if (open) close();
    *n_runs = count;
    return count > cap_runs ? RT_ERR_CAPACITY : RT_OK;
}

int rt_expand_command(const rt_alloc_info *registry, size_t n_alloc, uint64_t generation,
                      const char *line, uint64_t page, rt_id_range *out, size_t cap, size_t *n_out,
                      const char **error) {
    if ((!registry && n_alloc) || !line || !n_out || (!out && cap)) return RT_ERR_INVALID_ARGUMENT;
    if (!page) {
        long os_page = sysconf(_SC_PAGESIZE);
        page = os_page > 0 ? (uint64_t)os_page : 4096;
    }
    std::vector<rt_id_range> ranges;
    const char *why = rt::expand_plan_line(registry, n_alloc, generation, line, page, ranges);
    if (error) *error = why;
    *n_out = 0;
    if (why) return RT_ERR_PLAN;
    *n_out = ranges.size();
    size_t n = ranges.size() < cap ? ranges.size() : cap;
    if (n) memcpy(out, ranges.data(), n * sizeof(rt_id_range));
    return ranges.size() > cap ? RT_ERR_CAPACITY : RT_OK;
}

}  // extern "C"
