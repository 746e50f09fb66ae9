// The two scheduler-facing controllers as native state machines.
//
// Stands in for CacheWindowController (experiments/cache_window.py:71-148) and
// SlotPlacementController (experiments/slot_placement.py:55-162).  What talks
// to the outside world -- the Prometheus scrape, the control socket, the
// snapshot file -- stays with the caller; an update is therefore cut where the
// reference talks to the socket:
//
//   begin   gates and selection; says whether there is anything to send
//   plan    registry snapshot in, command line + accounting out
//   commit  the job has completed: the new state becomes current
//   fail    the job failed: forget, so that the next update starts over
//
// Every decision and every number is made here; a binding only moves data.
#include <algorithm>
#include <cinttypes>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <limits>
#include <map>
#include <new>
#include <string>
#include <vector>

#include "rt_internal.h"

namespace {

constexpr double kNever = -std::numeric_limits<double>::infinity();

struct Signature {
    std::vector<rt_alloc_info> cache;        // id, bytes, device of every cache allocation, registry order
    bool known = false;

    bool same(const std::vector<rt_alloc_info> &other) const {
        if (!known || cache.size() != other.size()) return false;
        for (size_t i = 0; i < cache.size(); ++i)
            if (cache[i].id != other[i].id || cache[i].bytes != other[i].bytes || cache[i].device != other[i].device)
                return false;
        return true;
    }
};

// cache allocations of a registry snapshot: the ones whose size is the spec's
std::vector<rt_alloc_info> cache_of(const rt_alloc_info *allocs, size_t n, uint64_t allocation_bytes,
                                    uint64_t *other_bytes) {
    std::vector<rt_alloc_info> cache;
    uint64_t other = 0;
    for (size_t i = 0; i < n; ++i) {
        if (allocs[i].bytes == allocation_bytes) cache.push_back(allocs[i]);
        else other += allocs[i].bytes;
    }
    if (other_bytes) *other_bytes = other;
    return cache;
}

}  // namespace

// ---------------------------------------------------------------------------
// window controller
// ---------------------------------------------------------------------------
struct rt_window_controller {
    rt_window_spec spec;
    bool has_current = false;
    uint64_t current[2] = {0, 0};
    Signature signature;
    double last_update = kNever;
    double highwater = 0.0;
    // between begin and commit
    bool armed = false, planned = false, initial = false;
    uint64_t window[2] = {0, 0};
    std::vector<rt_alloc_info> next_signature;
};

namespace {

enum { kHasPrompt = 1, kHasGeneration = 2, kHasRunning = 4, kHasQueue = 8 };

// _counters, experiments/cache_window.py:79-87
int completed_tokens(rt_window_controller *c, const rt_metrics *m, double *completed) {
    if ((m->present & (kHasPrompt | kHasGeneration)) != (kHasPrompt | kHasGeneration))
        return RT_ERR_METRICS_MISSING;
    const double v[2] = {m->prompt_tokens_total, m->generation_tokens_total};
    for (double x : v)
        if (!std::isfinite(x) || x < 0) return RT_ERR_METRICS_INVALID;
    const double sum = 0.0 + v[0] + v[1];
    if (sum > c->highwater) c->highwater = sum;
    *completed = c->highwater;
    return RT_OK;
}

bool same_window(const rt_window_controller *c, const uint64_t w[2]) {
    return c->has_current && c->current[0] == w[0] && c->current[1] == w[1];
}

}  // namespace

extern "C" {

int rt_window_controller_create(const rt_window_spec *spec, rt_window_controller **out) {
    if (!spec || !out) return RT_ERR_INVALID_ARGUMENT;
    *out = nullptr;
    int st = rt_window_spec_check(spec, nullptr);
    if (st != RT_OK) return st;
    rt_window_controller *c = new (std::nothrow) rt_window_controller();
    if (!c) return RT_ERR_OUT_OF_MEMORY;
    c->spec = *spec;
    *out = c;
    return RT_OK;
}

int rt_window_controller_destroy(rt_window_controller *c) {
    delete c;
    return RT_OK;
}

// due, experiments/cache_window.py:142-148.  1 / 0, or a negative status.
int rt_window_controller_due(rt_window_controller *c, const rt_metrics *m, double now) {
    if (!c || !m) return RT_ERR_INVALID_ARGUMENT;
    if (c->spec.update_mode == 1) return 0;                       // initial_only
    double completed;
    int st = completed_tokens(c, m, &completed);
    if (st != RT_OK) return st;
    uint64_t w[2];
    if ((st = rt_window(&c->spec, completed, w)) != RT_OK) return st;
    if (same_window(c, w)) return 0;
    if (!(now - c->last_update >= c->spec.min_update_seconds)) return 0;
    if (!c->spec.idle_only) return 1;
    if (!(m->present & kHasRunning)) return RT_ERR_METRICS_KEY_RUNNING;
    if (!(m->num_running_reqs == 0)) return 0;
    if (!(m->present & kHasQueue)) return RT_ERR_METRICS_KEY_QUEUE;
    return m->num_queue_reqs == 0 ? 1 : 0;
}

// update up to the first socket call, experiments/cache_window.py:90-100.
// 1: go on (wait for idle, take the registry snapshot, call _plan); 0: nothing to do.
int rt_window_controller_begin(rt_window_controller *c, const rt_metrics *m, double now, int initial) {
    if (!c || !m) return RT_ERR_INVALID_ARGUMENT;
    c->armed = c->planned = false;
    double completed;
    int st = completed_tokens(c, m, &completed);
    if (st != RT_OK) return st;
    uint64_t w[2];
    if ((st = rt_window(&c->spec, completed, w)) != RT_OK) return st;
    if (!initial) {
        if (c->spec.update_mode == 1) return 0;
        if (same_window(c, w) || now - c->last_update < c->spec.min_update_seconds) return 0;
        if (c->spec.idle_only) {
            if (!(m->present & kHasRunning)) return RT_ERR_METRICS_KEY_RUNNING;
            if (m->num_running_reqs > 0) return 0;
            if (!(m->present & kHasQueue)) return RT_ERR_METRICS_KEY_QUEUE;
            if (m->num_queue_reqs > 0) return 0;
        }
    }
    c->window[0] = w[0];
    c->window[1] = w[1];
    c->initial = initial != 0;
    c->armed = true;
    return 1;
}

// registry snapshot -> command and accounting, experiments/cache_window.py:102-113,122-131
int rt_window_controller_plan(rt_window_controller *c, const rt_alloc_info *allocs, size_t n,
                              uint64_t generation, char *command, size_t cap, rt_window_update *out) {
    if (!c || (!allocs && n) || !command || !cap || !out) return RT_ERR_INVALID_ARGUMENT;
    if (!c->armed) return RT_ERR_INVALID_ARGUMENT;
    uint64_t other = 0;
    std::vector<rt_alloc_info> cache = cache_of(allocs, n, c->spec.allocation_bytes, &other);
    memset(out, 0, sizeof(*out));
    out->cache_count = cache.size();
    if (cache.size() != c->spec.allocation_count) return RT_ERR_LAYOUT_MISMATCH;
    const bool full = c->initial || !c->signature.same(cache) || !c->has_current;
    const bool refresh = !full && c->spec.update_mode == 2;       // full_cache
    const uint64_t old0 = full ? RT_INITIAL : c->current[0], old1 = full ? RT_INITIAL : c->current[1];
    int len = snprintf(command, cap, "%s %" PRIu64 " %" PRIu64 " %" PRIu64 " %" PRIu64 " %" PRIu64 " %" PRIu64 " %" PRIu64,
                       refresh ? "windowfullv" : "windowv", generation, c->spec.allocation_bytes,
                       c->spec.allocation_count, old0, old1, c->window[0], c->window[1]);
    if (len < 0 || (size_t)len >= cap) return RT_ERR_CAPACITY;
    out->full = full;
    out->refresh = refresh;
    out->old_window[0] = old0;
    out->old_window[1] = old1;
    out->new_window[0] = c->window[0];
    out->new_window[1] = c->window[1];
    out->generation = generation;
    out->completed_highwater = c->highwater;
    const uint64_t old_pair[2] = {full ? 0 : old0, full ? 0 : old1};
    int st = rt_window_accounting(&c->spec, cache.size(), other, old_pair, c->window, full, refresh,
                                  &out->gpu_bytes, &out->cpu_bytes);
    if (st != RT_OK) return st;
    c->next_signature.swap(cache);
    c->planned = true;
    return RT_OK;
}

// experiments/cache_window.py:132
int rt_window_controller_commit(rt_window_controller *c, double now) {
    if (!c || !c->planned) return RT_ERR_INVALID_ARGUMENT;
    c->current[0] = c->window[0];
    c->current[1] = c->window[1];
    c->has_current = true;
    c->signature.cache.swap(c->next_signature);
    c->signature.known = true;
    c->last_update = now;
    c->armed = c->planned = false;
    return RT_OK;
}

// the job failed, experiments/cache_window.py:115-118
int rt_window_controller_fail(rt_window_controller *c) {
    if (!c) return RT_ERR_INVALID_ARGUMENT;
    c->signature.known = false;
    c->signature.cache.clear();
    c->has_current = false;
    c->armed = c->planned = false;
    return RT_OK;
}

int rt_window_controller_get(const rt_window_controller *c, rt_window_state *out) {
    if (!c || !out) return RT_ERR_INVALID_ARGUMENT;
    out->has_current = c->has_current;
    out->has_signature = c->signature.known;
    out->current[0] = c->current[0];
    out->current[1] = c->current[1];
    out->last_update = c->last_update;
    out->completed_highwater = c->highwater;
    out->signature_count = c->signature.cache.size();
    return RT_OK;
}

int rt_window_controller_set(rt_window_controller *c, const rt_window_state *in) {
    if (!c || !in) return RT_ERR_INVALID_ARGUMENT;
    c->has_current = in->has_current != 0;
    c->current[0] = in->current[0];
    c->current[1] = in->current[1];
    c->last_update = in->last_update;
    c->highwater = in->completed_highwater;
    return RT_OK;
}

int rt_window_controller_get_signature(const rt_window_controller *c, rt_alloc_info *out, size_t cap, size_t *n) {
    if (!c || !n || (!out && cap)) return RT_ERR_INVALID_ARGUMENT;
    *n = c->signature.cache.size();
    if (!c->signature.known) return 1;                            // no signature on record
    if (*n > cap) return RT_ERR_CAPACITY;
    std::copy(c->signature.cache.begin(), c->signature.cache.end(), out);
    return RT_OK;
}

int rt_window_controller_set_signature(rt_window_controller *c, const rt_alloc_info *sig, size_t n, int known) {
    if (!c || (!sig && n)) return RT_ERR_INVALID_ARGUMENT;
    c->signature.cache.assign(sig, sig + n);
    c->signature.known = known != 0;
    return RT_OK;
}

}  // extern "C"

// ---------------------------------------------------------------------------
// slot-placement controller
// ---------------------------------------------------------------------------
namespace {

struct Commit {
    int32_t version;
    double at;
};

// the part of a feedback snapshot the controller reads, copied (it outlives the call)
struct Snapshot {
    uint64_t epoch = 0;
    int64_t sequence = 0;
    double observed = 0;
    std::vector<int32_t> versions;
    std::vector<rt_block_stamp> reads, writes;
    std::vector<uint32_t> free_head;

    void take(const rt_snapshot_doc &s) {
        epoch = s.epoch;
        sequence = s.sequence;
        observed = s.observed_monotonic_s;
        versions.assign(s.block_versions, s.block_versions + s.n_versions);
        reads.assign(s.recent_reads, s.recent_reads + s.n_reads);
        writes.assign(s.recent_writes, s.recent_writes + s.n_writes);
        free_head.assign(s.free_head_blocks, s.free_head_blocks + s.n_free);
    }
};

bool snapshot_ok(const rt_snapshot_doc *s) {
    return s && (s->block_versions || !s->n_versions) && (s->recent_reads || !s->n_reads) &&
           (s->recent_writes || !s->n_writes) && (s->free_head_blocks || !s->n_free);
}

// target_blocks, experiments/slot_placement.py:37-44: recently active reads,
// recently active writes, the sampled free-list head, then everything by
// recency (stable: reads before writes among equal stamps); first mention
// wins; cut at the budget.
void rank_blocks(const Snapshot &s, const rt_slot_spec &spec, uint64_t budget, double now,
                 std::vector<uint32_t> *ranked) {
    ranked->clear();
    std::vector<uint32_t> order;
    order.reserve(2 * (s.reads.size() + s.writes.size()) + s.free_head.size());
    for (const rt_block_stamp &e : s.reads)
        if (now - e.t <= spec.active_seconds) order.push_back(e.block);
    for (const rt_block_stamp &e : s.writes)
        if (now - e.t <= spec.active_seconds) order.push_back(e.block);
    order.insert(order.end(), s.free_head.begin(), s.free_head.end());
    std::vector<rt_block_stamp> history(s.reads);
    history.insert(history.end(), s.writes.begin(), s.writes.end());
    std::stable_sort(history.begin(), history.end(),
                     [](const rt_block_stamp &a, const rt_block_stamp &b) { return -a.t < -b.t; });
    for (const rt_block_stamp &e : history) order.push_back(e.block);
    std::vector<uint32_t> seen_sorted;
    for (uint32_t b : order) {
        if (ranked->size() >= budget) break;
        auto at = std::lower_bound(seen_sorted.begin(), seen_sorted.end(), b);
        if (at != seen_sorted.end() && *at == b) continue;
        seen_sorted.insert(at, b);
        ranked->push_back(b);
    }
}

}  // namespace

struct rt_slot_controller {
    rt_window_controller window;          // the controller it extends: window state and signature
    rt_slot_spec spec;
    uint64_t pid = 0;
    uint64_t budget = 0;
    std::map<uint32_t, Commit> committed;
    bool has_epoch = false;
    uint64_t epoch = 0;
    double last_attempt = kNever;
    // between begin and commit
    bool armed = false, planned = false;
    double now = 0;
    Snapshot snap;
    std::vector<uint32_t> desired, selected;
    std::vector<rt_alloc_info> next_signature;
};

namespace {

// choose, experiments/slot_placement.py:83-94
int choose_blocks(const rt_slot_controller *c, const Snapshot &s, double now, std::vector<uint32_t> *desired,
                  std::vector<uint32_t> *selected) {
    rank_blocks(s, c->spec, c->budget, now, desired);
    selected->clear();
    for (uint32_t block : *desired) {
        if (block >= s.versions.size()) return RT_ERR_INVALID_ARGUMENT;   // the snapshot does not cover the block
        auto old = c->committed.find(block);
        bool todo = old == c->committed.end() || old->second.version != s.versions[block];
        if (!todo && now - old->second.at >= c->spec.refresh_seconds) {
            auto active = [&](const std::vector<rt_block_stamp> &list) {
                for (const rt_block_stamp &e : list)
                    if (e.block == block && now - e.t <= c->spec.active_seconds) return true;
                return false;
            };
            todo = active(s.reads) || active(s.writes);
        }
        if (todo && selected->size() < c->spec.max_blocks_per_update) selected->push_back(block);
    }
    return RT_OK;
}

}  // namespace

extern "C" {

// SlotPlacementSpec.__post_init__, experiments/slot_placement.py:28-34
int rt_slot_spec_check(const rt_slot_spec *s, int *bad_field) {
    if (!s) return RT_ERR_INVALID_ARGUMENT;
    const uint64_t ints[3] = {s->block_tokens, s->lookahead_tokens, s->max_blocks_per_update};
    const int int_field[3] = {0, 1, 3};
    for (int k = 0; k < 3; ++k)
        if (!ints[k] || ints[k] >= (1ull << 63)) {
            if (bad_field) *bad_field = int_field[k];
            return RT_ERR_SLOT_SPEC;
        }
    const double reals[4] = {s->min_update_seconds, s->active_seconds, s->refresh_seconds,
                             s->max_feedback_lag_seconds};
    const int real_field[4] = {2, 4, 5, 6};
    for (int k = 0; k < 4; ++k)
        if (!std::isfinite(reals[k]) || reals[k] <= 0) {
            if (bad_field) *bad_field = real_field[k];
            return RT_ERR_SLOT_SPEC;
        }
    return RT_OK;
}

int rt_target_blocks(const rt_snapshot_doc *snapshot, const rt_slot_spec *spec, uint64_t budget, double now,
                     uint32_t *out, size_t cap, size_t *n) {
    if (!snapshot_ok(snapshot) || !spec || !n || (!out && cap)) return RT_ERR_INVALID_ARGUMENT;
    Snapshot s;
    s.take(*snapshot);
    std::vector<uint32_t> ranked;
    rank_blocks(s, *spec, budget, now, &ranked);
    *n = ranked.size();
    if (ranked.size() > cap) return RT_ERR_CAPACITY;
    std::copy(ranked.begin(), ranked.end(), out);
    return RT_OK;
}

// __init__, experiments/slot_placement.py:56-67
int rt_slot_controller_create(const rt_window_spec *cache_spec, const rt_slot_spec *slot_spec, uint64_t pid,
                              rt_slot_controller **out) {
    if (!cache_spec || !slot_spec || !out) return RT_ERR_INVALID_ARGUMENT;
    *out = nullptr;
    int st = rt_window_spec_check(cache_spec, nullptr);
    if (st == RT_OK) st = rt_slot_spec_check(slot_spec, nullptr);
    uint64_t budget = 0;
    if (st == RT_OK) st = rt_slot_budget(cache_spec, slot_spec->block_tokens, &budget);
    if (st != RT_OK) return st;
    rt_slot_controller *c = new (std::nothrow) rt_slot_controller();
    if (!c) return RT_ERR_OUT_OF_MEMORY;
    c->window.spec = *cache_spec;
    c->spec = *slot_spec;
    c->pid = pid;
    c->budget = budget;
    *out = c;
    return RT_OK;
}

int rt_slot_controller_destroy(rt_slot_controller *c) {
    delete c;
    return RT_OK;
}

// the window controller inside: borrowed, lives as long as `c`
rt_window_controller *rt_slot_controller_window(rt_slot_controller *c) { return c ? &c->window : nullptr; }

uint64_t rt_slot_controller_budget(const rt_slot_controller *c) { return c ? c->budget : 0; }

// the checks of snapshot(), experiments/slot_placement.py:74-78.
// 1: usable; 0: too old to act on; RT_ERR_FEEDBACK_IDENTITY: not ours.
int rt_slot_controller_accept(const rt_slot_controller *c, const rt_snapshot_doc *s) {
    if (!c || !snapshot_ok(s)) return RT_ERR_INVALID_ARGUMENT;
    if (s->pid != c->pid || s->block_tokens != c->spec.block_tokens) return RT_ERR_FEEDBACK_IDENTITY;
    const double lag = s->published_monotonic_s - s->observed_monotonic_s;
    return lag > c->spec.max_feedback_lag_seconds ? 0 : 1;
}

int rt_slot_controller_choose(const rt_slot_controller *c, const rt_snapshot_doc *snapshot, double now,
                              uint32_t *desired, size_t cap_desired, size_t *n_desired, uint32_t *selected,
                              size_t cap_selected, size_t *n_selected) {
    if (!c || !snapshot_ok(snapshot) || !n_desired || !n_selected) return RT_ERR_INVALID_ARGUMENT;
    Snapshot s;
    s.take(*snapshot);
    std::vector<uint32_t> d, sel;
    int st = choose_blocks(c, s, now, &d, &sel);
    if (st != RT_OK) return st;
    *n_desired = d.size();
    *n_selected = sel.size();
    if (d.size() > cap_desired || sel.size() > cap_selected) return RT_ERR_CAPACITY;
    if (desired) std::copy(d.begin(), d.end(), desired);
    if (selected) std::copy(sel.begin(), sel.end(), selected);
    return RT_OK;
}

// due, experiments/slot_placement.py:96-104.  `snapshot` is NULL when there is
// none to act on (no file yet, or accept() said 0).
int rt_slot_controller_due(const rt_slot_controller *c, const rt_snapshot_doc *snapshot, double now) {
    if (!c) return RT_ERR_INVALID_ARGUMENT;
    if (now - c->last_attempt < c->spec.min_update_seconds) return 0;
    if (!snapshot) return 0;
    if (!snapshot_ok(snapshot)) return RT_ERR_INVALID_ARGUMENT;
    if (!c->has_epoch || c->epoch != snapshot->epoch) return 1;
    Snapshot s;
    s.take(*snapshot);
    std::vector<uint32_t> d, sel;
    int st = choose_blocks(c, s, now, &d, &sel);
    if (st != RT_OK) return st;
    return sel.empty() ? 0 : 1;
}

// whether an update would be attempted at all (the first line of due())
int rt_slot_controller_attempt_allowed(const rt_slot_controller *c, double now) {
    if (!c) return RT_ERR_INVALID_ARGUMENT;
    return now - c->last_attempt < c->spec.min_update_seconds ? 0 : 1;
}

// update up to the first socket call, experiments/slot_placement.py:119-132
int rt_slot_controller_begin(rt_slot_controller *c, const rt_snapshot_doc *snapshot, double now) {
    if (!c) return RT_ERR_INVALID_ARGUMENT;
    c->armed = c->planned = false;
    c->last_attempt = now;
    if (!snapshot) return 0;
    if (!snapshot_ok(snapshot)) return RT_ERR_INVALID_ARGUMENT;
    if (!c->has_epoch || c->epoch != snapshot->epoch) {
        c->committed.clear();
        c->epoch = snapshot->epoch;
        c->has_epoch = true;
    }
    c->snap.take(*snapshot);
    c->now = now;
    int st = choose_blocks(c, c->snap, now, &c->desired, &c->selected);
    if (st != RT_OK) return st;
    if (c->selected.empty()) return 0;
    c->armed = true;
    return 1;
}

// registry snapshot -> blocksv command, experiments/slot_placement.py:133-139,154
int rt_slot_controller_plan(rt_slot_controller *c, const rt_alloc_info *allocs, size_t n, uint64_t generation,
                            char *command, size_t cap, rt_slot_update *out) {
    if (!c || (!allocs && n) || !command || !cap || !out || !c->armed) return RT_ERR_INVALID_ARGUMENT;
    const rt_window_spec &w = c->window.spec;
    std::vector<rt_alloc_info> cache = cache_of(allocs, n, w.allocation_bytes, nullptr);
    memset(out, 0, sizeof(*out));
    out->cache_count = cache.size();
    if (cache.size() != w.allocation_count) return RT_ERR_LAYOUT_MISMATCH;
    if (!c->window.signature.same(cache)) {
        // another set of cache allocations: nothing of the record applies to it
        c->committed.clear();
        c->window.signature.cache = cache;
        c->window.signature.known = true;
        int st = choose_blocks(c, c->snap, c->now, &c->desired, &c->selected);
        if (st != RT_OK) return st;
    }
    const uint64_t block_bytes = c->spec.block_tokens * w.bytes_per_token;
    std::vector<char> mask(c->selected.empty() ? 2 : *std::max_element(c->selected.begin(), c->selected.end()) / 4 + 3);
    int st = rt_encode_mask(c->selected.data(), c->selected.size(), mask.data(), mask.size());
    if (st < 0) return st;
    int len = snprintf(command, cap, "blocksv %" PRIu64 " %" PRIu64 " %" PRIu64 " %" PRIu64 " %s", generation,
                       w.allocation_bytes, w.allocation_count, block_bytes, mask.data());
    if (len < 0 || (size_t)len >= cap) return RT_ERR_CAPACITY;
    uint64_t covered = 0;
    for (uint32_t b : c->selected) {
        const uint64_t left = w.allocation_bytes - (uint64_t)b * block_bytes;
        covered += block_bytes < left ? block_bytes : left;
    }
    out->generation = generation;
    out->epoch = c->epoch;
    out->sequence = c->snap.sequence;
    out->observed_monotonic_s = c->snap.observed;
    out->gpu_bytes = covered * cache.size();
    out->n_desired = c->desired.size();
    out->n_selected = c->selected.size();
    c->planned = true;
    return RT_OK;
}

// desired / selected of the update in progress (valid after begin / plan)
int rt_slot_controller_pending(const rt_slot_controller *c, uint32_t *desired, size_t cap_desired,
                               uint32_t *selected, size_t cap_selected) {
    if (!c || !c->armed) return RT_ERR_INVALID_ARGUMENT;
    if (c->desired.size() > cap_desired || c->selected.size() > cap_selected) return RT_ERR_CAPACITY;
    if (desired) std::copy(c->desired.begin(), c->desired.end(), desired);
    if (selected) std::copy(c->selected.begin(), c->selected.end(), selected);
    return RT_OK;
}

// the job has completed, experiments/slot_placement.py:149-153
int rt_slot_controller_commit(rt_slot_controller *c, double commit_time) {
    if (!c || !c->planned) return RT_ERR_INVALID_ARGUMENT;
    std::map<uint32_t, Commit> kept;
    for (uint32_t b : c->desired) {
        auto at = c->committed.find(b);
        if (at != c->committed.end()) kept.insert(*at);
    }
    for (uint32_t b : c->selected) kept[b] = Commit{c->snap.versions[b], commit_time};
    c->committed.swap(kept);
    c->window.last_update = commit_time;
    c->armed = c->planned = false;
    return RT_OK;
}

// rejected command or failed job, experiments/slot_placement.py:140-147
int rt_slot_controller_fail(rt_slot_controller *c) {
    if (!c) return RT_ERR_INVALID_ARGUMENT;
    c->committed.clear();
    c->armed = c->planned = false;
    return RT_OK;
}

// after the initial window plan, experiments/slot_placement.py:107-118: the
// blocks of the window are on record with the snapshot's versions
int rt_slot_controller_seed(rt_slot_controller *c, const rt_snapshot_doc *snapshot, double commit_time) {
    if (!c || !snapshot_ok(snapshot) || !c->window.has_current) return RT_ERR_INVALID_ARGUMENT;
    const uint64_t unit = c->spec.block_tokens * c->window.spec.bytes_per_token;
    const uint64_t first = c->window.current[0] / unit, last = c->window.current[1] / unit;
    if (last > snapshot->n_versions) return RT_ERR_INVALID_ARGUMENT;
    c->epoch = snapshot->epoch;
    c->has_epoch = true;
    c->committed.clear();
    for (uint64_t b = first; b < last; ++b) c->committed[(uint32_t)b] = Commit{snapshot->block_versions[b], commit_time};
    return RT_OK;
}

int rt_slot_controller_get(const rt_slot_controller *c, rt_slot_state *out) {
    if (!c || !out) return RT_ERR_INVALID_ARGUMENT;
    out->has_epoch = c->has_epoch;
    out->epoch = c->epoch;
    out->last_attempt = c->last_attempt;
    out->committed_count = c->committed.size();
    return RT_OK;
}

int rt_slot_controller_set(rt_slot_controller *c, const rt_slot_state *in) {
    if (!c || !in) return RT_ERR_INVALID_ARGUMENT;
    c->has_epoch = in->has_epoch != 0;
    c->epoch = in->epoch;
    c->last_attempt = in->last_attempt;
    return RT_OK;
}

int rt_slot_controller_get_committed(const rt_slot_controller *c, rt_block_commit *out, size_t cap, size_t *n) {
    if (!c || !n || (!out && cap)) return RT_ERR_INVALID_ARGUMENT;
    *n = c->committed.size();
    if (*n > cap) return RT_ERR_CAPACITY;
    size_t k = 0;
    for (const auto &e : c->committed) out[k++] = rt_block_commit{e.first, e.second.version, e.second.at};
    return RT_OK;
}

int rt_slot_controller_set_committed(rt_slot_controller *c, const rt_block_commit *in, size_t n) {
    if (!c || (!in && n)) return RT_ERR_INVALID_ARGUMENT;
    c->committed.clear();
    for (size_t k = 0; k < n; ++k) c->committed[in[k].block] = Commit{in[k].version, in[k].at};
    return RT_OK;
}

}  // extern "C"
