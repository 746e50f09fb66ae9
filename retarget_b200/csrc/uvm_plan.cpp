// Plan-command expander.  Behaviour (word limits, validation order, error
// strings, range order) follows the command handler of the reference preload
// library, select.cpp:24045-24309; the structure here is a table-driven parser
// over an array snapshot of the registry rather than a walk of its linked list.
#include "uvm_plan.h"

#include <cstring>
#include <string>

namespace rt {
namespace {

struct Word {
    const char *p;
    size_t n;
    bool is(const char *s) const { return strlen(s) == n && !memcmp(p, s, n); }
};

// select.cpp:24047-24054: space, tab and CR separate words; a ninth word is an error.
int split(const char *line, Word words[8]) {
    int count = 0;
    const char *p = line;
    while (*p) {
        while (*p == ' ' || *p == '\t' || *p == '\r') ++p;
        if (!*p) break;
        const char *b = p;
        while (*p && *p != ' ' && *p != '\t' && *p != '\r') ++p;
        if (count == 8) return -1;
        words[count].p = b;
        words[count].n = (size_t)(p - b);
        ++count;
    }
    return count;
}

struct Emitter {
    std::vector<rt_id_range> &out;
    void operator()(const rt_alloc_info &a, uint64_t offset, uint64_t bytes, int32_t dst) {
        if (!bytes) return;                      // select.cpp:23927
        rt_id_range r;
        r.id = a.id;
        r.offset = offset;
        r.bytes = bytes;
        r.dst = dst;
        r.reserved = 0;
        out.push_back(r);
    }
};

int hex_value(char ch) {
    if (ch >= '0' && ch <= '9') return ch - '0';
    if (ch >= 'a' && ch <= 'f') return ch - 'a' + 10;
    return -1;
}

// select.cpp:24147-24195
const char *blocks_plan(const rt_alloc_info *reg, size_t n, uint64_t generation, uint64_t gen,
                        uint64_t alloc_bytes, uint64_t count, uint64_t block_bytes, Word mask,
                        uint64_t page, Emitter emit) {
    if (gen != generation) return "stale_allocations";
    if (!alloc_bytes || !block_bytes || block_bytes > alloc_bytes || block_bytes % page || !count)
        return "invalid_block_geometry";
    if (!mask.n || mask.n > 256) return "invalid_block_mask";
    const uint64_t whole = alloc_bytes / block_bytes;
    const uint64_t n_blocks = whole + (alloc_bytes % block_bytes != 0);
    // bit i of the mask = hex digit i/4 counted from the END of the text
    bool bits[RT_MAX_BLOCKS] = {false};
    bool any = false;
    for (size_t d = 0; d < mask.n; ++d) {
        int v = hex_value(mask.p[mask.n - 1 - d]);
        if (v < 0) return "invalid_block_mask";
        bool beyond = false;
        for (unsigned bit = 0; bit < 4; ++bit)
            if (v & (1 << bit)) {
                any = true;
                if (d * 4 + bit >= n_blocks) beyond = true;
                else bits[d * 4 + bit] = true;
            }
        if (beyond) return "block_out_of_range";
    }
    if (!any) return "empty_block_mask";
    uint64_t matched = 0;
    for (size_t i = 0; i < n; ++i) {
        if (reg[i].bytes != alloc_bytes) continue;
        ++matched;
        if (!reg[i].concurrent) return "concurrent_managed_access_required";
    }
    if (matched != count) return "cache_allocation_count_mismatch";
    for (size_t i = 0; i < n; ++i) {
        if (reg[i].bytes != alloc_bytes) continue;
        // the mask has at most 1024 bits; an allocation may have more blocks than that
        const uint64_t scan_end = n_blocks < RT_MAX_BLOCKS ? n_blocks : RT_MAX_BLOCKS;
        uint64_t b = 0;
        while (b < scan_end) {
            if (!bits[b]) { ++b; continue; }
            uint64_t e = b;
            while (e < scan_end && bits[e]) ++e;
            // a run that reaches the partial last block ends at the allocation end
            uint64_t end_byte = e > whole ? alloc_bytes : e * block_bytes;
            emit(reg[i], b * block_bytes, end_byte - b * block_bytes, reg[i].device);
            b = e;
        }
    }
    return nullptr;
}

bool window_ok(uint64_t lo, uint64_t hi, uint64_t alloc_bytes, uint64_t page) {
    return lo <= hi && hi <= alloc_bytes && lo % page == 0 && (hi == alloc_bytes || hi % page == 0);
}

// select.cpp:24196-24249
const char *window_plan(const rt_alloc_info *reg, size_t n, uint64_t generation, uint64_t gen,
                        uint64_t alloc_bytes, uint64_t count, uint64_t ob, uint64_t oe, uint64_t nb,
                        uint64_t ne, bool refresh, uint64_t page, Emitter emit) {
    const bool initial = ob == UINT64_MAX && oe == UINT64_MAX;
    if (gen != generation) return "stale_allocations";
    if (!alloc_bytes || !count || !window_ok(nb, ne, alloc_bytes, page) ||
        (!initial && !window_ok(ob, oe, alloc_bytes, page)))
        return "invalid_window";
    uint64_t matched = 0;
    for (size_t i = 0; i < n; ++i) {
        const bool cache = reg[i].bytes == alloc_bytes;
        if (cache) ++matched;
        if ((initial || cache) && !reg[i].concurrent) return "concurrent_managed_access_required";
    }
    if (matched != count) return "cache_allocation_count_mismatch";
    const bool whole = initial || refresh;
    for (int to_gpu = 0; to_gpu < 2; ++to_gpu) {          // everything CPU-bound first
        for (size_t i = 0; i < n; ++i) {
            const rt_alloc_info &a = reg[i];
            if (a.bytes != alloc_bytes) {
                if (initial && to_gpu) emit(a, 0, a.bytes, a.device);
                continue;
            }
            const int32_t dst = to_gpu ? a.device : RT_DST_CPU;
            if (whole) {
                if (to_gpu) {
                    emit(a, nb, ne - nb, dst);
                } else {
                    emit(a, 0, nb, dst);
                    emit(a, ne, alloc_bytes - ne, dst);
                }
                continue;
            }
            // pieces of (src) not covered by (other): src = old when evicting, new when growing
            const uint64_t sb = to_gpu ? nb : ob, se = to_gpu ? ne : oe;
            const uint64_t tb = to_gpu ? ob : nb, te = to_gpu ? oe : ne;
            uint64_t hi = se < tb ? se : tb;
            if (hi > sb) emit(a, sb, hi - sb, dst);
            uint64_t lo = sb > te ? sb : te;
            if (se > lo) emit(a, lo, se - lo, dst);
        }
    }
    return nullptr;
}

// Prefix-split alignment walk shared by target/targetv/retarget.
const char *check_prefix(const rt_alloc_info *reg, size_t n, uint64_t target, uint64_t page) {
    uint64_t remaining = target;
    for (size_t i = 0; i < n; ++i) {
        uint64_t gpu = remaining > reg[i].bytes ? reg[i].bytes : remaining;
        remaining -= gpu;
        if (gpu != reg[i].bytes && gpu % page) return "unaligned_target";
        if (!reg[i].concurrent) return "concurrent_managed_access_required";
    }
    return nullptr;
}

uint64_t managed_bytes(const rt_alloc_info *reg, size_t n) {
    uint64_t total = 0;
    for (size_t i = 0; i < n; ++i) total += reg[i].bytes;
    return total;
}

// select.cpp:24281-24309
const char *target_plan(const rt_alloc_info *reg, size_t n, uint64_t generation, bool versioned,
                        uint64_t gen, uint64_t bytes, uint64_t page, Emitter emit) {
    if (versioned && gen != generation) return "stale_allocations";
    if (bytes > managed_bytes(reg, n)) return "target_exceeds_managed_bytes";
    if (const char *e = check_prefix(reg, n, bytes, page)) return e;
    for (int to_gpu = 0; to_gpu < 2; ++to_gpu) {
        uint64_t remaining = bytes;
        for (size_t i = 0; i < n; ++i) {
            uint64_t gpu = remaining > reg[i].bytes ? reg[i].bytes : remaining;
            remaining -= gpu;
            if (to_gpu) emit(reg[i], 0, gpu, reg[i].device);
            else emit(reg[i], gpu, reg[i].bytes - gpu, RT_DST_CPU);
        }
    }
    return nullptr;
}

// select.cpp:24250-24280
const char *retarget_plan(const rt_alloc_info *reg, size_t n, uint64_t generation, uint64_t gen,
                          uint64_t old_target, uint64_t new_target, uint64_t page, Emitter emit) {
    if (gen != generation) return "stale_allocations";
    const uint64_t managed = managed_bytes(reg, n);
    if (old_target > managed || new_target > managed) return "target_exceeds_managed_bytes";
    if (const char *e = check_prefix(reg, n, old_target, page)) return e;
    if (const char *e = check_prefix(reg, n, new_target, page)) return e;
    if (old_target == new_target) return nullptr;
    const bool grow = new_target > old_target;
    const uint64_t lower = grow ? old_target : new_target, upper = grow ? new_target : old_target;
    uint64_t base = 0;
    for (size_t i = 0; i < n; ++i) {
        uint64_t end = base + reg[i].bytes;
        uint64_t lo = lower > base ? lower : base, hi = upper < end ? upper : end;
        if (hi > lo) emit(reg[i], lo - base, hi - lo, grow ? reg[i].device : RT_DST_CPU);
        base = end;
    }
    return nullptr;
}

// select.cpp:24136-24146
const char *prefetch_plan(const rt_alloc_info *reg, size_t n, uint64_t id, uint64_t offset,
                          uint64_t bytes, bool to_cpu, uint64_t page, Emitter emit) {
    const rt_alloc_info *a = nullptr;
    for (size_t i = 0; i < n && !a; ++i)
        if (reg[i].id == id) a = &reg[i];
    if (!a) return "unknown_id";
    if (!bytes || offset >= a->bytes || bytes > a->bytes - offset) return "invalid_range";
    if (offset % page || (bytes % page && bytes != a->bytes - offset)) return "unaligned_range";
    if (!a->concurrent) return "concurrent_managed_access_required";
    emit(*a, offset, bytes, to_cpu ? RT_DST_CPU : a->device);
    return nullptr;
}

}  // namespace

bool parse_u64(const char *word, size_t len, uint64_t *out) {
    if (!len) return false;
    uint64_t v = 0;
    for (size_t i = 0; i < len; ++i) {
        char ch = word[i];
        if (ch < '0' || ch > '9') return false;
        uint64_t d = (uint64_t)(ch - '0');
        if (v > (UINT64_MAX - d) / 10) return false;
        v = v * 10 + d;
    }
    *out = v;
    return true;
}

const char *expand_plan_line(const rt_alloc_info *reg, size_t n, uint64_t generation,
                             const char *line, uint64_t page, std::vector<rt_id_range> &ranges) {
    ranges.clear();
    Word w[8];
    int count = split(line, w);
    if (count <= 0) return "invalid_command";
    // command name -> (word count, how many leading numeric arguments)
    static const struct { const char *name; int words; int numbers; } kCommands[] = {
        {"blocksv", 6, 4}, {"prefetch", 5, 3}, {"target", 2, 1}, {"targetv", 3, 2},
        {"retarget", 4, 3}, {"windowv", 8, 7}, {"windowfullv", 8, 7}};
    int which = -1;
    for (int i = 0; i < 7; ++i)
        if (count == kCommands[i].words && w[0].is(kCommands[i].name)) which = i;
    if (which < 0) return "invalid_command";
    uint64_t v[7] = {0};
    for (int i = 0; i < kCommands[which].numbers; ++i)
        if (!parse_u64(w[1 + i].p, w[1 + i].n, &v[i])) return "invalid_command";
    if (which == 1 && !w[4].is("cpu") && !w[4].is("gpu")) return "invalid_command";
    Emitter emit{ranges};
    const char *err = nullptr;
    switch (which) {
        case 0: err = blocks_plan(reg, n, generation, v[0], v[1], v[2], v[3], w[5], page, emit); break;
        case 1: err = prefetch_plan(reg, n, v[0], v[1], v[2], w[4].is("cpu"), page, emit); break;
        case 2: err = target_plan(reg, n, generation, false, 0, v[0], page, emit); break;
        case 3: err = target_plan(reg, n, generation, true, v[0], v[1], page, emit); break;
        case 4: err = retarget_plan(reg, n, generation, v[0], v[1], v[2], page, emit); break;
        default:
            err = window_plan(reg, n, generation, v[0], v[1], v[2], v[3], v[4], v[5], v[6], which == 6,
                              page, emit);
    }
    if (err) ranges.clear();
    return err;
}

}  // namespace rt
