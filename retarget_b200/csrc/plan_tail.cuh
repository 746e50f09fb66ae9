// Plan tail: wanted bitmaps -> budget cut -> diff against the resident set ->
// coalesced byte ranges in queue order.  Runs in ONE CTA (the one that retired
// the last scan unit, or the single CTA of the bitmap-only kernel) and is laid
// out to keep dependent global round trips off the critical path: one parallel
// load of every bitmap's wanted + resident words, everything else in shared
// memory, then the range stores.
#pragma once
#include "plan_device.cuh"

namespace rt {

#ifdef RT_TRACE
static __device__ unsigned long long g_tail_trace[8];
#define RT_TAIL_MARK(k)                                                          \
    do {                                                                         \
        if (threadIdx.x == 0) {                                                  \
            unsigned long long t__;                                              \
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t__));             \
            g_tail_trace[k] = t__;                                               \
        }                                                                        \
    } while (0)
#else
#define RT_TAIL_MARK(k)
#endif

// --------------------------------------------------------------------------
// small warp helpers
// --------------------------------------------------------------------------
__device__ __forceinline__ uint32_t warp_inclusive_sum(uint32_t v, uint32_t lane) {
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        uint32_t n = __shfl_up_sync(0xffffffffu, v, d);
        if (lane >= (uint32_t)d) v += n;
    }
    return v;
}

__device__ __forceinline__ uint32_t warp_sum(uint32_t v) {
    return __reduce_add_sync(0xffffffffu, v);
}

// Lowest `k` set bits of x: binary search for the shortest low mask that holds
// k set bits (six steps of popc; __fns is emulated in software and much slower).
__device__ __forceinline__ uint32_t lowest_bits(uint32_t x, uint32_t k) {
    if (k >= (uint32_t)__popc(x)) return x;
    uint32_t lo = 0, hi = 32;                        // mask width
    while (lo < hi) {
        uint32_t mid = (lo + hi) >> 1;
        uint32_t have = __popc(x & (mid >= 32 ? 0xffffffffu : ((1u << mid) - 1u)));
        if (have >= k) hi = mid; else lo = mid + 1;
    }
    return x & (lo >= 32 ? 0xffffffffu : ((1u << lo) - 1u));
}

// --------------------------------------------------------------------------
// CTA-scope barriers.  The TMA kernel keeps a producer warp out of the
// consumers' barriers, so those go through a named barrier of kThreads threads.
// --------------------------------------------------------------------------
template <int kBar, int kThreads>
__device__ __forceinline__ void cta_sync() {
    if (kBar == 0) __syncthreads();
    else asm volatile("bar.sync %0, %1;" ::"n"(kBar), "n"(kThreads) : "memory");
}

template <int kBar, int kThreads>
__device__ __forceinline__ bool cta_or(bool pred) {
    if (kBar == 0) return __syncthreads_or(pred);
    uint32_t r;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.u32 p, %1, 0;\n\t"
        "bar.red.or.pred q, %2, %3, p;\n\t"
        "selp.u32 %0, 1, 0, q;\n\t}"
        : "=r"(r)
        : "r"((uint32_t)pred), "n"(kBar), "n"(kThreads)
        : "memory");
    return r != 0;
}

// --------------------------------------------------------------------------
// shared-memory layout of the tail (carved from a raw, 16-byte aligned buffer)
// --------------------------------------------------------------------------
constexpr int kTailWarps = kScanThreads / 32;
// Words per bitmap in the tail's shared staging: [evict|want][add|resident] plus
// one word of padding, so that thread-per-bitmap accesses fall in different banks.
constexpr uint32_t kMaskStride = 2 * kWords + 1;

struct TailShared {
    unsigned long long *bytes;   // [2]   CPU-bound / GPU-bound byte totals
    uint32_t *stats;             // [8]   touched, desired, added, evicted, [4] = some bitmap has runs
    uint32_t *warp_tot;          // [kTailWarps]
    uint32_t *counts;            // [n_groups][2]        runs per (bitmap, phase)
    uint32_t *off;               // [2*n_buffers + 1]    first range of every (phase, buffer)
    uint32_t *masks;             // [n_groups][kMaskStride] evict / add words
    uint16_t *stage;             // [kTailWarps][2][kMaxRuns] run begin / end per warp
};

__host__ __device__ constexpr size_t tail_smem_bytes(uint32_t n_groups, uint32_t n_buffers) {
    return ((4 + 8 + kTailWarps + 2 * (size_t)n_groups + (2 * (size_t)n_buffers + 1) +
             (size_t)kMaskStride * n_groups) * 4 +
            (size_t)kTailWarps * 2 * kMaxRuns * 2 + 15) & ~(size_t)15;
}

__device__ __forceinline__ TailShared carve_tail(unsigned char *raw, uint32_t n_groups, uint32_t n_buffers) {
    TailShared s;
    uint32_t *w = reinterpret_cast<uint32_t *>(raw);
    s.bytes = reinterpret_cast<unsigned long long *>(w);  w += 4;
    s.stats = w;                                           w += 8;
    s.warp_tot = w;                                        w += kTailWarps;
    s.counts = w;                                          w += 2 * n_groups;
    s.off = w;                                             w += 2 * n_buffers + 1;
    s.masks = w;                                           w += kMaskStride * n_groups;
    s.stage = reinterpret_cast<uint16_t *>(w);
    return s;
}

// First and last bits of every run of set bits; lane = word index.
__device__ __forceinline__ void run_edges(uint32_t m, uint32_t lane, uint32_t &starts, uint32_t &lasts) {
    uint32_t prev_top = __shfl_up_sync(0xffffffffu, m, 1) >> 31;
    uint32_t next_low = __shfl_down_sync(0xffffffffu, m, 1) & 1u;
    if (lane == 0) prev_top = 0;
    if (lane == 31) next_low = 0;
    starts = m & ~((m << 1) | prev_top);
    lasts = m & ~((m >> 1) | (next_low << 31));
}

// --------------------------------------------------------------------------
// the tail itself: kScanThreads threads of one CTA
// --------------------------------------------------------------------------
// `want` holds n_groups x kWords words; `consume` zeroes them after reading
// (they are the scan's accumulation words).
template <int kBar>
__device__ void plan_tail(const PlanArgs &p, uint32_t *want, bool consume, unsigned char *raw) {
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t G = p.n_groups, n = p.n_buffers;
    const TailShared sh = carve_tail(raw, G, n);
    RT_TAIL_MARK(0);
    if (tid < 8) sh.stats[tid] = 0;
    if (tid < 2) sh.bytes[tid] = 0;
    cta_sync<kBar, kScanThreads>();
    // counters written by other CTAs: fetched now, used at the very end
    unsigned long long invalid = 0, ignored = 0;
    uint32_t eflags = 0;
    if (tid == 0) {
        invalid = __ldcg(&p.global->invalid_slots);
        ignored = __ldcg(&p.global->ignored_slots);
        eflags = __ldcg(&p.global->error_flags);
    }
    // Stage every bitmap's wanted and resident words in shared memory with ONE
    // round trip (all loads in flight together); a load per loop iteration of
    // pass A would cost a dependent L2 round trip per bitmap.
    // Loads first (kBatch pairs per thread in flight at once), stores second: a
    // plain load-store loop would serialise one L2 round trip per iteration.
    constexpr uint32_t kBatch = 8;
    uint32_t resident_bits = 0;
    for (uint32_t base = 0; base < G * kWords; base += kBatch * kScanThreads) {
        uint32_t a_w[kBatch], b_w[kBatch];
#pragma unroll
        for (uint32_t k = 0; k < kBatch; ++k) {
            const uint32_t i = base + k * kScanThreads + tid;
            a_w[k] = b_w[k] = 0;
            if (i < G * kWords) {
                const uint32_t g = i / kWords, l = i % kWords;
                if (p.explicit_sets) {
                    a_w[k] = __ldcg(&want[(g * 2 + 0) * kWords + l]);
                    b_w[k] = __ldcg(&want[(g * 2 + 1) * kWords + l]);
                    resident_bits += __popc(__ldcg(&p.resident[i]));   // already the new set
                } else {
                    a_w[k] = __ldcg(&want[i]);
                    if (!p.scan_only) b_w[k] = __ldcg(&p.resident[i]);
                }
            }
        }
#pragma unroll
        for (uint32_t k = 0; k < kBatch; ++k) {
            const uint32_t i = base + k * kScanThreads + tid;
            if (i < G * kWords) {
                const uint32_t g = i / kWords, l = i % kWords;
                sh.masks[g * kMaskStride + l] = a_w[k];
                sh.masks[g * kMaskStride + kWords + l] = b_w[k];
                if (consume && !p.explicit_sets) want[i] = 0;
            }
        }
    }
    if (p.explicit_sets && resident_bits) atomicAdd(&sh.stats[1], resident_bits);
    cta_sync<kBar, kScanThreads>();
    RT_TAIL_MARK(1);

    // ---- pass A: one THREAD per bitmap, walking its words in order ----
    // A running count replaces the cross-lane prefix sums, the carry bit of the
    // previous word replaces the neighbour shuffles, and all bitmaps advance in
    // parallel (a warp per bitmap left 8 warps to do 40 bitmaps in 5 dependent
    // rounds and took 3.2 us; this takes a fraction of that).
    // Scalars of `p` are copied to locals first: `p` lives in parameter space and
    // every global store in the loop would otherwise force them to be re-read.
    const uint32_t n_blocks = p.n_blocks, budget = p.budget, flags = p.flags;
    const bool explicit_sets = p.explicit_sets != 0, scan_only = p.scan_only != 0;
    uint32_t *const resident = p.resident, *const bitmaps_out = p.bitmaps_out;
    const uint32_t n_words = (n_blocks + 31) / 32;
    uint32_t n_touched = 0, n_des = 0, n_add = 0, n_ev = 0, some_runs = 0;
    for (uint32_t g = tid; g < G; g += kScanThreads) {
        uint32_t *m = sh.masks + g * kMaskStride;
        uint32_t kept = 0, c_ev = 0, c_add = 0, carry_ev = 0, carry_add = 0;
        for (uint32_t w = 0; w < n_words; ++w) {
            const uint32_t left = n_blocks - w * 32;
            const uint32_t valid = left >= 32 ? 0xffffffffu : ((1u << left) - 1u);
            uint32_t evict, add, desired;
            if (explicit_sets) {
                // the caller (the recency ranking) already chose what moves and
                // has updated the resident words: staging holds [evict | add]
                evict = m[w];
                add = m[kWords + w];
                desired = 0;            // counted from the resident words while staging
            } else {
                const uint32_t raw_w = m[w] & valid, res = m[kWords + w];
                n_touched += __popc(raw_w);
                if (scan_only) {
                    if (bitmaps_out) bitmaps_out[g * kWords + w] = raw_w;
                    evict = add = desired = 0;
                } else {
                    // budget cut: lowest block ids first (one event: every stamp
                    // ties, and ties rank by ascending block id)
                    const uint32_t room = budget > kept ? budget - kept : 0;
                    desired = room ? lowest_bits(raw_w, room) : 0u;
                    kept += __popc(desired);
                    add = desired & ~res;
                    evict = (flags & RT_PLAN_EVICT) ? (res & ~desired) : 0u;
                    if (!(flags & RT_PLAN_DRY_RUN)) resident[g * kWords + w] = desired;
                }
            }
            m[w] = evict;
            m[kWords + w] = add;
            n_des += __popc(desired);
            n_add += __popc(add);
            n_ev += __popc(evict);
            // a run starts at every set bit whose lower neighbour is clear
            c_ev += __popc(evict & ~((evict << 1) | carry_ev));
            c_add += __popc(add & ~((add << 1) | carry_add));
            carry_ev = evict >> 31;
            carry_add = add >> 31;
        }
        if (scan_only && bitmaps_out)
            for (uint32_t w = n_words; w < kWords; ++w) bitmaps_out[g * kWords + w] = 0;
        for (uint32_t w = n_words; w < kWords; ++w) { m[w] = 0; m[kWords + w] = 0; }
        sh.counts[g * 2 + 0] = c_ev;
        sh.counts[g * 2 + 1] = c_add;
        some_runs |= c_ev | c_add;
    }
    // totals: one reduction per warp, then at most one shared atomic per warp and counter
    n_touched = warp_sum(n_touched);
    n_des = warp_sum(n_des);
    n_add = warp_sum(n_add);
    n_ev = warp_sum(n_ev);
    some_runs = __any_sync(0xffffffffu, some_runs != 0);
    if (lane == 0) {
        if (n_touched) atomicAdd(&sh.stats[0], n_touched);
        if (n_des) atomicAdd(&sh.stats[1], n_des);
        if (n_add) atomicAdd(&sh.stats[2], n_add);
        if (n_ev) atomicAdd(&sh.stats[3], n_ev);
        if (some_runs) sh.stats[4] = 1;
    }
    cta_sync<kBar, kScanThreads>();
    RT_TAIL_MARK(2);
    // steady state: nothing moves, so there is nothing to lay out
    const bool any_runs = sh.stats[4] != 0;

    // ---- exclusive prefix sum of run counts over (phase, buffer) ----
    const uint32_t items = (p.scan_only || !any_runs) ? 0 : 2 * n;
    const uint32_t per = (items + kScanThreads - 1) / kScanThreads;
    const uint32_t first = tid * per;
    uint32_t local = 0;
    for (uint32_t k = 0; k < per; ++k) {
        uint32_t i = first + k;
        if (i < items) {
            uint32_t phase = i >= n, j = i - phase * n;
            local += sh.counts[p.buffer_group[j] * 2 + phase];
        }
    }
    const uint32_t incl = warp_inclusive_sum(local, lane);
    if (lane == 31) sh.warp_tot[warp] = incl;
    cta_sync<kBar, kScanThreads>();
    uint32_t base = 0, total = 0;
    for (uint32_t w = 0; w < (uint32_t)kTailWarps; ++w) {
        if (w < warp) base += sh.warp_tot[w];
        total += sh.warp_tot[w];
    }
    uint32_t run = base + incl - local;
    for (uint32_t k = 0; k < per; ++k) {
        uint32_t i = first + k;
        if (i < items) {
            sh.off[i] = run;
            uint32_t phase = i >= n, j = i - phase * n;
            run += sh.counts[p.buffer_group[j] * 2 + phase];
        }
    }
    if (tid == 0) sh.off[items] = total;
    cta_sync<kBar, kScanThreads>();
    const uint32_t n_cpu = items ? sh.off[n] : 0;
    RT_TAIL_MARK(3);

    // ---- pass B: one warp per (bitmap, phase): stage its run list in shared
    //      memory, then write it once for every buffer of the bitmap ----
    uint16_t *sb = sh.stage + (size_t)warp * 2 * kMaxRuns, *se = sb + kMaxRuns;
    unsigned long long my_bytes[2] = {0, 0};
    for (uint32_t t = warp; t < 2 * G && items; t += kTailWarps) {
        const uint32_t count = sh.counts[t];
        if (!count) continue;                                   // uniform over the warp
        const uint32_t g = t >> 1, phase = t & 1;
        uint32_t starts, lasts;
        run_edges(sh.masks[g * kMaskStride + phase * kWords + lane], lane, starts, lasts);
        uint32_t bpos = warp_inclusive_sum(__popc(starts), lane) - __popc(starts);
        uint32_t epos = warp_inclusive_sum(__popc(lasts), lane) - __popc(lasts);
        while (starts) {
            uint32_t b = __ffs(starts) - 1;
            starts &= starts - 1;
            sb[bpos++] = (uint16_t)(lane * 32 + b);
        }
        while (lasts) {
            uint32_t b = __ffs(lasts) - 1;
            lasts &= lasts - 1;
            se[epos++] = (uint16_t)(lane * 32 + b + 1);
        }
        __syncwarp();
        const int32_t dst = phase ? p.dst_device : RT_DST_CPU;
        for (uint32_t j0 = 0; j0 < n; j0 += 32) {
            const uint32_t j = j0 + lane;
            uint32_t mine = __ballot_sync(0xffffffffu, j < n && p.buffer_group[j] == g);
            while (mine) {
                const uint32_t jj = j0 + (uint32_t)__ffs(mine) - 1;
                mine &= mine - 1;
                const uint32_t at = sh.off[phase * n + jj];
                for (uint32_t k = lane; k < count; k += 32) {
                    unsigned long long b = (unsigned long long)sb[k] * p.block_bytes;
                    unsigned long long e = (unsigned long long)se[k] * p.block_bytes;
                    if (e > p.alloc_bytes) e = p.alloc_bytes;   // final partial block, select.cpp:24188
                    my_bytes[phase] += e - b;
                    if (at + k < p.cap) {
                        rt_range r;
                        r.buffer = jj;
                        r.dst = dst;
                        r.offset = b;
                        r.bytes = e - b;
                        p.out[at + k] = r;
                    }
                }
            }
        }
        __syncwarp();
    }
    RT_TAIL_MARK(4);
    if (my_bytes[0]) atomicAdd(&sh.bytes[0], my_bytes[0]);
    if (my_bytes[1]) atomicAdd(&sh.bytes[1], my_bytes[1]);
    cta_sync<kBar, kScanThreads>();
    if (tid == 0) {
        rt_plan_result res;
        res.n_ranges = total;
        res.n_cpu_ranges = n_cpu;
        res.flags = (total > p.cap ? RT_RESULT_OVERFLOW : 0u) | (invalid ? RT_RESULT_SLOT_RANGE : 0u) | eflags;
        res.blocks_touched = sh.stats[0];
        res.blocks_desired = sh.stats[1];
        res.blocks_added = sh.stats[2];
        res.blocks_evicted = sh.stats[3];
        res.reserved = 0;
        res.invalid_slots = invalid;
        res.ignored_slots = ignored;
        res.cpu_bytes = sh.bytes[0];
        res.gpu_bytes = sh.bytes[1];
        *p.result = res;
        // leave the scratch clean for the next launch
        GlobalScratch &gl = *p.global;
        gl.invalid_slots = 0;
        gl.ignored_slots = 0;
        gl.units_done = 0;
        gl.error_flags = 0;
    }
    RT_TAIL_MARK(5);
}

}  // namespace rt
