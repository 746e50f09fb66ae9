// Plan tail: wanted bitmaps -> budget cut -> diff against the resident set ->
// coalesced byte ranges in queue order.  Runs in ONE CTA (the one that retired
// the last scan unit, or the single CTA of the bitmap-only kernel).  One CTA is
// latency bound -- about eleven cycles per instruction per warp in measurement,
// whatever the instruction -- so the design goal is the shortest dependent
// instruction chain: one global round trip for every bitmap's words, one thread
// per mask word with warp shuffles for everything that crosses words, then one
// thread per (phase, buffer) for the range stores.
#pragma once
#include "plan_device.cuh"

namespace rt {

#ifdef RT_TRACE
static __device__ unsigned long long g_tail_trace[8];
#define RT_TAIL_MARK(k)                                                          \
    do {                                                                         \
        if (threadIdx.x == 0) {                                                  \
            unsigned long long t__;                                              \
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t__)::"memory");   \
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

__device__ __forceinline__ unsigned long long warp_sum64(unsigned long long v) {
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
    return v;
}

// Lowest `k` set bits of x.  The answer keeps the low `pos` bits of x, pos the
// largest width whose low bits hold at most k set bits: five unrolled steps of
// popc (a loop costs compares and branches on the tail's critical path; __fns
// is emulated in software and much slower).
__device__ __forceinline__ uint32_t lowest_bits(uint32_t x, uint32_t k) {
    if (k >= (uint32_t)__popc(x)) return x;
    uint32_t pos = 0;
#pragma unroll
    for (uint32_t s = 16; s >= 1; s >>= 1)
        if ((uint32_t)__popc(x & ((1u << (pos + s)) - 1u)) <= k) pos += s;
    return x & ((1u << pos) - 1u);
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
// Words per bitmap in the tail's shared staging:
//   [0, kWords)          evict words
//   [kWords, 2*kWords)   add words
//   [2*kWords, 3*kWords) per word, the number of runs that start in lower words:
//                        low half = evict runs, high half = add runs
// plus one word of padding, so that threads working on different bitmaps and
// the same word index fall in different banks.
constexpr uint32_t kMaskStride = 3 * kWords + 1;

struct TailShared {
    unsigned long long *warp_bytes;  // [kTailWarps][2]  CPU-bound / GPU-bound bytes per warp
    uint32_t *warp_stats;            // [kTailWarps][4]  touched, desired, added, evicted per warp
    uint32_t *counts;                // [n_groups][2]        runs per (bitmap, phase)
    uint32_t *off;                   // [2*n_buffers + 1]    first range of every (phase, buffer)
    uint32_t *masks;                 // [n_groups][kMaskStride]
    uint8_t *group_of;               // [n_buffers]          bitmap of every buffer
};

__host__ __device__ constexpr size_t tail_smem_bytes(uint32_t n_groups, uint32_t n_buffers) {
    return ((4 * kTailWarps + 4 * kTailWarps + 2 * (size_t)n_groups +
             (2 * (size_t)n_buffers + 1) + (size_t)kMaskStride * n_groups) * 4 +
            (size_t)n_buffers + 15) & ~(size_t)15;
}

__device__ __forceinline__ TailShared carve_tail(unsigned char *raw, uint32_t n_groups, uint32_t n_buffers) {
    TailShared s;
    uint32_t *w = reinterpret_cast<uint32_t *>(raw);
    s.warp_bytes = reinterpret_cast<unsigned long long *>(w);  w += 4 * kTailWarps;
    s.warp_stats = w;                                          w += 4 * kTailWarps;
    s.counts = w;                                              w += 2 * n_groups;
    s.off = w;                                                 w += 2 * n_buffers + 1;
    s.masks = w;                                               w += kMaskStride * n_groups;
    s.group_of = reinterpret_cast<uint8_t *>(w);
    return s;
}

// Inclusive sum over segments of `seg` consecutive lanes (seg a power of two).
__device__ __forceinline__ uint32_t segment_inclusive_sum(uint32_t v, uint32_t w, uint32_t seg) {
    for (uint32_t d = 1; d < seg; d <<= 1) {
        const uint32_t t = __shfl_up_sync(0xffffffffu, v, d);
        if (w >= d) v += t;
    }
    return v;
}

// --------------------------------------------------------------------------
// the tail itself: kScanThreads threads of one CTA
// --------------------------------------------------------------------------
// `want` holds n_groups x kWords words; `consume` zeroes them after reading
// (they are the scan's accumulation words).
template <int kBar>
__device__ void plan_tail(const PlanArgs &p, uint32_t *want, bool consume, unsigned char *raw) {
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // Scalars of `p` are copied to locals first: `p` lives in parameter space and
    // every global store below would otherwise force them to be re-read.
    const uint32_t G = p.n_groups, n = p.n_buffers;
    const uint32_t n_blocks = p.n_blocks, budget = p.budget, flags = p.flags;
    const bool explicit_sets = p.explicit_sets != 0, scan_only = p.scan_only != 0;
    uint32_t *const resident = p.resident, *const bitmaps_out = p.bitmaps_out;
    const uint32_t n_words = (n_blocks + 31) / 32;
    const TailShared sh = carve_tail(raw, G, n);
    RT_TAIL_MARK(0);
    // counters written by other CTAs: fetched now, used at the very end
    unsigned long long invalid = 0, ignored = 0;
    uint32_t eflags = 0;
    if (tid == 0) {
        invalid = __ldcg(&p.global->invalid_slots);
        ignored = __ldcg(&p.global->ignored_slots);
        eflags = __ldcg(&p.global->error_flags);
    }
    // the buffer -> bitmap table goes to shared memory; its load is in flight
    // together with the first mask words below
    const uint8_t *const table = p.buffer_group;
    const uint32_t table_first = tid < n ? __ldcg(&table[tid]) : 0u;
    RT_TAIL_MARK(6);

    // ---- pass A: one THREAD per (bitmap, word) ----
    // A warp holds 32/seg bitmaps, seg = the power of two that covers the words
    // in use; sums and neighbour bits cross words by shuffles inside a segment.
    // The words of two rounds are loaded before the first is processed, so the
    // one global round trip of the tail is paid once.
    uint32_t seg = 1;
    while (seg < n_words) seg <<= 1;
    const uint32_t per_warp = 32 / seg, sub = lane / seg, w = lane & (seg - 1);
    const uint32_t round_stride = kTailWarps * per_warp;
    const uint32_t left = w < n_words ? n_blocks - w * 32 : 0;
    const uint32_t valid = left >= 32 ? 0xffffffffu : ((1u << left) - 1u);
    uint32_t n_touched = 0, n_des = 0, n_add = 0, n_ev = 0, some_runs = 0;
    constexpr int kRounds = 2;
    for (uint32_t g0 = warp * per_warp; g0 < G; g0 += kRounds * round_stride) {
        uint32_t a_w[kRounds], b_w[kRounds], r_w[kRounds];
#pragma unroll
        for (int k = 0; k < kRounds; ++k) {
            const uint32_t g = g0 + k * round_stride + sub;
            a_w[k] = b_w[k] = r_w[k] = 0;
            if (g < G && w < n_words) {
                if (explicit_sets) {
                    // the caller (the recency ranking) already chose what moves and
                    // has updated the resident words: `want` holds [evict | add]
                    a_w[k] = __ldcg(&want[(g * 2 + 0) * kWords + w]);
                    b_w[k] = __ldcg(&want[(g * 2 + 1) * kWords + w]);
                    r_w[k] = __ldcg(&resident[g * kWords + w]);
                } else {
                    a_w[k] = __ldcg(&want[g * kWords + w]);
                    if (!scan_only) r_w[k] = __ldcg(&resident[g * kWords + w]);
                }
            }
        }
#ifdef RT_TRACE
        if (tid == 0 && (a_w[0] | r_w[0]) == 0x12345u) g_tail_trace[7] = 1;   // forces the loads to land
        else RT_TAIL_MARK(7);
#endif
        // no early exit for a round past the last bitmap: its lanes hold zeros,
        // and straight-line code lets the rounds' dependent chains interleave
#pragma unroll
        for (int k = 0; k < kRounds; ++k) {
            const uint32_t g = g0 + k * round_stride + sub;
            const bool live = g < G && w < n_words;
            uint32_t evict, add, desired;
            if (explicit_sets) {
                evict = a_w[k];
                add = b_w[k];
                desired = r_w[k];                                   // already the new set
            } else {
                const uint32_t raw_w = a_w[k] & valid;
                if (live && consume) want[g * kWords + w] = 0;
                n_touched += __popc(raw_w);
                if (scan_only) {
                    if (live && bitmaps_out) bitmaps_out[g * kWords + w] = raw_w;
                    evict = add = desired = 0;
                } else {
                    // budget cut: lowest block ids first (one event: every stamp
                    // ties, and ties rank by ascending block id)
                    const uint32_t cnt = __popc(raw_w);
                    const uint32_t before = segment_inclusive_sum(cnt, w, seg) - cnt;
                    const uint32_t room = budget > before ? budget - before : 0;
                    desired = room >= cnt ? raw_w : lowest_bits(raw_w, room);
                    add = desired & ~r_w[k];
                    evict = (flags & RT_PLAN_EVICT) ? (r_w[k] & ~desired) : 0u;
                    if (live && !(flags & RT_PLAN_DRY_RUN)) resident[g * kWords + w] = desired;
                }
            }
            n_des += __popc(desired);
            n_add += __popc(add);
            n_ev += __popc(evict);
            // a run starts at every set bit whose lower neighbour is clear
            const uint32_t below_ev = __shfl_up_sync(0xffffffffu, evict, 1);
            const uint32_t below_add = __shfl_up_sync(0xffffffffu, add, 1);
            const uint32_t c = __popc(evict & ~((evict << 1) | (w ? below_ev >> 31 : 0u))) |
                               (__popc(add & ~((add << 1) | (w ? below_add >> 31 : 0u))) << 16);
            const uint32_t upto = segment_inclusive_sum(c, w, seg);   // both halves at once: each <= 512
            if (live) {
                uint32_t *m = sh.masks + g * kMaskStride;
                m[w] = evict;
                m[kWords + w] = add;
                m[2 * kWords + w] = upto - c;                         // runs that start below this word
                if (w == n_words - 1) {
                    sh.counts[g * 2 + 0] = upto & 0xffffu;
                    sh.counts[g * 2 + 1] = upto >> 16;
                    some_runs |= upto;
                }
            }
        }
    }
    if (tid < n) sh.group_of[tid] = (uint8_t)table_first;
    for (uint32_t j = tid + kScanThreads; j < n; j += kScanThreads) sh.group_of[j] = __ldcg(&table[j]);
    RT_TAIL_MARK(1);
    if (scan_only && bitmaps_out)                                    // words past the ones in use
        for (uint32_t i = tid; i < G * kWords; i += kScanThreads)
            if ((i & (kWords - 1)) >= n_words) bitmaps_out[i] = 0;
    n_touched = warp_sum(n_touched);
    n_des = warp_sum(n_des);
    n_add = warp_sum(n_add);
    n_ev = warp_sum(n_ev);
    if (lane == 0) {
        uint32_t *ws = sh.warp_stats + warp * 4;
        ws[0] = n_touched; ws[1] = n_des; ws[2] = n_add; ws[3] = n_ev;
    }
    // steady state: nothing moves, so there is nothing to lay out
    const bool any_runs = cta_or<kBar, kScanThreads>(some_runs != 0);
    RT_TAIL_MARK(2);

    // ---- exclusive prefix sum of run counts over (phase, buffer): warp 0 ----
    // One warp, consecutive items per lane, one shuffle scan: a CTA-wide scan
    // costs a second barrier and a pass through shared memory, which is more
    // than 2*n_buffers/32 additions per lane.
    const uint32_t items = (scan_only || !any_runs) ? 0 : 2 * n;
    uint32_t total = 0;
    if (warp == 0 && items) {
        const uint32_t per = (items + 31) / 32, first = lane * per;
        uint32_t local = 0;
        for (uint32_t k = 0; k < per; ++k) {
            const uint32_t i = first + k;
            if (i < items) {
                const uint32_t phase = i >= n, j = i - phase * n;
                local += sh.counts[sh.group_of[j] * 2 + phase];
            }
        }
        const uint32_t incl = warp_inclusive_sum(local, lane);
        uint32_t run = incl - local;
        for (uint32_t k = 0; k < per; ++k) {
            const uint32_t i = first + k;
            if (i < items) {
                sh.off[i] = run;
                const uint32_t phase = i >= n, j = i - phase * n;
                run += sh.counts[sh.group_of[j] * 2 + phase];
            }
        }
        if (lane == 31) sh.off[items] = incl;
    }
    cta_sync<kBar, kScanThreads>();
    if (items) total = sh.off[items];
    const uint32_t n_cpu = items ? sh.off[n] : 0;
    RT_TAIL_MARK(3);

    // ---- pass B: one thread per (phase, buffer) ----
    // The thread walks the words of its bitmap's evict or add mask and writes
    // the runs; where they go is the prefix sum above.  (A warp per (bitmap,
    // phase) handing its run list to every buffer in turn took ten dependent
    // rounds for 40 bitmaps: 17 us for 160 ranges.)
    const unsigned long long block_bytes = p.block_bytes, alloc_bytes = p.alloc_bytes;
    const uint32_t cap = p.cap;
    const int32_t dst_gpu = p.dst_device;
    rt_range *const out = p.out;
    unsigned long long cpu_bytes = 0, gpu_bytes = 0;
    for (uint32_t i = tid; i < items; i += kScanThreads) {
        const uint32_t phase = i >= n, j = i - phase * n, g = sh.group_of[j];
        if (!sh.counts[g * 2 + phase]) continue;
        const uint32_t *m = sh.masks + g * kMaskStride + phase * kWords;
        uint32_t at = sh.off[i], below_top = 0;
        unsigned long long moved = 0;
        for (uint32_t k = 0; k < n_words; ++k) {
            const uint32_t word = m[k];
            uint32_t starts = word & ~((word << 1) | below_top);
            below_top = word >> 31;
            while (starts) {
                const uint32_t b = __ffs(starts) - 1;
                starts &= starts - 1;
                // first clear bit above b, in this word or the following ones
                const uint32_t clear = ~(word >> b);        // zero only for b == 0 and a full word
                uint32_t e = clear ? b + (uint32_t)__ffs(clear) - 1 : 32u;
                if (e == 32) {
                    uint32_t k2 = k + 1;
                    while (k2 < n_words && m[k2] == 0xffffffffu) ++k2;
                    e = (k2 - k) * 32 + (k2 < n_words ? (uint32_t)__ffs(~m[k2]) - 1 : 0u);
                }
                const unsigned long long lo = (unsigned long long)(k * 32 + b) * block_bytes;
                unsigned long long hi = (unsigned long long)(k * 32 + e) * block_bytes;
                if (hi > alloc_bytes) hi = alloc_bytes;             // final partial block, select.cpp:24188
                moved += hi - lo;
                if (at < cap) {
                    rt_range rg;
                    rg.buffer = j;
                    rg.dst = phase ? dst_gpu : RT_DST_CPU;
                    rg.offset = lo;
                    rg.bytes = hi - lo;
                    out[at] = rg;
                }
                ++at;
            }
        }
        if (phase) gpu_bytes += moved; else cpu_bytes += moved;
    }
    RT_TAIL_MARK(4);
    if (items) {
        cpu_bytes = warp_sum64(cpu_bytes);
        gpu_bytes = warp_sum64(gpu_bytes);
    }
    if (lane == 0) {
        sh.warp_bytes[warp * 2 + 0] = cpu_bytes;
        sh.warp_bytes[warp * 2 + 1] = gpu_bytes;
    }
    cta_sync<kBar, kScanThreads>();
    if (tid == 0) {
        rt_plan_result res;
        uint32_t st[4] = {0, 0, 0, 0};
        unsigned long long by[2] = {0, 0};
#pragma unroll
        for (int k = 0; k < kTailWarps; ++k) {
#pragma unroll
            for (int q = 0; q < 4; ++q) st[q] += sh.warp_stats[k * 4 + q];
            by[0] += sh.warp_bytes[k * 2 + 0];
            by[1] += sh.warp_bytes[k * 2 + 1];
        }
        res.n_ranges = total;
        res.n_cpu_ranges = n_cpu;
        res.flags = (total > cap ? RT_RESULT_OVERFLOW : 0u) | (invalid ? RT_RESULT_SLOT_RANGE : 0u) | eflags;
        res.blocks_touched = st[0];
        res.blocks_desired = st[1];
        res.blocks_added = st[2];
        res.blocks_evicted = st[3];
        res.reserved = 0;
        res.invalid_slots = invalid;
        res.ignored_slots = ignored;
        res.cpu_bytes = by[0];
        res.gpu_bytes = by[1];
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
