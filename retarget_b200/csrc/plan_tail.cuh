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

// Lowest `k` set bits of x, without a branch.  The answer keeps the low `pos`
// bits of x, pos the largest width below 32 whose low bits hold at most k set
// bits: five unrolled steps of popc.  (A search loop costs compares and
// branches on the tail's critical path and keeps the compiler from overlapping
// independent bitmaps; __fns is emulated in software and much slower.)
__device__ __forceinline__ uint32_t lowest_bits(uint32_t x, uint32_t k) {
    uint32_t pos = 0;
#pragma unroll
    for (uint32_t s = 16; s >= 1; s >>= 1)
        pos += ((uint32_t)__popc(x & ((1u << (pos + s)) - 1u)) <= k) ? s : 0u;
    const uint32_t cut = x & ((1u << pos) - 1u);
    return k >= (uint32_t)__popc(x) ? x : cut;
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
//   [0, kWords)          words that leave the resident set (announced as CPU-bound
//                        ranges only under RT_PLAN_EVICT)
//   [kWords, 2*kWords)   add words
// plus one word of padding, so that threads working on different bitmaps and
// the same word index fall in different banks.
constexpr uint32_t kMaskStride = 2 * kWords + 1;
// Run lists of at most kFew runs per (bitmap, phase) are written out by pass A
// as (begin, end) block pairs, so the common plans -- a window that moves, a
// few blocks that change -- need no second look at the mask words.
constexpr uint32_t kFew = 2;
constexpr int kWarpStats = 8;   // touched, desired, added, evicted, buffer-blocks to CPU / GPU, partial last blocks to CPU / GPU

struct TailShared {
    uint32_t *warp_stats;            // [kTailWarps][kWarpStats]
    uint32_t *warp_tot;              // [kTailWarps]
    uint32_t *counts;                // [n_groups][2]        runs per (bitmap, phase)
    uint32_t *off;                   // [2*n_buffers + 1]    first range of every (phase, buffer)
    uint32_t *masks;                 // [n_groups][kMaskStride]
    uint16_t *few;                   // [n_groups][2][kFew][2]  begin, end of the first runs
    uint32_t *verdict;               // [1]  the scan saw ids above capacity or gave up a wait
    uint8_t *group_of;               // [n_buffers]          bitmap of every buffer
};

__host__ __device__ constexpr size_t tail_smem_bytes(uint32_t n_groups, uint32_t n_buffers) {
    return ((kWarpStats * kTailWarps + kTailWarps + 2 * (size_t)n_groups + (2 * (size_t)n_buffers + 1) +
             (size_t)kMaskStride * n_groups + 2 * kFew * (size_t)n_groups + 1) * 4 +
            (size_t)n_buffers + 15) & ~(size_t)15;
}

__device__ __forceinline__ TailShared carve_tail(unsigned char *raw, uint32_t n_groups, uint32_t n_buffers) {
    TailShared s;
    uint32_t *w = reinterpret_cast<uint32_t *>(raw);
    s.warp_stats = w;                                          w += kWarpStats * kTailWarps;
    s.warp_tot = w;                                            w += kTailWarps;
    s.counts = w;                                              w += 2 * n_groups;
    s.off = w;                                                 w += 2 * n_buffers + 1;
    s.masks = w;                                               w += kMaskStride * n_groups;
    s.few = reinterpret_cast<uint16_t *>(w);                   w += 2 * kFew * n_groups;
    s.verdict = w;                                             w += 1;
    s.group_of = reinterpret_cast<uint8_t *>(w);
    return s;
}

// Inclusive sum over segments of consecutive lanes; `w` is the lane's index in
// its segment.  Always five steps: a lane only adds what lies inside its own
// segment (w >= d), and a fixed count keeps the code free of branches.
__device__ __forceinline__ uint32_t segment_inclusive_sum(uint32_t v, uint32_t w) {
#pragma unroll
    for (uint32_t d = 1; d < 32; d <<= 1) {
        const uint32_t t = __shfl_up_sync(0xffffffffu, v, d);
        v += w >= d ? t : 0u;
    }
    return v;
}

// Pass A helper for one phase's mask word: number of runs that start in it and,
// for the first kFew runs of the bitmap, their begin / end blocks.
//   below_top  bit 31 of the word below (0 for word 0)
//   above_low  bit 0 of the word above (0 for the last word)
__device__ __forceinline__ uint32_t run_starts(uint32_t x, uint32_t below_top) {
    return x & ~((x << 1) | below_top);
}
__device__ __forceinline__ void note_few(uint16_t *few, uint32_t x, uint32_t w, uint32_t below_top,
                                         uint32_t above_low, uint32_t starts_below) {
    uint32_t starts = run_starts(x, below_top);
    uint32_t lasts = x & ~((x >> 1) | (above_low << 31));
    uint32_t si = starts_below;
    // a run that crosses in from the word below has started but not ended there
    uint32_t ei = starts_below - (below_top & x & 1u);
#pragma unroll
    for (uint32_t q = 0; q < kFew; ++q) {
        if (starts && si < kFew) {
            few[2 * si] = (uint16_t)(w * 32 + __ffs(starts) - 1);
            starts &= starts - 1;
            ++si;
        }
        if (lasts && ei < kFew) {
            few[2 * ei + 1] = (uint16_t)(w * 32 + __ffs(lasts));
            lasts &= lasts - 1;
            ++ei;
        }
    }
}

__device__ __forceinline__ void store_range(rt_range *out, uint32_t at, uint32_t cap, uint32_t buffer,
                                            int32_t dst, uint32_t begin, uint32_t end,
                                            unsigned long long block_bytes, unsigned long long alloc_bytes) {
    if (at >= cap) return;
    const unsigned long long lo = (unsigned long long)begin * block_bytes;
    unsigned long long hi = (unsigned long long)end * block_bytes;
    if (hi > alloc_bytes) hi = alloc_bytes;                     // final partial block, select.cpp:24188
    // 24 bytes as one 16-byte and one 8-byte store (which half is 16-byte aligned
    // alternates with `at`): when a plan has thousands of ranges the tail is bound
    // by the number of store instructions one SM can retire
    const unsigned long long head = (unsigned long long)buffer | ((unsigned long long)(uint32_t)dst << 32);
    unsigned long long *q = reinterpret_cast<unsigned long long *>(out + at);
    if ((reinterpret_cast<uintptr_t>(q) & 15u) == 0) {
        *reinterpret_cast<ulonglong2 *>(q) = make_ulonglong2(head, lo);
        q[2] = hi - lo;
    } else {
        q[0] = head;
        *reinterpret_cast<ulonglong2 *>(q + 1) = make_ulonglong2(lo, hi - lo);
    }
}

// --------------------------------------------------------------------------
// pass A: one THREAD per (bitmap, word)
// --------------------------------------------------------------------------
// A warp holds 32/seg bitmaps, seg = the power of two that covers the words in
// use; sums and neighbour bits cross words by shuffles inside a segment.  The
// words of two rounds are loaded before the first is processed, so the one
// global round trip of the tail is paid once.  The mode is a template parameter
// and the arithmetic of both rounds comes before any of their stores, so that
// the compiler sees straight-line code and overlaps the two dependent chains (a
// run-time mode test inside the loop kept them apart: 1.6 us instead of 0.9).
enum TailMode { kTailPlan = 0, kTailExplicit = 1, kTailScanOnly = 2 };

struct PassA {
    uint32_t G, n_words, n_blocks, budget, flags;
    bool consume;
    uint32_t *want, *resident, *bitmaps_out;
    const uint16_t *group_size;
};

template <int kMode>
__device__ __forceinline__ void pass_a(const PassA &in, const TailShared &sh, uint32_t (&st)[kWarpStats],
                                       uint32_t &some_runs) {
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t G = in.G, n_words = in.n_words;
    uint32_t seg = 1;
    while (seg < n_words) seg <<= 1;
    const uint32_t per_warp = 32 / seg, sub = lane / seg, w = lane & (seg - 1);
    const uint32_t round_stride = kTailWarps * per_warp;
    const uint32_t seg_lanes = (seg >= 32 ? 0xffffffffu : ((1u << seg) - 1u)) << (sub * seg);   // lanes of this thread's bitmap
    const uint32_t left = w < n_words ? in.n_blocks - w * 32 : 0;
    const uint32_t valid = left >= 32 ? 0xffffffffu : ((1u << left) - 1u);
    const uint32_t last_bit = (w == n_words - 1) ? 1u << ((in.n_blocks - 1) & 31) : 0u;
    const bool evicting = (in.flags & RT_PLAN_EVICT) != 0, dry = (in.flags & RT_PLAN_DRY_RUN) != 0;
    constexpr int kRounds = 2;
    for (uint32_t g0 = warp * per_warp; g0 < G; g0 += kRounds * round_stride) {
        uint32_t a_w[kRounds], b_w[kRounds], r_w[kRounds], size_g[kRounds];
#pragma unroll
        for (int k = 0; k < kRounds; ++k) {
            const uint32_t g = g0 + k * round_stride + sub;
            a_w[k] = b_w[k] = r_w[k] = size_g[k] = 0;
            if (g < G && w < n_words) {
                size_g[k] = __ldcg(&in.group_size[g]);
                if (kMode == kTailExplicit) {
                    // the caller (the recency ranking) already chose what moves and
                    // commits it itself: `want` holds [evict | add | new resident]
                    a_w[k] = __ldcg(&in.want[(g * 3 + 0) * kWords + w]);
                    b_w[k] = __ldcg(&in.want[(g * 3 + 1) * kWords + w]);
                    r_w[k] = __ldcg(&in.want[(g * 3 + 2) * kWords + w]);
                } else {
                    a_w[k] = __ldcg(&in.want[g * kWords + w]);
                    if (kMode == kTailPlan) r_w[k] = __ldcg(&in.resident[g * kWords + w]);
                }
            }
        }
        // arithmetic of both rounds (a round past the last bitmap is not skipped:
        // its lanes hold zeros)
        uint32_t raw[kRounds], evict[kRounds], add[kRounds], desired[kRounds], gone[kRounds];
        uint32_t below_ev[kRounds], below_add[kRounds], above_ev[kRounds], above_add[kRounds];
        uint32_t c[kRounds], upto[kRounds];
#pragma unroll
        for (int k = 0; k < kRounds; ++k) {
            raw[k] = 0;
            gone[k] = 0;
            if (kMode == kTailExplicit) {
                evict[k] = a_w[k];
                add[k] = b_w[k];
                desired[k] = r_w[k];                                // already the new set
            } else {
                raw[k] = a_w[k] & valid;
                st[0] += __popc(raw[k]);
                if (kMode == kTailScanOnly) {
                    evict[k] = add[k] = desired[k] = 0;
                } else {
                    // budget cut: lowest block ids first (one event: every stamp
                    // ties, and ties rank by ascending block id)
                    const uint32_t cnt = __popc(raw[k]);
                    const uint32_t before = segment_inclusive_sum(cnt, w) - cnt;
                    desired[k] = lowest_bits(raw[k], in.budget > before ? in.budget - before : 0u);
                    add[k] = desired[k] & ~r_w[k];
                    // what leaves the resident set; only announced when evicting
                    gone[k] = r_w[k] & ~desired[k];
                    evict[k] = evicting ? gone[k] : 0u;
                    // A bitmap whose plan moves nothing keeps its record as it is:
                    // the reference's controller returns before it touches
                    // `committed` when nothing was selected
                    // (experiments/slot_placement.py:131-132).  Only without
                    // eviction can that differ from the desired set.
                    if (!evicting && (__ballot_sync(0xffffffffu, add[k] != 0) & seg_lanes) == 0) gone[k] = 0;
                }
            }
            st[1] += __popc(desired[k]);
            st[2] += __popc(add[k]);
            st[3] += __popc(evict[k]);
            // bytes moved are counted in blocks x buffers of the bitmap here; the
            // last block of a buffer may be partial and is counted separately
            st[4] += __popc(evict[k]) * size_g[k];
            st[5] += __popc(add[k]) * size_g[k];
            st[6] += (evict[k] & last_bit) ? size_g[k] : 0u;
            st[7] += (add[k] & last_bit) ? size_g[k] : 0u;
            // neighbour bits across the word boundaries of the bitmap
            const uint32_t dn_ev = __shfl_up_sync(0xffffffffu, evict[k], 1);
            const uint32_t dn_add = __shfl_up_sync(0xffffffffu, add[k], 1);
            const uint32_t up_ev = __shfl_down_sync(0xffffffffu, evict[k], 1);
            const uint32_t up_add = __shfl_down_sync(0xffffffffu, add[k], 1);
            below_ev[k] = w ? dn_ev >> 31 : 0u;
            below_add[k] = w ? dn_add >> 31 : 0u;
            above_ev[k] = w + 1 < seg ? up_ev & 1u : 0u;
            above_add[k] = w + 1 < seg ? up_add & 1u : 0u;
            // a run starts at every set bit whose lower neighbour is clear
            c[k] = __popc(run_starts(evict[k], below_ev[k])) | (__popc(run_starts(add[k], below_add[k])) << 16);
            upto[k] = segment_inclusive_sum(c[k], w);               // both halves at once: each <= 512
        }
        // stores of both rounds
#pragma unroll
        for (int k = 0; k < kRounds; ++k) {
            const uint32_t g = g0 + k * round_stride + sub;
            if (!(g < G && w < n_words)) continue;
            if (kMode != kTailExplicit && in.consume) in.want[g * kWords + w] = 0;
            if (kMode == kTailScanOnly && in.bitmaps_out) in.bitmaps_out[g * kWords + w] = raw[k];
            // new resident word = (old | add) & ~gone: the desired set, or the old
            // record when the bitmap's plan moved nothing
            if (kMode == kTailPlan && !dry) in.resident[g * kWords + w] = (r_w[k] | add[k]) & ~gone[k];
            // (the old resident word is (new & ~add) | gone: the tail puts it back
            // when the plan turns out not to be deliverable)
            uint32_t *m = sh.masks + g * kMaskStride;
            m[w] = kMode == kTailPlan ? gone[k] : evict[k];
            m[kWords + w] = add[k];
            uint16_t *few = sh.few + g * 4 * kFew;
            note_few(few, evict[k], w, below_ev[k], above_ev[k], (upto[k] - c[k]) & 0xffffu);
            note_few(few + 2 * kFew, add[k], w, below_add[k], above_add[k], (upto[k] - c[k]) >> 16);
            if (w == n_words - 1) {
                sh.counts[g * 2 + 0] = upto[k] & 0xffffu;
                sh.counts[g * 2 + 1] = upto[k] >> 16;
                some_runs |= upto[k];
            }
        }
    }
}

// --------------------------------------------------------------------------
// tail of a launch whose scan failed in the CTA that would plan: no plan, the
// resident words stay as they are, the scratch is cleaned for the next launch
// --------------------------------------------------------------------------
__device__ __forceinline__ void tail_abort(const PlanArgs &p) {
    uint32_t *want = &p.groups[0].want[0];
    for (uint32_t i = threadIdx.x; i < p.n_groups * kWords; i += kScanThreads) want[i] = 0;
    if (threadIdx.x == 0) {
        GlobalScratch &gl = *p.global;
        rt_plan_result res = {};
        res.flags = __ldcg(&gl.error_flags) | RT_RESULT_TIMEOUT |
                    (__ldcg(&gl.invalid_slots) ? RT_RESULT_SLOT_RANGE : 0u);
        res.invalid_slots = __ldcg(&gl.invalid_slots);
        res.ignored_slots = __ldcg(&gl.ignored_slots);
        *p.result = res;
        gl.invalid_slots = 0;
        gl.ignored_slots = 0;
        gl.units_done = 0;
        gl.error_flags = 0;
    }
}

// --------------------------------------------------------------------------
// the tail itself: kScanThreads threads of one CTA
// --------------------------------------------------------------------------
// `want` holds n_groups x kWords words; `consume` zeroes them after reading
// (they are the scan's accumulation words).
//
// Returns whether the plan is deliverable (the same answer in every thread).  It
// is not when the scan saw an id above the capacity, when a bounded wait of the
// scan gave up, or when there are more ranges than `cap`: the resident words
// are then put back to what they were before the call -- a plan that cannot be
// executed must not count as resident on the next step (the reference drops
// its record on any failure, experiments/slot_placement.py:140-147, and checks
// the slot range before it stamps anything, experiments/slot_feedback.py:42).
template <int kBar>
__device__ bool plan_tail(const PlanArgs &p, uint32_t *want, bool consume, unsigned char *raw) {
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // Scalars of `p` are copied to locals first: `p` lives in parameter space and
    // every global store below would otherwise force them to be re-read.
    const uint32_t G = p.n_groups, n = p.n_buffers;
    const uint32_t n_blocks = p.n_blocks, budget = p.budget, flags = p.flags;
    const bool explicit_sets = p.explicit_sets != 0, scan_only = p.scan_only != 0;
    uint32_t *const resident = p.resident, *const bitmaps_out = p.bitmaps_out;
    const uint32_t n_words = (n_blocks + 31) / 32;
    const TailShared sh = carve_tail(raw, G, n);
    // counters written by other CTAs: fetched now, used at the very end
    unsigned long long invalid = 0, ignored = 0;
    uint32_t eflags = 0;
    if (tid == 0) {
        invalid = __ldcg(&p.global->invalid_slots);
        ignored = __ldcg(&p.global->ignored_slots);
        eflags = __ldcg(&p.global->error_flags);
        sh.verdict[0] = (invalid != 0) | ((eflags & RT_RESULT_TIMEOUT) != 0);   // read after the barrier below
    }
    // the buffer -> bitmap table goes to shared memory; its load is in flight
    // together with the first mask words below
    const uint8_t *const table = p.buffer_group;
    const uint32_t table_first = tid < n ? __ldcg(&table[tid]) : 0u;

    // ---- pass A: one THREAD per (bitmap, word) ----
    PassA pa;
    pa.G = G; pa.n_words = n_words; pa.n_blocks = n_blocks; pa.budget = budget; pa.flags = flags;
    pa.consume = consume; pa.want = want; pa.resident = resident; pa.bitmaps_out = bitmaps_out;
    pa.group_size = p.group_size;
    uint32_t st[kWarpStats] = {0, 0, 0, 0, 0, 0, 0, 0};
    uint32_t some_runs = 0;
    if (explicit_sets) pass_a<kTailExplicit>(pa, sh, st, some_runs);
    else if (scan_only) pass_a<kTailScanOnly>(pa, sh, st, some_runs);
    else pass_a<kTailPlan>(pa, sh, st, some_runs);
    if (tid < n) sh.group_of[tid] = (uint8_t)table_first;
    for (uint32_t j = tid + kScanThreads; j < n; j += kScanThreads) sh.group_of[j] = __ldcg(&table[j]);
    if (scan_only && bitmaps_out)                                    // words past the ones in use
        for (uint32_t i = tid; i < G * kWords; i += kScanThreads)
            if ((i & (kWords - 1)) >= n_words) bitmaps_out[i] = 0;
#pragma unroll
    for (int q = 0; q < kWarpStats; ++q) st[q] = warp_sum(st[q]);
    if (lane == 0) {
#pragma unroll
        for (int q = 0; q < kWarpStats; ++q) sh.warp_stats[warp * kWarpStats + q] = st[q];
    }
    // steady state: nothing moves, so there is nothing to lay out
    const bool any_runs = cta_or<kBar, kScanThreads>(some_runs != 0);

    // ---- exclusive prefix sum of run counts over (phase, buffer) ----
    // With at most one item per thread (2*n_buffers <= 256, the usual case) the
    // thread that computed an item's offset is the one that writes its ranges,
    // so the offsets stay in registers and one barrier is saved.
    const uint32_t items = (scan_only || !any_runs) ? 0 : 2 * n;
    const bool one_each = items <= (uint32_t)kScanThreads;
    uint32_t total = 0, n_cpu = 0, my_at = 0;
    if (items) {
        const uint32_t per = one_each ? 1u : (items + kScanThreads - 1) / kScanThreads;
        const uint32_t first = tid * per;
        uint32_t local = 0;
        for (uint32_t k = 0; k < per; ++k) {
            const uint32_t i = first + k;
            if (i < items) {
                const uint32_t phase = i >= n, j = i - phase * n;
                local += sh.counts[sh.group_of[j] * 2 + phase];
            }
        }
        const uint32_t incl = warp_inclusive_sum(local, lane);
        if (lane == 31) sh.warp_tot[warp] = incl;
        cta_sync<kBar, kScanThreads>();
        uint32_t base = 0;
#pragma unroll
        for (uint32_t k = 0; k < (uint32_t)kTailWarps; ++k) {
            const uint32_t t = sh.warp_tot[k];
            base += k < warp ? t : 0u;
            total += t;
        }
        my_at = base + incl - local;
        if (one_each) {
            if (tid == n) sh.off[n] = my_at;                  // ranges of phase 0, for the result record
        } else {
            uint32_t run = my_at;
            for (uint32_t k = 0; k < per; ++k) {
                const uint32_t i = first + k;
                if (i < items) {
                    sh.off[i] = run;
                    const uint32_t phase = i >= n, j = i - phase * n;
                    run += sh.counts[sh.group_of[j] * 2 + phase];
                }
            }
            cta_sync<kBar, kScanThreads>();
        }
    }

    // ---- pass B: one thread per (phase, buffer) ----
    // Short run lists come ready-made from pass A; longer ones are read off the
    // mask words.  Where a buffer's ranges go is the prefix sum above.  (A warp
    // per (bitmap, phase) handing its run list to every buffer in turn took ten
    // dependent rounds for 40 bitmaps: 17 us for 160 ranges.)
    const unsigned long long block_bytes = p.block_bytes, alloc_bytes = p.alloc_bytes;
    const uint32_t cap = p.cap;
    const int32_t dst_gpu = p.dst_device;
    rt_range *const out = p.out;
    for (uint32_t i = tid; i < items; i += kScanThreads) {
        const uint32_t phase = i >= n, j = i - phase * n, g = sh.group_of[j];
        const uint32_t count = sh.counts[g * 2 + phase];
        if (!count) continue;
        const int32_t dst = phase ? dst_gpu : RT_DST_CPU;
        uint32_t at = one_each ? my_at : sh.off[i];
        if (count <= kFew) {
            const uint16_t *few = sh.few + (g * 2 + phase) * 2 * kFew;
            for (uint32_t q = 0; q < count; ++q)
                store_range(out, at + q, cap, j, dst, few[2 * q], few[2 * q + 1], block_bytes, alloc_bytes);
            continue;
        }
        const uint32_t *m = sh.masks + g * kMaskStride + phase * kWords;
        uint32_t below_top = 0;
        for (uint32_t k = 0; k < n_words; ++k) {
            const uint32_t word = m[k];
            uint32_t starts = run_starts(word, below_top);
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
                store_range(out, at, cap, j, dst, k * 32 + b, k * 32 + e, block_bytes, alloc_bytes);
                ++at;
            }
        }
    }
    cta_sync<kBar, kScanThreads>();
    // ---- deliverable? ----
    const bool scan_failed = sh.verdict[0] != 0;
    const bool delivered = !scan_failed && total <= cap;
    if (!delivered && !explicit_sets && !scan_only && !(flags & RT_PLAN_DRY_RUN)) {
        // pass A has stored the new resident words: put the old ones back
        for (uint32_t i = tid; i < G * n_words; i += kScanThreads) {
            const uint32_t g = i / n_words, w = i - g * n_words;
            const uint32_t *m = sh.masks + g * kMaskStride;
            resident[g * kWords + w] = (resident[g * kWords + w] & ~m[kWords + w]) | m[w];
        }
    }
    if (tid == 0) {
        if (items) n_cpu = sh.off[n];
        rt_plan_result res;
        uint32_t sum[kWarpStats] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
        for (int k = 0; k < kTailWarps; ++k)
#pragma unroll
            for (int q = 0; q < kWarpStats; ++q) sum[q] += sh.warp_stats[k * kWarpStats + q];
        // what the last block of a buffer lacks to a whole block
        const unsigned long long short_by = (unsigned long long)n_blocks * block_bytes - alloc_bytes;
        // after a failed scan the ranges come from incomplete bitmaps: none is reported
        res.n_ranges = scan_failed ? 0u : total;
        res.n_cpu_ranges = scan_failed ? 0u : n_cpu;
        res.flags = (total > cap ? RT_RESULT_OVERFLOW : 0u) | (invalid ? RT_RESULT_SLOT_RANGE : 0u) | eflags;
        res.blocks_touched = sum[0];
        res.blocks_desired = sum[1];
        res.blocks_added = sum[2];
        res.blocks_evicted = sum[3];
        res.reserved = 0;
        res.invalid_slots = invalid;
        res.ignored_slots = ignored;
        res.cpu_bytes = (scan_only || scan_failed) ? 0 : sum[4] * block_bytes - sum[6] * short_by;
        res.gpu_bytes = (scan_only || scan_failed) ? 0 : sum[5] * block_bytes - sum[7] * short_by;
        *p.result = res;
        // leave the scratch clean for the next launch
        GlobalScratch &gl = *p.global;
        gl.invalid_slots = 0;
        gl.ignored_slots = 0;
        gl.units_done = 0;
        gl.error_flags = 0;
    }
    return delivered;
}

}  // namespace rt
