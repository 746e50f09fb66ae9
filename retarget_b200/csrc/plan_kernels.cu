// Planner kernels for sm_100a.
//
// One launch per decode step does all of:
//   scan     slot ids -> per-bitmap "touched block" words (shared-memory bitmap
//            per CTA, one global atomicOr per non-zero word per CTA and bitmap)
//   tail     per bitmap, by the CTA that retires the bitmap's last work unit: budget
//            cut, diff against the resident words, run coalescing (one warp,
//            one 32-bit word per lane, ballot/popc/shuffle only)
//   finalize by the CTA that retires the last bitmap: prefix sum over
//            (phase, buffer) and emission of the byte ranges in queue order
// CTAs never wait for each other: hand-over is by arrival counters ("last one
// out does the next stage"), so nothing in here can hang.
//
// The path is index arithmetic bound by HBM reads; there is no contraction in
// it and no tensor-core work.
#include <cuda_runtime.h>

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

// Lowest `k` set bits of x.
__device__ __forceinline__ uint32_t lowest_bits(uint32_t x, uint32_t k) {
    if (k >= (uint32_t)__popc(x)) return x;
    if (k == 0) return 0;
    uint32_t pos = __fns(x, 0, (int)k + 1);      // position of the (k+1)-th set bit
    return x & ((1u << pos) - 1u);
}

// --------------------------------------------------------------------------
// scan: mark one slot id in the CTA's shared bitmap
// --------------------------------------------------------------------------
struct ScanCounters {
    uint32_t invalid;    // id above capacity
    uint32_t ignored;    // id below 1
};

__device__ __forceinline__ void mark_slot(long long s, const ScanArgs &a, uint32_t *s_bits,
                                          ScanCounters &c) {
    // valid ids are 1..capacity: one unsigned compare covers both ends
    unsigned long long u = (unsigned long long)(s - 1);
    if (u < a.capacity) {
        uint32_t v = (uint32_t)s;
        uint32_t blk = a.shift >= 0 ? (v >> a.shift) : (v / a.block_tokens);
        uint32_t w = blk >> 5, bit = 1u << (blk & 31);
        // Bitmaps saturate after the first few ids: test with a plain
        // shared load and only fall into the atomic when the bit is new.  Lanes
        // that need the same word elect one leader for a single atomicOr.
        if (!(s_bits[w] & bit)) {
            uint32_t active = __activemask();
            uint32_t peers = __match_any_sync(active, w);
            uint32_t bits = __reduce_or_sync(peers, bit);
            if ((uint32_t)(__ffs(peers) - 1) == (threadIdx.x & 31u)) atomicOr(&s_bits[w], bits);
        }
    } else if (s < 1) {
        ++c.ignored;
    } else {
        ++c.invalid;
    }
}

// One work unit: kChunkElems ids starting at the even index e0, of which
// [begin, end) belong to the unit's group.  Every thread holds kUnroll 16-byte
// pairs; bit 2u / 2u+1 of `mask` says whether v[u].x / v[u].y is a real id.
struct Chunk {
    longlong2 v[kUnroll];
    uint32_t mask;
};

__device__ __forceinline__ void load_chunk(const long long *slots, long long e0, long long begin,
                                           long long end, Chunk &ch) {
    const int tid = threadIdx.x;
    if (e0 >= begin && e0 + kChunkElems <= end) {
        // interior: kUnroll independent, fully coalesced 128-bit loads per thread
#pragma unroll
        for (int u = 0; u < kUnroll; ++u)
            ch.v[u] = __ldcs(reinterpret_cast<const longlong2 *>(
                slots + e0 + 2 * (u * kScanThreads + tid)));
        ch.mask = (1u << (2 * kUnroll)) - 1u;
    } else {
        ch.mask = 0;
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            long long i = e0 + 2 * (u * kScanThreads + tid);
            ch.v[u].x = ch.v[u].y = 0;
            if (i >= begin && i < end) { ch.v[u].x = __ldcs(slots + i); ch.mask |= 1u << (2 * u); }
            if (i + 1 >= begin && i + 1 < end) {
                ch.v[u].y = __ldcs(slots + i + 1);
                ch.mask |= 2u << (2 * u);
            }
        }
    }
}

__device__ __forceinline__ void mark_chunk(const Chunk &ch, const ScanArgs &a, uint32_t *s_bits,
                                           ScanCounters &c) {
    if (ch.mask == (1u << (2 * kUnroll)) - 1u) {
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            mark_slot(ch.v[u].x, a, s_bits, c);
            mark_slot(ch.v[u].y, a, s_bits, c);
        }
    } else {
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            if (ch.mask & (1u << (2 * u))) mark_slot(ch.v[u].x, a, s_bits, c);
            if (ch.mask & (2u << (2 * u))) mark_slot(ch.v[u].y, a, s_bits, c);
        }
    }
}

// Where work unit q lives.  `g` is a running hint (units are visited in
// ascending order), advanced past every group that ends before q.
struct UnitPos {
    uint32_t g;
    long long e0, begin, end;
};

template <bool kTable>
__device__ __forceinline__ UnitPos locate_unit(const ScanArgs &a, int q, uint32_t g_hint) {
    UnitPos u;
    long long lo, hi;
    int k;
    if (kTable) {
        int row = q / a.units_per_row;
        k = q - row * a.units_per_row;
        int len = a.lens[row];
        if (len < 0) len = 0;
        if ((long long)len > a.stride) len = (int)a.stride;
        lo = (long long)row * a.stride;
        hi = lo + len;
        u.g = 0;
    } else {
        uint32_t g = g_hint;
        while (q >= a.unit_first[g + 1]) ++g;
        k = q - a.unit_first[g];
        lo = a.group_off[g];
        hi = a.group_off[g + 1];
        u.g = g;
    }
    u.e0 = (lo & ~1LL) + (long long)k * kChunkElems;
    u.end = u.e0 + kChunkElems < hi ? u.e0 + kChunkElems : hi;
    u.begin = u.e0 > lo ? u.e0 : lo;
    if (u.begin > u.end) u.begin = u.end;
    return u;
}

// --------------------------------------------------------------------------
// tail: one warp turns a bitmap into evict/add run lists
// --------------------------------------------------------------------------
__device__ __forceinline__ void emit_runs(uint32_t m, uint32_t lane, uint16_t *run_begin,
                                          uint16_t *run_end, uint32_t *n_runs) {
    uint32_t prev_top = __shfl_up_sync(0xffffffffu, m, 1) >> 31;
    uint32_t next_low = __shfl_down_sync(0xffffffffu, m, 1) & 1u;
    if (lane == 0) prev_top = 0;
    if (lane == 31) next_low = 0;
    uint32_t starts = m & ~((m << 1) | prev_top);
    uint32_t lasts = m & ~((m >> 1) | (next_low << 31));
    uint32_t sb = warp_inclusive_sum(__popc(starts), lane);
    uint32_t eb = warp_inclusive_sum(__popc(lasts), lane);
    uint32_t total = __shfl_sync(0xffffffffu, sb, 31);
    sb -= __popc(starts);
    eb -= __popc(lasts);
    while (starts) {
        uint32_t b = __ffs(starts) - 1;
        starts &= starts - 1;
        run_begin[sb++] = (uint16_t)(lane * 32 + b);
    }
    while (lasts) {
        uint32_t b = __ffs(lasts) - 1;
        lasts &= lasts - 1;
        run_end[eb++] = (uint16_t)(lane * 32 + b + 1);
    }
    if (lane == 0) *n_runs = total;
}

// `raw` = this lane's word of the touched bitmap.
__device__ void group_tail(const PlanArgs &p, uint32_t g, uint32_t raw, uint32_t lane) {
    GroupScratch &gs = p.groups[g];
    // bits at or above n_blocks cannot be produced by valid ids; drop them anyway
    uint32_t lo_bit = lane * 32;
    uint32_t valid = p.n_blocks >= lo_bit + 32 ? 0xffffffffu
                     : (p.n_blocks > lo_bit ? ((1u << (p.n_blocks - lo_bit)) - 1u) : 0u);
    raw &= valid;
    uint32_t touched = warp_sum(__popc(raw));
    if (p.scan_only) {
        if (p.bitmaps_out) p.bitmaps_out[g * kWords + lane] = raw;
        if (lane == 0) {
            gs.touched = touched; gs.desired = 0; gs.added = 0; gs.evicted = 0;
            gs.n_runs[0] = 0; gs.n_runs[1] = 0;
        }
        return;
    }
    // budget cut: lowest block ids first (one event => all stamps tie, and ties
    // rank by ascending block id)
    uint32_t before = warp_inclusive_sum(__popc(raw), lane) - __popc(raw);
    uint32_t keep = p.budget > before ? p.budget - before : 0;
    uint32_t desired = lowest_bits(raw, keep);
    uint32_t res = p.resident[g * kWords + lane];
    uint32_t add = desired & ~res;
    uint32_t evict = (p.flags & RT_PLAN_EVICT) ? (res & ~desired) : 0u;
    if (!(p.flags & RT_PLAN_DRY_RUN)) p.resident[g * kWords + lane] = desired;
    emit_runs(evict, lane, gs.run_begin[0], gs.run_end[0], &gs.n_runs[0]);
    emit_runs(add, lane, gs.run_begin[1], gs.run_end[1], &gs.n_runs[1]);
    uint32_t n_des = warp_sum(__popc(desired));
    uint32_t n_add = warp_sum(__popc(add));
    uint32_t n_ev = warp_sum(__popc(evict));
    if (lane == 0) { gs.touched = touched; gs.desired = n_des; gs.added = n_add; gs.evicted = n_ev; }
}

// --------------------------------------------------------------------------
// finalize: the whole CTA lays the ranges out in queue order
// --------------------------------------------------------------------------
struct FinalizeShared {
    uint32_t off[2 * RT_MAX_BUFFERS + 1];
    uint32_t warp_tot[kScanThreads / 32];
    uint32_t stats[4];
    unsigned long long bytes[2];
};

__device__ void finalize(const PlanArgs &p, FinalizeShared &sh) {
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t nthr = blockDim.x, nwarp = nthr >> 5;
    const uint32_t items = p.scan_only ? 0 : 2 * p.n_buffers;
    if (tid < 4) sh.stats[tid] = 0;
    if (tid < 2) sh.bytes[tid] = 0;
    __syncthreads();
    // group statistics
    for (uint32_t g = tid; g < p.n_groups; g += nthr) {
        const GroupScratch &gs = p.groups[g];      // written by other CTAs: read through L2
        atomicAdd(&sh.stats[0], __ldcg(&gs.touched));
        atomicAdd(&sh.stats[1], __ldcg(&gs.desired));
        atomicAdd(&sh.stats[2], __ldcg(&gs.added));
        atomicAdd(&sh.stats[3], __ldcg(&gs.evicted));
    }
    // exclusive prefix sum of run counts over (phase, buffer)
    const uint32_t per = (items + nthr - 1) / nthr;
    const uint32_t first = tid * per;
    uint32_t local = 0;
    for (uint32_t k = 0; k < per; ++k) {
        uint32_t i = first + k;
        if (i < items) {
            uint32_t phase = i >= p.n_buffers;
            uint32_t j = i - phase * p.n_buffers;
            local += __ldcg(&p.groups[p.buffer_group[j]].n_runs[phase]);
        }
    }
    uint32_t incl = warp_inclusive_sum(local, lane);
    if (lane == 31) sh.warp_tot[warp] = incl;
    __syncthreads();
    uint32_t base = 0;
    for (uint32_t w = 0; w < warp; ++w) base += sh.warp_tot[w];
    uint32_t total = 0;
    for (uint32_t w = 0; w < nwarp; ++w) total += sh.warp_tot[w];
    uint32_t run = base + incl - local;
    for (uint32_t k = 0; k < per; ++k) {
        uint32_t i = first + k;
        if (i < items) {
            sh.off[i] = run;
            uint32_t phase = i >= p.n_buffers;
            uint32_t j = i - phase * p.n_buffers;
            run += __ldcg(&p.groups[p.buffer_group[j]].n_runs[phase]);
        }
    }
    if (tid == 0) sh.off[items] = total;
    __syncthreads();
    const uint32_t n_cpu = items ? sh.off[p.n_buffers] : 0;
    unsigned long long my_bytes[2] = {0, 0};
    for (uint32_t r = tid; r < total; r += nthr) {
        // last item whose offset is <= r
        uint32_t lo = 0, hi = items;
        while (hi - lo > 1) {
            uint32_t mid = (lo + hi) >> 1;
            if (sh.off[mid] <= r) lo = mid; else hi = mid;
        }
        uint32_t phase = lo >= p.n_buffers;
        uint32_t j = lo - phase * p.n_buffers;
        const GroupScratch &gs = p.groups[p.buffer_group[j]];
        uint32_t k = r - sh.off[lo];
        unsigned long long b = (unsigned long long)__ldcg(&gs.run_begin[phase][k]) * p.block_bytes;
        unsigned long long e = (unsigned long long)__ldcg(&gs.run_end[phase][k]) * p.block_bytes;
        if (e > p.alloc_bytes) e = p.alloc_bytes;       // final partial block, select.cpp:24188
        my_bytes[phase] += e - b;
        if (r < p.cap) {
            rt_range out;
            out.buffer = j;
            out.dst = phase ? p.dst_device : RT_DST_CPU;
            out.offset = b;
            out.bytes = e - b;
            p.out[r] = out;
        }
    }
    if (my_bytes[0]) atomicAdd(&sh.bytes[0], my_bytes[0]);
    if (my_bytes[1]) atomicAdd(&sh.bytes[1], my_bytes[1]);
    __syncthreads();
    if (tid == 0) {
        GlobalScratch &gl = *p.global;
        rt_plan_result res;
        res.n_ranges = total;
        res.n_cpu_ranges = n_cpu;
        unsigned long long invalid = *(volatile unsigned long long *)&gl.invalid_slots;
        uint32_t eflags = *(volatile uint32_t *)&gl.error_flags;
        res.flags = (total > p.cap ? RT_RESULT_OVERFLOW : 0u) | (invalid ? RT_RESULT_SLOT_RANGE : 0u) | eflags;
        res.blocks_touched = sh.stats[0];
        res.blocks_desired = sh.stats[1];
        res.blocks_added = sh.stats[2];
        res.blocks_evicted = sh.stats[3];
        res.reserved = 0;
        res.invalid_slots = invalid;
        res.ignored_slots = *(volatile unsigned long long *)&gl.ignored_slots;
        res.cpu_bytes = sh.bytes[0];
        res.gpu_bytes = sh.bytes[1];
        *p.result = res;
        // leave the scratch clean for the next launch
        gl.invalid_slots = 0;
        gl.ignored_slots = 0;
        gl.groups_done = 0;
        gl.error_flags = 0;
        __threadfence_system();
    }
}

// Hand-over after a CTA's bits for bitmap g reached the global words.  Returns after the
// CTA has done whatever stage fell to it.
struct HandoverShared {
    int role;      // 0 nothing, 1 run the group's tail, 2 tail + finalize
};

__device__ __forceinline__ void retire_units(const PlanArgs &p, uint32_t g, uint32_t count,
                                             uint32_t units_in_group, HandoverShared &hs,
                                             FinalizeShared &fs) {
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        uint32_t prev = atomicAdd(&p.groups[g].units_done, count);
        hs.role = prev + count == units_in_group;
    }
    __syncthreads();
    if (!hs.role) return;
    __threadfence();
    if (threadIdx.x < 32) {
        uint32_t lane = threadIdx.x;
        uint32_t raw = atomicExch(&p.groups[g].want[lane], 0u);   // consume + clean
        if (lane == 0) p.groups[g].units_done = 0;
        group_tail(p, g, raw, lane);
        __threadfence();
        __syncwarp();
        if (lane == 0) {
            uint32_t prev = atomicAdd(&p.global->groups_done, 1u);
            hs.role = prev + 1 == p.n_groups ? 2 : 1;
        }
    }
    __syncthreads();
    if (hs.role == 2) {
        __threadfence();
        finalize(p, fs);
    }
    __syncthreads();
}

__device__ __forceinline__ void flush_counters(const PlanArgs &p, ScanCounters &c) {
    // rare path: any thread of the CTA saw an id outside 1..capacity
    if (__syncthreads_or(c.invalid | c.ignored)) {
        uint32_t inv = warp_sum(c.invalid), ign = warp_sum(c.ignored);
        if ((threadIdx.x & 31) == 0) {
            if (inv) atomicAdd(&p.global->invalid_slots, (unsigned long long)inv);
            if (ign) atomicAdd(&p.global->ignored_slots, (unsigned long long)ign);
        }
        c.invalid = c.ignored = 0;
    }
}

// --------------------------------------------------------------------------
// kernel: plain 128-bit loads, register double buffering
// --------------------------------------------------------------------------
// CSR input: every CTA owns one contiguous span of work units, keeps its shared
// bitmap across the units of a group and hands over once per (CTA, group).
// Table input: units are dealt round-robin (rows have ragged lengths) and all
// belong to bitmap 0.
template <bool kTable>
__global__ void __launch_bounds__(kScanThreads)
scan_plan_kernel(const __grid_constant__ ScanArgs a, const __grid_constant__ PlanArgs p) {
    __shared__ uint32_t s_bits[kWords];
    __shared__ HandoverShared hs;
    __shared__ FinalizeShared fs;
    ScanCounters c = {0, 0};
    int q, q_end, q_step;
    if (kTable) {
        q = blockIdx.x; q_end = a.n_units; q_step = gridDim.x;
    } else {
        q = (int)((long long)a.n_units * blockIdx.x / gridDim.x);
        q_end = (int)((long long)a.n_units * (blockIdx.x + 1) / gridDim.x);
        q_step = 1;
    }
    if (q >= q_end) return;
    if (threadIdx.x < kWords) s_bits[threadIdx.x] = 0;
    uint32_t g0 = 0;
    if (!kTable) {
        // last group whose first unit is <= q
        int gl = 0, gh = a.n_groups;
        while (gh - gl > 1) {
            int mid = (gl + gh) >> 1;
            if (a.unit_first[mid] <= q) gl = mid; else gh = mid;
        }
        g0 = gl;
    }
    UnitPos cur = locate_unit<kTable>(a, q, g0);
    Chunk ch;
    load_chunk(a.slots, cur.e0, cur.begin, cur.end, ch);
    __syncthreads();
    uint32_t units_done = 0;
    for (;;) {
        int qn = q + q_step;
        UnitPos nxt = cur;
        Chunk chn;
        chn.mask = 0;
        if (qn < q_end) {                       // next unit's loads fly while this one is marked
            nxt = locate_unit<kTable>(a, qn, cur.g);
            load_chunk(a.slots, nxt.e0, nxt.begin, nxt.end, chn);
        }
        mark_chunk(ch, a, s_bits, c);
        ++units_done;
        bool last = qn >= q_end;
        if (last || nxt.g != cur.g) {
            uint32_t in_group = kTable ? (uint32_t)a.n_units
                                       : (uint32_t)(a.unit_first[cur.g + 1] - a.unit_first[cur.g]);
            __syncthreads();
            if (threadIdx.x < kWords && s_bits[threadIdx.x])
                atomicOr(&p.groups[cur.g].want[threadIdx.x], s_bits[threadIdx.x]);
            flush_counters(p, c);
            retire_units(p, cur.g, units_done, in_group, hs, fs);
            units_done = 0;
            if (threadIdx.x < kWords) s_bits[threadIdx.x] = 0;
            __syncthreads();
        }
        if (last) break;
        q = qn;
        cur = nxt;
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) ch.v[u] = chn.v[u];
        ch.mask = chn.mask;
    }
}

// --------------------------------------------------------------------------
// kernel: slot ids staged through shared memory with bulk async copies (TMA)
// --------------------------------------------------------------------------
// One elected thread keeps kStages 16 KiB copies in flight per CTA
// (cp.async.bulk global -> shared, completion counted on an mbarrier); all
// threads then read their ids from shared memory with conflict-free 128-bit
// loads.  Registers hold no staging data, so the bytes in flight per SM are set
// by shared memory (kStages x 16 KiB per CTA), not by occupancy.
//
// Every wait on an mbarrier is bounded; when the bound is hit the CTA records
// RT_RESULT_TIMEOUT, skips the unit and still retires it, so the grid always
// drains.
constexpr int kStages = 4;
constexpr int kStageBytes = kChunkElems * 8;
constexpr uint32_t kWaitLimit = 1u << 24;

__device__ __forceinline__ uint32_t smem_addr(const void *ptr) {
    return (uint32_t)__cvta_generic_to_shared(ptr);
}
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_test(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_addr(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t *bar, uint32_t parity) {
    for (uint32_t it = 0; it < kWaitLimit; ++it)
        if (mbar_test(bar, parity)) return true;
    return false;
}
__device__ __forceinline__ void bulk_load(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
            smem_addr(dst)),
        "l"(src), "r"(bytes), "r"(smem_addr(bar))
        : "memory");
}

__global__ void __launch_bounds__(kScanThreads)
scan_plan_tma_kernel(const __grid_constant__ ScanArgs a, const __grid_constant__ PlanArgs p) {
    extern __shared__ __align__(128) unsigned char stage_mem[];
    __shared__ __align__(8) uint64_t full_bar[kStages];
    __shared__ uint32_t s_bits[kWords];
    __shared__ HandoverShared hs;
    __shared__ FinalizeShared fs;
    const int tid = threadIdx.x;
    const int q_begin = (int)((long long)a.n_units * blockIdx.x / gridDim.x);
    const int q_end = (int)((long long)a.n_units * (blockIdx.x + 1) / gridDim.x);
    if (q_begin >= q_end) return;
    const long long copy_limit = a.group_off[a.n_groups] & ~1LL;   // whole 16-byte pairs only
    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) mbar_init(&full_bar[s], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (tid < kWords) s_bits[tid] = 0;
    uint32_t g0;
    {
        int gl = 0, gh = a.n_groups;
        while (gh - gl > 1) {
            int mid = (gl + gh) >> 1;
            if (a.unit_first[mid] <= q_begin) gl = mid; else gh = mid;
        }
        g0 = gl;
    }
    __syncthreads();

    // producer state (thread 0 only)
    int q_issue = q_begin;
    uint32_t g_issue = g0;
    auto issue = [&](int stage) {
        UnitPos u = locate_unit<false>(a, q_issue, g_issue);
        g_issue = u.g;
        long long hi = (u.end + 1) & ~1LL;
        if (hi > copy_limit) hi = copy_limit;
        long long n = hi - u.e0;
        if (n > 0) {
            mbar_expect_tx(&full_bar[stage], (uint32_t)(n * 8));
            bulk_load(stage_mem + stage * kStageBytes, a.slots + u.e0, (uint32_t)(n * 8), &full_bar[stage]);
        } else {
            mbar_arrive(&full_bar[stage]);
        }
        ++q_issue;
    };
    if (tid == 0)
        for (int s = 0; s < kStages && q_issue < q_end; ++s) issue(s);

    ScanCounters c = {0, 0};
    uint32_t units_done = 0, g_cur = g0;
    bool gave_up = false;
    for (int q = q_begin; q < q_end; ++q) {
        const int i = q - q_begin;
        const int stage = i % kStages;
        const uint32_t parity = (uint32_t)(i / kStages) & 1u;
        UnitPos u = locate_unit<false>(a, q, g_cur);
        if (u.g != g_cur) {
            // the CTA crosses into the next bitmap: hand the finished one over
            __syncthreads();
            if (tid < kWords && s_bits[tid]) atomicOr(&p.groups[g_cur].want[tid], s_bits[tid]);
            flush_counters(p, c);
            retire_units(p, g_cur, units_done, (uint32_t)(a.unit_first[g_cur + 1] - a.unit_first[g_cur]),
                         hs, fs);
            units_done = 0;
            if (tid < kWords) s_bits[tid] = 0;
            __syncthreads();
            g_cur = u.g;
        }
        long long copied_to = (u.end + 1) & ~1LL;
        if (copied_to > copy_limit) copied_to = copy_limit;
        bool ok = mbar_wait_bounded(&full_bar[stage], parity);
        if (ok) {
            const longlong2 *src = reinterpret_cast<const longlong2 *>(stage_mem + stage * kStageBytes);
            const bool interior = u.e0 >= u.begin && u.e0 + kChunkElems <= u.end;
            longlong2 v[kUnroll];
            if (interior) {
#pragma unroll
                for (int k = 0; k < kUnroll; ++k) v[k] = src[k * kScanThreads + tid];
#pragma unroll
                for (int k = 0; k < kUnroll; ++k) {
                    mark_slot(v[k].x, a, s_bits, c);
                    mark_slot(v[k].y, a, s_bits, c);
                }
            } else {
#pragma unroll
                for (int k = 0; k < kUnroll; ++k) {
                    long long idx = u.e0 + 2 * (k * kScanThreads + tid);
                    if (idx < copied_to) {
                        longlong2 w = src[k * kScanThreads + tid];
                        if (idx >= u.begin && idx < u.end) mark_slot(w.x, a, s_bits, c);
                        if (idx + 1 >= u.begin && idx + 1 < u.end) mark_slot(w.y, a, s_bits, c);
                    } else if (idx >= u.begin && idx < u.end) {
                        // odd last id of the whole array: not part of any 16-byte pair
                        mark_slot(__ldcs(a.slots + idx), a, s_bits, c);
                    }
                }
            }
        } else {
            gave_up = true;
        }
        ++units_done;
        __syncthreads();                     // everyone is done reading this stage
        if (tid == 0 && q_issue < q_end) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            issue(stage);
        }
    }
    if (gave_up) {
        if ((tid & 31) == 0) atomicOr(&p.global->error_flags, RT_RESULT_TIMEOUT);
        // give copies that may still be in flight one more bounded chance to land
        for (int s = 0; s < kStages; ++s) {
            int uses = (q_end - q_begin - s + kStages - 1) / kStages;
            if (uses > 0) mbar_wait_bounded(&full_bar[s], (uint32_t)(uses - 1) & 1u);
        }
    }
    __syncthreads();
    if (tid < kWords && s_bits[tid]) atomicOr(&p.groups[g_cur].want[tid], s_bits[tid]);
    flush_counters(p, c);
    retire_units(p, g_cur, units_done, (uint32_t)(a.unit_first[g_cur + 1] - a.unit_first[g_cur]), hs, fs);
}

// --------------------------------------------------------------------------
// kernel: wanted bitmaps given, no scan
// --------------------------------------------------------------------------
__global__ void __launch_bounds__(kScanThreads)
plan_tail_kernel(const uint32_t *want, const __grid_constant__ PlanArgs p) {
    __shared__ FinalizeShared fs;
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (uint32_t g = warp; g < p.n_groups; g += blockDim.x >> 5)
        group_tail(p, g, want[g * kWords + lane], lane);
    __threadfence();
    __syncthreads();
    finalize(p, fs);
}

// --------------------------------------------------------------------------
// host-side launchers (called from the C ABI)
// --------------------------------------------------------------------------
cudaError_t launch_scan_plan(const ScanArgs &a, const PlanArgs &p, bool table, int grid,
                             cudaStream_t stream) {
    if (table)
        scan_plan_kernel<true><<<grid, kScanThreads, 0, stream>>>(a, p);
    else
        scan_plan_kernel<false><<<grid, kScanThreads, 0, stream>>>(a, p);
    return cudaGetLastError();
}

cudaError_t launch_plan_tail(const uint32_t *want, const PlanArgs &p, cudaStream_t stream) {
    plan_tail_kernel<<<1, kScanThreads, 0, stream>>>(want, p);
    return cudaGetLastError();
}

cudaError_t launch_scan_plan_tma(const ScanArgs &a, const PlanArgs &p, int grid, cudaStream_t stream) {
    scan_plan_tma_kernel<<<grid, kScanThreads, kStages * kStageBytes, stream>>>(a, p);
    return cudaGetLastError();
}

cudaError_t scan_plan_occupancy(int *plain_blocks_per_sm, int *tma_blocks_per_sm) {
    cudaError_t e = cudaFuncSetAttribute(scan_plan_tma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         kStages * kStageBytes);
    if (e != cudaSuccess) return e;
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(plain_blocks_per_sm, scan_plan_kernel<false>,
                                                      kScanThreads, 0);
    if (e != cudaSuccess) return e;
    return cudaOccupancyMaxActiveBlocksPerMultiprocessor(tma_blocks_per_sm, scan_plan_tma_kernel,
                                                         kScanThreads, kStages * kStageBytes);
}

}  // namespace rt
