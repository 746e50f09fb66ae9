// Planner kernels for sm_100a.
//
// One launch per decode step does all of:
//   scan  slot ids -> per-bitmap "touched block" words: every CTA owns a
//         contiguous span of 16 KiB work units, marks blocks in a shared byte map
//         and folds it into the bitmap's global words (one atomicOr per non-zero
//         word) whenever it leaves a bitmap
//   tail  by the CTA that retires the launch's last work unit (plan_tail.cuh):
//         budget cut, diff against the resident words, run coalescing, prefix sum
//         over (phase, buffer), byte ranges in queue order, result record
// CTAs never wait for each other: hand-over is by one arrival counter ("last one
// out does the tail"), so nothing in here can hang.
//
// Chained launches (RT_PLAN_CHAINED): the kernel is launched with programmatic
// stream serialization.  Its scanning CTAs need nothing from the launch before
// it, so each of them executes griddepcontrol.launch_dependents as its first
// instruction.  CTA 0 of every launch is a GATEKEEPER: it scans nothing, it
// executes griddepcontrol.wait (the launch before this one has completed), then
// griddepcontrol.launch_dependents, and exits.  The next launch can therefore
// start once this launch's CTAs are all running AND the launch before this one
// has completed: its CTAs move onto an SM as soon as this launch's CTAs leave it
// (the ramp of step i+1 overlaps the drain of step i, and the one-CTA tail of
// step i runs under the scan of step i+1), yet no more than two consecutive
// launches are ever in flight, which is what lets them alternate between two
// scratch sets.  The CTA that runs a tail executes griddepcontrol.wait before it
// reads the resident words.  Nothing polls, nothing spins.
//
// The path is index arithmetic bound by HBM reads; there is no contraction in
// it and no tensor-core work.
#include <cuda_runtime.h>

#include "plan_device.cuh"
#include "plan_tail.cuh"

// Streaming load of slot ids: read once, never reused.
#ifndef RT_LOAD
#define RT_LOAD(ptr) __ldcs(ptr)
#endif

namespace rt {


// --------------------------------------------------------------------------
// scan: mark slot ids in the CTA's shared block map
// --------------------------------------------------------------------------
// The map is one BYTE per block (1 KiB for 1024 blocks).  Marking a block is a
// single plain shared store of 1: idempotent, so it needs no read, no atomic
// and no branch.  (A bit map with test + atomicOr cost ~39 instructions per id
// in measurement and left the kernel issue-bound at a third of HBM speed.)  The
// bytes are folded into 32-bit words with warp ballots when the CTA leaves a
// bitmap.
struct ScanCounters {
    uint32_t invalid;    // id above capacity
    uint32_t ignored;    // id below 1
};

// slot -> block.  Power-of-two block sizes shift; others use an exact
// multiply-shift division (round-up magic with the 33-bit "add" fix-up, valid
// for every 32-bit numerator), so no hardware-emulated divide sits in the loop.
template <bool kPow2>
__device__ __forceinline__ uint32_t block_of(uint32_t slot, const ScanArgs &a) {
    if (kPow2) return slot >> a.shift;
    uint32_t q = __umulhi(slot, a.magic);
    return (((slot - q) >> 1) + q) >> a.magic_shift;
}

// Exact classification of one id (slow path).
template <bool kPow2>
__device__ __forceinline__ void mark_slot(long long s, const ScanArgs &a, uint8_t *s_map,
                                          ScanCounters &c) {
    unsigned long long u = (unsigned long long)(s - 1);
    if (u < a.capacity) s_map[block_of<kPow2>((uint32_t)s, a)] = 1;
    else if (s < 1) ++c.ignored;
    else ++c.invalid;
}

// Slot ids arrive as int64 (the CSR tables the planner was first written for)
// or as int32 (the serving engine's own kv_indices / req_to_token tensors).  A
// thread always loads 16 bytes at a time: two or four ids.
template <typename Id> struct IdTraits;
template <> struct IdTraits<long long> {
    using Vec = longlong2;
    static constexpr int kPer = 2;
};
template <> struct IdTraits<int> {
    using Vec = int4;
    static constexpr int kPer = 4;
};
// ids of one work unit (16 KiB): 2048 int64 or 4096 int32
template <typename Id>
constexpr int kChunkIds = kScanThreads * IdTraits<Id>::kPer * kUnroll;
static_assert(kChunkIds<long long> == kChunkElems, "unit size mismatch");
template <typename Id>
constexpr uint32_t kAllIdsOf = (1u << (IdTraits<Id>::kPer * kUnroll)) - 1u;
constexpr uint32_t kAllIds = kAllIdsOf<long long>;

__device__ __forceinline__ long long vec_get(const longlong2 &v, int k) { return k ? v.y : v.x; }
__device__ __forceinline__ int vec_get(const int4 &v, int k) {
    return k == 0 ? v.x : k == 1 ? v.y : k == 2 ? v.z : v.w;
}
__device__ __forceinline__ void vec_set(longlong2 &v, int k, long long x) { (k ? v.y : v.x) = x; }
__device__ __forceinline__ void vec_set(int4 &v, int k, int x) {
    (k == 0 ? v.x : k == 1 ? v.y : k == 2 ? v.z : v.w) = x;
}
template <typename Vec> struct VecIds;
template <> struct VecIds<longlong2> { static constexpr int kPer = 2; };
template <> struct VecIds<int4> { static constexpr int kPer = 4; };

// Folds one 16-byte vector into the batch test: OR of the high words (int64
// only) and the largest (id - 1) as an unsigned 32-bit number -- an id of 0, and
// every negative int32, wraps to a value no capacity reaches.
__device__ __forceinline__ void batch_test(const longlong2 &v, uint32_t &hi_or, uint32_t &worst) {
    hi_or |= (uint32_t)((unsigned long long)v.x >> 32) | (uint32_t)((unsigned long long)v.y >> 32);
    worst = max(worst, max((uint32_t)v.x - 1u, (uint32_t)v.y - 1u));
}
__device__ __forceinline__ void batch_test(const int4 &v, uint32_t &hi_or, uint32_t &worst) {
    worst = max(max(worst, max((uint32_t)v.x - 1u, (uint32_t)v.y - 1u)),
                max((uint32_t)v.z - 1u, (uint32_t)v.w - 1u));
}

// kUnroll 16-byte vectors, all of them real ids.
template <bool kPow2, typename Vec>
__device__ __forceinline__ void mark_full(const Vec (&v)[kUnroll], const ScanArgs &a,
                                          uint8_t *s_map, ScanCounters &c) {
    constexpr int kPer = VecIds<Vec>::kPer;
    // Fast path: one test for the whole batch.  Every id must be 1..capacity
    // (< 2^32); then the stores run unconditionally.
    uint32_t hi_or = 0, worst = 0;
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) batch_test(v[u], hi_or, worst);
    if (hi_or == 0 && worst < (uint32_t)a.capacity) {
#pragma unroll
        for (int u = 0; u < kUnroll; ++u)
#pragma unroll
            for (int k = 0; k < kPer; ++k) s_map[block_of<kPow2>((uint32_t)vec_get(v[u], k), a)] = 1;
        return;
    }
    // some id is 0, negative or above capacity: classify each one exactly
#pragma unroll
    for (int u = 0; u < kUnroll; ++u)
#pragma unroll
        for (int k = 0; k < kPer; ++k) mark_slot<kPow2>((long long)vec_get(v[u], k), a, s_map, c);
}

// Same with a validity mask: bit kPer*u + k says whether id k of v[u] is real.
// A vector whose ids are all real still gets the one-test fast path; only the
// vectors that straddle the ends of the id list are classified id by id.
template <bool kPow2, typename Vec>
__device__ __forceinline__ void mark_masked(const Vec (&v)[kUnroll], uint32_t mask,
                                            const ScanArgs &a, uint8_t *s_map, ScanCounters &c) {
    constexpr int kPer = VecIds<Vec>::kPer;
    constexpr uint32_t kWhole = (1u << kPer) - 1u;
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
        const uint32_t bits = (mask >> (kPer * u)) & kWhole;
        if (bits == kWhole) {
            uint32_t hi_or = 0, worst = 0;
            batch_test(v[u], hi_or, worst);
            if (hi_or == 0 && worst < (uint32_t)a.capacity) {
#pragma unroll
                for (int k = 0; k < kPer; ++k) s_map[block_of<kPow2>((uint32_t)vec_get(v[u], k), a)] = 1;
                continue;
            }
        }
#pragma unroll
        for (int k = 0; k < kPer; ++k)
            if (bits & (1u << k)) mark_slot<kPow2>((long long)vec_get(v[u], k), a, s_map, c);
    }
}

// One work unit as registers: kChunkIds ids starting at the 16-byte aligned
// index e0, of which [begin, end) belong to the unit's group.
template <typename Id>
struct Chunk {
    typename IdTraits<Id>::Vec v[kUnroll];
    uint32_t mask;
};

// `mine` points at this thread's first vector of the unit (slots + e0 + kPer*tid).
template <typename Id>
__device__ __forceinline__ void load_chunk(const Id *mine, long long e0, long long begin,
                                           long long end, Chunk<Id> &ch) {
    using Vec = typename IdTraits<Id>::Vec;
    constexpr int kPer = IdTraits<Id>::kPer;
    if (e0 >= begin && e0 + kChunkIds<Id> <= end) {
        // interior: kUnroll independent, fully coalesced 128-bit loads per thread
#pragma unroll
        for (int u = 0; u < kUnroll; ++u)
            ch.v[u] = RT_LOAD(reinterpret_cast<const Vec *>(mine + kPer * u * kScanThreads));
        ch.mask = kAllIdsOf<Id>;
    } else {
        ch.mask = 0;
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const long long i = e0 + kPer * (u * kScanThreads + (int)threadIdx.x);
            if (i >= begin && i + kPer <= end) {         // whole vector inside: one 128-bit load
                ch.v[u] = RT_LOAD(reinterpret_cast<const Vec *>(mine + kPer * u * kScanThreads));
                ch.mask |= ((1u << kPer) - 1u) << (kPer * u);
                continue;
            }
#pragma unroll
            for (int k = 0; k < kPer; ++k) {
                Id x = 0;
                if (i + k >= begin && i + k < end) {
                    x = RT_LOAD(mine + kPer * u * kScanThreads + k);
                    ch.mask |= 1u << (kPer * u + k);
                }
                vec_set(ch.v[u], k, x);
            }
        }
    }
}

template <bool kPow2, typename Id>
__device__ __forceinline__ void mark_chunk(const Chunk<Id> &ch, const ScanArgs &a, uint8_t *s_map,
                                           ScanCounters &c) {
    if (ch.mask == kAllIdsOf<Id>) mark_full<kPow2>(ch.v, a, s_map, c);
    else mark_masked<kPow2>(ch.v, ch.mask, a, s_map, c);
}

// The part of bitmap g that falls to a CTA owning work units [q_begin, q_end).
struct GroupSpan {
    int q_lo, q_hi;          // units of this group handled here
    int units_in_group;
    long long lo, hi;        // the group's ids
    long long e0;            // even start index of unit q_lo
};

template <typename Id = long long>
__device__ __forceinline__ GroupSpan group_span(const ScanArgs &a, uint32_t g, int q_begin, int q_end) {
    GroupSpan s;
    const int uf = a.unit_first[g], ul = a.unit_first[g + 1];
    s.q_lo = q_begin > uf ? q_begin : uf;
    s.q_hi = q_end < ul ? q_end : ul;
    s.units_in_group = ul - uf;
    s.lo = a.group_off[g];
    s.hi = a.group_off[g + 1];
    s.e0 = (s.lo & ~(long long)(IdTraits<Id>::kPer - 1)) + (long long)(s.q_lo - uf) * kChunkIds<Id>;
    return s;
}

__device__ __forceinline__ uint32_t first_group(const ScanArgs &a, int q) {
    // last group whose first unit is <= q
    int gl = 0, gh = a.n_groups;
    while (gh - gl > 1) {
        int mid = (gl + gh) >> 1;
        if (a.unit_first[mid] <= q) gl = mid; else gh = mid;
    }
    return (uint32_t)gl;
}

// --------------------------------------------------------------------------
// hand-over between the scan and the tail
// --------------------------------------------------------------------------
struct HandoverShared {
    int last;      // this CTA retired the last work unit of the launch
};

// Programmatic dependent launch.  Both are no-ops in a kernel that was launched
// without the attribute.
__device__ __forceinline__ void griddep_wait() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
}
__device__ __forceinline__ void griddep_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// First statement of every scan kernel.  Returns true in the gatekeeper CTA,
// which has then done all it is there for; the others continue as worker
// number blockIdx.x - 1 of gridDim.x - 1.
__device__ __forceinline__ bool gatekeeper() {
    if (blockIdx.x != 0) {
        griddep_launch_dependents();
        return false;
    }
    griddep_wait();                 // the launch before this one has completed ...
    griddep_launch_dependents();    // ... so the one after this one may use its scratch set
    return true;
}

template <int kBar>
__device__ __forceinline__ void flush_counters(const PlanArgs &p, ScanCounters &c) {
    // rare path: any thread of the CTA saw an id outside 1..capacity
    if (cta_or<kBar, kScanThreads>((c.invalid | c.ignored) != 0)) {
        uint32_t inv = warp_sum(c.invalid), ign = warp_sum(c.ignored);
        if ((threadIdx.x & 31) == 0) {
            if (inv) atomicAdd(&p.global->invalid_slots, (unsigned long long)inv);
            if (ign) atomicAdd(&p.global->ignored_slots, (unsigned long long)ign);
        }
        c.invalid = c.ignored = 0;
    }
}

__device__ __forceinline__ void clear_map(uint8_t *s_map) {
    reinterpret_cast<uint32_t *>(s_map)[threadIdx.x] = 0;      // 256 threads x 4 bytes
}

// Byte map -> 32-bit words by ballot, OR-ed into the bitmap's global words.
// Call between two CTA barriers.
__device__ __forceinline__ void flush_map(const PlanArgs &p, uint32_t g, const uint8_t *s_map) {
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    constexpr int kPerWarp = kWords / (kScanThreads / 32);
#pragma unroll
    for (int k = 0; k < kPerWarp; ++k) {
        uint32_t word = warp * kPerWarp + k;
        uint32_t bits = __ballot_sync(0xffffffffu, s_map[word * 32 + lane] != 0);
        if (lane == 0 && bits) atomicOr(&p.groups[g].want[word], bits);
    }
}

// The CTA leaves bitmap g: publish its bits and counters, start a clean map.
template <int kBar>
__device__ __forceinline__ void leave_group(const PlanArgs &p, uint32_t g, uint8_t *s_map,
                                            ScanCounters &c) {
    cta_sync<kBar, kScanThreads>();
    flush_map(p, g, s_map);
    flush_counters<kBar>(p, c);
    clear_map(s_map);
    cta_sync<kBar, kScanThreads>();
}

// The CTA is done with its `count` work units.  Whoever brings the launch-wide
// counter to the total runs the tail; nobody waits for anybody.
// `tail_mem_unsafe`: this CTA gave up waiting for a bulk copy into the memory
// the tail would work in.  A copy that lands late could overwrite the tail's
// working set, so the CTA then only cleans up (tail_abort) and plans nothing.
template <int kBar>
__device__ __forceinline__ void finish_cta(const PlanArgs &p, uint32_t count, HandoverShared &hs,
                                           unsigned char *tail_mem, bool tail_mem_unsafe = false) {
    __threadfence();                      // this CTA's atomicOr / atomicAdd before the arrival
    cta_sync<kBar, kScanThreads>();
    if (threadIdx.x == 0) {
        uint32_t prev = atomicAdd(&p.global->units_done, count);
        hs.last = prev + count == p.n_units;
    }
    cta_sync<kBar, kScanThreads>();
    if (!hs.last) return;
    __threadfence();
    // the launch before this one has completed: its resident words, ranges and result are final
    griddep_wait();
    if (tail_mem_unsafe) tail_abort(p);
    else plan_tail<kBar>(p, &p.groups[0].want[0], true, tail_mem);
}

// --------------------------------------------------------------------------
// kernel: CSR input, plain 128-bit loads, register double buffering
// --------------------------------------------------------------------------
// Every CTA owns one contiguous span of work units (16 KiB each), walks it
// bitmap by bitmap, keeps its shared block map across a bitmap's part of the
// span and hands over once per (CTA, bitmap).  Inside a bitmap the next unit's
// loads are issued before the current unit is marked.  (Dealing the work out in
// 4 KiB units instead, so that no CTA is a whole unit short of the others,
// measured 1.5-5 % slower: the launch is bound by HBM, not by its slowest CTA,
// and the part-units at both ends of every span cost more than they save.)
#ifdef RT_MIN_CTAS
#define RT_SCAN_BOUNDS __launch_bounds__(kScanThreads, RT_MIN_CTAS)
#else
#define RT_SCAN_BOUNDS __launch_bounds__(kScanThreads)
#endif
template <bool kPow2, typename Id>
__global__ void RT_SCAN_BOUNDS
scan_plan_kernel(const __grid_constant__ ScanArgs a, const __grid_constant__ PlanArgs p) {
    using Vec = typename IdTraits<Id>::Vec;
    constexpr int kPer = IdTraits<Id>::kPer;
    constexpr int kChunk = kChunkIds<Id>;
    extern __shared__ __align__(16) unsigned char tail_mem[];
    __shared__ __align__(16) uint8_t s_map[RT_MAX_BLOCKS];
    __shared__ HandoverShared hs;
    if (gatekeeper()) return;
    const uint32_t worker = blockIdx.x - 1, n_workers = gridDim.x - 1;
    const int q_begin = (int)((long long)a.n_units * worker / n_workers);
    const int q_end = (int)((long long)a.n_units * (worker + 1) / n_workers);
    if (q_begin >= q_end) return;
    const Id *slots = reinterpret_cast<const Id *>(a.slots);
    ScanCounters c = {0, 0};
    clear_map(s_map);
    __syncthreads();
    for (uint32_t g = first_group(a, q_begin);; ++g) {
        const GroupSpan sp = group_span<Id>(a, g, q_begin, q_end);
        // this CTA's part of the bitmap's ids: [begin, end), read from the 16-byte
        // aligned index e0 <= begin on
        long long e0 = sp.e0;
        const long long span_end = sp.e0 + (long long)(sp.q_hi - sp.q_lo) * kChunk;
        const long long begin = e0 > sp.lo ? e0 : sp.lo, end = span_end < sp.hi ? span_end : sp.hi;
        const Id *mine = slots + e0 + kPer * (int)threadIdx.x;
        // ragged first chunk of the bitmap (its first id is not on a 16-byte boundary)
        if (e0 < begin && begin < end) {
            Chunk<Id> ch;
            load_chunk<Id>(mine, e0, begin, end, ch);
            mark_chunk<kPow2, Id>(ch, a, s_map, c);
            e0 += kChunk; mine += kChunk;
        }
        // whole chunks: two register sets alternate, so the loads of one chunk are
        // in flight while the other is marked, with no copies between them
        const int n_whole = end > e0 ? (int)((end - e0) / kChunk) : 0;
        if (n_whole > 0) {
            Vec va[kUnroll], vb[kUnroll];
#pragma unroll
            for (int u = 0; u < kUnroll; ++u)
                va[u] = RT_LOAD(reinterpret_cast<const Vec *>(mine + kPer * u * kScanThreads));
            int left = n_whole;
            while (left >= 2) {
#pragma unroll
                for (int u = 0; u < kUnroll; ++u)
                    vb[u] = RT_LOAD(reinterpret_cast<const Vec *>(mine + kChunk + kPer * u * kScanThreads));
                mark_full<kPow2>(va, a, s_map, c);
                mine += 2 * kChunk;
                left -= 2;
                if (left > 0) {
#pragma unroll
                    for (int u = 0; u < kUnroll; ++u)
                        va[u] = RT_LOAD(reinterpret_cast<const Vec *>(mine + kPer * u * kScanThreads));
                }
                mark_full<kPow2>(vb, a, s_map, c);
            }
            if (left == 1) {
                mark_full<kPow2>(va, a, s_map, c);
                mine += kChunk;
            }
            e0 += (long long)n_whole * kChunk;
        }
        // what is left of the part: less than a chunk
        if (e0 < end) {
            Chunk<Id> ch;
            load_chunk<Id>(mine, e0, begin, end, ch);
            mark_chunk<kPow2, Id>(ch, a, s_map, c);
        }
        leave_group<0>(p, g, s_map, c);
        if (sp.q_hi >= q_end) break;
    }
    finish_cta<0>(p, (uint32_t)(q_end - q_begin), hs, tail_mem);
}

// --------------------------------------------------------------------------
// kernel: padded [rows, stride] table (the serving engine's req_to_token)
// --------------------------------------------------------------------------
// Row r holds lens[r] valid ids at table[r * stride ..]; the rest of the row is
// padding that is never read.  Work is dealt by ROW SEGMENT (seg_ids ids of one
// row).  All ids feed bitmap 0.  Two ways to walk the segments, chosen by the
// host from the segment length:
//
//   kWarpSegs   segments of a few hundred ids or more (the serving engine's
//               request rows): one WARP per segment, segments dealt round-robin
//               over all warps of the grid.  A lane takes every 32nd 16-byte
//               vector, kUnroll of them in flight with the next kUnroll issued
//               before these are marked; the next segment's length is fetched
//               while this one streams, so no dependent load sits between rows.
//   otherwise   short rows: segments are dealt round-robin over the CTAs.  A CTA
//               first turns its segments into a list of 16-byte vectors (per
//               segment the number of vectors that hold valid ids, exclusive
//               prefix sum in shared memory) and streams the flattened list --
//               256 threads x kUnroll loads per batch, each thread finding its
//               vector's segment with a cursor that only moves forward -- so
//               rows of a few ids still fill every lane.
constexpr int kSegsPerPass = 1024;
constexpr int kWarpSegVectors = 64;     // shortest segment (in 16-byte vectors) that gets a warp of its own

struct TableSeg {
    long long lo, hi;        // valid ids of the segment: flat indices [lo, hi)
};

struct TableShared {
    TableSeg seg[kSegsPerPass];
    unsigned int vec_before[kSegsPerPass + 1];   // exclusive prefix of the segments' vector counts
    unsigned int warp_sum[kScanThreads / 32];
};

// Batch `b` of the flattened list: kUnroll vectors per thread.  `cur` is the
// thread's cursor into the segment list; it only moves forward.
template <typename Id>
__device__ __forceinline__ void fetch_table_batch(const Id *slots, const TableShared &sh, int n_segs,
                                                  unsigned int total, unsigned int base, int &cur,
                                                  Chunk<Id> &ch) {
    using Vec = typename IdTraits<Id>::Vec;
    constexpr int kPer = IdTraits<Id>::kPer;
    constexpr uint32_t kWhole = (1u << kPer) - 1u;
    ch.mask = 0;
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
        const unsigned int vi = base + (unsigned int)(u * kScanThreads) + threadIdx.x;
        if (vi >= total) continue;
        while (cur + 1 < n_segs && vi >= sh.vec_before[cur + 1]) ++cur;
        const long long lo = sh.seg[cur].lo, hi = sh.seg[cur].hi;
        // the segment's first vector starts at the 16-byte boundary at or below `lo`
        const long long i0 = (lo & ~(long long)(kPer - 1)) + (long long)(vi - sh.vec_before[cur]) * kPer;
        if (i0 >= lo && i0 + kPer <= hi) {
            ch.v[u] = RT_LOAD(reinterpret_cast<const Vec *>(slots + i0));
            ch.mask |= kWhole << (kPer * u);
        } else {
            // first or last vector of a segment: only the ids inside it are read
#pragma unroll
            for (int k = 0; k < kPer; ++k) {
                Id x = 0;
                if (i0 + k >= lo && i0 + k < hi) {
                    x = RT_LOAD(slots + i0 + k);
                    ch.mask |= 1u << (kPer * u + k);
                }
                vec_set(ch.v[u], k, x);
            }
        }
    }
}

// Valid ids [lo, hi) of segment `seg` of row `row` (flat indices into the table).
__device__ __forceinline__ void table_segment(const ScanArgs &a, uint32_t row, uint32_t seg, long long len,
                                              long long &lo, long long &hi) {
    if (len < 0) len = 0;
    if (len > a.stride) len = a.stride;
    const long long row_lo = (long long)row * a.stride;
    lo = row_lo + (long long)seg * a.seg_ids;
    hi = lo + a.seg_ids;
    if (hi > row_lo + len) hi = row_lo + len;
    if (hi < lo) hi = lo;
}

// A warp's walk over its segments (kWarpSegs).  The segments of a warp, laid end
// to end, form one sequence of 16-byte vectors; lane l takes vectors l, l + 32,
// ... of that sequence, so every batch of 32 * kUnroll vectors is full whatever
// the segment lengths are.  Each lane keeps its own cursor (all lanes walk the
// same segments, a few vectors apart); the length of the segment after the
// current one is always already on its way.  Segment numbers advance by the
// number of warps in the grid; (row, segment-in-row) are stepped along with
// precomputed quotient and remainder, so the walk contains no division.
struct SegCursor {
    uint32_t row, seg;           // current segment
    uint32_t row_next, seg_next; // the one after it
    uint32_t first;              // index of the current segment's first vector in the warp's sequence
    uint32_t n_vec;              // vectors in it
    long long lo, hi, i0;        // its valid ids [lo, hi); its first vector starts at flat index i0
    long long len_next;          // valid ids of row_next
    bool done;
};

struct SegStride {
    uint32_t rows, segs;         // advance of (row, segment-in-row) from one of a warp's segments to the next
};

template <typename Id>
__device__ __forceinline__ void enter_segment(const ScanArgs &a, const SegStride &step, SegCursor &c) {
    constexpr int kPer = IdTraits<Id>::kPer;
    c.row = c.row_next;
    c.seg = c.seg_next;
    table_segment(a, c.row, c.seg, c.len_next, c.lo, c.hi);
    c.i0 = c.lo & ~(long long)(kPer - 1);
    c.n_vec = c.hi > c.lo ? (uint32_t)((c.hi - c.i0 + kPer - 1) / kPer) : 0u;
    c.seg_next = c.seg + step.segs;
    c.row_next = c.row + step.rows;
    if (c.seg_next >= a.segs_per_row) {
        c.seg_next -= a.segs_per_row;
        ++c.row_next;
    }
    // (a row number past the table marks the end; rows * segments is below 2^32 * 2^32, the sum cannot wrap
    //  before it passes n_rows because step.rows < n_rows whenever a warp has a second segment)
    c.len_next = c.row_next < a.n_rows ? (long long)__ldg(a.lens + c.row_next) : 0;
}

// Vectors base + lane + 32 u (u < kUnroll) of the warp's sequence.
template <typename Id>
__device__ __forceinline__ void fetch_warp_batch(const Id *slots, const ScanArgs &a, const SegStride &step,
                                                 uint32_t base, uint32_t lane, SegCursor &c, Chunk<Id> &ch) {
    using Vec = typename IdTraits<Id>::Vec;
    constexpr int kPer = IdTraits<Id>::kPer;
    constexpr uint32_t kWhole = (1u << kPer) - 1u;
    // Common case: all of this lane's vectors lie strictly inside the current
    // segment (neither its first nor its last vector, which may be partly
    // padding): kUnroll whole-vector loads off one pointer, nothing to test.
    const uint32_t rel = base + lane - c.first;               // wraps far above n_vec once the segment is behind
    if (!c.done && rel >= 1u && (unsigned long long)rel + 32u * (kUnroll - 1) + 1u < c.n_vec) {
        const Vec *src = reinterpret_cast<const Vec *>(slots + c.i0) + rel;
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) ch.v[u] = RT_LOAD(src + 32 * u);
        ch.mask = kAllIdsOf<Id>;
        return;
    }
    ch.mask = 0;
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
        const uint32_t vi = base + lane + 32u * (unsigned)u;
        while (!c.done && vi - c.first >= c.n_vec) {
            c.first += c.n_vec;
            if (c.row_next >= a.n_rows) c.done = true;
            else enter_segment<Id>(a, step, c);
        }
        if (c.done) continue;
        const long long at = c.i0 + (long long)((vi - c.first) * (uint32_t)kPer);
        if (at >= c.lo && at + kPer <= c.hi) {
            ch.v[u] = RT_LOAD(reinterpret_cast<const Vec *>(slots + at));
            ch.mask |= kWhole << (kPer * u);
        } else {
            // first or last vector of a segment: only the ids inside it are read
#pragma unroll
            for (int k = 0; k < kPer; ++k) {
                Id x = 0;
                if (at + k >= c.lo && at + k < c.hi) {
                    x = RT_LOAD(slots + at + k);
                    ch.mask |= 1u << (kPer * u + k);
                }
                vec_set(ch.v[u], k, x);
            }
        }
    }
}

template <bool kPow2, typename Id, bool kWarpSegs>
__global__ void __launch_bounds__(kScanThreads, 4)
scan_table_kernel(const __grid_constant__ ScanArgs a, const __grid_constant__ PlanArgs p) {
    constexpr int kPer = IdTraits<Id>::kPer;
    extern __shared__ __align__(16) unsigned char tail_mem[];
    __shared__ __align__(16) uint8_t s_map[RT_MAX_BLOCKS];
    __shared__ HandoverShared hs;
    const Id *slots = reinterpret_cast<const Id *>(a.slots);
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (gatekeeper()) return;
    const uint32_t worker = blockIdx.x - 1, n_workers = gridDim.x - 1;
    ScanCounters c = {0, 0};
    clear_map(s_map);
    const unsigned long long n_virtual = (unsigned long long)a.n_rows * a.segs_per_row;
    if (kWarpSegs) {
        __syncthreads();                         // the map is clear before any warp marks
        // this warp's segments: its global index, then every n_warps-th
        const unsigned long long n_warps = (unsigned long long)n_workers * (kScanThreads / 32);
        const unsigned long long mine0 = (unsigned long long)worker * (kScanThreads / 32) + warp;
        SegStride step;
        step.rows = (uint32_t)(n_warps / a.segs_per_row);
        step.segs = (uint32_t)(n_warps % a.segs_per_row);
        SegCursor cur;
        cur.row = cur.seg = cur.first = cur.n_vec = 0;
        cur.lo = cur.hi = cur.i0 = 0;
        cur.row_next = (uint32_t)(mine0 / a.segs_per_row);
        cur.seg_next = (uint32_t)(mine0 % a.segs_per_row);
        cur.done = mine0 >= n_virtual;
        cur.len_next = cur.done ? 0 : (long long)__ldg(a.lens + cur.row_next);
        if (!cur.done) enter_segment<Id>(a, step, cur);
        constexpr uint32_t kWarpBatch = 32u * kUnroll;
        Chunk<Id> now, nxt;
        uint32_t base = 0;
        fetch_warp_batch<Id>(slots, a, step, base, lane, cur, now);
        // the next batch is in flight while this one is marked; a batch that is
        // empty in every lane is past the warp's last vector
        while (__any_sync(0xffffffffu, now.mask != 0)) {
            base += kWarpBatch;
            fetch_warp_batch<Id>(slots, a, step, base, lane, cur, nxt);
            if (now.mask) mark_chunk<kPow2, Id>(now, a, s_map, c);
            now = nxt;
        }
        leave_group<0>(p, 0, s_map, c);
        finish_cta<0>(p, 1u, hs, tail_mem);
        return;
    }
    __shared__ TableShared sh;
    // this CTA's segments: worker, worker + n_workers, ...
    const unsigned long long mine = n_virtual > worker ? (n_virtual - worker + n_workers - 1) / n_workers : 0;
    for (unsigned long long pass = 0; pass < mine; pass += kSegsPerPass) {
        const int n_segs = (int)(mine - pass < (unsigned long long)kSegsPerPass ? mine - pass : kSegsPerPass);
        __syncthreads();                         // the previous pass is done with the lists
        // ---- the segment list: 4 consecutive entries per thread ----
        unsigned int cnt[4], local = 0;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int k = (int)tid * 4 + e;
            cnt[e] = 0;
            if (k < n_segs) {
                const unsigned long long v = worker + (pass + k) * n_workers;
                const uint32_t row = (uint32_t)(a.segs_per_row == 1 ? v : v / a.segs_per_row);
                const uint32_t seg = (uint32_t)(v - (unsigned long long)row * a.segs_per_row);
                long long lo, hi;
                table_segment(a, row, seg, (long long)__ldg(a.lens + row), lo, hi);
                const long long v0 = lo / kPer, v1 = (hi + kPer - 1) / kPer;
                sh.seg[k].lo = lo;
                sh.seg[k].hi = hi;
                cnt[e] = hi > lo ? (unsigned int)(v1 - v0) : 0u;
            }
            local += cnt[e];
        }
        const unsigned int incl = warp_inclusive_sum(local, lane);
        if (lane == 31) sh.warp_sum[warp] = incl;
        __syncthreads();
        unsigned int before = incl - local;
#pragma unroll
        for (int w = 0; w < kScanThreads / 32; ++w) before += (uint32_t)w < warp ? sh.warp_sum[w] : 0u;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int k = (int)tid * 4 + e;
            if (k < n_segs) sh.vec_before[k] = before;
            before += cnt[e];
        }
        if (tid == kScanThreads - 1) sh.vec_before[n_segs] = before;     // the last thread's running sum is the total
        __syncthreads();
        const unsigned int total = sh.vec_before[n_segs];
        // ---- stream the flattened vector list ----
        constexpr unsigned int kBatch = kScanThreads * kUnroll;
        int cur = 0;                              // batches are fetched in order: one cursor serves them all
        Chunk<Id> now, nxt;
        fetch_table_batch<Id>(slots, sh, n_segs, total, 0, cur, now);
        for (unsigned int base = 0; base < total; base += kBatch) {
            if (base + kBatch < total) fetch_table_batch<Id>(slots, sh, n_segs, total, base + kBatch, cur, nxt);
            else nxt.mask = 0;
            if (now.mask) mark_chunk<kPow2, Id>(now, a, s_map, c);
            now = nxt;
        }
    }
    leave_group<0>(p, 0, s_map, c);
    finish_cta<0>(p, 1u, hs, tail_mem);
}

// --------------------------------------------------------------------------
// kernel: slot ids staged through shared memory with bulk async copies (TMA)
// --------------------------------------------------------------------------
// A producer warp keeps kStages 16 KiB copies in flight per CTA
// (cp.async.bulk global -> shared, completion counted on a "full" mbarrier);
// eight consumer warps read their ids from shared memory with conflict-free
// 128-bit loads and hand each stage back through an "empty" mbarrier, so no
// CTA-wide barrier sits in the streaming loop.  Registers hold no staging
// data: the bytes in flight per SM are set by shared memory (kStages x 16 KiB
// per CTA), not by occupancy.
//
// Every wait on an mbarrier is bounded in time.  The first wait of a CTA that
// runs out records RT_RESULT_TIMEOUT; from then on the CTA waits for nothing
// any more, it only retires its remaining units, so the grid always drains and
// a failed launch costs a few waits, not one per unit.  A plan made from an
// incomplete scan is never committed (see plan_tail).
#ifndef RT_STAGES
#define RT_STAGES 4
#endif
constexpr int kStages = RT_STAGES;
#ifndef RT_TMA_MIN_CTAS
#define RT_TMA_MIN_CTAS 3
#endif
constexpr int kStageBytes = kChunkElems * 8;
// the staging ring is reused as the tail's working memory once streaming is over
static_assert((size_t)kStages * kStageBytes >= tail_smem_bytes(RT_MAX_GROUPS, RT_MAX_BUFFERS),
              "staging ring too small to host the plan tail");
// Longest time one wait on an mbarrier may take.  A 16 KiB copy lands in a few
// microseconds; a wait that lasts milliseconds means the copy is not coming.
#ifndef RT_WAIT_NS
#define RT_WAIT_NS 4000000ull
#endif
constexpr unsigned long long kWaitNs = RT_WAIT_NS;

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
// try_wait suspends the thread in hardware for a bounded time before it
// reports "not yet", so the polling loop issues few instructions.
__device__ __forceinline__ bool mbar_test(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_addr(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Waits at most kWaitNs of wall-clock time (the device's nanosecond timer), so
// the bound does not depend on how long the hardware suspends a try_wait.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t *bar, uint32_t parity) {
    if (mbar_test(bar, parity)) return true;
    const unsigned long long until = global_ns() + kWaitNs;
    while (!mbar_test(bar, parity))
        if (global_ns() > until) return false;
    return true;
}
__device__ __forceinline__ void bulk_load(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
            smem_addr(dst)),
        "l"(src), "r"(bytes), "r"(smem_addr(bar))
        : "memory");
}

// Threads 0..255 consume; warp 8 is the producer (lane 0 issues the copies).
constexpr int kTmaThreads = kScanThreads + 32;
constexpr int kConsumerBar = 1;

// Ids [e0, copy_end) of a unit travel by bulk copy: whole 16-byte pairs only,
// never past the last whole pair of the array.
__device__ __forceinline__ long long copy_end_of(long long e0, long long hi, long long copy_limit) {
    long long end = e0 + kChunkElems < hi ? e0 + kChunkElems : hi;
    end = (end + 1) & ~1LL;
    return end < copy_limit ? end : copy_limit;
}

template <bool kPow2>
__global__ void __launch_bounds__(kTmaThreads, RT_TMA_MIN_CTAS)
scan_plan_tma_kernel(const __grid_constant__ ScanArgs a, const __grid_constant__ PlanArgs p) {
    extern __shared__ __align__(128) unsigned char stage_mem[];
    __shared__ __align__(8) uint64_t full_bar[kStages];    // copy landed (tx bytes)
    __shared__ __align__(8) uint64_t empty_bar[kStages];   // all consumer warps done with the stage
    __shared__ __align__(16) uint8_t s_map[RT_MAX_BLOCKS];
    __shared__ HandoverShared hs;
    const int tid = threadIdx.x;
    if (gatekeeper()) return;
    const uint32_t worker = blockIdx.x - 1, n_workers = gridDim.x - 1;
    const int q_begin = (int)((long long)a.n_units * worker / n_workers);
    const int q_end = (int)((long long)a.n_units * (worker + 1) / n_workers);
    if (q_begin >= q_end) return;
    const long long copy_limit = a.group_off[a.n_groups] & ~1LL;
    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], kScanThreads / 32);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (tid < kScanThreads) clear_map(s_map);
    const uint32_t g0 = first_group(a, q_begin);
    __syncthreads();

    if (tid >= kScanThreads) {
        // ---- producer warp: keeps up to kStages copies in flight ----
        if (tid == kScanThreads) {
            int i = 0;
            bool alive = true;
            for (uint32_t g = g0; alive; ++g) {
                const GroupSpan sp = group_span(a, g, q_begin, q_end);
                long long e0 = sp.e0;
                for (int q = sp.q_lo; q < sp.q_hi; ++q, ++i, e0 += kChunkElems) {
                    const int stage = i % kStages, round = i / kStages;
                    if (round > 0 && !mbar_wait_bounded(&empty_bar[stage], (uint32_t)(round - 1) & 1u)) {
                        atomicOr(&p.global->error_flags, RT_RESULT_TIMEOUT);
                        alive = false;
                        break;
                    }
                    const long long n = copy_end_of(e0, sp.hi, copy_limit) - e0;
#ifdef RT_TEST_STALL
                    // test build only: the first worker "loses" its first copy, so that the
                    // consumers' bounded wait runs out (nothing faults, nothing hangs)
                    if (blockIdx.x == 1 && i == 0) continue;
#endif
                    if (n > 0) {
                        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                        mbar_expect_tx(&full_bar[stage], (uint32_t)(n * 8));
                        bulk_load(stage_mem + stage * kStageBytes, a.slots + e0, (uint32_t)(n * 8),
                                  &full_bar[stage]);
                    } else {
                        mbar_arrive(&full_bar[stage]);
                    }
                }
                if (sp.q_hi >= q_end) break;
            }
        }
        return;
    }

    // ---- consumer warps ----
    ScanCounters c = {0, 0};
    bool gave_up = false;
    int i = 0;
    for (uint32_t g = g0;; ++g) {
        const GroupSpan sp = group_span(a, g, q_begin, q_end);
        long long e0 = sp.e0;
        for (int q = sp.q_lo; q < sp.q_hi; ++q, ++i, e0 += kChunkElems) {
            const int stage = i % kStages;
            const uint32_t parity = (uint32_t)(i / kStages) & 1u;
            const longlong2 *src =
                reinterpret_cast<const longlong2 *>(stage_mem + stage * kStageBytes) + tid;
            const bool landed = !gave_up && mbar_wait_bounded(&full_bar[stage], parity);
            longlong2 v[kUnroll];
            uint32_t mask = 0;
            if (landed) {
                if (e0 >= sp.lo && e0 + kChunkElems <= sp.hi) {
#pragma unroll
                    for (int k = 0; k < kUnroll; ++k) v[k] = src[k * kScanThreads];
                    mask = kAllIds;
                } else {
                    const long long copied_to = copy_end_of(e0, sp.hi, copy_limit);
                    const long long end = e0 + kChunkElems < sp.hi ? e0 + kChunkElems : sp.hi;
#pragma unroll
                    for (int k = 0; k < kUnroll; ++k) {
                        long long idx = e0 + 2 * (k * kScanThreads + tid);
                        v[k].x = v[k].y = 0;
                        if (idx < copied_to) {
                            v[k] = src[k * kScanThreads];
                            if (idx >= sp.lo && idx < end) mask |= 1u << (2 * k);
                            if (idx + 1 >= sp.lo && idx + 1 < end) mask |= 2u << (2 * k);
                        } else if (idx >= sp.lo && idx < end) {
                            // odd last id of the whole array: not part of any 16-byte pair
                            v[k].x = RT_LOAD(a.slots + idx);
                            mask |= 1u << (2 * k);
                        }
                    }
                }
            } else {
                gave_up = true;
            }
            // the ids are in registers: give the stage back before marking
            __syncwarp();
            if ((tid & 31) == 0) mbar_arrive(&empty_bar[stage]);
            if (mask == kAllIds) mark_full<kPow2>(v, a, s_map, c);
            else mark_masked<kPow2>(v, mask, a, s_map, c);
        }
        leave_group<kConsumerBar>(p, g, s_map, c);
        if (sp.q_hi >= q_end) break;
    }
    // (one thread's wait running out means the whole CTA stops trusting its ring)
    gave_up = cta_or<kConsumerBar, kScanThreads>(gave_up);
    if (gave_up) {
        if (tid == 0) atomicOr(&p.global->error_flags, RT_RESULT_TIMEOUT);
        // copies that never signalled may still be in flight: give them one more
        // bounded chance to land before the CTA's shared memory is released
        if (tid == 0)
            for (int s = 0; s < kStages; ++s) {
                int uses = (q_end - q_begin - s + kStages - 1) / kStages;
                if (uses > 0) mbar_wait_bounded(&full_bar[s], (uint32_t)(uses - 1) & 1u);
            }
    }
    // every stage has been consumed: the staging memory now serves the tail
    // (unless this CTA gave up on a copy, which might still land there)
    finish_cta<kConsumerBar>(p, (uint32_t)(q_end - q_begin), hs, stage_mem, gave_up);
}

// --------------------------------------------------------------------------
// kernel: wanted bitmaps given, no scan
// --------------------------------------------------------------------------
__global__ void __launch_bounds__(kScanThreads)
plan_tail_kernel(uint32_t *want, const __grid_constant__ PlanArgs p) {
    extern __shared__ __align__(16) unsigned char tail_mem[];
    plan_tail<0>(p, want, false, tail_mem);
}

// --------------------------------------------------------------------------
// host-side launchers (called from the C ABI)
// --------------------------------------------------------------------------
// `chained`: launch with programmatic stream serialization, so that the scan may
// start while the kernel before it in the stream is still in its tail.
template <typename Kernel>
static cudaError_t launch_scan(Kernel kernel, int grid, int threads, size_t smem, cudaStream_t stream,
                               bool chained, const ScanArgs &a, const PlanArgs &p) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid + 1u);          // the workers and, as CTA 0, the gatekeeper
    cfg.blockDim = dim3((unsigned)threads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = chained ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, a, p);
}

cudaError_t launch_scan_plan(const ScanArgs &a, const PlanArgs &p, bool table, bool ids32, int grid,
                             cudaStream_t stream, bool chained) {
    const bool pow2 = a.shift >= 0;
    const size_t smem = tail_smem_bytes(p.n_groups, p.n_buffers);
    if (table) {
        // one warp per segment when a segment holds at least kWarpSegVectors 16-byte vectors
        const bool warps = a.seg_ids / (ids32 ? 4 : 2) >= kWarpSegVectors;
#define RT_TABLE(P, T)                                                                                        \
    (warps ? launch_scan(scan_table_kernel<P, T, true>, grid, kScanThreads, smem, stream, chained, a, p)      \
           : launch_scan(scan_table_kernel<P, T, false>, grid, kScanThreads, smem, stream, chained, a, p))
        if (ids32) return pow2 ? RT_TABLE(true, int) : RT_TABLE(false, int);
        return pow2 ? RT_TABLE(true, long long) : RT_TABLE(false, long long);
#undef RT_TABLE
    }
    if (ids32)
        return pow2 ? launch_scan(scan_plan_kernel<true, int>, grid, kScanThreads, smem, stream, chained, a, p)
                    : launch_scan(scan_plan_kernel<false, int>, grid, kScanThreads, smem, stream, chained, a, p);
    return pow2 ? launch_scan(scan_plan_kernel<true, long long>, grid, kScanThreads, smem, stream, chained, a, p)
                : launch_scan(scan_plan_kernel<false, long long>, grid, kScanThreads, smem, stream, chained, a, p);
}

cudaError_t launch_plan_tail(const uint32_t *want, const PlanArgs &p, cudaStream_t stream) {
    plan_tail_kernel<<<1, kScanThreads, tail_smem_bytes(p.n_groups, p.n_buffers), stream>>>(
        const_cast<uint32_t *>(want), p);
    return cudaGetLastError();
}

cudaError_t launch_scan_plan_tma(const ScanArgs &a, const PlanArgs &p, int grid, cudaStream_t stream,
                                 bool chained) {
    const size_t smem = kStages * kStageBytes;
    return a.shift >= 0 ? launch_scan(scan_plan_tma_kernel<true>, grid, kTmaThreads, smem, stream, chained, a, p)
                        : launch_scan(scan_plan_tma_kernel<false>, grid, kTmaThreads, smem, stream, chained, a, p);
}

// Opt in to the dynamic shared memory the kernels need and report how many CTAs
// of each streaming kernel fit on one SM for this plan's geometry.
cudaError_t scan_plan_occupancy(uint32_t n_groups, uint32_t n_buffers, int *plain_blocks_per_sm,
                                int *tma_blocks_per_sm, int *table_blocks_per_sm) {
    const int tail = (int)tail_smem_bytes(n_groups, n_buffers);
    const int tma = kStages * kStageBytes;
    // The attribute belongs to the kernel, not to a plan: it is set to what the
    // largest plan needs, so that plans of different geometry can live in one
    // process (set per plan, a smaller plan created later made the launches of a
    // larger one fail with "invalid value").
    const int tail_max = (int)tail_smem_bytes(RT_MAX_GROUPS, RT_MAX_BUFFERS);
    cudaError_t e;
#define RT_SET_SMEM(kernel, bytes)                                                           \
    if ((e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes)) != \
        cudaSuccess)                                                                         \
        return e;
    RT_SET_SMEM(scan_plan_tma_kernel<true>, tma)
    RT_SET_SMEM(scan_plan_tma_kernel<false>, tma)
    RT_SET_SMEM((scan_plan_kernel<true, long long>), tail_max)
    RT_SET_SMEM((scan_plan_kernel<false, long long>), tail_max)
    RT_SET_SMEM((scan_plan_kernel<true, int>), tail_max)
    RT_SET_SMEM((scan_plan_kernel<false, int>), tail_max)
    RT_SET_SMEM((scan_table_kernel<true, long long, true>), tail_max)
    RT_SET_SMEM((scan_table_kernel<false, long long, true>), tail_max)
    RT_SET_SMEM((scan_table_kernel<true, int, true>), tail_max)
    RT_SET_SMEM((scan_table_kernel<false, int, true>), tail_max)
    RT_SET_SMEM((scan_table_kernel<true, long long, false>), tail_max)
    RT_SET_SMEM((scan_table_kernel<false, long long, false>), tail_max)
    RT_SET_SMEM((scan_table_kernel<true, int, false>), tail_max)
    RT_SET_SMEM((scan_table_kernel<false, int, false>), tail_max)
    RT_SET_SMEM(plan_tail_kernel, tail_max)
#undef RT_SET_SMEM
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(plain_blocks_per_sm, scan_plan_kernel<true, long long>,
                                                      kScanThreads, tail);
    if (e != cudaSuccess) return e;
    // (the list-building form has the larger footprint of the two)
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(table_blocks_per_sm, scan_table_kernel<true, int, false>,
                                                      kScanThreads, tail);
    if (e != cudaSuccess) return e;
    return cudaOccupancyMaxActiveBlocksPerMultiprocessor(tma_blocks_per_sm, scan_plan_tma_kernel<true>,
                                                         kTmaThreads, tma);
}

}  // namespace rt
