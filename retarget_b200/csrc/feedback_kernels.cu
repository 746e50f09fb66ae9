// Slot-feedback state kept in GPU memory, and the recency-ranked block plan.
//
// Stands in for experiments/slot_feedback.py (per-slot generation counters,
// per-block version / last-read / last-write stamps, free-list head) and for
// the ranking + selection of experiments/slot_placement.py:37-44,83-94, so that
// the serving engine's index tensors never leave the device: no pinned copy,
// no Python loop per slot, no JSON file per 50 ms.
//
// One bitmap (the reference plans one mask for all KV allocations).  Events are
// small (at most a few hundred thousand ids), so these kernels favour simplicity
// over streaming tricks; the bulk scan of the planner is a different kernel.
#include <cuda_runtime.h>

#include <cmath>
#include <new>

#include "plan_device.cuh"
#include "plan_tail.cuh"
#include "rt_internal.h"

namespace rt {

constexpr int kFreeHeadMax = 4096;     // the probe samples the first 4096 free slots
constexpr int kRankThreads = 1024;     // one thread per block id

struct FeedbackState {
    int32_t *generations;      // [capacity + 1]
    int32_t *versions;         // [n_blocks]
    double *read_seen;         // [n_blocks], -inf = never
    double *write_seen;        // [n_blocks]
    int32_t *commit_version;   // [n_blocks], valid where `resident` has the bit
    double *commit_time;       // [n_blocks]
    long long *free_head;      // [kFreeHeadMax] slot ids, queue order
    int32_t *free_count;       // [1]
    uint32_t *event_blocks;    // [3 * kWords] scratch: blocks touched by the current event's lists
                               //   (one event: [a | b]; a whole step: [allocated | read | written])
    uint32_t *arrivals;        // [1] scratch: CTAs of the current event that have finished marking
    uint32_t *slot_marks;      // [(capacity + 32) / 32] scratch: slots of the current alloc event
    unsigned long long *bad;   // [2] invalid / ignored ids seen so far
};

struct Geometry {
    unsigned long long capacity;
    uint32_t block_tokens;
    int shift;
    uint32_t magic, magic_shift;
    uint32_t n_blocks;
};

__device__ __forceinline__ uint32_t block_of_slot(uint32_t slot, const Geometry &g) {
    if (g.shift >= 0) return slot >> g.shift;
    uint32_t q = __umulhi(slot, g.magic);
    return (((slot - q) >> 1) + q) >> g.magic_shift;
}

// --------------------------------------------------------------------------
// one launch per event
// --------------------------------------------------------------------------
// Every CTA marks the blocks its share of the ids falls in (a byte map per
// list in shared memory, folded into the event words with one atomicOr per
// non-zero word); for allocations it also does generations[id] += 1 -- once per
// occurrence, like `generations[begin:end] += 1` over order-preserving runs --
// and sets a mark per slot for the free-head filter.  The CTA that arrives last
// then does what needs the whole event: the stamps, the free-list head, the
// clean-up of the scratch words.  Nobody waits for anybody.
// The id lists are int64 or int32 (template parameter of the kernel).
struct EventArgs {
    const void *ids_a;         // attention: read ids; allocation: the allocated slots
    long long n_a;
    const void *ids_b;         // attention: written ids; allocation: unused
    long long n_b;
    const void *fresh;         // allocation: the new free-list head, or null
    int n_fresh;
    int alloc;                 // 0 attention, 1 allocation
    double t;
};

template <typename Id>
__device__ __forceinline__ void mark_ids(const Id *ids, long long n, const Geometry &geo,
                                         const FeedbackState &st, int alloc, uint8_t *s_map, int *s_ver,
                                         uint32_t &invalid, uint32_t &ignored) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (long long)gridDim.x * blockDim.x) {
        long long s = (long long)__ldcs(ids + i);
        if ((unsigned long long)(s - 1) < geo.capacity) {
            const uint32_t v = (uint32_t)s, block = block_of_slot(v, geo);
            s_map[block] = 1;
            if (alloc) {
                // the slot's new generation is a candidate for its block's version
                atomicMax(&s_ver[block], atomicAdd(&st.generations[v], 1) + 1);
                atomicOr(&st.slot_marks[v >> 5], 1u << (v & 31));
            }
        } else if (s < 1) {
            if (alloc && s == 0) atomicOr(&st.slot_marks[0], 1u);   // only matters to the free-head filter
            ++ignored;
        } else {
            ++invalid;
        }
    }
}

// Byte map -> the event's words (call between two CTA barriers).
__device__ __forceinline__ void flush_event_map(const uint8_t *s_map, uint32_t *words) {
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (warp >= 8) return;                      // eight warps x four words cover the map
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        uint32_t word = warp * 4 + k;
        uint32_t bits = __ballot_sync(0xffffffffu, s_map[word * 32 + lane] != 0);
        if (lane == 0 && bits) atomicOr(&words[word], bits);
    }
}

// Allocation events: a block's version is the largest generation among its
// slots (slot_feedback.py:61).  Generations only ever grow, and only in the
// slots an event allocates, so the largest generation of a touched block after
// the event is the larger of its version before and the new generations of the
// slots just allocated: no slot of the block has to be read again.
__device__ __forceinline__ void flush_versions(const uint8_t *s_map, const int *s_ver, const FeedbackState &st) {
    for (uint32_t b = threadIdx.x; b < (uint32_t)RT_MAX_BLOCKS; b += blockDim.x)
        if (s_map[b]) atomicMax(&st.versions[b], s_ver[b]);
}

// Free-list head, by one CTA.  With a fresh head the event replaces it
// (slot_feedback.py:63-64); without, the slots this event allocated are dropped
// from the known head, order kept (slot_feedback.py:65-70).  One pass: every
// thread takes a contiguous piece of the head into registers (all its loads in
// flight together), a CTA-wide prefix sum places what it keeps.
constexpr int kHeadPerThread = kFreeHeadMax / 256;       // CTAs have at least 256 threads
static_assert(kWords == 32, "a lane per bitmap word");

template <typename Id>
__device__ void update_free_head(const FeedbackState &st, const Id *fresh, int n_fresh,
                                 unsigned long long capacity, int *s_warp) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (fresh) {
        int n = n_fresh < kFreeHeadMax ? n_fresh : kFreeHeadMax;
        for (int i = tid; i < n; i += blockDim.x) st.free_head[i] = (long long)fresh[i];
        if (tid == 0) *st.free_count = n;
        return;
    }
    const int n = *st.free_count;
    const int per = (n + (int)blockDim.x - 1) / (int)blockDim.x;      // <= kHeadPerThread
    const int first = tid * per;
    long long slot[kHeadPerThread];
    uint32_t keep = 0;
#pragma unroll
    for (int k = 0; k < kHeadPerThread; ++k)
        slot[k] = (k < per && first + k < n) ? __ldcg(&st.free_head[first + k]) : -1;
#pragma unroll
    for (int k = 0; k < kHeadPerThread; ++k) {
        if (!(k < per && first + k < n)) continue;
        bool stays = true;
        if ((unsigned long long)slot[k] <= capacity)
            stays = !((__ldcg(&st.slot_marks[(uint32_t)slot[k] >> 5]) >> ((uint32_t)slot[k] & 31)) & 1u);
        keep |= (uint32_t)stays << k;
    }
    // exclusive prefix of the kept counts over the CTA
    const int mine = __popc(keep);
    int incl = mine;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        int up = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += up;
    }
    if (lane == 31) s_warp[warp] = incl;
    __syncthreads();                            // every thread has read its piece of the head
    int before = incl - mine;
    for (int w = 0; w < warp; ++w) before += s_warp[w];
#pragma unroll
    for (int k = 0; k < kHeadPerThread; ++k)
        if ((keep >> k) & 1u) st.free_head[before++] = slot[k];
    if (tid == (int)blockDim.x - 1) *st.free_count = before;
}

// What needs a whole allocation event, by the CTA that arrived last:
// write_seen = t for every touched block (slot_feedback.py:62), the free-list
// head, and the clean-up of the slot marks.  `words`: the event's touched-block
// words.  (The versions were brought up to date while the ids were marked.)
template <typename Id>
__device__ void finish_alloc_event(const EventArgs &ev, const Geometry &geo, const FeedbackState &st,
                                   const uint32_t *words, int *s_warp) {
    const Id *ids_a = static_cast<const Id *>(ev.ids_a);
    for (uint32_t b = threadIdx.x; b < geo.n_blocks; b += blockDim.x)
        if ((__ldcg(&words[b >> 5]) >> (b & 31)) & 1u) st.write_seen[b] = ev.t;
    update_free_head(st, static_cast<const Id *>(ev.fresh), ev.n_fresh, geo.capacity, s_warp);
    __syncthreads();
    // the slot marks served the free-head filter: clear them again
    for (long long i = threadIdx.x; i < ev.n_a; i += blockDim.x) {
        long long s = (long long)ids_a[i];
        if ((unsigned long long)s <= geo.capacity) st.slot_marks[(uint32_t)s >> 5] = 0;
    }
}

// read_seen = t (slot_feedback.py:72-73), write_seen = t (:74-75)
__device__ __forceinline__ void finish_attention_event(double t, const Geometry &geo, const FeedbackState &st,
                                                       const uint32_t *read_words, const uint32_t *write_words) {
    for (uint32_t b = threadIdx.x; b < geo.n_blocks; b += blockDim.x) {
        if ((__ldcg(&read_words[b >> 5]) >> (b & 31)) & 1u) st.read_seen[b] = t;
        if ((__ldcg(&write_words[b >> 5]) >> (b & 31)) & 1u) st.write_seen[b] = t;
    }
}

template <typename Id>
__global__ void __launch_bounds__(256)
feedback_event_kernel(EventArgs ev, Geometry geo, FeedbackState st) {
    const Id *ids_a = static_cast<const Id *>(ev.ids_a), *ids_b = static_cast<const Id *>(ev.ids_b);
    __shared__ uint8_t s_map[2][RT_MAX_BLOCKS];
    __shared__ int s_ver[RT_MAX_BLOCKS], s_warp[32], s_last;
    reinterpret_cast<uint32_t *>(s_map[0])[threadIdx.x] = 0;
    reinterpret_cast<uint32_t *>(s_map[1])[threadIdx.x] = 0;
    if (ev.alloc)
        for (uint32_t b = threadIdx.x; b < (uint32_t)RT_MAX_BLOCKS; b += blockDim.x) s_ver[b] = 0;
    __syncthreads();
    uint32_t invalid = 0, ignored = 0;
    mark_ids(ids_a, ev.n_a, geo, st, ev.alloc, s_map[0], s_ver, invalid, ignored);
    mark_ids(ids_b, ev.n_b, geo, st, 0, s_map[1], nullptr, invalid, ignored);
    __syncthreads();
    if (ev.alloc) flush_versions(s_map[0], s_ver, st);
    flush_event_map(s_map[0], st.event_blocks);
    if (ev.n_b) flush_event_map(s_map[1], st.event_blocks + kWords);
    const uint32_t lane = threadIdx.x & 31;
    uint32_t inv = warp_sum(invalid), ign = warp_sum(ignored);
    if (lane == 0) {
        if (inv) atomicAdd(&st.bad[0], (unsigned long long)inv);
        if (ign) atomicAdd(&st.bad[1], (unsigned long long)ign);
    }
    // arrival: the last CTA finishes the event
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) s_last = atomicAdd(st.arrivals, 1u) == gridDim.x - 1;
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    if (!ev.alloc) finish_attention_event(ev.t, geo, st, st.event_blocks, st.event_blocks + kWords);
    else finish_alloc_event<Id>(ev, geo, st, st.event_blocks, s_warp);
    __syncthreads();
    if (threadIdx.x < 2 * kWords) st.event_blocks[threadIdx.x] = 0;
    if (threadIdx.x == 0) *st.arrivals = 0;
}


// --------------------------------------------------------------------------
// ranking + selection: one CTA, one thread per block id
// --------------------------------------------------------------------------
struct RankPolicy {
    uint32_t budget;
    uint32_t max_blocks;       // max_blocks_per_update
    uint32_t flags;            // RT_PLAN_EVICT, RT_PLAN_DRY_RUN
    double at;                 // time of the snapshot (30 s horizon), slot_feedback.py:82-85
    double now;
    double commit;             // stamp given to newly committed blocks
    double active_seconds;
    double refresh_seconds;
};

// Doubles -> unsigned integers with the same order.
__device__ __forceinline__ unsigned long long ordered_bits(double x) {
    unsigned long long u = (unsigned long long)__double_as_longlong(x);
    return (u >> 63) ? ~u : (u | 0x8000000000000000ull);
}

// Rank key of a block as two 64-bit words that compare like the tuple
// (class, -t, aux, block id):
//   class  0 active read, 1 active write, 2 free-list head, 3 history, 7 unranked
//   -t     sortable image of the stamp (0 where time does not matter)
//   aux    class 2: position in the free head (< 4096); class 3: 0 read entry, 1 write entry
//   hi = class:3 | tkey[63:3]        lo = tkey[2:0]:3 | aux:32 | block id:10
// Block ids are distinct, so no two keys are equal.
struct RankKey {
    unsigned long long hi, lo;
};
__device__ __forceinline__ RankKey make_key(uint32_t cls, unsigned long long tkey, uint32_t aux, uint32_t id) {
    RankKey k;
    k.hi = ((unsigned long long)cls << 61) | (tkey >> 3);
    k.lo = ((tkey & 7ull) << 61) | ((unsigned long long)aux << 10) | id;
    return k;
}
__device__ __forceinline__ bool key_less(const RankKey &a, const RankKey &b) {
    return a.hi < b.hi || (a.hi == b.hi && a.lo < b.lo);
}

// One compare-exchange step of the bitonic network: this thread keeps the
// smaller or the larger of its key and its partner's.
__device__ __forceinline__ void keep_one(RankKey &mine, const RankKey &theirs, bool keep_min) {
    if (key_less(theirs, mine) == keep_min) mine = theirs;
}

// Working memory of the plan tail inside the ranking kernel: the sort buffers,
// free once the order is known.
static_assert(2 * 2 * kRankThreads * sizeof(unsigned long long) >= tail_smem_bytes(1, RT_MAX_BUFFERS),
              "sort buffers too small to host the plan tail");

// Ranking, selection and range emission in one launch.  blockDim = the power of
// two that covers the blocks (at least kScanThreads, which the tail needs).
//   sets: [0..31] evict words, [32..63] add words, [64..95] the resident words
//   after this plan (read back by the tail part)
// Nothing is committed before the tail has said that the plan is deliverable,
// and nothing at all when no block moves: the reference's controller returns
// before it touches `committed` when nothing was selected
// (experiments/slot_placement.py:131-132), so a committed block that drops out
// of the desired set for a while is not sent again when it comes back with its
// version unchanged.
struct RankShared {
    unsigned long long swap[2][2][kRankThreads];   // [buffer][hi|lo][thread]
    int free_pos[kRankThreads];
    uint32_t warp[32];
    uint8_t sel[kRankThreads], des[kRankThreads];
    int delivered;
};

__device__ void rank_and_plan(const Geometry &geo, const FeedbackState &st, const RankPolicy &pol, uint32_t *resident,
                              uint32_t *sets, const PlanArgs &tail, RankShared &sh) {
    auto &s_swap = sh.swap;
    auto &s_free_pos = sh.free_pos;
    auto &s_warp = sh.warp;
    auto &s_sel = sh.sel;
    auto &s_des = sh.des;
    int &s_delivered = sh.delivered;
    const uint32_t b = threadIdx.x, lane = b & 31, warp = b >> 5, n_threads = blockDim.x;
    s_free_pos[b] = 0x7fffffff;
    __syncthreads();
    const int n_free = *st.free_count;
#pragma unroll 4
    for (int i = b; i < n_free; i += n_threads) {
        long long slot = st.free_head[i];
        if (slot >= 0) {
            unsigned long long blk = geo.shift >= 0 ? ((unsigned long long)slot >> geo.shift)
                                                    : ((unsigned long long)slot / geo.block_tokens);
            if (blk < n_threads) atomicMin(&s_free_pos[blk], i);
        }
    }
    __syncthreads();
    const bool real = b < geo.n_blocks;
    const double r = real ? st.read_seen[b] : -INFINITY, w = real ? st.write_seen[b] : -INFINITY;
    // what `choose` will ask about block b if it ends up inside the budget (slot_placement.py:86-93);
    // none of it depends on the rank, so it is settled here, while thread b still speaks for block b
    const int32_t version_b = real ? st.versions[b] : 0;
    const int32_t commit_version_b = real ? st.commit_version[b] : 0;
    const double commit_time_b = real ? st.commit_time[b] : 0.0;
    const bool held_b = (resident[b >> 5] >> (b & 31)) & 1u;
    const bool recent_r = isfinite(r) && pol.at - r <= 30.0, recent_w = isfinite(w) && pol.at - w <= 30.0;
    const bool active_r = recent_r && pol.now - r <= pol.active_seconds;
    const bool active_w = recent_w && pol.now - w <= pol.active_seconds;
    RankKey k = make_key(7, 0, 0, b);
    if (active_r) k = make_key(0, ordered_bits(-r), 0, b);
    else if (active_w) k = make_key(1, ordered_bits(-w), 0, b);
    else if (real && s_free_pos[b] != 0x7fffffff) k = make_key(2, 0, (uint32_t)s_free_pos[b], b);
    else if (recent_r || recent_w) {
        // first of the block's entries in reads+writes sorted by -t (stable: reads first)
        const bool use_r = recent_r && (!recent_w || r >= w);
        k = make_key(3, ordered_bits(-(use_r ? r : w)), use_r ? 0u : 1u, b);
    }
    s_sel[b] = !held_b || commit_version_b != version_b ||
               (pol.now - commit_time_b >= pol.refresh_seconds && (active_r || active_w));
    // Bitonic sort, one key per thread, keys in registers: partners up to 16
    // lanes away trade by shuffle, farther ones through shared memory (two
    // buffers in turn, so one barrier per step is enough).  Only the power of
    // two that covers the blocks is sorted as a whole; the threads beyond it hold
    // "never" keys and merely permute them among themselves.
    uint32_t sort_n = 32;
    while (sort_n < geo.n_blocks) sort_n <<= 1;
    uint32_t turn = 0;
    for (uint32_t size = 2; size <= sort_n; size <<= 1) {
        for (uint32_t stride = size >> 1; stride > 0; stride >>= 1) {
            RankKey other;
            if (stride < 32) {
                other.hi = __shfl_xor_sync(0xffffffffu, k.hi, stride);
                other.lo = __shfl_xor_sync(0xffffffffu, k.lo, stride);
            } else {
                s_swap[turn][0][b] = k.hi;
                s_swap[turn][1][b] = k.lo;
                __syncthreads();
                other.hi = s_swap[turn][0][b ^ stride];
                other.lo = s_swap[turn][1][b ^ stride];
                turn ^= 1;
            }
            // ascending runs keep the minimum at the lower index
            keep_one(k, other, ((b & size) == 0) == ((b & stride) == 0));
        }
    }
    // position b of the sorted order holds block `blk`
    const uint32_t blk = (uint32_t)(k.lo & 1023u);
    const bool desired = (k.hi >> 61) != 7 && b < pol.budget;
    __syncthreads();                        // s_sel[] of every block is in shared memory (sort_n may be one warp)
    const bool todo = desired && s_sel[blk];
    // first max_blocks of `todo` in rank order
    uint32_t mask = __ballot_sync(0xffffffffu, todo);
    if (lane == 0) s_warp[warp] = __popc(mask);
    __syncthreads();
    uint32_t before = __popc(mask & ((1u << lane) - 1u));
    for (uint32_t wv = 0; wv < warp; ++wv) before += s_warp[wv];
    const bool selected = todo && before < pol.max_blocks;
    s_sel[blk] = selected;                  // (every thread read its s_sel[blk] before the barrier above)
    s_des[blk] = desired;
    __syncthreads();
    // back to block-id order: thread b speaks for block b, warp = bitmap word
    const bool sel_b = s_sel[b], des_b = s_des[b];
    const bool evict_b = (pol.flags & RT_PLAN_EVICT) && held_b && !des_b;
    const uint32_t add_word = __ballot_sync(0xffffffffu, sel_b);
    const uint32_t evict_word = __ballot_sync(0xffffffffu, evict_b);
    const uint32_t keep_word = __ballot_sync(0xffffffffu, (held_b && des_b) || sel_b);
    const uint32_t held_word = __ballot_sync(0xffffffffu, held_b);
    // does anything move?  (also the barrier after which every thread has read `resident`)
    const bool moves = __syncthreads_or(sel_b || evict_b);
    const uint32_t new_word = moves ? keep_word : held_word;
    if (lane == 0) {
        sets[warp] = evict_word;
        sets[kWords + warp] = add_word;
        sets[2 * kWords + warp] = new_word;
    }
    if (b == 0)                             // words of blocks beyond this launch's threads
        for (uint32_t wv = n_threads >> 5; wv < (uint32_t)kWords; ++wv)
            sets[wv] = sets[kWords + wv] = sets[2 * kWords + wv] = 0;
    __syncthreads();                        // the words above are visible to the whole CTA
    // ---- byte ranges: the plan tail, run by the first kScanThreads threads ----
    if (b < (uint32_t)kScanThreads) {
        const bool ok = plan_tail<1>(tail, sets, false, reinterpret_cast<unsigned char *>(&s_swap[0][0][0]));
        if (b == 0) s_delivered = ok;
    }
    __syncthreads();
    // ---- commit, now that the plan is known to fit the caller's range buffer ----
    if (!s_delivered || !moves || (pol.flags & RT_PLAN_DRY_RUN)) return;
    if (sel_b) {
        st.commit_version[b] = version_b;
        st.commit_time[b] = pol.commit;
    }
    if (lane == 0) resident[warp] = new_word;
}

__global__ void __launch_bounds__(kRankThreads)
feedback_rank_kernel(Geometry geo, FeedbackState st, RankPolicy pol, uint32_t *resident, uint32_t *sets,
                     const __grid_constant__ PlanArgs tail) {
    __shared__ __align__(16) RankShared sh;
    rank_and_plan(geo, st, pol, resident, sets, tail, sh);
}

// --------------------------------------------------------------------------
// one launch per decode step: allocation event + attention event + plan
// --------------------------------------------------------------------------
// What a serving engine does every decode step -- hand out pages, run
// attention, ask for a plan -- folded into ONE launch.  Every CTA marks its
// share of the three id lists (allocated, read, written); the CTA that arrives
// last then does, in the order the separate calls would have: the allocation
// event's finishing work, the attention event's stamps, the ranking and the
// plan.  blockDim is the ranking's (a power of two covering the blocks).
struct StepArgs {
    EventArgs alloc;           // n_a == 0 and no fresh head: no allocation event this step
    EventArgs attention;
};

template <typename Id>
__global__ void __launch_bounds__(kRankThreads)
feedback_step_kernel(StepArgs ev, Geometry geo, FeedbackState st, RankPolicy pol, uint32_t *resident,
                     uint32_t *sets, const __grid_constant__ PlanArgs tail) {
    __shared__ __align__(16) RankShared sh;
    __shared__ int s_last;
    // the three byte maps and the version candidates live in the sort buffers
    // until the ranking needs them
    uint8_t(*s_map)[RT_MAX_BLOCKS] = reinterpret_cast<uint8_t(*)[RT_MAX_BLOCKS]>(&sh.swap[0][0][0]);
    int *s_ver = reinterpret_cast<int *>(&sh.swap[0][0][0]) + 3 * RT_MAX_BLOCKS / 4;
    static_assert(sizeof(sh.swap) >= 7 * RT_MAX_BLOCKS, "sort buffers too small for the maps");
    for (uint32_t i = threadIdx.x; i < (ev.alloc.n_a ? 7u : 3u) * RT_MAX_BLOCKS / 4; i += blockDim.x)
        reinterpret_cast<uint32_t *>(&s_map[0][0])[i] = 0;
    __syncthreads();
    const bool has_alloc = ev.alloc.n_a > 0 || ev.alloc.fresh != nullptr;
    uint32_t invalid = 0, ignored = 0;
    mark_ids(static_cast<const Id *>(ev.alloc.ids_a), ev.alloc.n_a, geo, st, 1, s_map[0], s_ver, invalid, ignored);
    mark_ids(static_cast<const Id *>(ev.attention.ids_a), ev.attention.n_a, geo, st, 0, s_map[1], nullptr, invalid,
             ignored);
    mark_ids(static_cast<const Id *>(ev.attention.ids_b), ev.attention.n_b, geo, st, 0, s_map[2], nullptr, invalid,
             ignored);
    __syncthreads();
    if (ev.alloc.n_a) flush_versions(s_map[0], s_ver, st);
    if (ev.alloc.n_a) flush_event_map(s_map[0], st.event_blocks);
    if (ev.attention.n_a) flush_event_map(s_map[1], st.event_blocks + kWords);
    if (ev.attention.n_b) flush_event_map(s_map[2], st.event_blocks + 2 * kWords);
    const uint32_t lane = threadIdx.x & 31;
    uint32_t inv = warp_sum(invalid), ign = warp_sum(ignored);
    if (lane == 0) {
        if (inv) atomicAdd(&st.bad[0], (unsigned long long)inv);
        if (ign) atomicAdd(&st.bad[1], (unsigned long long)ign);
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) s_last = atomicAdd(st.arrivals, 1u) == gridDim.x - 1;
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    if (has_alloc) {
        finish_alloc_event<Id>(ev.alloc, geo, st, st.event_blocks, reinterpret_cast<int *>(sh.warp));
        __syncthreads();
    }
    finish_attention_event(ev.attention.t, geo, st, st.event_blocks + kWords, st.event_blocks + 2 * kWords);
    __syncthreads();
    if (threadIdx.x < 3 * kWords) st.event_blocks[threadIdx.x] = 0;
    if (threadIdx.x == 0) *st.arrivals = 0;
    __syncthreads();                       // the state is final; the maps are no longer needed
    rank_and_plan(geo, st, pol, resident, sets, tail, sh);
}

}  // namespace rt

// --------------------------------------------------------------------------
// C ABI
// --------------------------------------------------------------------------
#include "plan_internal.h"

struct rt_feedback {
    rt_plan *plan = nullptr;
    rt::PlanView view;
    rt::Geometry geo;
    rt::FeedbackState st;
    uint32_t *d_sets = nullptr;       // [3 * kWords] evict | add | resident after the plan
    uint64_t epoch = 0;
    void *block = nullptr;            // one allocation behind all state arrays
    size_t block_bytes = 0;
};

namespace {

int fb_fail(cudaError_t e) {
    rt::last_cuda_error_set((int)e);
    return e == cudaErrorMemoryAllocation ? RT_ERR_OUT_OF_MEMORY : RT_ERR_CUDA;
}
#define FB_CUDA(call)                                \
    do {                                             \
        cudaError_t e__ = (call);                    \
        if (e__ != cudaSuccess) return fb_fail(e__); \
    } while (0)

struct FbDevice {
    int prev = -1;
    explicit FbDevice(int d) { cudaGetDevice(&prev); cudaSetDevice(d); }
    ~FbDevice() { if (prev >= 0) cudaSetDevice(prev); }
};

size_t align_up(size_t x) { return (x + 255) & ~(size_t)255; }

// -inf stamps, zero everything else
__global__ void feedback_clear_kernel(rt::FeedbackState st, uint32_t n_blocks) {
    for (uint32_t b = threadIdx.x; b < n_blocks; b += blockDim.x) {
        st.read_seen[b] = -INFINITY;
        st.write_seen[b] = -INFINITY;
        st.commit_time[b] = -INFINITY;
    }
}

int clear_state(rt_feedback *fb, cudaStream_t s) {
    FB_CUDA(cudaMemsetAsync(fb->block, 0, fb->block_bytes, s));
    feedback_clear_kernel<<<1, 256, 0, s>>>(fb->st, fb->geo.n_blocks);
    FB_CUDA(cudaGetLastError());
    FB_CUDA(cudaMemsetAsync(fb->view.d_resident, 0, sizeof(uint32_t) * rt::kWords, s));
    return RT_OK;
}

int launch_event(rt_feedback *fb, const rt::EventArgs &ev, bool ids32, cudaStream_t s) {
    // 32-bit ids: a negative id must never look like a valid large one
    if (ids32 && fb->geo.capacity > 0x7fffffffull) return RT_ERR_INVALID_ARGUMENT;
    long long blocks = (ev.n_a + ev.n_b + 255) / 256;
    int grid = (int)(blocks < 1 ? 1 : blocks < 1184 ? blocks : 1184);
    if (ids32) rt::feedback_event_kernel<int><<<grid, 256, 0, s>>>(ev, fb->geo, fb->st);
    else rt::feedback_event_kernel<long long><<<grid, 256, 0, s>>>(ev, fb->geo, fb->st);
    FB_CUDA(cudaGetLastError());
    return RT_OK;
}

}  // namespace

extern "C" {

int rt_feedback_create(rt_plan *plan, rt_feedback **out) {
    if (!plan || !out) return RT_ERR_INVALID_ARGUMENT;
    *out = nullptr;
    rt_feedback *fb = new (std::nothrow) rt_feedback();
    if (!fb) return RT_ERR_OUT_OF_MEMORY;
    fb->plan = plan;
    rt::plan_view(plan, &fb->view);
    if (fb->view.layout.n_groups != 1) { delete fb; return RT_ERR_INVALID_ARGUMENT; }
    const uint64_t cap = fb->view.layout.capacity_slots;
    const uint32_t nb = fb->view.n_blocks;
    fb->geo = {cap, fb->view.block_tokens, fb->view.shift, fb->view.magic, fb->view.magic_shift, nb};
    FbDevice guard(fb->view.device);
    // one allocation, carved into the state arrays (all of it starts at zero)
    size_t off = 0;
    auto take = [&](size_t bytes) { size_t at = off; off += align_up(bytes); return at; };
    size_t o_gen = take(4 * (cap + 1)), o_ver = take(4 * nb), o_rs = take(8 * nb), o_ws = take(8 * nb),
           o_cv = take(4 * nb), o_ct = take(8 * nb), o_fh = take(8 * rt::kFreeHeadMax), o_fc = take(4),
           o_eb = take(4 * 3 * rt::kWords), o_arr = take(4), o_sm = take(4 * ((cap + 32) / 32 + 1)), o_bad = take(16),
           o_sets = take(4 * 3 * rt::kWords);
    fb->block_bytes = off;
    cudaError_t e = cudaMalloc(&fb->block, off);
    if (e != cudaSuccess) { delete fb; return fb_fail(e); }
    char *base = static_cast<char *>(fb->block);
    fb->st.generations = reinterpret_cast<int32_t *>(base + o_gen);
    fb->st.versions = reinterpret_cast<int32_t *>(base + o_ver);
    fb->st.read_seen = reinterpret_cast<double *>(base + o_rs);
    fb->st.write_seen = reinterpret_cast<double *>(base + o_ws);
    fb->st.commit_version = reinterpret_cast<int32_t *>(base + o_cv);
    fb->st.commit_time = reinterpret_cast<double *>(base + o_ct);
    fb->st.free_head = reinterpret_cast<long long *>(base + o_fh);
    fb->st.free_count = reinterpret_cast<int32_t *>(base + o_fc);
    fb->st.event_blocks = reinterpret_cast<uint32_t *>(base + o_eb);
    fb->st.arrivals = reinterpret_cast<uint32_t *>(base + o_arr);
    fb->st.slot_marks = reinterpret_cast<uint32_t *>(base + o_sm);
    fb->st.bad = reinterpret_cast<unsigned long long *>(base + o_bad);
    fb->d_sets = reinterpret_cast<uint32_t *>(base + o_sets);
    int st = clear_state(fb, fb->view.stream);
    if (st == RT_OK && cudaStreamSynchronize(fb->view.stream) != cudaSuccess) st = RT_ERR_CUDA;
    if (st != RT_OK) { cudaFree(fb->block); delete fb; return st; }
    fb->epoch = 1;                      // reset() on the first allocator event, slot_feedback.py:25-33
    *out = fb;
    return RT_OK;
}

int rt_feedback_destroy(rt_feedback *fb) {
    if (!fb) return RT_OK;
    FbDevice guard(fb->view.device);
    cudaStreamSynchronize(fb->view.stream);
    cudaFree(fb->block);
    delete fb;
    return RT_OK;
}

int rt_feedback_reset(rt_feedback *fb, void *stream) {
    if (!fb) return RT_ERR_INVALID_ARGUMENT;
    FbDevice guard(fb->view.device);
    int st = clear_state(fb, stream ? (cudaStream_t)stream : fb->view.stream);
    if (st == RT_OK) ++fb->epoch;
    return st;
}

static int feedback_alloc(rt_feedback *fb, const void *d_slots, uint64_t n, const void *d_free_head,
                          uint32_t n_free, double t, void *stream, bool ids32) {
    if (!fb || (!d_slots && n) || (!d_free_head && n_free)) return RT_ERR_INVALID_ARGUMENT;
    FbDevice guard(fb->view.device);
    cudaStream_t s = stream ? (cudaStream_t)stream : fb->view.stream;
    rt::EventArgs ev = {};
    ev.ids_a = d_slots;
    ev.n_a = (long long)n;
    ev.fresh = d_free_head;
    ev.n_fresh = (int)n_free;
    ev.alloc = 1;
    ev.t = t;
    return launch_event(fb, ev, ids32, s);
}

static int feedback_attention(rt_feedback *fb, const void *d_read, uint64_t n_read, const void *d_write,
                              uint64_t n_write, double t, void *stream, bool ids32) {
    if (!fb || (!d_read && n_read) || (!d_write && n_write)) return RT_ERR_INVALID_ARGUMENT;
    FbDevice guard(fb->view.device);
    cudaStream_t s = stream ? (cudaStream_t)stream : fb->view.stream;
    rt::EventArgs ev = {};
    ev.ids_a = d_read;
    ev.n_a = (long long)n_read;
    ev.ids_b = d_write;
    ev.n_b = (long long)n_write;
    ev.t = t;
    return launch_event(fb, ev, ids32, s);
}

int rt_feedback_alloc(rt_feedback *fb, const int64_t *d_slots, uint64_t n, const int64_t *d_free_head,
                      uint32_t n_free, double t, void *stream) {
    return feedback_alloc(fb, d_slots, n, d_free_head, n_free, t, stream, false);
}

int rt_feedback_alloc_i32(rt_feedback *fb, const int32_t *d_slots, uint64_t n, const int32_t *d_free_head,
                          uint32_t n_free, double t, void *stream) {
    return feedback_alloc(fb, d_slots, n, d_free_head, n_free, t, stream, true);
}

int rt_feedback_attention(rt_feedback *fb, const int64_t *d_read, uint64_t n_read, const int64_t *d_write,
                          uint64_t n_write, double t, void *stream) {
    return feedback_attention(fb, d_read, n_read, d_write, n_write, t, stream, false);
}

int rt_feedback_attention_i32(rt_feedback *fb, const int32_t *d_read, uint64_t n_read, const int32_t *d_write,
                              uint64_t n_write, double t, void *stream) {
    return feedback_attention(fb, d_read, n_read, d_write, n_write, t, stream, true);
}

int rt_feedback_snapshot(rt_feedback *fb, int32_t *versions, double *read_seen, double *write_seen,
                         int64_t *free_head, uint32_t *n_free, uint64_t *epoch, uint64_t *invalid_slots) {
    if (!fb) return RT_ERR_INVALID_ARGUMENT;
    FbDevice guard(fb->view.device);
    cudaStream_t s = fb->view.stream;
    const uint32_t nb = fb->geo.n_blocks;
    int32_t count = 0;
    unsigned long long bad[2] = {0, 0};
    if (versions) FB_CUDA(cudaMemcpyAsync(versions, fb->st.versions, 4 * nb, cudaMemcpyDeviceToHost, s));
    if (read_seen) FB_CUDA(cudaMemcpyAsync(read_seen, fb->st.read_seen, 8 * nb, cudaMemcpyDeviceToHost, s));
    if (write_seen) FB_CUDA(cudaMemcpyAsync(write_seen, fb->st.write_seen, 8 * nb, cudaMemcpyDeviceToHost, s));
    if (free_head)
        FB_CUDA(cudaMemcpyAsync(free_head, fb->st.free_head, 8 * rt::kFreeHeadMax, cudaMemcpyDeviceToHost, s));
    FB_CUDA(cudaMemcpyAsync(&count, fb->st.free_count, 4, cudaMemcpyDeviceToHost, s));
    FB_CUDA(cudaMemcpyAsync(bad, fb->st.bad, 16, cudaMemcpyDeviceToHost, s));
    FB_CUDA(cudaStreamSynchronize(s));
    if (n_free) *n_free = (uint32_t)count;
    if (epoch) *epoch = fb->epoch;
    if (invalid_slots) *invalid_slots = bad[0];
    return RT_OK;
}

static bool policy_ok(const rt_feedback_policy *policy) {
    return policy && policy->active_seconds > 0 && policy->refresh_seconds > 0;
}

static rt::RankPolicy rank_policy(const rt_feedback_policy *policy, double at, double now) {
    rt::RankPolicy pol;
    pol.budget = policy->budget;
    pol.max_blocks = policy->max_blocks_per_update;
    pol.flags = policy->flags;
    pol.at = at;
    pol.now = now;
    pol.commit = now;
    pol.active_seconds = policy->active_seconds;
    pol.refresh_seconds = policy->refresh_seconds;
    return pol;
}

// one thread per block id, a power of two for the sorting network, and at
// least the CTA the tail part needs
static uint32_t rank_threads(const rt_feedback *fb) {
    uint32_t threads = rt::kScanThreads;
    while (threads < fb->geo.n_blocks) threads <<= 1;
    return threads;
}

static int feedback_step(rt_feedback *fb, const rt_feedback_step_ids *ids, const rt_feedback_policy *policy,
                         double now, rt_range *out, uint32_t cap, rt_plan_result *result, void *stream,
                         bool ids32) {
    if (!fb || !ids || !policy_ok(policy) || !result || (!out && cap) || (!ids->d_allocated && ids->n_allocated) ||
        (!ids->d_free_head && ids->n_free) || (!ids->d_read && ids->n_read) || (!ids->d_written && ids->n_written))
        return RT_ERR_INVALID_ARGUMENT;
    if (ids32 && fb->geo.capacity > 0x7fffffffull) return RT_ERR_INVALID_ARGUMENT;
    FbDevice guard(fb->view.device);
    cudaStream_t s = stream ? (cudaStream_t)stream : fb->view.stream;
    rt::StepArgs ev = {};
    ev.alloc.ids_a = ids->d_allocated;
    ev.alloc.n_a = (long long)ids->n_allocated;
    ev.alloc.fresh = ids->d_free_head;
    ev.alloc.n_fresh = (int)ids->n_free;
    ev.alloc.alloc = 1;
    ev.alloc.t = ids->t_allocated;
    ev.attention.ids_a = ids->d_read;
    ev.attention.n_a = (long long)ids->n_read;
    ev.attention.ids_b = ids->d_written;
    ev.attention.n_b = (long long)ids->n_written;
    ev.attention.t = ids->t_attention;
    rt::RankPolicy pol = rank_policy(policy, ids->t_attention, now);
    rt::PlanArgs p;
    rt::plan_fill_args(fb->plan, p, RT_MAX_BLOCKS, policy->flags | RT_PLAN_DRY_RUN, out, cap, result);
    p.explicit_sets = 1;
    const uint32_t threads = rank_threads(fb);
    // a CTA per `threads` ids of the longest list, at most one wave of the device
    uint64_t longest = ids->n_allocated > ids->n_read ? ids->n_allocated : ids->n_read;
    if (ids->n_written > longest) longest = ids->n_written;
    uint64_t want = (longest + threads - 1) / threads;
    const uint64_t wave = (uint64_t)fb->view.sm_count * (2048 / threads);
    int grid = (int)(want < 1 ? 1 : want < wave ? want : wave);
    if (ids32)
        rt::feedback_step_kernel<int><<<grid, threads, 0, s>>>(ev, fb->geo, fb->st, pol, fb->view.d_resident,
                                                               fb->d_sets, p);
    else
        rt::feedback_step_kernel<long long><<<grid, threads, 0, s>>>(ev, fb->geo, fb->st, pol,
                                                                     fb->view.d_resident, fb->d_sets, p);
    FB_CUDA(cudaGetLastError());
    return RT_OK;
}

int rt_feedback_step(rt_feedback *fb, const rt_feedback_step_ids *ids, const rt_feedback_policy *policy, double now,
                     rt_range *out, uint32_t cap, rt_plan_result *result, void *stream) {
    return feedback_step(fb, ids, policy, now, out, cap, result, stream, false);
}

int rt_feedback_step_i32(rt_feedback *fb, const rt_feedback_step_ids *ids, const rt_feedback_policy *policy,
                         double now, rt_range *out, uint32_t cap, rt_plan_result *result, void *stream) {
    return feedback_step(fb, ids, policy, now, out, cap, result, stream, true);
}

int rt_feedback_plan(rt_feedback *fb, const rt_feedback_policy *policy, double at, double now, rt_range *out,
                     uint32_t cap, rt_plan_result *result, void *stream) {
    if (!fb || !policy_ok(policy) || !result || (!out && cap)) return RT_ERR_INVALID_ARGUMENT;
    FbDevice guard(fb->view.device);
    cudaStream_t s = stream ? (cudaStream_t)stream : fb->view.stream;
    rt::RankPolicy pol;
    pol.budget = policy->budget;
    pol.max_blocks = policy->max_blocks_per_update;
    pol.flags = policy->flags;
    pol.at = at;
    pol.now = now;
    pol.commit = now;
    pol.active_seconds = policy->active_seconds;
    pol.refresh_seconds = policy->refresh_seconds;
    rt::PlanArgs p;
    rt::plan_fill_args(fb->plan, p, RT_MAX_BLOCKS, policy->flags | RT_PLAN_DRY_RUN, out, cap, result);
    p.explicit_sets = 1;
    // one thread per block id, a power of two for the sorting network, and at
    // least the CTA the tail part needs
    uint32_t threads = rt::kScanThreads;
    while (threads < fb->geo.n_blocks) threads <<= 1;
    rt::feedback_rank_kernel<<<1, threads, 0, s>>>(fb->geo, fb->st, pol, fb->view.d_resident, fb->d_sets, p);
    FB_CUDA(cudaGetLastError());
    return RT_OK;
}

}  // extern "C"
