// C ABI of the device planner: plan handles, argument checks, launches.
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <new>
#include <vector>

#include "plan_device.cuh"
#include "rt_internal.h"
#include "plan_internal.h"
#include "host_pack.h"

namespace rt {
void division_magic(uint32_t d, uint32_t *magic, uint32_t *shift);
cudaError_t launch_scan_plan(const ScanArgs &a, const PlanArgs &p, bool table, bool ids32, int grid,
                             cudaStream_t stream, bool chained);
cudaError_t launch_scan_plan_tma(const ScanArgs &a, const PlanArgs &p, int grid, cudaStream_t stream,
                                 bool chained);
cudaError_t launch_plan_tail(const uint32_t *want, const PlanArgs &p, cudaStream_t stream);
cudaError_t scan_plan_occupancy(uint32_t n_groups, uint32_t n_buffers, int *plain_blocks_per_sm,
                                int *tma_blocks_per_sm, int *table_blocks_per_sm);
}  // namespace rt

constexpr unsigned kUnset = ~0u;

struct rt_plan {
    rt_layout layout;
    int device = 0;
    int sm_count = 0;
    int plain_blocks_per_sm = 1;
    int tma_blocks_per_sm = 1;
    int table_blocks_per_sm = 1;
    uint32_t n_blocks = 0;
    uint32_t block_tokens = 0;
    int shift = -1;
    uint32_t magic = 0, magic_shift = 0;
    cudaStream_t stream = nullptr;
    rt::GroupScratch *d_groups = nullptr;    // two sets of n_groups, used by the scan launches in turn
    rt::GlobalScratch *d_global = nullptr;   // two sets
    uint32_t scans = 0;                      // scan launches issued so far
    uint32_t *d_resident = nullptr;
    uint8_t *d_buffer_group = nullptr;  // bitmap of every buffer, registry order
    uint16_t *d_group_size = nullptr;   // buffers per bitmap
    long long *d_stage = nullptr;      // host-buffer call: slot ids land here
    int32_t *h_narrow = nullptr;       // host-buffer call: pinned staging for ids narrowed to 32 bits
    unsigned narrow_threads = kUnset;  // host threads that do the narrowing (0: never narrow)
    uint64_t max_indices = 0;
    rt_range *h_out = nullptr;         // pinned + mapped: the kernel writes ranges here
    rt_plan_result *h_result = nullptr;
    uint32_t max_ranges = 0;
};

namespace {

thread_local int g_last_cuda_error = 0;

int cuda_fail(cudaError_t e) {
    g_last_cuda_error = (int)e;
    if (e == cudaErrorNoDevice || e == cudaErrorInsufficientDriver || e == cudaErrorInitializationError)
        return RT_ERR_NO_DEVICE;
    if (e == cudaErrorMemoryAllocation) return RT_ERR_OUT_OF_MEMORY;
    return RT_ERR_CUDA;
}

#define RT_CUDA(call)                                  \
    do {                                               \
        cudaError_t e__ = (call);                      \
        if (e__ != cudaSuccess) return cuda_fail(e__); \
    } while (0)

struct DeviceGuard {
    int prev = -1;
    bool ok = false;
    explicit DeviceGuard(int device) {
        if (cudaGetDevice(&prev) != cudaSuccess) prev = -1;
        ok = cudaSetDevice(device) == cudaSuccess;
    }
    ~DeviceGuard() {
        if (prev >= 0) cudaSetDevice(prev);
    }
};

void fill_plan_args(const rt_plan *pl, rt::PlanArgs &p, uint32_t budget, uint32_t flags,
                    rt_range *out, uint32_t cap, rt_plan_result *result) {
    p.groups = pl->d_groups;                 // set 0; scan launches choose theirs with next_scratch()
    p.global = pl->d_global;
    p.resident = pl->d_resident;
    p.buffer_group = pl->d_buffer_group;
    p.group_size = pl->d_group_size;
    p.n_units = 0;
    p.bitmaps_out = nullptr;
    p.out = out;
    p.result = result;
    p.cap = cap;
    p.n_buffers = pl->layout.n_buffers;
    p.n_groups = pl->layout.n_groups;
    p.n_blocks = pl->n_blocks;
    p.budget = budget;
    p.flags = flags;
    p.dst_device = pl->layout.dst_device;
    p.scan_only = 0;
    p.explicit_sets = 0;
    p.alloc_bytes = pl->layout.alloc_bytes;
    p.block_bytes = pl->layout.block_bytes;
}

// Scan launches alternate between the plan's two scratch sets (plan_device.cuh).
void next_scratch(rt_plan *pl, rt::PlanArgs &p) {
    const uint32_t set = pl->scans++ & 1u;
    p.groups = pl->d_groups + (size_t)set * pl->layout.n_groups;
    p.global = pl->d_global + set;
}

// CSR work-unit table.  Every group gets at least one unit so that its tail
// runs even when it has no ids this step.
// ids of one 16-byte load and of one 16 KiB work unit, by id width
inline long long ids_per_vec(bool ids32) { return ids32 ? 4 : 2; }
inline long long ids_per_unit(bool ids32) { return ids32 ? 2 * rt::kChunkElems : rt::kChunkElems; }

int fill_scan_args_csr(const rt_plan *pl, rt::ScanArgs &a, const void *d_slots,
                       const int64_t *group_off, bool ids32) {
    const uint32_t G = pl->layout.n_groups;
    // int32 ids: a negative id must never look like a valid large one
    if (ids32 && pl->layout.capacity_slots > 0x7fffffffull) return RT_ERR_INVALID_ARGUMENT;
    const long long per_vec = ids_per_vec(ids32), per_unit = ids_per_unit(ids32);
    a.slots = reinterpret_cast<const long long *>(d_slots);
    a.lens = nullptr;
    a.stride = 0;
    a.seg_ids = 0;
    a.n_rows = 0;
    a.segs_per_row = 0;
    a.n_groups = (int)G;
    a.capacity = pl->layout.capacity_slots;
    a.block_tokens = pl->block_tokens;
    a.shift = pl->shift;
    a.magic = pl->magic;
    a.magic_shift = pl->magic_shift;
    long long units = 0;
    for (uint32_t g = 0; g < G; ++g) {
        long long lo = group_off[g], hi = group_off[g + 1];
        if (lo < 0 || hi < lo) return RT_ERR_INVALID_ARGUMENT;
        a.group_off[g] = lo;
        a.unit_first[g] = (int)units;
        long long span = hi - (lo & ~(per_vec - 1));
        long long n = (span + per_unit - 1) / per_unit;
        units += n > 0 ? n : 1;
        if (units > 0x7fffffffLL) return RT_ERR_CAPACITY;
    }
    a.group_off[G] = group_off[G];
    a.unit_first[G] = (int)units;
    a.n_units = (int)units;
    if ((reinterpret_cast<uintptr_t>(d_slots) & 15u) && group_off[G] > 0) return RT_ERR_ALIGNMENT;
    return RT_OK;
}

// Worker CTAs of a launch.  One wave: every CTA is resident from the start and
// owns one contiguous span; one slot of the wave is left for the gatekeeper CTA
// the launcher adds.  A chained launch leaves a second slot free: the one the
// launch before it is still running its tail in.  Without it one worker starts
// late by the length of that tail and, the spans being fixed, finishes late.
int grid_for(const rt_plan *pl, int units, bool tma, bool chained) {
    const int per_sm = tma ? pl->tma_blocks_per_sm : pl->plain_blocks_per_sm;
    long long slots = (long long)pl->sm_count * per_sm - 1 - (chained ? 1 : 0);
    if (slots < 1) slots = 1;
    return (int)(units < slots ? units : slots);
}

bool want_tma(uint32_t flags) { return (flags & RT_PLAN_TMA) != 0; }

}  // namespace

namespace rt {
// Multiplier and shift for dividing any 32-bit n by d (d not a power of two):
//   q = mulhi(n, magic);  n / d == (((n - q) >> 1) + q) >> shift
// This is the round-up method with a 33-bit multiplier whose top bit is
// folded into the add (Granlund & Montgomery; the "branch-free" libdivide form).
void division_magic(uint32_t d, uint32_t *magic, uint32_t *shift) {
    uint32_t k = 31;
    while (!(d >> k)) --k;                       // floor(log2 d)
    const uint64_t two_k = 1ull << (32 + k);
    uint64_t m = two_k / d, rem = two_k % d;     // floor(2^(32+k) / d)
    m *= 2;
    uint64_t twice = rem * 2;
    if (twice >= d) m += 1;
    *magic = (uint32_t)(m + 1);
    *shift = k;
}
// What other translation units (the feedback state) need to know about a plan.
void plan_view(const rt_plan *pl, PlanView *v) {
    v->layout = pl->layout;
    v->device = pl->device;
    v->stream = pl->stream;
    v->d_resident = pl->d_resident;
    v->n_blocks = pl->n_blocks;
    v->block_tokens = pl->block_tokens;
    v->shift = pl->shift;
    v->magic = pl->magic;
    v->magic_shift = pl->magic_shift;
    v->sm_count = pl->sm_count;
}
void plan_fill_args(const rt_plan *pl, PlanArgs &p, uint32_t budget, uint32_t flags, rt_range *out,
                    uint32_t cap, rt_plan_result *result) {
    fill_plan_args(pl, p, budget, flags, out, cap, result);
}
int last_cuda_error_get() { return g_last_cuda_error; }
void last_cuda_error_set(int e) { g_last_cuda_error = e; }
}  // namespace rt

extern "C" {

int rt_plan_create(const rt_layout *layout, int device, uint64_t max_indices, uint32_t max_ranges,
                   rt_plan **out) {
    if (!layout || !out) return RT_ERR_INVALID_ARGUMENT;
    *out = nullptr;
    const rt_layout &L = *layout;
    if (!L.n_buffers || L.n_buffers > RT_MAX_BUFFERS || !L.n_groups || L.n_groups > RT_MAX_GROUPS ||
        !L.alloc_bytes || !L.bytes_per_slot || !L.block_bytes || L.block_bytes > L.alloc_bytes ||
        L.block_bytes % L.bytes_per_slot || !L.capacity_slots || L.capacity_slots > 0xfffffffeull)
        return RT_ERR_INVALID_ARGUMENT;
    uint64_t n_blocks = L.alloc_bytes / L.block_bytes + (L.alloc_bytes % L.block_bytes != 0);
    uint32_t block_tokens = L.block_bytes / L.bytes_per_slot;
    if (n_blocks > RT_MAX_BLOCKS || L.capacity_slots / block_tokens >= n_blocks)
        return RT_ERR_INVALID_ARGUMENT;
    if (L.buffer_group)
        for (uint32_t j = 0; j < L.n_buffers; ++j)
            if (L.buffer_group[j] >= L.n_groups) return RT_ERR_INVALID_ARGUMENT;
    if (!L.buffer_group && L.n_groups != 1) return RT_ERR_INVALID_ARGUMENT;

    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess) return cuda_fail(e);
    if (device < 0 || device >= count) return RT_ERR_NO_DEVICE;
    DeviceGuard guard(device);
    if (!guard.ok) return RT_ERR_NO_DEVICE;

    rt_plan *pl = new (std::nothrow) rt_plan();
    if (!pl) return RT_ERR_OUT_OF_MEMORY;
    pl->layout = L;
    pl->layout.buffer_group = nullptr;
    pl->device = device;
    pl->n_blocks = (uint32_t)n_blocks;
    pl->block_tokens = block_tokens;
    pl->shift = -1;
    if ((block_tokens & (block_tokens - 1)) == 0) {
        int s = 0;
        while ((1u << s) != block_tokens) ++s;
        pl->shift = s;
    } else {
        rt::division_magic(block_tokens, &pl->magic, &pl->magic_shift);
    }
    pl->max_indices = max_indices;
    pl->max_ranges = max_ranges;
    int status = RT_OK;
    auto fail = [&](cudaError_t err) { status = cuda_fail(err); };
    do {
        if ((e = cudaDeviceGetAttribute(&pl->sm_count, cudaDevAttrMultiProcessorCount, device))) { fail(e); break; }
        if ((e = rt::scan_plan_occupancy(L.n_groups, L.n_buffers, &pl->plain_blocks_per_sm,
                                         &pl->tma_blocks_per_sm, &pl->table_blocks_per_sm))) { fail(e); break; }
        if (pl->plain_blocks_per_sm < 1) pl->plain_blocks_per_sm = 1;
        if (pl->table_blocks_per_sm < 1) pl->table_blocks_per_sm = 1;
        if (pl->tma_blocks_per_sm < 1) pl->tma_blocks_per_sm = 1;
        if ((e = cudaStreamCreateWithFlags(&pl->stream, cudaStreamNonBlocking))) { fail(e); break; }
        size_t gbytes = 2 * sizeof(rt::GroupScratch) * L.n_groups;
        if ((e = cudaMalloc(&pl->d_groups, gbytes))) { fail(e); break; }
        if ((e = cudaMemset(pl->d_groups, 0, gbytes))) { fail(e); break; }
        if ((e = cudaMalloc(&pl->d_global, 2 * sizeof(rt::GlobalScratch)))) { fail(e); break; }
        if ((e = cudaMemset(pl->d_global, 0, 2 * sizeof(rt::GlobalScratch)))) { fail(e); break; }
        size_t rbytes = sizeof(uint32_t) * rt::kWords * L.n_groups;
        if ((e = cudaMalloc(&pl->d_resident, rbytes))) { fail(e); break; }
        if ((e = cudaMemset(pl->d_resident, 0, rbytes))) { fail(e); break; }
        {
            uint8_t table[RT_MAX_BUFFERS] = {0};
            if (L.buffer_group)
                for (uint32_t j = 0; j < L.n_buffers; ++j) table[j] = (uint8_t)L.buffer_group[j];
            uint16_t sizes[RT_MAX_GROUPS] = {0};
            for (uint32_t j = 0; j < L.n_buffers; ++j) ++sizes[table[j]];
            if ((e = cudaMalloc(&pl->d_buffer_group, L.n_buffers))) { fail(e); break; }
            if ((e = cudaMemcpy(pl->d_buffer_group, table, L.n_buffers, cudaMemcpyHostToDevice))) { fail(e); break; }
            if ((e = cudaMalloc(&pl->d_group_size, sizeof(uint16_t) * L.n_groups))) { fail(e); break; }
            if ((e = cudaMemcpy(pl->d_group_size, sizes, sizeof(uint16_t) * L.n_groups, cudaMemcpyHostToDevice))) { fail(e); break; }
        }
        if (max_indices) {
            // +2 ids of slack so a 16-byte load at the very end stays in bounds
            if ((e = cudaMalloc(&pl->d_stage, sizeof(long long) * (max_indices + 2)))) { fail(e); break; }
        }
        if ((e = cudaHostAlloc(&pl->h_out, sizeof(rt_range) * (max_ranges ? max_ranges : 1),
                               cudaHostAllocMapped))) { fail(e); break; }
        if ((e = cudaHostAlloc(&pl->h_result, sizeof(rt_plan_result), cudaHostAllocMapped))) { fail(e); break; }
        if ((e = cudaDeviceSynchronize())) { fail(e); break; }
    } while (0);
    if (status != RT_OK) {
        rt_plan_destroy(pl);
        return status;
    }
    *out = pl;
    return RT_OK;
}

int rt_plan_destroy(rt_plan *pl) {
    if (!pl) return RT_OK;
    DeviceGuard guard(pl->device);
    if (pl->stream) {
        cudaStreamSynchronize(pl->stream);
        cudaStreamDestroy(pl->stream);
    }
    cudaFree(pl->d_groups);
    cudaFree(pl->d_global);
    cudaFree(pl->d_resident);
    cudaFree(pl->d_buffer_group);
    cudaFree(pl->d_group_size);
    cudaFree(pl->d_stage);
    if (pl->h_out) cudaFreeHost(pl->h_out);
    if (pl->h_narrow) cudaFreeHost(pl->h_narrow);
    if (pl->h_result) cudaFreeHost(pl->h_result);
    delete pl;
    return RT_OK;
}

int rt_plan_set_resident(rt_plan *pl, const uint32_t *words) {
    if (!pl || !words) return RT_ERR_INVALID_ARGUMENT;
    DeviceGuard guard(pl->device);
    size_t bytes = sizeof(uint32_t) * rt::kWords * pl->layout.n_groups;
    RT_CUDA(cudaMemcpyAsync(pl->d_resident, words, bytes, cudaMemcpyHostToDevice, pl->stream));
    RT_CUDA(cudaStreamSynchronize(pl->stream));
    return RT_OK;
}

int rt_plan_get_resident(rt_plan *pl, uint32_t *words) {
    if (!pl || !words) return RT_ERR_INVALID_ARGUMENT;
    DeviceGuard guard(pl->device);
    size_t bytes = sizeof(uint32_t) * rt::kWords * pl->layout.n_groups;
    RT_CUDA(cudaMemcpyAsync(words, pl->d_resident, bytes, cudaMemcpyDeviceToHost, pl->stream));
    RT_CUDA(cudaStreamSynchronize(pl->stream));
    return RT_OK;
}

}  // extern "C"

namespace {

int step_device_impl(rt_plan *pl, const void *d_slots, bool ids32, const int64_t *group_off,
                     uint32_t budget, uint32_t flags, rt_range *out, uint32_t cap,
                     rt_plan_result *result, void *stream) {
    if (!pl || !group_off || !result || (!out && cap)) return RT_ERR_INVALID_ARGUMENT;
    if (!d_slots && group_off[pl->layout.n_groups] > 0) return RT_ERR_INVALID_ARGUMENT;
    DeviceGuard guard(pl->device);
    rt::ScanArgs a;
    const bool tma = !ids32 && want_tma(flags);      // the bulk-copy kernel reads int64 ids only
    int st = fill_scan_args_csr(pl, a, d_slots, group_off, ids32);
    if (st != RT_OK) return st;
    rt::PlanArgs p;
    fill_plan_args(pl, p, budget, flags, out, cap, result);
    p.n_units = (uint32_t)a.n_units;
    next_scratch(pl, p);
    cudaStream_t s = stream ? (cudaStream_t)stream : pl->stream;
    const bool chained = (flags & RT_PLAN_CHAINED) != 0;
    int grid = grid_for(pl, a.n_units, tma, chained);
    RT_CUDA(tma ? rt::launch_scan_plan_tma(a, p, grid, s, chained)
                : rt::launch_scan_plan(a, p, false, ids32, grid, s, chained));
    return RT_OK;
}

unsigned plan_narrow_threads(rt_plan *pl) {
    if (pl->narrow_threads == kUnset) {
        int devices = 1;
        if (cudaGetDeviceCount(&devices) != cudaSuccess || devices < 1) devices = 1;
        pl->narrow_threads = rt::narrow_threads((unsigned)devices);
    }
    return pl->narrow_threads;
}

constexpr int64_t kNarrowMinIds = 1 << 20;       // below this the wide copy takes well under a millisecond
constexpr size_t kNarrowChunkIds = 1 << 20;      // 8 MiB in, 4 MiB out per chunk

int step_host_impl(rt_plan *pl, const void *h_slots, bool ids32, const int64_t *group_off,
                   uint32_t budget, uint32_t flags, rt_range *out, uint32_t cap,
                   rt_plan_result *result) {
    if (!pl || !group_off || !result || (!out && cap)) return RT_ERR_INVALID_ARGUMENT;
    const uint32_t G = pl->layout.n_groups;
    int64_t n = group_off[G];
    if (n < 0 || (uint64_t)n > pl->max_indices || group_off[0] < 0) return RT_ERR_CAPACITY;
    if (n && !h_slots) return RT_ERR_INVALID_ARGUMENT;
    DeviceGuard guard(pl->device);
    // 64-bit ids of a pool that 32 bits can number cross the host link as 32-bit
    // ids: narrowed on the host cores into pinned memory, each chunk copied as soon
    // as it is complete while the chunks after it are being narrowed.  Half the bytes on
    // the link, which is what bounds this call; the caller's buffer need not be
    // pinned.  (The bulk-copy kernel has no 32-bit form; short lists are not
    // worth the hand-over to the worker threads.)
    bool narrow = !ids32 && !(flags & (RT_PLAN_WIDE_COPY | RT_PLAN_TMA)) && n >= kNarrowMinIds &&
                  pl->layout.capacity_slots < 0x7fffffffull;
    narrow = narrow && plan_narrow_threads(pl) > 0;
    if (narrow && !pl->h_narrow &&
        cudaHostAlloc(reinterpret_cast<void **>(&pl->h_narrow), 4 * (size_t)pl->max_indices + 64,
                      cudaHostAllocDefault) != cudaSuccess) {
        // no pinned memory for the staging buffer: this plan copies its ids as they are
        cudaGetLastError();
        pl->h_narrow = nullptr;
        pl->narrow_threads = 0;
        narrow = false;
    }
    if (narrow) {
        // every chunk is copied as soon as it is narrowed, while the host threads go on
        struct Copier {
            rt_plan *pl;
            cudaError_t err;
        } copier = {pl, cudaSuccess};
        rt::narrow_ids_streamed(
            static_cast<const int64_t *>(h_slots), pl->h_narrow, (size_t)n, pl->narrow_threads, kNarrowChunkIds,
            [](void *ctx, size_t first, size_t count) {
                Copier *c = static_cast<Copier *>(ctx);
                if (c->err != cudaSuccess) return;
                c->err = cudaMemcpyAsync(reinterpret_cast<int32_t *>(c->pl->d_stage) + first, c->pl->h_narrow + first,
                                         4 * count, cudaMemcpyHostToDevice, c->pl->stream);
            },
            &copier);
        RT_CUDA(copier.err);
        ids32 = true;
    } else if (n) {
        RT_CUDA(cudaMemcpyAsync(pl->d_stage, h_slots, (ids32 ? 4 : 8) * (size_t)n, cudaMemcpyHostToDevice,
                                pl->stream));
    }
    uint32_t dev_cap = cap < pl->max_ranges ? cap : pl->max_ranges;
    // (the copy precedes the kernel in the stream: nothing to chain to)
    int st = step_device_impl(pl, pl->d_stage, ids32, group_off, budget, flags & ~RT_PLAN_CHAINED,
                              pl->h_out, dev_cap, pl->h_result, pl->stream);
    if (st != RT_OK) return st;
    RT_CUDA(cudaStreamSynchronize(pl->stream));
    *result = *pl->h_result;
    uint32_t n_copy = result->n_ranges < dev_cap ? result->n_ranges : dev_cap;
    if (n_copy) memcpy(out, pl->h_out, sizeof(rt_range) * n_copy);
    // none of these plans was committed: the resident bitmaps are what they were
    if (result->flags & RT_RESULT_TIMEOUT) return RT_ERR_TIMEOUT;
    if (result->flags & RT_RESULT_SLOT_RANGE) return RT_ERR_SLOT_RANGE;
    if (result->flags & RT_RESULT_OVERFLOW) return RT_ERR_CAPACITY;
    return RT_OK;
}

int step_table_impl(rt_plan *pl, const void *d_table, bool ids32, const int32_t *d_lens,
                    uint32_t n_rows, uint64_t stride, uint32_t budget, uint32_t flags, rt_range *out,
                    uint32_t cap, rt_plan_result *result, void *stream) {
    if (!pl || !result || (!out && cap) || pl->layout.n_groups != 1) return RT_ERR_INVALID_ARGUMENT;
    if (!n_rows || !stride || !d_table || !d_lens) return RT_ERR_INVALID_ARGUMENT;
    if (ids32 && pl->layout.capacity_slots > 0x7fffffffull) return RT_ERR_INVALID_ARGUMENT;
    if (reinterpret_cast<uintptr_t>(d_table) & 15u) return RT_ERR_ALIGNMENT;
    DeviceGuard guard(pl->device);
    rt::ScanArgs a;
    memset(&a, 0, sizeof(a));
    a.slots = reinterpret_cast<const long long *>(d_table);
    a.lens = d_lens;
    a.stride = (long long)stride;
    if (stride > (1ull << 40) || n_rows > 0x7fffffffu) return RT_ERR_INVALID_ARGUMENT;
    // Work is dealt by row segment: to warps (8 per CTA) when rows are long enough
    // for a warp each, else to CTAs.  Rows are cut into segments of at least 1024
    // ids until there are about four segments per worker, so that the last round
    // of the round-robin leaves few workers idle.
    // one wave, less the gatekeeper and, when chained, the slot the previous launch's tail still runs in
    const unsigned long long ctas = (unsigned long long)pl->sm_count * pl->table_blocks_per_sm - 1 -
                                    ((flags & RT_PLAN_CHAINED) ? 1 : 0);
    const unsigned long long workers = stride >= 1024 ? ctas * (rt::kScanThreads / 32) : ctas;
    unsigned long long segs = 1;
    if (n_rows < 4 * workers) {
        segs = (4 * workers + n_rows - 1) / n_rows;
        const unsigned long long most = stride / 1024 ? stride / 1024 : 1;
        if (segs > most) segs = most;
    }
    unsigned long long seg_ids = (stride + segs - 1) / segs;
    seg_ids = (seg_ids + 3) & ~3ull;                              // segments start on the row's own 16-byte grid
    if (seg_ids > (1ull << 20)) seg_ids = 1ull << 20;             // keeps a pass's vector count in 32 bits
    segs = (stride + seg_ids - 1) / seg_ids;
    if (segs > 0xffffffffull) return RT_ERR_CAPACITY;
    a.seg_ids = (long long)seg_ids;
    a.n_rows = n_rows;
    a.segs_per_row = (uint32_t)segs;
    const unsigned long long n_virtual = (unsigned long long)n_rows * segs;
    const int grid = (int)(n_virtual < ctas ? n_virtual : ctas);
    a.n_units = grid;                                             // every CTA arrives once
    a.n_groups = 1;
    a.capacity = pl->layout.capacity_slots;
    a.block_tokens = pl->block_tokens;
    a.shift = pl->shift;
    a.magic = pl->magic;
    a.magic_shift = pl->magic_shift;
    rt::PlanArgs p;
    fill_plan_args(pl, p, budget, flags, out, cap, result);
    p.n_units = (uint32_t)a.n_units;
    next_scratch(pl, p);
    cudaStream_t s = stream ? (cudaStream_t)stream : pl->stream;
    RT_CUDA(rt::launch_scan_plan(a, p, true, ids32, grid, s, (flags & RT_PLAN_CHAINED) != 0));
    return RT_OK;
}

int scan_slots_impl(rt_plan *pl, const void *d_slots, bool ids32, const int64_t *group_off,
                    uint32_t *d_bitmaps, rt_plan_result *result, void *stream) {
    if (!pl || !group_off || !result || !d_bitmaps) return RT_ERR_INVALID_ARGUMENT;
    if (!d_slots && group_off[pl->layout.n_groups] > 0) return RT_ERR_INVALID_ARGUMENT;
    DeviceGuard guard(pl->device);
    rt::ScanArgs a;
    int st = fill_scan_args_csr(pl, a, d_slots, group_off, ids32);
    if (st != RT_OK) return st;
    rt::PlanArgs p;
    fill_plan_args(pl, p, 0, 0, nullptr, 0, result);
    p.n_units = (uint32_t)a.n_units;
    p.scan_only = 1;
    p.bitmaps_out = d_bitmaps;
    next_scratch(pl, p);
    cudaStream_t s = stream ? (cudaStream_t)stream : pl->stream;
    RT_CUDA(rt::launch_scan_plan(a, p, false, ids32, grid_for(pl, a.n_units, false, false), s, false));
    return RT_OK;
}

}  // namespace

extern "C" {

int rt_plan_step_device(rt_plan *pl, const int64_t *d_slots, const int64_t *group_off,
                        uint32_t budget, uint32_t flags, rt_range *out, uint32_t cap,
                        rt_plan_result *result, void *stream) {
    return step_device_impl(pl, d_slots, false, group_off, budget, flags, out, cap, result, stream);
}

int rt_plan_step_device_i32(rt_plan *pl, const int32_t *d_slots, const int64_t *group_off,
                            uint32_t budget, uint32_t flags, rt_range *out, uint32_t cap,
                            rt_plan_result *result, void *stream) {
    return step_device_impl(pl, d_slots, true, group_off, budget, flags, out, cap, result, stream);
}

int rt_plan_step(rt_plan *pl, const int64_t *h_slots, const int64_t *group_off, uint32_t budget,
                 uint32_t flags, rt_range *out, uint32_t cap, rt_plan_result *result) {
    return step_host_impl(pl, h_slots, false, group_off, budget, flags, out, cap, result);
}

int rt_plan_step_i32(rt_plan *pl, const int32_t *h_slots, const int64_t *group_off, uint32_t budget,
                     uint32_t flags, rt_range *out, uint32_t cap, rt_plan_result *result) {
    return step_host_impl(pl, h_slots, true, group_off, budget, flags, out, cap, result);
}

int rt_plan_narrow_threads(rt_plan *pl, uint32_t *threads) {
    if (!pl || !threads) return RT_ERR_INVALID_ARGUMENT;
    *threads = plan_narrow_threads(pl);
    return RT_OK;
}

int rt_narrow_ids(const int64_t *src, int32_t *dst, uint64_t n, uint32_t threads) {
    if ((!src || !dst) && n) return RT_ERR_INVALID_ARGUMENT;
    if (!threads) {
        int devices = 1;
        if (cudaGetDeviceCount(&devices) != cudaSuccess || devices < 1) devices = 1;
        threads = rt::narrow_threads((unsigned)devices);
        if (!threads) threads = 1;
    }
    rt::narrow_ids_parallel(src, dst, (size_t)n, threads);
    return RT_OK;
}

int rt_plan_step_table(rt_plan *pl, const int64_t *d_table, const int32_t *d_lens, uint32_t n_rows,
                       uint64_t stride, uint32_t budget, uint32_t flags, rt_range *out, uint32_t cap,
                       rt_plan_result *result, void *stream) {
    return step_table_impl(pl, d_table, false, d_lens, n_rows, stride, budget, flags, out, cap, result,
                           stream);
}

int rt_plan_step_table_i32(rt_plan *pl, const int32_t *d_table, const int32_t *d_lens, uint32_t n_rows,
                           uint64_t stride, uint32_t budget, uint32_t flags, rt_range *out,
                           uint32_t cap, rt_plan_result *result, void *stream) {
    return step_table_impl(pl, d_table, true, d_lens, n_rows, stride, budget, flags, out, cap, result,
                           stream);
}

int rt_scan_slots(rt_plan *pl, const int64_t *d_slots, const int64_t *group_off, uint32_t *d_bitmaps,
                  rt_plan_result *result, void *stream) {
    return scan_slots_impl(pl, d_slots, false, group_off, d_bitmaps, result, stream);
}

int rt_scan_slots_i32(rt_plan *pl, const int32_t *d_slots, const int64_t *group_off,
                      uint32_t *d_bitmaps, rt_plan_result *result, void *stream) {
    return scan_slots_impl(pl, d_slots, true, group_off, d_bitmaps, result, stream);
}

int rt_plan_from_bitmaps(rt_plan *pl, const uint32_t *d_want, uint32_t budget, uint32_t flags,
                         rt_range *out, uint32_t cap, rt_plan_result *result, void *stream) {
    if (!pl || !d_want || !result || (!out && cap)) return RT_ERR_INVALID_ARGUMENT;
    DeviceGuard guard(pl->device);
    rt::PlanArgs p;
    fill_plan_args(pl, p, budget, flags, out, cap, result);
    cudaStream_t s = stream ? (cudaStream_t)stream : pl->stream;
    RT_CUDA(rt::launch_plan_tail(d_want, p, s));
    return RT_OK;
}

int rt_plan_sync(rt_plan *pl) {
    if (!pl) return RT_ERR_INVALID_ARGUMENT;
    DeviceGuard guard(pl->device);
    RT_CUDA(cudaStreamSynchronize(pl->stream));
    return RT_OK;
}

}  // extern "C"
