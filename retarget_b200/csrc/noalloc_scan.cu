// rt_scan_slots_static: the slot scan for callers that must not allocate.
//
// Who cannot allocate, and why.  The scan is also wanted from inside the
// LD_PRELOAD library itself (its control thread lives in the serving process).
// There a cudaMalloc is not neutral: it passes through the library's own
// cuMemAlloc hook, comes back as a *registered managed* allocation and bumps
// the allocation generation that every plan command is checked against -- so a
// planner that allocates invalidates the very plan it is computing.  The same
// holds for processes whose device memory is handed over, to the last byte, to
// the serving engine's pool: there is nothing left to ask for, and a failed
// cudaMalloc in the middle of a decode step is not an option.
//
// So this entry point owns no plan handle and calls no cudaMalloc / cudaFree or
// any other allocating routine.  Its working memory (the per-bitmap
// accumulation words and the arrival counters that rt_scan_slots keeps in
// cudaMalloc'ed scratch) is a file-scope __device__ array, 8.25 KiB, which every
// GPU that loads the library holds until the process exits.  That fixes the
// limit: at most RT_STATIC_MAX_GROUPS (64) bitmaps per call; the number of slot
// ids is not limited.
//
// The array's name is only a host-side stand-in for the device object, so the
// host code below never passes it to a kernel: once per device, with that device
// current, it asks cudaGetSymbolAddress for the real device address and keeps
// it.  That set-up happens inside the FIRST call on each device; make that first
// call before any stream capture begins.
//
// All calls on a device share the one array.  It keeps whatever the last call
// left, so every call clears the part it uses (a cudaMemsetAsync on the caller's
// stream, ahead of the kernel).  Two calls that overlap on the GPU (different
// streams, or different threads) race on it: serialise them.
#include <cuda_runtime.h>

#include <cstddef>
#include <mutex>

#include "plan_device.cuh"
#include "plan_tail.cuh"
#include "rt_internal.h"

namespace {

using namespace rt;

struct StaticScratch {
    GlobalScratch global;
    unsigned char pad[256 - sizeof(GlobalScratch)];
    GroupScratch groups[RT_STATIC_MAX_GROUPS];
};

static __device__ __align__(256) unsigned char g_static_scratch[sizeof(StaticScratch)];

struct StaticArgs {
    StaticScratch *scratch;       // device address of g_static_scratch (from cudaGetSymbolAddress)
    uint32_t *bitmaps_out;        // n_groups x kWords
    rt_plan_result *result;
    uint32_t n_blocks;
    uint32_t n_units;
};

__device__ __forceinline__ void mark_one(long long s, const ScanArgs &a, uint8_t *s_map, uint32_t &invalid,
                                         uint32_t &ignored) {
    unsigned long long u = (unsigned long long)(s - 1);
    if (u < a.capacity) {
        uint32_t v = (uint32_t)s;
        uint32_t blk;
        if (a.shift >= 0) {
            blk = v >> a.shift;
        } else {
            uint32_t q = __umulhi(v, a.magic);
            blk = (((v - q) >> 1) + q) >> a.magic_shift;
        }
        s_map[blk] = 1;
    } else if (s < 1) {
        ++ignored;
    } else {
        ++invalid;
    }
}

// Same decomposition as the planner's scan: work units of kChunkElems ids, one
// contiguous span of units per CTA, a shared byte map per bitmap, ballots to
// fold it into words, arrival counter, last CTA writes the outputs.
__global__ void __launch_bounds__(kScanThreads)
scan_static_kernel(const __grid_constant__ ScanArgs a, const __grid_constant__ StaticArgs s) {
    __shared__ __align__(16) uint8_t s_map[RT_MAX_BLOCKS];
    __shared__ int s_last;
    __shared__ uint32_t s_touched;
    const int tid = threadIdx.x;
    const uint32_t lane = tid & 31, warp = tid >> 5;
    const int q_begin = (int)((long long)a.n_units * blockIdx.x / gridDim.x);
    const int q_end = (int)((long long)a.n_units * (blockIdx.x + 1) / gridDim.x);
    if (q_begin >= q_end) return;
    uint32_t invalid = 0, ignored = 0;
    reinterpret_cast<uint32_t *>(s_map)[tid] = 0;
    __syncthreads();
    int gl = 0, gh = a.n_groups;
    while (gh - gl > 1) {
        int mid = (gl + gh) >> 1;
        if (a.unit_first[mid] <= q_begin) gl = mid; else gh = mid;
    }
    for (uint32_t g = (uint32_t)gl;; ++g) {
        const int uf = a.unit_first[g], ul = a.unit_first[g + 1];
        const int q_lo = q_begin > uf ? q_begin : uf, q_hi = q_end < ul ? q_end : ul;
        const long long lo = a.group_off[g], hi = a.group_off[g + 1];
        long long e0 = (lo & ~1LL) + (long long)(q_lo - uf) * kChunkElems;
        for (int q = q_lo; q < q_hi; ++q, e0 += kChunkElems) {
            if (e0 >= lo && e0 + kChunkElems <= hi) {
                longlong2 v[kUnroll];
#pragma unroll
                for (int u = 0; u < kUnroll; ++u)
                    v[u] = __ldcs(reinterpret_cast<const longlong2 *>(a.slots + e0 + 2 * (u * kScanThreads + tid)));
#pragma unroll
                for (int u = 0; u < kUnroll; ++u) {
                    mark_one(v[u].x, a, s_map, invalid, ignored);
                    mark_one(v[u].y, a, s_map, invalid, ignored);
                }
            } else {
#pragma unroll
                for (int u = 0; u < kUnroll; ++u) {
                    long long i = e0 + 2 * (u * kScanThreads + tid);
                    if (i >= lo && i < hi) mark_one(__ldcs(a.slots + i), a, s_map, invalid, ignored);
                    if (i + 1 >= lo && i + 1 < hi) mark_one(__ldcs(a.slots + i + 1), a, s_map, invalid, ignored);
                }
            }
        }
        // leave bitmap g: bytes -> words, OR into the static scratch, clean map
        __syncthreads();
        constexpr int kPerWarp = kWords / (kScanThreads / 32);
#pragma unroll
        for (int k = 0; k < kPerWarp; ++k) {
            uint32_t word = warp * kPerWarp + k;
            uint32_t bits = __ballot_sync(0xffffffffu, s_map[word * 32 + lane] != 0);
            if (lane == 0 && bits) atomicOr(&s.scratch->groups[g].want[word], bits);
        }
        __syncthreads();
        reinterpret_cast<uint32_t *>(s_map)[tid] = 0;
        __syncthreads();
        if (q_hi >= q_end) break;
    }
    uint32_t inv = warp_sum(invalid), ign = warp_sum(ignored);
    if (lane == 0) {
        if (inv) atomicAdd(&s.scratch->global.invalid_slots, (unsigned long long)inv);
        if (ign) atomicAdd(&s.scratch->global.ignored_slots, (unsigned long long)ign);
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        uint32_t count = (uint32_t)(q_end - q_begin);
        uint32_t prev = atomicAdd(&s.scratch->global.units_done, count);
        s_last = prev + count == s.n_units;
        s_touched = 0;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    // last CTA: copy the accumulated words out, one warp per bitmap
    for (uint32_t g = warp; g < (uint32_t)a.n_groups; g += kScanThreads / 32) {
        uint32_t w = __ldcg(&s.scratch->groups[g].want[lane]);
        const uint32_t lo_bit = lane * 32;
        const uint32_t valid = s.n_blocks >= lo_bit + 32 ? 0xffffffffu
                               : (s.n_blocks > lo_bit ? ((1u << (s.n_blocks - lo_bit)) - 1u) : 0u);
        w &= valid;
        s.bitmaps_out[g * kWords + lane] = w;
        uint32_t n = warp_sum(__popc(w));
        if (lane == 0) atomicAdd(&s_touched, n);
    }
    __syncthreads();
    if (tid == 0) {
        rt_plan_result res = {};
        unsigned long long bad = __ldcg(&s.scratch->global.invalid_slots);
        res.flags = bad ? RT_RESULT_SLOT_RANGE : 0u;
        res.blocks_touched = s_touched;
        res.invalid_slots = bad;
        res.ignored_slots = __ldcg(&s.scratch->global.ignored_slots);
        *s.result = res;
    }
}

// Per-device address of the scratch array, resolved on first use.
constexpr int kMaxDevices = 64;
std::mutex g_setup_lock;
StaticScratch *g_scratch_addr[kMaxDevices];
int g_sm_count[kMaxDevices];

}  // namespace

namespace rt {
void division_magic(uint32_t d, uint32_t *magic, uint32_t *shift);
}

extern "C" int rt_scan_slots_static(const int64_t *d_slots, const int64_t *group_off, uint32_t n_groups,
                                    uint64_t capacity_slots, uint32_t block_tokens, uint32_t n_blocks,
                                    uint32_t *d_bitmaps, rt_plan_result *d_result, void *stream) {
    if (!group_off || !d_bitmaps || !d_result || !n_groups || !block_tokens || !capacity_slots ||
        capacity_slots > 0xfffffffeull || !n_blocks || n_blocks > RT_MAX_BLOCKS ||
        capacity_slots / block_tokens >= n_blocks)
        return RT_ERR_INVALID_ARGUMENT;
    if (n_groups > RT_STATIC_MAX_GROUPS) return RT_ERR_CAPACITY;   // beyond the static scratch
    if (!d_slots && group_off[n_groups] > 0) return RT_ERR_INVALID_ARGUMENT;
    if ((reinterpret_cast<uintptr_t>(d_slots) & 15u) && group_off[n_groups] > 0) return RT_ERR_ALIGNMENT;

    int device = -1;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) { rt::last_cuda_error_set((int)e); return RT_ERR_NO_DEVICE; }
    if (device < 0 || device >= kMaxDevices) return RT_ERR_INVALID_ARGUMENT;
    StaticScratch *scratch;
    {
        // once per device, with that device current: the symbol's device address
        std::lock_guard<std::mutex> lock(g_setup_lock);
        if (!g_scratch_addr[device]) {
            void *ptr = nullptr;
            e = cudaGetSymbolAddress(&ptr, g_static_scratch);
            if (e != cudaSuccess || !ptr) { rt::last_cuda_error_set((int)e); return RT_ERR_CUDA; }
            e = cudaDeviceGetAttribute(&g_sm_count[device], cudaDevAttrMultiProcessorCount, device);
            if (e != cudaSuccess) { rt::last_cuda_error_set((int)e); return RT_ERR_CUDA; }
            g_scratch_addr[device] = static_cast<StaticScratch *>(ptr);
        }
        scratch = g_scratch_addr[device];
    }

    ScanArgs a = {};
    a.slots = reinterpret_cast<const long long *>(d_slots);
    a.n_groups = (int)n_groups;
    a.capacity = capacity_slots;
    a.block_tokens = block_tokens;
    a.shift = -1;
    if ((block_tokens & (block_tokens - 1)) == 0) {
        int s = 0;
        while ((1u << s) != block_tokens) ++s;
        a.shift = s;
    } else {
        rt::division_magic(block_tokens, &a.magic, &a.magic_shift);
    }
    long long units = 0;
    for (uint32_t g = 0; g < n_groups; ++g) {
        long long lo = group_off[g], hi = group_off[g + 1];
        if (lo < 0 || hi < lo) return RT_ERR_INVALID_ARGUMENT;
        a.group_off[g] = lo;
        a.unit_first[g] = (int)units;
        long long n = (hi - (lo & ~1LL) + kChunkElems - 1) / kChunkElems;
        units += n > 0 ? n : 1;
        if (units > 0x7fffffffLL) return RT_ERR_CAPACITY;
    }
    a.group_off[n_groups] = group_off[n_groups];
    a.unit_first[n_groups] = (int)units;
    a.n_units = (int)units;

    StaticArgs s;
    s.scratch = scratch;
    s.bitmaps_out = d_bitmaps;
    s.result = d_result;
    s.n_blocks = n_blocks;
    s.n_units = (uint32_t)units;
    cudaStream_t cs = static_cast<cudaStream_t>(stream);
    // the array still holds the previous call's words and counters: clear the part this call uses
    e = cudaMemsetAsync(scratch, 0, offsetof(StaticScratch, groups) + sizeof(GroupScratch) * n_groups, cs);
    if (e != cudaSuccess) { rt::last_cuda_error_set((int)e); return RT_ERR_CUDA; }
    long long slots = (long long)g_sm_count[device] * 4;
    int grid = (int)(units < slots ? units : slots);
    scan_static_kernel<<<grid, kScanThreads, 0, cs>>>(a, s);
    e = cudaGetLastError();
    if (e != cudaSuccess) { rt::last_cuda_error_set((int)e); return RT_ERR_CUDA; }
    return RT_OK;
}
