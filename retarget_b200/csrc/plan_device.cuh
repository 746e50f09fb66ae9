// Device-side data structures shared by the planner kernels.
#pragma once
#include <stdint.h>

#include "retarget_b200.h"

namespace rt {

constexpr int kWords = RT_BITMAP_WORDS;      // 32 x 32 bits = RT_MAX_BLOCKS

constexpr int kScanThreads = 256;
#ifndef RT_UNROLL
#define RT_UNROLL 4
#endif
constexpr int kUnroll = RT_UNROLL;                   // independent 16-byte loads per thread
constexpr int kChunkElems = kScanThreads * 2 * kUnroll;   // 2048 slot ids = 16 KiB

// Per-bitmap accumulation words, filled with atomicOr by the scan.  The tail
// zeroes them after reading, so back-to-back launches need no memset.
//
// A plan owns TWO sets of scratch (words + counters) and its scan launches use
// them in turn.  A chained launch (RT_PLAN_CHAINED) may run while the launch
// before it is still running, but never while the launch two before it is: one
// CTA of every launch does nothing but wait for the launch before it to
// complete and only then lets the next launch start (the gatekeeper in
// plan_kernels.cu).  So at most two consecutive launches are in flight at any
// time, and they use different sets.
struct GroupScratch {
    uint32_t want[kWords];
};

struct GlobalScratch {
    unsigned long long invalid_slots;
    unsigned long long ignored_slots;
    uint32_t units_done;          // arrival counter of scanned work units
    uint32_t error_flags;
};

// Kernel arguments, passed by value (about 1.7 KiB + 0.1 KiB): no per-step upload.
struct ScanArgs {
    const long long *slots;
    const int *lens;                          // table mode: valid ids per row
    long long group_off[RT_MAX_GROUPS + 1];   // CSR mode
    int unit_first[RT_MAX_GROUPS + 1];        // CSR mode: first work unit of each group
    long long stride;                         // table mode: ids from one row to the next
    long long seg_ids;                        // table mode: ids per row segment (a multiple of 4)
    uint32_t n_rows;                          // table mode
    uint32_t segs_per_row;                    // table mode: ceil(stride / seg_ids)
    int n_units;                              // CSR mode: work units of kChunkElems ids each
    int n_groups;
    unsigned long long capacity;              // largest valid slot id
    uint32_t block_tokens;
    int shift;                                // log2(block_tokens) or -1
    uint32_t magic;                           // exact division by block_tokens when it is not
    uint32_t magic_shift;                     //   a power of two: see block_of()
};

struct PlanArgs {
    GroupScratch *groups;
    GlobalScratch *global;
    uint32_t *resident;                       // n_groups x kWords
    uint32_t *bitmaps_out;                    // scan-only: n_groups x kWords (or null)
    rt_range *out;
    rt_plan_result *result;
    uint32_t cap;
    uint32_t n_buffers;
    uint32_t n_groups;
    uint32_t n_blocks;
    uint32_t budget;
    uint32_t flags;
    int32_t dst_device;
    int scan_only;
    int explicit_sets;                        // `want` holds [evict | add] words per bitmap
    uint32_t n_units;                         // work units of this launch (scan kernels)
    unsigned long long alloc_bytes;
    unsigned long long block_bytes;
    const uint8_t *buffer_group;              // device: bitmap of every buffer, registry order
    const uint16_t *group_size;               // device: buffers per bitmap
};

}  // namespace rt
