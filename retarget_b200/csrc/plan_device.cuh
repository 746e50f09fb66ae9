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
// them in turn: launch number n (counted by the host from 2) uses set n & 1.
// A chained launch (RT_PLAN_CHAINED) may start scanning while the launches
// before it are still running; the set it uses was last used by launch n - 2,
// whose tail writes its own number into the set's `cleaned` word when it has
// left the set clean.  A CTA of launch n reads that word when it starts and
// looks at it again (a bounded number of times) before its first write to the
// set; in steady state the first read already says n - 2.
struct GroupScratch {
    uint32_t want[kWords];
};

struct GlobalScratch {
    unsigned long long invalid_slots;
    unsigned long long ignored_slots;
    uint32_t units_done;          // arrival counter of scanned work units
    uint32_t error_flags;
    uint32_t cleaned;             // number of the last launch whose tail left this set clean
    uint32_t reserved;
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
    uint32_t launch_no;                       // scan launches: this launch's number (set = launch_no & 1)
    unsigned long long alloc_bytes;
    unsigned long long block_bytes;
    const uint8_t *buffer_group;              // device: bitmap of every buffer, registry order
    const uint16_t *group_size;               // device: buffers per bitmap
};

}  // namespace rt
