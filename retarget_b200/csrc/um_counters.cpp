// Unified-memory counters for the prefetch experiment: GPU page-fault groups
// and bytes migrated by the driver, read through CUPTI's activity records
// (CUPTI_ACTIVITY_KIND_UNIFIED_MEMORY_COUNTER).  Built as a library of its own
// (libretarget_umcount.so) so that the planner library carries no CUPTI
// dependency; the experiment loads it when it is there and reports
// "unavailable" with CUPTI's own error text when a call is refused.
//
// The reference vendors CUPTI activity tracing but compiles it out
// (select.cpp:17193,17422-17860); its evaluation counts faults with external
// tools.  Nothing here is on the planning path.
#include <cupti.h>

#include <atomic>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>

namespace {

std::atomic<uint64_t> g_gpu_fault_groups{0}, g_cpu_faults{0}, g_bytes_htod{0}, g_bytes_dtoh{0}, g_records{0};
std::atomic<uint64_t> g_dropped{0};
char g_error[256] = "";
bool g_enabled = false;
int g_kinds = 0;

bool ok(CUptiResult r, const char *what) {
    if (r == CUPTI_SUCCESS) return true;
    const char *text = nullptr;
    cuptiGetResultString(r, &text);
    snprintf(g_error, sizeof(g_error), "%s: %s", what, text ? text : "unknown CUPTI error");
    return false;
}

void CUPTIAPI buffer_requested(uint8_t **buffer, size_t *size, size_t *max_records) {
    *size = 4u << 20;
    *buffer = static_cast<uint8_t *>(aligned_alloc(8, *size));
    *max_records = 0;
}

void CUPTIAPI buffer_completed(CUcontext ctx, uint32_t stream, uint8_t *buffer, size_t, size_t valid) {
    CUpti_Activity *record = nullptr;
    while (buffer && valid && cuptiActivityGetNextRecord(buffer, valid, &record) == CUPTI_SUCCESS) {
        if (record->kind != CUPTI_ACTIVITY_KIND_UNIFIED_MEMORY_COUNTER) continue;
        auto *r = reinterpret_cast<CUpti_ActivityUnifiedMemoryCounter3 *>(record);
        g_records.fetch_add(1);
        switch (r->counterKind) {
            case CUPTI_ACTIVITY_UNIFIED_MEMORY_COUNTER_KIND_GPU_PAGE_FAULT: g_gpu_fault_groups.fetch_add(r->value); break;
            case CUPTI_ACTIVITY_UNIFIED_MEMORY_COUNTER_KIND_CPU_PAGE_FAULT_COUNT: g_cpu_faults.fetch_add(1); break;
            case CUPTI_ACTIVITY_UNIFIED_MEMORY_COUNTER_KIND_BYTES_TRANSFER_HTOD: g_bytes_htod.fetch_add(r->value); break;
            case CUPTI_ACTIVITY_UNIFIED_MEMORY_COUNTER_KIND_BYTES_TRANSFER_DTOH: g_bytes_dtoh.fetch_add(r->value); break;
            default: break;
        }
    }
    size_t dropped = 0;
    if (cuptiActivityGetNumDroppedRecords(ctx, stream, &dropped) == CUPTI_SUCCESS) g_dropped.fetch_add(dropped);
    free(buffer);
}

}  // namespace

extern "C" {

// Enables the counters for the calling process (the CUDA driver must be
// initialised).  Returns 0, or -1 with the reason in rt_um_counters_error().
int rt_um_counters_enable(void) {
    if (g_enabled) return 0;
    if (!ok(cuptiActivityRegisterCallbacks(buffer_requested, buffer_completed), "cuptiActivityRegisterCallbacks"))
        return -1;
    // Not every counter kind is offered everywhere: ask for all four first, then
    // for fewer.  g_kinds says how many were accepted (in the order below).
    const CUpti_ActivityUnifiedMemoryCounterKind kinds[4] = {
        CUPTI_ACTIVITY_UNIFIED_MEMORY_COUNTER_KIND_BYTES_TRANSFER_HTOD,
        CUPTI_ACTIVITY_UNIFIED_MEMORY_COUNTER_KIND_BYTES_TRANSFER_DTOH,
        CUPTI_ACTIVITY_UNIFIED_MEMORY_COUNTER_KIND_GPU_PAGE_FAULT,
        CUPTI_ACTIVITY_UNIFIED_MEMORY_COUNTER_KIND_CPU_PAGE_FAULT_COUNT};
    bool on = false;
    for (int n = 4; n >= 2 && !on; --n) {
        CUpti_ActivityUnifiedMemoryCounterConfig config[4];
        for (int i = 0; i < n; ++i) {
            config[i].scope = CUPTI_ACTIVITY_UNIFIED_MEMORY_COUNTER_SCOPE_PROCESS_SINGLE_DEVICE;
            config[i].kind = kinds[i];
            config[i].deviceId = 0;
            config[i].enable = 1;
        }
        if (!ok(cuptiActivityConfigureUnifiedMemoryCounter(config, n), "cuptiActivityConfigureUnifiedMemoryCounter"))
            continue;
        on = ok(cuptiActivityEnable(CUPTI_ACTIVITY_KIND_UNIFIED_MEMORY_COUNTER), "cuptiActivityEnable");
        if (on) g_kinds = n;
    }
    if (!on) return -1;
    g_enabled = true;
    return 0;
}

// Flushes the activity buffers and returns the totals since the last call:
// out[0] GPU page-fault groups, out[1] CPU page faults, out[2] bytes host->device,
// out[3] bytes device->host, out[4] records seen, out[5] records dropped.
int rt_um_counters_read(uint64_t out[6]) {
    if (!g_enabled) return -1;
    if (!ok(cuptiActivityFlushAll(1), "cuptiActivityFlushAll")) return -1;
    out[0] = g_gpu_fault_groups.exchange(0);
    out[1] = g_cpu_faults.exchange(0);
    out[2] = g_bytes_htod.exchange(0);
    out[3] = g_bytes_dtoh.exchange(0);
    out[4] = g_records.exchange(0);
    out[5] = g_dropped.exchange(0);
    return 0;
}

int rt_um_counters_disable(void) {
    if (!g_enabled) return 0;
    g_enabled = false;
    return ok(cuptiActivityDisable(CUPTI_ACTIVITY_KIND_UNIFIED_MEMORY_COUNTER), "cuptiActivityDisable") ? 0 : -1;
}

const char *rt_um_counters_error(void) { return g_error; }

// How many counter kinds were accepted: 4 all, 3 no CPU page faults, 2 bytes only.
int rt_um_counters_kinds(void) { return g_kinds; }

}  // extern "C"
