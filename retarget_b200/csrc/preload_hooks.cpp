// LD_PRELOAD face of the library: the driver-API entry points an application's
// CUDA runtime resolves, interposed so that device allocations become managed,
// every managed allocation is registered with the UVM server, and the control
// socket comes up right after a successful cuInit.
//
// Scope: the allocation / lifetime hooks and the symbol redirection of the
// reference preload library (select.cpp:24723-24901, 25347-25564).  Its launch
// gate, time-slice control, SM masking and memory-limit hooks are other control
// paths and are not reproduced: those symbols are not exported here, so the
// application reaches the driver directly for them.
//
// Environment (select.cpp:23849-23856):
//   SELECT_UVM_ENABLE=1          turn the UVM server on
//   SELECT_UVM_CONVERT_ALLOC=1   turn cuMemAlloc into cuMemAllocManaged
//   SELECT_UVM_CHUNK_MB=1..256   bytes per cuMemPrefetchAsync call
#include <dlfcn.h>
#include <pthread.h>
#include <unistd.h>

#include <climits>
#include <initializer_list>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "rt_internal.h"
#include "uvm_server.h"

// cuda.h maps several public names onto their _v2 symbols; the hooks below
// export the literal names on purpose.
#undef cuDevicePrimaryCtxRelease
#undef cuDevicePrimaryCtxReset
#undef cuGetProcAddress
#undef cuMemAlloc
#undef cuMemFree
#undef cuCtxDestroy

namespace {

std::once_flag g_init_once, g_start_once;
bool g_enabled = false, g_convert = false;
pid_t g_owner = 0;

bool inherited() {
    pid_t owner = __atomic_load_n(&g_owner, __ATOMIC_ACQUIRE);
    return owner && owner != getpid();
}

void init() {
    const char *s = getenv("SELECT_UVM_ENABLE");
    g_enabled = s && !strcmp(s, "1");
    s = getenv("SELECT_UVM_CONVERT_ALLOC");
    g_convert = s && !strcmp(s, "1");
    __atomic_store_n(&g_owner, getpid(), __ATOMIC_RELEASE);
    if (pthread_atfork(nullptr, nullptr, rt::uvm_fork_child) != 0) g_enabled = false;
    if (!rt::driver_api()) g_enabled = false;
}

const rt::DriverApi *api() {
    std::call_once(g_init_once, init);
    return rt::driver_api();
}

bool active() { return g_enabled && !inherited(); }

void start_server() {
    if (!active()) return;
    const rt::DriverApi *d = rt::driver_api();
    if (!d || !d->mem_alloc_managed || !d->can_prefetch() || !d->ctx_get_current || !d->ctx_get_device ||
        !d->ctx_set_current || !d->device_get_attribute || !d->stream_create || !d->stream_synchronize ||
        !d->stream_destroy || !d->mem_free || !d->ctx_destroy)
        return;
    rt_uvm_config cfg = {};
    cfg.listen = 1;
    if (rt_uvm_start(&cfg) == RT_OK) atexit([] { rt_uvm_stop(); });
}

}  // namespace

extern "C" {

CUresult cuMemAllocManaged(CUdeviceptr *dptr, size_t bytes, unsigned int flags);
CUresult cuMemAlloc_v2(CUdeviceptr *dptr, size_t bytes);
CUresult cuMemFree_v2(CUdeviceptr dptr);
CUresult cuCtxDestroy_v2(CUcontext ctx);
CUresult cuDevicePrimaryCtxRelease(CUdevice device);
CUresult cuDevicePrimaryCtxRelease_v2(CUdevice device);
CUresult cuDevicePrimaryCtxReset(CUdevice device);
CUresult cuDevicePrimaryCtxReset_v2(CUdevice device);
CUresult cuGetProcAddress(const char *symbol, void **pfn, int version, cuuint64_t flags);
CUresult cuGetProcAddress_v2(const char *symbol, void **pfn, int version, cuuint64_t flags,
                             CUdriverProcAddressQueryResult *status);

CUresult cuInit(unsigned int flags) {
    if (inherited()) return CUDA_ERROR_NOT_INITIALIZED;
    const rt::DriverApi *d = api();
    CUresult result = d && d->init ? d->init(flags) : CUDA_ERROR_NOT_INITIALIZED;
    if (result == CUDA_SUCCESS) std::call_once(g_start_once, start_server);
    return result;
}

CUresult cuMemAllocManaged(CUdeviceptr *dptr, size_t bytes, unsigned int flags) {
    if (inherited()) return CUDA_ERROR_NOT_INITIALIZED;
    const rt::DriverApi *d = api();
    if (!d || !d->mem_alloc_managed) return CUDA_ERROR_NOT_SUPPORTED;
    if (!active()) return d->mem_alloc_managed(dptr, bytes, flags);
    return rt::uvm_tracked_alloc(dptr, bytes, flags);
}

CUresult cuMemAlloc_v2(CUdeviceptr *dptr, size_t bytes) {
    if (inherited()) return CUDA_ERROR_NOT_INITIALIZED;
    const rt::DriverApi *d = api();
    if (active() && g_convert) return cuMemAllocManaged(dptr, bytes, CU_MEM_ATTACH_GLOBAL);
    return d && d->mem_alloc ? d->mem_alloc(dptr, bytes) : CUDA_ERROR_NOT_SUPPORTED;
}

CUresult cuMemFree_v2(CUdeviceptr dptr) {
    if (inherited()) return CUDA_ERROR_NOT_INITIALIZED;
    const rt::DriverApi *d = api();
    if (!d || !d->mem_free) return CUDA_ERROR_NOT_SUPPORTED;
    if (!active()) return d->mem_free(dptr);
    return rt::uvm_tracked_free(dptr);
}

CUresult cuCtxDestroy_v2(CUcontext ctx) {
    if (inherited()) return CUDA_ERROR_NOT_INITIALIZED;
    const rt::DriverApi *d = api();
    if (!d || !d->ctx_destroy) return CUDA_ERROR_NOT_SUPPORTED;
    if (!active()) return d->ctx_destroy(ctx);
    return rt::uvm_tracked_ctx_destroy(ctx);
}

static CUresult primary_call(CUdevice device, CUresult (*rt::DriverApi::*slot)(CUdevice), const char *name) {
    if (inherited()) return CUDA_ERROR_NOT_INITIALIZED;
    const rt::DriverApi *d = api();
    if (!d || !(d->*slot)) return CUDA_ERROR_NOT_SUPPORTED;
    if (!active()) return (d->*slot)(device);
    return rt::uvm_tracked_primary(device, d->*slot, name);
}

// Both generations stay exported: the argument ABI agrees, the driver behaviour
// does not, so each forwards to the symbol of its own name.
CUresult cuDevicePrimaryCtxRelease(CUdevice device) {
    return primary_call(device, &rt::DriverApi::primary_release_v1, "cuDevicePrimaryCtxRelease");
}
CUresult cuDevicePrimaryCtxRelease_v2(CUdevice device) {
    return primary_call(device, &rt::DriverApi::primary_release_v2, "cuDevicePrimaryCtxRelease_v2");
}
CUresult cuDevicePrimaryCtxReset(CUdevice device) {
    return primary_call(device, &rt::DriverApi::primary_reset_v1, "cuDevicePrimaryCtxReset");
}
CUresult cuDevicePrimaryCtxReset_v2(CUdevice device) {
    return primary_call(device, &rt::DriverApi::primary_reset_v2, "cuDevicePrimaryCtxReset_v2");
}

// Which hook stands in for the driver pointer `real` that a lookup of `symbol`
// produced.  The pointer must match: version-1 cuMemAlloc / cuMemFree have a
// different ABI and are passed through (select.cpp:24839-24863).
static void *replacement_for(const char *symbol, void *real, int version) {
    const rt::DriverApi *d = rt::driver_api();
    if (!real || !d) return nullptr;
    auto is = [&](const char *a, const char *b) { return !strcmp(symbol, a) || !strcmp(symbol, b); };
    if (is("cuDevicePrimaryCtxRelease", "cuDevicePrimaryCtxRelease_v2") && version >= 7000) {
        if (real == (void *)d->primary_release_v1) return (void *)cuDevicePrimaryCtxRelease;
        if (real == (void *)d->primary_release_v2) return (void *)cuDevicePrimaryCtxRelease_v2;
    }
    if (is("cuDevicePrimaryCtxReset", "cuDevicePrimaryCtxReset_v2") && version >= 7000) {
        if (real == (void *)d->primary_reset_v1) return (void *)cuDevicePrimaryCtxReset;
        if (real == (void *)d->primary_reset_v2) return (void *)cuDevicePrimaryCtxReset_v2;
    }
    if (!strcmp(symbol, "cuMemAllocManaged") && version >= 6000 && real == (void *)d->mem_alloc_managed)
        return (void *)cuMemAllocManaged;
    if (is("cuMemAlloc", "cuMemAlloc_v2") && version >= 3020 && real == (void *)d->mem_alloc)
        return (void *)cuMemAlloc_v2;
    if (is("cuMemFree", "cuMemFree_v2") && version >= 3020 && real == (void *)d->mem_free)
        return (void *)cuMemFree_v2;
    if (is("cuCtxDestroy", "cuCtxDestroy_v2") && version >= 4000 && real == (void *)d->ctx_destroy)
        return (void *)cuCtxDestroy_v2;
    return nullptr;
}

static void redirect(const char *symbol, void **pfn, int version) {
    if (void *mine = replacement_for(symbol, *pfn, version)) { *pfn = mine; return; }
    if (!strcmp(symbol, "cuInit")) *pfn = (void *)cuInit;
    else if (!strcmp(symbol, "cuGetProcAddress"))
        *pfn = version >= 12000 ? (void *)cuGetProcAddress_v2 : (void *)cuGetProcAddress;
}

CUresult cuGetProcAddress(const char *symbol, void **pfn, int version, cuuint64_t flags) {
    const rt::DriverApi *d = api();
    if (!d || !d->get_proc_address_v1) return CUDA_ERROR_NOT_SUPPORTED;
    CUresult query = d->get_proc_address_v1(symbol, pfn, version, flags);
    if (query != CUDA_SUCCESS || !symbol || !pfn || !*pfn) return query;
    redirect(symbol, pfn, version);
    return query;
}

CUresult cuGetProcAddress_v2(const char *symbol, void **pfn, int version, cuuint64_t flags,
                             CUdriverProcAddressQueryResult *status) {
    const rt::DriverApi *d = api();
    if (!d || !d->get_proc_address_v2) return CUDA_ERROR_NOT_SUPPORTED;
    CUresult query = d->get_proc_address_v2(symbol, pfn, version, flags, status);
    if (query != CUDA_SUCCESS || !symbol || !pfn || !*pfn) return query;
    redirect(symbol, pfn, version);
    return query;
}

// dlsym interposer: CUDA runtimes look the driver entry points up by name.
void *dlsym(void *handle, const char *symbol) {
    using dlsym_fn = void *(*)(void *, const char *);
    static dlsym_fn real_dlsym = [] {
        for (const char *v : {"GLIBC_2.34", "GLIBC_2.2.5", "GLIBC_2.17"})
            if (void *p = dlvsym(RTLD_NEXT, "dlsym", v)) return (dlsym_fn)p;
        return (dlsym_fn) nullptr;
    }();
    if (!real_dlsym || !symbol) return nullptr;
    void *real = real_dlsym(handle, symbol);
    // only names this library hooks are ever redirected, and only when the
    // lookup really landed in the driver
    static const char *const hooked[] = {
        "cuInit", "cuMemAllocManaged", "cuMemAlloc_v2", "cuMemFree_v2", "cuCtxDestroy_v2",
        "cuDevicePrimaryCtxRelease", "cuDevicePrimaryCtxRelease_v2", "cuDevicePrimaryCtxReset",
        "cuDevicePrimaryCtxReset_v2", "cuGetProcAddress", "cuGetProcAddress_v2"};
    bool mine = false;
    for (const char *name : hooked) mine |= !strcmp(symbol, name);
    if (!mine || !real) return real;
    // loading the driver may itself call dlsym: never re-enter the set-up
    static thread_local bool busy = false;
    if (busy) return real;
    busy = true;
    const rt::DriverApi *d = api();
    busy = false;
    if (!d) return real;
    if (!strcmp(symbol, "cuInit")) return real == (void *)d->init ? (void *)cuInit : real;
    if (!strcmp(symbol, "cuGetProcAddress"))
        return real == (void *)d->get_proc_address_v1 ? (void *)cuGetProcAddress : real;
    if (!strcmp(symbol, "cuGetProcAddress_v2"))
        return real == (void *)d->get_proc_address_v2 ? (void *)cuGetProcAddress_v2 : real;
    void *replacement = replacement_for(symbol, real, INT_MAX);
    return replacement ? replacement : real;
}

}  // extern "C"
