#include "driver_api.h"

#include <dlfcn.h>

#include <cstdlib>
#include <initializer_list>
#include <mutex>

namespace rt {
namespace {

using dlsym_fn = void *(*)(void *, const char *);

// The C library's own dlsym, even when this code sits inside a preload library
// that exports a `dlsym` of its own.
dlsym_fn libc_dlsym() {
    static dlsym_fn fn = [] {
        for (const char *version : {"GLIBC_2.34", "GLIBC_2.2.5", "GLIBC_2.17", "GLIBC_2.0"}) {
            void *p = dlvsym(RTLD_NEXT, "dlsym", version);
            if (p) return reinterpret_cast<dlsym_fn>(p);
        }
        return reinterpret_cast<dlsym_fn>(dlvsym(RTLD_DEFAULT, "dlsym", "GLIBC_2.2.5"));
    }();
    return fn;
}

DriverApi g_api;
std::once_flag g_once;
bool g_ok = false;

template <class F>
void bind(F &slot, const char *name) {
    slot = reinterpret_cast<F>(driver_symbol(name));
}

void load() {
    const char *path = getenv("RETARGET_B200_LIBCUDA");
    void *h = nullptr;
    if (path && *path) {
        h = dlopen(path, RTLD_NOW | RTLD_GLOBAL);
    } else {
        h = dlopen("libcuda.so.1", RTLD_NOW | RTLD_GLOBAL);
        if (!h) h = dlopen("libcuda.so", RTLD_NOW | RTLD_GLOBAL);
    }
    if (!h || !libc_dlsym()) return;
    g_api.handle = h;
    bind(g_api.init, "cuInit");
    bind(g_api.ctx_get_current, "cuCtxGetCurrent");
    bind(g_api.ctx_set_current, "cuCtxSetCurrent");
    bind(g_api.ctx_get_device, "cuCtxGetDevice");
    bind(g_api.device_get_attribute, "cuDeviceGetAttribute");
    bind(g_api.stream_create, "cuStreamCreate");
    bind(g_api.stream_synchronize, "cuStreamSynchronize");
    bind(g_api.stream_destroy, "cuStreamDestroy_v2");
    if (!g_api.stream_destroy) bind(g_api.stream_destroy, "cuStreamDestroy");
    bind(g_api.mem_alloc, "cuMemAlloc_v2");
    bind(g_api.mem_alloc_managed, "cuMemAllocManaged");
    bind(g_api.mem_free, "cuMemFree_v2");
    bind(g_api.prefetch_v1, "cuMemPrefetchAsync");
    bind(g_api.prefetch_v2, "cuMemPrefetchAsync_v2");
    bind(g_api.ctx_destroy, "cuCtxDestroy_v2");
    bind(g_api.primary_release_v1, "cuDevicePrimaryCtxRelease");
    bind(g_api.primary_release_v2, "cuDevicePrimaryCtxRelease_v2");
    bind(g_api.primary_reset_v1, "cuDevicePrimaryCtxReset");
    bind(g_api.primary_reset_v2, "cuDevicePrimaryCtxReset_v2");
    bind(g_api.primary_get_state, "cuDevicePrimaryCtxGetState");
    bind(g_api.get_proc_address_v1, "cuGetProcAddress");
    bind(g_api.get_proc_address_v2, "cuGetProcAddress_v2");
    g_ok = true;
}

}  // namespace

CUresult DriverApi::prefetch(CUdeviceptr ptr, size_t bytes, int dst, CUstream stream) const {
    if (prefetch_v1) return prefetch_v1(ptr, bytes, dst < 0 ? CU_DEVICE_CPU : (CUdevice)dst, stream);
    if (!prefetch_v2) return CUDA_ERROR_NOT_SUPPORTED;
    CUmemLocation where = {};
    where.type = dst < 0 ? CU_MEM_LOCATION_TYPE_HOST : CU_MEM_LOCATION_TYPE_DEVICE;
    where.id = dst < 0 ? 0 : dst;
    return prefetch_v2(ptr, bytes, where, 0, stream);
}

const DriverApi *driver_api() {
    std::call_once(g_once, load);
    return g_ok ? &g_api : nullptr;
}

void *driver_symbol(const char *name) {
    if (!g_api.handle || !libc_dlsym()) return nullptr;
    return libc_dlsym()(g_api.handle, name);
}

}  // namespace rt
