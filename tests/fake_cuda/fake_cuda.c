/*
 * Stub CUDA driver for CPU-only tests of the UVM server, the prefetch executor
 * and the preload hooks.  It exports the few driver entry points those parts
 * resolve, records every call in an in-memory log, hands out fake managed
 * pointers, and can be told to fail the N-th prefetch.  Nothing here touches a
 * GPU.
 */
#define _GNU_SOURCE
#include <dlfcn.h>
#include <pthread.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>

typedef int CUresult;
typedef int CUdevice;
typedef unsigned long long CUdeviceptr;
typedef void *CUcontext;
typedef void *CUstream;
typedef struct { int type; int id; } CUmemLocation;

#define LOG_CAP (1 << 20)
static pthread_mutex_t lock = PTHREAD_MUTEX_INITIALIZER;
static char log_buf[LOG_CAP];
static size_t log_len;
static int fail_after = -1;          /* fail the prefetch with this 0-based index */
static int fail_code = 1;
static int prefetch_calls;
static int concurrent_access = 1;
static __thread CUcontext current_ctx;
static CUdeviceptr next_ptr = 0x7f0000000000ull;
static uintptr_t next_stream = 0x1000;
static int sync_delay_us;

static void logf_(const char *fmt, ...) __attribute__((format(printf, 1, 2)));
#include <stdarg.h>
static void logf_(const char *fmt, ...)
{
    va_list ap;
    pthread_mutex_lock(&lock);
    va_start(ap, fmt);
    int n = vsnprintf(log_buf + log_len, LOG_CAP - log_len, fmt, ap);
    va_end(ap);
    if (n > 0 && log_len + (size_t)n < LOG_CAP) log_len += (size_t)n;
    pthread_mutex_unlock(&lock);
}

/* ---- test controls ---- */
void fake_cuda_reset(void)
{
    pthread_mutex_lock(&lock);
    log_len = 0;
    log_buf[0] = 0;
    fail_after = -1;
    prefetch_calls = 0;
    concurrent_access = 1;
    sync_delay_us = 0;
    pthread_mutex_unlock(&lock);
}
void fake_cuda_fail_prefetch(int index, int code) { fail_after = index; fail_code = code; }
void fake_cuda_set_concurrent(int value) { concurrent_access = value; }
void fake_cuda_set_sync_delay_us(int us) { sync_delay_us = us; }
size_t fake_cuda_log(char *out, size_t cap)
{
    pthread_mutex_lock(&lock);
    size_t n = log_len < cap - 1 ? log_len : cap - 1;
    memcpy(out, log_buf, n);
    out[n] = 0;
    pthread_mutex_unlock(&lock);
    return n;
}

/* ---- driver entry points ---- */
CUresult cuInit(unsigned int flags) { logf_("init %u\n", flags); return 0; }
CUresult cuDriverGetVersion(int *v) { *v = 12090; return 0; }
CUresult cuCtxGetCurrent(CUcontext *ctx) { *ctx = current_ctx; return 0; }
CUresult cuCtxSetCurrent(CUcontext ctx)
{
    current_ctx = ctx;
    logf_("ctx_set %p\n", ctx);
    return 0;
}
CUresult cuCtxGetDevice(CUdevice *dev) { *dev = 0; return current_ctx ? 0 : 201; }
CUresult cuDeviceGetAttribute(int *value, int attribute, CUdevice dev)
{
    (void)dev;
    *value = attribute == 89 /* CONCURRENT_MANAGED_ACCESS */ ? concurrent_access : 0;
    return 0;
}
CUresult cuDevicePrimaryCtxRetain(CUcontext *ctx, CUdevice dev) { *ctx = (CUcontext)(uintptr_t)(0xC000 + dev); return 0; }
CUresult cuDevicePrimaryCtxRelease(CUdevice dev) { logf_("primary_release %d\n", dev); return 0; }
CUresult cuDevicePrimaryCtxRelease_v2(CUdevice dev) { logf_("primary_release %d\n", dev); return 0; }
CUresult cuDevicePrimaryCtxReset(CUdevice dev) { logf_("primary_reset %d\n", dev); return 0; }
CUresult cuDevicePrimaryCtxReset_v2(CUdevice dev) { logf_("primary_reset %d\n", dev); return 0; }
CUresult cuCtxDestroy_v2(CUcontext ctx) { logf_("ctx_destroy %p\n", ctx); return 0; }
CUresult cuStreamCreate(CUstream *s, unsigned int flags)
{
    pthread_mutex_lock(&lock);
    *s = (CUstream)(next_stream++);
    pthread_mutex_unlock(&lock);
    logf_("stream_create %p %u\n", *s, flags);
    return 0;
}
CUresult cuStreamSynchronize(CUstream s)
{
    if (sync_delay_us) {
        struct timespec ts = {sync_delay_us / 1000000, (sync_delay_us % 1000000) * 1000L};
        nanosleep(&ts, NULL);
    }
    logf_("sync %p\n", s);
    return 0;
}
CUresult cuStreamDestroy_v2(CUstream s) { logf_("stream_destroy %p\n", s); return 0; }
CUresult cuMemAllocManaged(CUdeviceptr *ptr, size_t bytes, unsigned int flags)
{
    pthread_mutex_lock(&lock);
    *ptr = next_ptr;
    next_ptr += (bytes + 0x1fffffull) & ~0x1fffffull;
    pthread_mutex_unlock(&lock);
    logf_("alloc_managed %llx %zu %u\n", *ptr, bytes, flags);
    return 0;
}
CUresult cuMemAlloc_v2(CUdeviceptr *ptr, size_t bytes)
{
    pthread_mutex_lock(&lock);
    *ptr = next_ptr;
    next_ptr += (bytes + 0x1fffffull) & ~0x1fffffull;
    pthread_mutex_unlock(&lock);
    logf_("alloc_device %llx %zu\n", *ptr, bytes);
    return 0;
}
CUresult cuMemFree_v2(CUdeviceptr ptr) { logf_("free %llx\n", ptr); return 0; }
CUresult cuMemPrefetchAsync(CUdeviceptr ptr, size_t bytes, CUdevice dst, CUstream s)
{
    pthread_mutex_lock(&lock);
    int index = prefetch_calls++;
    int fail = index == fail_after;
    pthread_mutex_unlock(&lock);
    logf_("prefetch %llx %zu %d %p\n", ptr, bytes, dst, s);
    return fail ? fail_code : 0;
}
CUresult cuGetProcAddress_v2(const char *symbol, void **fn, int version, unsigned long long flags, int *status);
CUresult cuGetProcAddress(const char *symbol, void **fn, int version, unsigned long long flags)
{
    return cuGetProcAddress_v2(symbol, fn, version, flags, NULL);
}
CUresult cuGetProcAddress_v2(const char *symbol, void **fn, int version, unsigned long long flags, int *status)
{
    (void)version; (void)flags;
    Dl_info info;
    void *self = NULL;
    if (dladdr((void *)&cuInit, &info)) self = dlopen(info.dli_fname, RTLD_NOW | RTLD_NOLOAD);
    *fn = self ? dlsym(self, symbol) : NULL;
    if (!*fn) {
        char name[128];
        snprintf(name, sizeof(name), "%s_v2", symbol);
        *fn = self ? dlsym(self, name) : NULL;
    }
    if (status) *status = *fn ? 0 : 1;
    return *fn ? 0 : 500;
}
