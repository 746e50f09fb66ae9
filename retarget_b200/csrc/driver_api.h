// The handful of CUDA driver entry points the UVM server and the preload hooks
// call, resolved at run time from libcuda (never linked), the way the reference
// preload library resolves them (select.cpp:23839-23848, 25851-25937).
#pragma once
#include <cuda.h>

namespace rt {

// Members carry neutral names: cuda.h turns several public names into macros.
struct DriverApi {
    void *handle = nullptr;
    CUresult (*init)(unsigned int) = nullptr;
    CUresult (*ctx_get_current)(CUcontext *) = nullptr;
    CUresult (*ctx_set_current)(CUcontext) = nullptr;
    CUresult (*ctx_get_device)(CUdevice *) = nullptr;
    CUresult (*device_get_attribute)(int *, CUdevice_attribute, CUdevice) = nullptr;
    CUresult (*stream_create)(CUstream *, unsigned int) = nullptr;
    CUresult (*stream_synchronize)(CUstream) = nullptr;
    CUresult (*stream_destroy)(CUstream) = nullptr;
    CUresult (*mem_alloc)(CUdeviceptr *, size_t) = nullptr;                  // the driver's cuMemAlloc_v2
    CUresult (*mem_alloc_managed)(CUdeviceptr *, size_t, unsigned int) = nullptr;
    CUresult (*mem_free)(CUdeviceptr) = nullptr;                              // cuMemFree_v2 in the driver
    // explicit signatures: the public header may alias the prefetch names
    CUresult (*prefetch_v1)(CUdeviceptr, size_t, CUdevice, CUstream) = nullptr;
    CUresult (*prefetch_v2)(CUdeviceptr, size_t, CUmemLocation, unsigned int, CUstream) = nullptr;
    CUresult (*ctx_destroy)(CUcontext) = nullptr;                             // cuCtxDestroy_v2 in the driver
    CUresult (*primary_release_v1)(CUdevice) = nullptr;
    CUresult (*primary_release_v2)(CUdevice) = nullptr;
    CUresult (*primary_reset_v1)(CUdevice) = nullptr;
    CUresult (*primary_reset_v2)(CUdevice) = nullptr;
    CUresult (*primary_get_state)(CUdevice, unsigned int *, int *) = nullptr;
    CUresult (*get_proc_address_v1)(const char *, void **, int, cuuint64_t) = nullptr;
    CUresult (*get_proc_address_v2)(const char *, void **, int, cuuint64_t,
                                    CUdriverProcAddressQueryResult *) = nullptr;

    bool can_prefetch() const { return prefetch_v1 || prefetch_v2; }
    // Prefetch to a device ordinal or to the CPU (dst < 0) with whichever entry
    // point the driver exports.
    CUresult prefetch(CUdeviceptr ptr, size_t bytes, int dst, CUstream stream) const;
};

// Loads libcuda once.  RETARGET_B200_LIBCUDA names another library (the tests
// point it at a stub driver).  `lookup` resolves a symbol in that library
// without going through any interposed dlsym.  Returns nullptr when the driver
// cannot be loaded.
const DriverApi *driver_api();
void *driver_symbol(const char *name);

}  // namespace rt
