// Entry points of the UVM server used by the preload hooks (same process, same
// library).  Each one runs the real driver call and the registry update under
// the server's lifetime lock, so a migration batch never overlaps an
// allocation, a free or a context teardown.
#pragma once
#include "driver_api.h"

namespace rt {

// Tracked managed allocation (the reference's cuMemAllocManaged hook,
// select.cpp:24724-24761): records context, device and whether the device
// supports concurrent managed access.
CUresult uvm_tracked_alloc(CUdeviceptr *dptr, size_t bytes, unsigned int flags);
// select.cpp:24772-24783
CUresult uvm_tracked_free(CUdeviceptr dptr);
// select.cpp:24785-24796
CUresult uvm_tracked_ctx_destroy(CUcontext ctx);
// select.cpp:24798-24815: on success every record of the device is dropped.
CUresult uvm_tracked_primary(CUdevice device, CUresult (*real)(CUdevice), const char *name);
// After fork(): the child closes the inherited descriptors and must not touch
// CUDA or the socket path (select.cpp:23817-23824).
void uvm_fork_child();

}  // namespace rt
