// Read-only bandwidth yardstick: streams a device buffer once, the way the slot
// scan does (one wave of 4 CTAs per SM, 16 KiB units dealt in contiguous runs,
// 128-bit streaming loads, two sets of registers in flight), and does nothing
// with the data but fold it into one word.  No reference counterpart: the bench
// quotes it beside the scan so that the scan's GB/s can be read against what a
// pure read of the same bytes reaches on the same device at the same moment
// (the measured copy peak counts a read AND a write stream).  Probes issued
// back to back overlap each other's ramp and drain, as chained scans do.
#include <cuda_runtime.h>

#include "rt_internal.h"

namespace {

constexpr int kThreads = 256;
constexpr int kVecPerThread = 4;                                  // 4 x 16 B x 256 threads = 16 KiB per unit

__global__ void __launch_bounds__(kThreads, 4)
read_probe_kernel(const uint4 *__restrict__ data, unsigned long long n_vec, unsigned long long *sink) {
    // back-to-back probes do not depend on one another: let the next one start
    // as soon as this one's CTAs are all running
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const unsigned long long unit_vec = (unsigned long long)kThreads * kVecPerThread;
    const unsigned long long units = n_vec / unit_vec;
    const unsigned long long q0 = units * blockIdx.x / gridDim.x, q1 = units * (blockIdx.x + 1) / gridDim.x;
    uint4 acc = make_uint4(0, 0, 0, 0);
    uint4 a[kVecPerThread], b[kVecPerThread];
    unsigned long long q = q0;
    if (q < q1) {
#pragma unroll
        for (int k = 0; k < kVecPerThread; ++k) a[k] = __ldcs(data + q * unit_vec + k * kThreads + threadIdx.x);
    }
    for (; q < q1; q += 2) {
        if (q + 1 < q1) {
#pragma unroll
            for (int k = 0; k < kVecPerThread; ++k)
                b[k] = __ldcs(data + (q + 1) * unit_vec + k * kThreads + threadIdx.x);
        }
#pragma unroll
        for (int k = 0; k < kVecPerThread; ++k) {
            acc.x ^= a[k].x; acc.y ^= a[k].y; acc.z ^= a[k].z; acc.w ^= a[k].w;
        }
        if (q + 2 < q1) {
#pragma unroll
            for (int k = 0; k < kVecPerThread; ++k)
                a[k] = __ldcs(data + (q + 2) * unit_vec + k * kThreads + threadIdx.x);
        }
        if (q + 1 < q1) {
#pragma unroll
            for (int k = 0; k < kVecPerThread; ++k) {
                acc.x ^= b[k].x; acc.y ^= b[k].y; acc.z ^= b[k].z; acc.w ^= b[k].w;
            }
        }
    }
    // the tail that is not a whole unit, by the last CTA
    if (blockIdx.x == gridDim.x - 1)
        for (unsigned long long i = units * unit_vec + threadIdx.x; i < n_vec; i += kThreads) {
            uint4 v = __ldcs(data + i);
            acc.x ^= v.x; acc.y ^= v.y; acc.z ^= v.z; acc.w ^= v.w;
        }
    unsigned long long word = ((unsigned long long)(acc.x ^ acc.z) << 32) | (acc.y ^ acc.w);
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) word ^= __shfl_xor_sync(0xffffffffu, word, d);
    if ((threadIdx.x & 31) == 0 && word) atomicXor(sink, word);
}

}  // namespace

extern "C" int rt_read_probe(const void *d_data, uint64_t bytes, uint64_t *d_sink, void *stream) {
    if (!d_data || !d_sink || (reinterpret_cast<uintptr_t>(d_data) & 15u) || bytes % 16)
        return RT_ERR_INVALID_ARGUMENT;
    int device = 0, sms = 148;
    cudaGetDevice(&device);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)sms * 4);
    cfg.blockDim = dim3(kThreads);
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, read_probe_kernel, static_cast<const uint4 *>(d_data),
                                       (unsigned long long)(bytes / 16),
                                       reinterpret_cast<unsigned long long *>(d_sink));
    if (e == cudaSuccess) e = cudaGetLastError();
    if (e != cudaSuccess) { rt::last_cuda_error_set((int)e); return RT_ERR_CUDA; }
    return RT_OK;
}
