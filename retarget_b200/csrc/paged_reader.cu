// Synthetic paged decode-attention reader: the consumer the prefetch plan is
// made for.  It touches what a decode step touches -- the K and V rows of every
// live slot in every layer buffer -- and reduces them to a per-buffer checksum,
// so a run with and without the placement plan can be compared (same bytes
// read; the difference is where the pages were when the kernel arrived).
//
// One warp per (buffer, slot) row: the row (bytes_per_slot, a multiple of 16) is
// read with 128-bit loads, viewed as 16-bit lanes (the KV dtype is bf16) and
// summed as unsigned integers, which keeps the check exact.
#include <cuda_runtime.h>

#include "rt_internal.h"

namespace {

__global__ void __launch_bounds__(256)
paged_reader_kernel(const unsigned char *const *buffers, uint32_t n_buffers, uint32_t bytes_per_slot,
                    const long long *slots, long long n_slots, unsigned long long capacity,
                    unsigned long long *sums) {
    const uint32_t lane = threadIdx.x & 31;
    const long long warps = (long long)gridDim.x * (blockDim.x >> 5);
    const long long rows = n_slots * n_buffers;
    for (long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); row < rows;
         row += warps) {
        // buffer-major inside a slot: consecutive warps read the same slot of
        // consecutive buffers, consecutive iterations walk the slot list
        const uint32_t j = (uint32_t)(row % n_buffers);
        const long long s = slots[row / n_buffers];
        if ((unsigned long long)(s - 1) >= capacity) continue;
        const uint4 *src = reinterpret_cast<const uint4 *>(buffers[j] + (unsigned long long)s * bytes_per_slot);
        unsigned long long acc = 0;
        for (uint32_t i = lane; i < bytes_per_slot / 16; i += 32) {
            uint4 v = src[i];
            acc += (v.x & 0xffffu) + (v.x >> 16) + (v.y & 0xffffu) + (v.y >> 16) + (v.z & 0xffffu) +
                   (v.z >> 16) + (v.w & 0xffffu) + (v.w >> 16);
        }
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) acc += __shfl_down_sync(0xffffffffu, acc, d);
        if (lane == 0) atomicAdd(&sums[j], acc);
    }
}

}  // namespace

extern "C" int rt_paged_read(const void *const *d_buffers, uint32_t n_buffers, uint32_t bytes_per_slot,
                             const int64_t *d_slots, uint64_t n_slots, uint64_t capacity_slots,
                             uint64_t *d_sums, void *stream) {
    if (!d_buffers || !n_buffers || !bytes_per_slot || bytes_per_slot % 16 || (!d_slots && n_slots) || !d_sums)
        return RT_ERR_INVALID_ARGUMENT;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    cudaError_t e = cudaMemsetAsync(d_sums, 0, sizeof(uint64_t) * n_buffers, s);
    if (e != cudaSuccess) { rt::last_cuda_error_set((int)e); return RT_ERR_CUDA; }
    if (!n_slots) return RT_OK;
    int device = 0, sms = 148;
    cudaGetDevice(&device);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    unsigned long long rows = (unsigned long long)n_slots * n_buffers;
    unsigned long long want = (rows + 7) / 8;
    int grid = (int)(want < (unsigned long long)sms * 8 ? want : (unsigned long long)sms * 8);
    paged_reader_kernel<<<grid, 256, 0, s>>>(reinterpret_cast<const unsigned char *const *>(d_buffers), n_buffers,
                                             bytes_per_slot, reinterpret_cast<const long long *>(d_slots),
                                             (long long)n_slots, capacity_slots,
                                             reinterpret_cast<unsigned long long *>(d_sums));
    e = cudaGetLastError();
    if (e != cudaSuccess) { rt::last_cuda_error_set((int)e); return RT_ERR_CUDA; }
    return RT_OK;
}
