// Host-side narrowing of slot ids before they cross the host link.
//
// The host-buffer planning call is bound by the host -> device copy of the slot
// ids (178 MB per step at the target size, a few milliseconds over PCIe against
// tens of microseconds of kernel).  A slot id of a pool with fewer than 2^31
// slots fits in 32 bits, so the call halves the bytes on the link by narrowing
// the caller's 64-bit ids into a pinned staging buffer on the host cores, chunk
// by chunk, each chunk's copy running while the next one is narrowed.
#pragma once
#include <cstddef>
#include <cstdint>

namespace rt {

// dst[i] = src[i] for ids in [0, 2^31); ids below zero become -1 and ids of 2^31
// and above become INT32_MAX, so that with capacity < INT32_MAX every id keeps
// its class (ignored: < 1, valid: 1..capacity, out of range: > capacity).
void narrow_ids(const int64_t *src, int32_t *dst, size_t n);

// The same over a pool of worker threads kept by the process (`threads` - 1
// workers, created by the first call and kept; the calling thread works too).
// Calls from several threads take turns.
void narrow_ids_parallel(const int64_t *src, int32_t *dst, size_t n, unsigned threads);

// The same, handing the result over in chunks: `ready(ctx, first, count)` is
// called on the calling thread for every `chunk_ids` ids (a multiple of 65,536;
// the last chunk may be short), in ascending order, as soon as that chunk is
// complete -- while the pool is already at work on the chunks after it.
using ChunkReady = void (*)(void *ctx, size_t first, size_t count);
void narrow_ids_streamed(const int64_t *src, int32_t *dst, size_t n, unsigned threads, size_t chunk_ids,
                         ChunkReady ready, void *ctx);

// Threads the host-buffer call narrows with, 0 for "do not narrow".
// RETARGET_B200_PACK_THREADS decides if set (0 switches narrowing off).  Else:
// 0 when `sharers` (processes expected to do the same at the same time: one per
// visible GPU) is more than one; otherwise three quarters of the CPUs this
// process may run on, at most 16 -- and 0 when that leaves fewer than 8.
unsigned narrow_threads(unsigned sharers);

}  // namespace rt
