// Synthetic paged bf16 decode attention: the consumer the placement plan is
// made for in the oversubscribed end-to-end configuration.
//
// One decode step reads, for every live request and every layer, the K and V
// rows of all of the request's cached slots: scores = q . K^T over the slots,
// softmax, output = scores . V.  What matters to the placement experiment is
// the access pattern (every live row of every layer buffer, gathered through
// the slot table) and that a page which is not resident stalls real arithmetic,
// so the kernel does the arithmetic for real: bf16 in, fp32 accumulate, one
// pass with a running maximum (the "online softmax" of flash decoding).
//
// Layout (the serving engine's): buffer of a layer = [pool_slots][heads][128]
// bf16, K and V separate; one slot row is heads * 256 bytes.
//
// Mapping: one CTA per (request, layer), one WARP per KV head.  A lane owns 4
// of the head's 128 dimensions: it loads 8 bytes of the K row and 8 bytes of
// the V row per slot.  Four slots are in flight per warp: their K and V
// fragments are loaded before the first dot product is reduced.  No tensor
// cores: with one query per request this is a matrix-vector product, bound by
// the row reads.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cmath>

#include "rt_internal.h"

namespace {

constexpr int kHeadDim = 128;
constexpr int kSlotsInFlight = 4;

struct Frag {
    float x[4];
};

__device__ __forceinline__ Frag load_frag(const unsigned char *row, uint32_t lane) {
    const uint2 raw = *reinterpret_cast<const uint2 *>(row + lane * 8);
    Frag f;
    f.x[0] = __uint_as_float(raw.x << 16);
    f.x[1] = __uint_as_float(raw.x & 0xffff0000u);
    f.x[2] = __uint_as_float(raw.y << 16);
    f.x[3] = __uint_as_float(raw.y & 0xffff0000u);
    return f;
}

__device__ __forceinline__ float warp_total(float v) {
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
    return v;
}

struct AttentionArgs {
    const unsigned char *const *k_buffers;     // [layers]
    const unsigned char *const *v_buffers;     // [layers]
    const __nv_bfloat16 *q;                    // [requests][layers][heads][128]
    const long long *slots;                    // request r owns slots[req_off[r] .. req_off[r+1])
    const long long *req_off;                  // [requests + 1]
    float *out;                                // [requests][layers][heads][128]
    unsigned long long capacity;
    uint32_t n_layers, n_heads;
    float scale;
};

__global__ void __launch_bounds__(256)
paged_attention_kernel(AttentionArgs a) {
    const uint32_t lane = threadIdx.x & 31, head = threadIdx.x >> 5;
    if (head >= a.n_heads) return;
    const uint32_t layer = blockIdx.x % a.n_layers;
    const uint32_t req = blockIdx.x / a.n_layers;
    const uint32_t row_bytes = a.n_heads * kHeadDim * 2;
    const unsigned char *kbuf = a.k_buffers[layer] + head * (kHeadDim * 2);
    const unsigned char *vbuf = a.v_buffers[layer] + head * (kHeadDim * 2);
    const size_t qo = (((size_t)req * a.n_layers + layer) * a.n_heads + head) * kHeadDim;
    Frag q;
    {
        const uint2 raw = *reinterpret_cast<const uint2 *>(reinterpret_cast<const unsigned char *>(a.q + qo) + lane * 8);
        q.x[0] = __uint_as_float(raw.x << 16) * a.scale;
        q.x[1] = __uint_as_float(raw.x & 0xffff0000u) * a.scale;
        q.x[2] = __uint_as_float(raw.y << 16) * a.scale;
        q.x[3] = __uint_as_float(raw.y & 0xffff0000u) * a.scale;
    }
    const long long lo = a.req_off[req], hi = a.req_off[req + 1];
    float m = -INFINITY, l = 0.f;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (long long i = lo; i < hi; i += kSlotsInFlight) {
        Frag k[kSlotsInFlight], v[kSlotsInFlight];
        bool live[kSlotsInFlight];
#pragma unroll
        for (int u = 0; u < kSlotsInFlight; ++u) {
            const long long s = i + u < hi ? a.slots[i + u] : 0;
            live[u] = (unsigned long long)(s - 1) < a.capacity;       // slot 0 is padding; ids outside the pool are skipped
            if (live[u]) {
                k[u] = load_frag(kbuf + (size_t)s * row_bytes, lane);
                v[u] = load_frag(vbuf + (size_t)s * row_bytes, lane);
            }
        }
#pragma unroll
        for (int u = 0; u < kSlotsInFlight; ++u) {
            if (!live[u]) continue;                                    // uniform over the warp
            const float score =
                warp_total(q.x[0] * k[u].x[0] + q.x[1] * k[u].x[1] + q.x[2] * k[u].x[2] + q.x[3] * k[u].x[3]);
            const float m_new = fmaxf(m, score);
            const float keep = __expf(m - m_new), w = __expf(score - m_new);
            l = l * keep + w;
#pragma unroll
            for (int d = 0; d < 4; ++d) acc[d] = acc[d] * keep + w * v[u].x[d];
            m = m_new;
        }
    }
    const float inv = l > 0.f ? 1.f / l : 0.f;
    float4 o = make_float4(acc[0] * inv, acc[1] * inv, acc[2] * inv, acc[3] * inv);
    *reinterpret_cast<float4 *>(a.out + qo + lane * 4) = o;
}

}  // namespace

extern "C" int rt_paged_attention(const void *const *d_k_buffers, const void *const *d_v_buffers, uint32_t n_layers,
                                  uint32_t n_kv_heads, const void *d_q, const int64_t *d_slots,
                                  const int64_t *d_req_off, uint32_t n_requests, uint64_t capacity_slots,
                                  float *d_out, void *stream) {
    if (!d_k_buffers || !d_v_buffers || !n_layers || !n_kv_heads || n_kv_heads > 8 || !d_q || !d_req_off || !d_out ||
        !capacity_slots)
        return RT_ERR_INVALID_ARGUMENT;
    if (!n_requests) return RT_OK;
    if ((unsigned long long)n_requests * n_layers > 0x7fffffffull) return RT_ERR_CAPACITY;
    AttentionArgs a;
    a.k_buffers = reinterpret_cast<const unsigned char *const *>(d_k_buffers);
    a.v_buffers = reinterpret_cast<const unsigned char *const *>(d_v_buffers);
    a.q = static_cast<const __nv_bfloat16 *>(d_q);
    a.slots = reinterpret_cast<const long long *>(d_slots);
    a.req_off = reinterpret_cast<const long long *>(d_req_off);
    a.out = d_out;
    a.capacity = capacity_slots;
    a.n_layers = n_layers;
    a.n_heads = n_kv_heads;
    a.scale = 1.0f / sqrtf((float)kHeadDim);
    paged_attention_kernel<<<n_requests * n_layers, 32 * n_kv_heads, 0, static_cast<cudaStream_t>(stream)>>>(a);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        rt::last_cuda_error_set((int)e);
        return RT_ERR_CUDA;
    }
    return RT_OK;
}
