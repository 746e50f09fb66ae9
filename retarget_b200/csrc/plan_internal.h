// A read-only view of a plan handle for the other device-side components.
#pragma once
#include <cuda_runtime.h>

#include "plan_device.cuh"

struct rt_plan;

namespace rt {

struct PlanView {
    rt_layout layout;
    int device;
    cudaStream_t stream;
    uint32_t *d_resident;
    uint32_t n_blocks, block_tokens;
    int shift;
    uint32_t magic, magic_shift;
    int sm_count;
};

void plan_view(const rt_plan *pl, PlanView *v);
void plan_fill_args(const rt_plan *pl, PlanArgs &p, uint32_t budget, uint32_t flags, rt_range *out,
                    uint32_t cap, rt_plan_result *result);
cudaError_t launch_plan_tail(const uint32_t *want, const PlanArgs &p, cudaStream_t stream);

}  // namespace rt
