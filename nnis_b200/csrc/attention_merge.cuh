// The merge of split attention: kernels that cut a query's key range into slices
// leave, per (token, head, slice), a record [running max, running sum, unnormalised
// output of d values]; this kernel adds the slices up in ascending order.
#pragma once

#include <float.h>

#include "common.cuh"

namespace nnis {

// Merge the splits of one (token, head) in ascending order of split.
template <typename T>
__global__ void attn_merge_kernel(const float* __restrict__ partial, T* __restrict__ out,
                                  size_t n_rows, int d, int n_splits) {
    size_t row = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    int lane = threadIdx.x & 31;
    if (row >= n_rows) return;
    const float* rec = partial + row * n_splits * (size_t)(d + 2);
    float m = -FLT_MAX;
    for (int s = 0; s < n_splits; ++s)
        if (rec[(size_t)s * (d + 2) + 1] > 0.f) m = fmaxf(m, rec[(size_t)s * (d + 2)]);
    float l = 0.f;
    for (int s = 0; s < n_splits; ++s) {
        float ls = rec[(size_t)s * (d + 2) + 1];
        if (ls > 0.f) l += ls * expf(rec[(size_t)s * (d + 2)] - m);
    }
    float inv = l > 0.f ? 1.0f / l : 0.f;
    for (int i = lane; i < d; i += 32) {
        float o = 0.f;
        for (int s = 0; s < n_splits; ++s) {
            float ls = rec[(size_t)s * (d + 2) + 1];
            if (ls > 0.f) o += rec[(size_t)s * (d + 2) + 2 + i] * expf(rec[(size_t)s * (d + 2)] - m);
        }
        out[row * d + i] = from_float<T>(o * inv);
    }
}

}  // namespace nnis
