// The merge of split attention: kernels that cut a query's key range into slices
// leave, per (token, head, slice), a record [running max, running sum, unnormalised
// output of d values]; this kernel adds the slices up in ascending order.
#pragma once

#include <float.h>

#include "async_copy.cuh"
#include "common.cuh"

namespace nnis {

// A CTA of 128 threads per (token, head); at most 64 slices.  The first warp works out the
// slices' weights exp(m_s - m) / l once (lane s holds slices s and s + 32); then every thread
// sums its output values over the slices, in ascending order of slice.
template <typename T>
__global__ void __launch_bounds__(128)
attn_merge_kernel(const float* __restrict__ partial, T* __restrict__ out, size_t n_rows, int d,
                  int n_splits) {
    __shared__ float share[64];
    pdl_wait();  // (a no-op unless launched as a programmatic dependent)
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31;
    const size_t row = blockIdx.x;
    const float* rec = partial + row * n_splits * (size_t)(d + 2);
    if (threadIdx.x < 32) {
        float ms[2], ls[2];
        float m = -FLT_MAX;
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            int s = lane + 32 * k;
            ms[k] = s < n_splits ? rec[(size_t)s * (d + 2)] : 0.f;
            ls[k] = s < n_splits ? rec[(size_t)s * (d + 2) + 1] : 0.f;
            if (ls[k] > 0.f) m = fmaxf(m, ms[k]);
        }
        m = warp_max(m);
        float l = 0.f;
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            ms[k] = ls[k] > 0.f ? expf(ms[k] - m) : 0.f;
            l += ls[k] * ms[k];
        }
        l = warp_sum(l);
        const float inv = l > 0.f ? 1.0f / l : 0.f;
        share[lane] = ms[0] * inv;
        share[lane + 32] = ms[1] * inv;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < d; i += 128) {
        float o = 0.f;
        for (int s = 0; s < n_splits; ++s) {
            float w = share[s];
            if (w > 0.f) o = fmaf(w, rec[(size_t)s * (d + 2) + 2 + i], o);
        }
        out[row * d + i] = from_float<T>(o);
    }
}

}  // namespace nnis
