// Retention: linear attention with a fixed decay per head, no softmax and no
// denominator.  Per head, with q and k rotated by position and k scaled by
// dim^-1/2:   S_t = g S_{t-1} + k_t v_t^T,   o_t = S_t^T q_t.
// The state S [dim, vdim] lives in float32 in a per-sequence state area and is
// carried from step to step; everything between the projections and the output
// (angles, rotation, decay, state, the head's unit norm, the gate) is float32.
//
//   retention_scan   a CTA per (sequence, head, 32 columns of vdim) walks the step's
//                    tokens of that sequence in order; warp w holds rows w, w+8, ...
//                    of the state tile in registers.  Serves prompts, later chunks
//                    (the state says where it stands) and single tokens.
//   retention_gate   o / rms(o) per head, times silu(g), rounded once.
//
// Packed input rows: [q (H dim) | k (H dim) | v (H vdim) | g (H vdim)].
#include "common.cuh"

namespace nnis {

template <typename T, int R>
__global__ void __launch_bounds__(256)
retention_scan_kernel(const T* __restrict__ qkvg, const float* __restrict__ freq,
                      const float* __restrict__ decay, float* __restrict__ state,
                      const int* __restrict__ token_pos, const int* __restrict__ token_seq,
                      const int* __restrict__ seq_slots, const int* __restrict__ seq_first_row,
                      const int* __restrict__ seq_start, const int* __restrict__ seq_count,
                      float* __restrict__ o_raw, int heads, int dim, int vdim, int rot_dims) {
    extern __shared__ float smem[];
    float* qs = smem;             // [dim]
    float* ks = smem + dim;       // [dim]
    float* red = smem + 2 * dim;  // [8][32]
    int unit = blockIdx.x, h = blockIdx.y, col = blockIdx.z * 32 + (threadIdx.x & 31);
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int first, start, count, slot;
    if (seq_first_row) {
        first = seq_first_row[unit];
        start = seq_start[unit];
        count = seq_count[unit];
        slot = seq_slots[unit];
    } else {  // one token per row; a row without a sequence has position -1
        first = unit;
        start = token_pos[unit];
        count = start < 0 ? 0 : 1;
        slot = seq_slots[token_seq[unit]];
    }
    if (count <= 0) return;
    const bool live = col < vdim;
    const float g = decay[h];
    const float k_scale = 1.0f / sqrtf((float)dim);
    float* S = state + (((size_t)slot * heads + h) * dim) * vdim;
    float s[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        int i = warp + 8 * r;
        s[r] = (live && i < dim) ? S[(size_t)i * vdim + col] : 0.f;
    }
    const size_t row_len = (size_t)2 * heads * dim + (size_t)2 * heads * vdim;
    const int half = rot_dims >> 1;
    for (int t = 0; t < count; ++t) {
        const T* row = qkvg + (size_t)(first + t) * row_len;
        const T* qh = row + (size_t)h * dim;
        const T* kh = row + (size_t)heads * dim + (size_t)h * dim;
        float pos = (float)(start + t);
        for (int j = threadIdx.x; j < dim - half; j += 256) {
            if (j < half) {
                float ang = pos * freq[j];
                float c = cosf(ang), sn = sinf(ang);
                float u = to_float(qh[j]), v = to_float(qh[j + half]);
                qs[j] = u * c - v * sn;
                qs[j + half] = v * c + u * sn;
                u = to_float(kh[j]);
                v = to_float(kh[j + half]);
                ks[j] = (u * c - v * sn) * k_scale;
                ks[j + half] = (v * c + u * sn) * k_scale;
            } else {
                qs[j + half] = to_float(qh[j + half]);
                ks[j + half] = to_float(kh[j + half]) * k_scale;
            }
        }
        __syncthreads();
        float v = live ? to_float(row[(size_t)2 * heads * dim + (size_t)h * vdim + col]) : 0.f;
        float o = 0.f;
#pragma unroll
        for (int r = 0; r < R; ++r) {
            int i = warp + 8 * r;
            if (i < dim) {
                s[r] = fmaf(g, s[r], ks[i] * v);
                o = fmaf(s[r], qs[i], o);
            }
        }
        red[warp * 32 + lane] = o;
        __syncthreads();
        if (warp == 0 && live) {
            float sum = 0.f;
#pragma unroll
            for (int w = 0; w < 8; ++w) sum += red[w * 32 + lane];
            o_raw[((size_t)(first + t) * heads + h) * vdim + col] = sum;
        }
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
        int i = warp + 8 * r;
        if (live && i < dim) S[(size_t)i * vdim + col] = s[r];
    }
}

// out[n, h, :] = o[n, h, :] / sqrt(mean(o[n, h, :]^2) + eps) * silu(g[n, h, :]); a warp
// per (token, head); a row at position -1 is left alone
template <typename T>
__global__ void __launch_bounds__(256)
retention_gate_kernel(const float* __restrict__ o_raw, const T* __restrict__ qkvg,
                      const int* __restrict__ token_pos, T* __restrict__ out, long long n_units,
                      int heads, int dim, int vdim, float eps) {
    long long unit = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (unit >= n_units) return;
    int lane = threadIdx.x & 31;
    long long n = unit / heads;
    int h = (int)(unit - n * heads);
    T* dst = out + (size_t)unit * vdim;
    if (token_pos[n] < 0) {
        for (int i = lane; i < vdim; i += 32) dst[i] = from_float<T>(0.f);
        return;
    }
    const float* o = o_raw + (size_t)unit * vdim;
    const T* gate = qkvg + (size_t)n * ((size_t)2 * heads * dim + (size_t)2 * heads * vdim) +
                    (size_t)2 * heads * dim + (size_t)heads * vdim + (size_t)h * vdim;
    float ss = 0.f;
    for (int i = lane; i < vdim; i += 32) ss = fmaf(o[i], o[i], ss);
    ss = warp_sum(ss);
    float s = 1.0f / sqrtf(ss / (float)vdim + eps);
    for (int i = lane; i < vdim; i += 32) {
        float z = to_float(gate[i]);
        dst[i] = from_float<T>((o[i] * s) * (z / (1.0f + expf(-z))));
    }
}

template <typename T>
static int launch_retention(const void* qkvg, const float* freq, const float* decay, float* state,
                            const int* token_pos, const int* token_seq, const int* seq_slots,
                            const int* seq_first_row, const int* seq_start, const int* seq_count,
                            float* o_raw, void* out, int n_tokens, int n_units, int heads, int dim,
                            int vdim, int rot_dims, float eps, cudaStream_t stream) {
    dim3 grid(n_units, heads, (vdim + 31) / 32);
    size_t smem = (2 * (size_t)dim + 256) * sizeof(float);
#define NNIS_RET_CASE(R) \
    retention_scan_kernel<T, R><<<grid, 256, smem, stream>>>( \
        (const T*)qkvg, freq, decay, state, token_pos, token_seq, seq_slots, seq_first_row, seq_start, \
        seq_count, o_raw, heads, dim, vdim, rot_dims)
    if (dim <= 32) NNIS_RET_CASE(4);
    else if (dim <= 64) NNIS_RET_CASE(8);
    else if (dim <= 128) NNIS_RET_CASE(16);
    else NNIS_RET_CASE(32);
#undef NNIS_RET_CASE
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;
    long long units = (long long)n_tokens * heads;
    retention_gate_kernel<T><<<(unsigned)((units + 7) / 8), 256, 0, stream>>>(
        o_raw, (const T*)qkvg, token_pos, (T*)out, units, heads, dim, vdim, eps);
    NNIS_RETURN_LAUNCH();
}

}  // namespace nnis

using namespace nnis;

// `seq_first_row` null: every row is a sequence of its own bringing one token
// (`n_units` = n_tokens); else `n_units` sequences with their first row, first
// position and token count.  `o_raw`: float32 scratch [n_tokens, heads * vdim].
NNIS_API int nnis_retention(const void* qkvg, const float* freq, const float* decay, float* state,
                            const int* token_pos, const int* token_seq, const int* seq_slots,
                            const int* seq_first_row, const int* seq_start, const int* seq_count,
                            float* o_raw, void* out, int n_tokens, int n_units, int heads, int dim,
                            int vdim, int rot_dims, float eps, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0 || n_units <= 0 || heads <= 0 || dim <= 0 || vdim <= 0 || rot_dims < 0 ||
        (rot_dims & 1) || rot_dims > dim || !(eps > 0.f) || !qkvg || !freq || !decay || !state ||
        !token_pos || !token_seq || !seq_slots || !o_raw || !out)
        return NNIS_ERR_ARGUMENT;
    if (seq_first_row && (!seq_start || !seq_count)) return NNIS_ERR_ARGUMENT;
    if (dim > 256 || heads > 65535 || (vdim + 31) / 32 > 65535) return NNIS_ERR_UNSUPPORTED;
    if (dtype == NNIS_DTYPE_F32)
        return launch_retention<float>(qkvg, freq, decay, state, token_pos, token_seq, seq_slots,
                                       seq_first_row, seq_start, seq_count, o_raw, out, n_tokens,
                                       n_units, heads, dim, vdim, rot_dims, eps, stream);
    if (dtype == NNIS_DTYPE_BF16)
        return launch_retention<bf16>(qkvg, freq, decay, state, token_pos, token_seq, seq_slots,
                                      seq_first_row, seq_start, seq_count, o_raw, out, n_tokens,
                                      n_units, heads, dim, vdim, rot_dims, eps, stream);
    return NNIS_ERR_UNSUPPORTED;
}
