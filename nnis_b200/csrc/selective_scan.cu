// Selective scan (the recurrence of a Mamba mixer) and the short causal convolution
// in front of it.  Per channel c and state index n, with a step size dt = softplus(.)
// per token and channel, A = -exp(A_log) [channels, N], B and C [N] per token:
//
//     S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n      y_c = sum_n S[c, n] C_n + D_c x_c
//
// and the output y * silu(z).  S is float32 in a per-sequence state area; the last
// taps - 1 inputs of the convolution are state too (float32 [taps - 1, channels], oldest
// first).  Both start at zero and are carried from step to step; step sizes, decays, the
// state and the sums are float32 in every dtype.
//
//   conv_silu        xc = silu(bias + sum_j conv[c, j] * input at (t - (taps - 1 - j))), inputs
//                    before the step's first token come from the state (zeros at a
//                    sequence's start)
//   selective_scan   a CTA of 128 threads per (sequence, run of channels); NS threads share
//                    a channel, each with NL of its N state values in registers; tokens go
//                    16 at a time through shared memory (B and C of the tile); the threads
//                    that own a channel move its convolution state on when the step is over
//
// A row whose position is -1 (padding) is skipped everywhere.
#include "async_copy.cuh"
#include "common.cuh"

namespace nnis {

// xz [n, 2 * inner]: the convolution reads the first `inner` columns
template <typename T>
__global__ void __launch_bounds__(256)
conv_silu_kernel(const T* __restrict__ xz, const float* __restrict__ conv_w, const float* __restrict__ conv_b,
                 const float* __restrict__ conv_state, const int* __restrict__ token_pos,
                 const int* __restrict__ token_seq, const int* __restrict__ seq_slots,
                 const int* __restrict__ seq_first_row, T* __restrict__ xc, int inner, int taps) {
    pdl_wait();
    pdl_launch_dependents();
    const int n = blockIdx.x;
    if (token_pos[n] < 0) return;
    const int seq = token_seq[n];
    const int slot = seq_slots[seq];
    const int first = seq_first_row ? seq_first_row[seq] : n;
    const int L = taps - 1;
    const float* tail = conv_state + (size_t)slot * L * inner;
    for (int c = blockIdx.y * 256 + threadIdx.x; c < inner; c += 256 * gridDim.y) {
        float acc = conv_b ? conv_b[c] : 0.f;
        for (int j = 0; j < taps; ++j) {
            int back = L - j;  // tokens before this one
            float in;
            if (n - back >= first) in = to_float(xz[(size_t)(n - back) * 2 * inner + c]);
            else in = tail[(size_t)(L - (back - (n - first))) * inner + c];
            acc = fmaf(conv_w[(size_t)c * taps + j], in, acc);
        }
        xc[(size_t)n * inner + c] = from_float<T>(acc / (1.0f + expf(-acc)));
    }
}

__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }

constexpr int kScanTile = 16;

// NL: state values a thread holds; NS (a power of two up to 32) threads share a channel.
// dt_raw float32 [n, inner] (before softplus, bias added); bc float32 [n, 2 N] (B then C)
template <typename T, int NL>
__global__ void __launch_bounds__(128)
selective_scan_kernel(const T* __restrict__ xc, const T* __restrict__ xz, const float* __restrict__ dt_raw,
                      const float* __restrict__ bc, const float* __restrict__ a_log, const float* __restrict__ dskip,
                      float* __restrict__ state, float* __restrict__ conv_state, const int* __restrict__ token_pos,
                      const int* __restrict__ token_seq, const int* __restrict__ seq_slots,
                      const int* __restrict__ seq_first_row, const int* __restrict__ seq_count,
                      T* __restrict__ y_out, int inner, int N, int NS, int taps) {
    extern __shared__ float smem[];  // [kScanTile][2 N]
    pdl_wait();
    pdl_launch_dependents();
    const int unit = blockIdx.x;
    int first, count, slot;
    if (seq_first_row) {
        first = seq_first_row[unit];
        count = seq_count[unit];
        slot = seq_slots[unit];
    } else {
        first = unit;
        count = token_pos[unit] < 0 ? 0 : 1;
        slot = seq_slots[token_seq[unit]];
    }
    if (count <= 0) return;
    const int per_cta = 128 / NS;
    const int c = blockIdx.y * per_cta + threadIdx.x / NS;
    const int part = threadIdx.x % NS, n0 = part * NL;
    const bool live = c < inner;
    float s[NL], a[NL];
    float* S = state + ((size_t)slot * inner + (live ? c : 0)) * N;
#pragma unroll
    for (int i = 0; i < NL; ++i) {
        bool in = live && n0 + i < N;
        s[i] = in ? S[n0 + i] : 0.f;
        a[i] = in ? -expf(a_log[(size_t)c * N + n0 + i]) : 0.f;
    }
    const float dsk = live ? dskip[c] : 0.f;
    for (int t0 = 0; t0 < count; t0 += kScanTile) {
        const int tn = min(kScanTile, count - t0);
        __syncthreads();
        for (int i = threadIdx.x; i < tn * 2 * N; i += 128) smem[i] = bc[(size_t)(first + t0) * 2 * N + i];
        __syncthreads();
        for (int t = 0; t < tn; ++t) {
            const size_t row = (size_t)(first + t0 + t);
            const float dt = live ? softplus_f(dt_raw[row * inner + c]) : 0.f;
            const float xv = live ? to_float(xc[row * inner + c]) : 0.f;
            const float* B = smem + t * 2 * N + n0;
            const float* C = B + N;
            const float dx = dt * xv;
            float y = 0.f;
#pragma unroll
            for (int i = 0; i < NL; ++i) {
                if (n0 + i < N) {
                    s[i] = fmaf(expf(dt * a[i]), s[i], dx * B[i]);
                    y = fmaf(s[i], C[i], y);
                }
            }
            for (int o = NS >> 1; o > 0; o >>= 1) y += __shfl_xor_sync(0xffffffffu, y, o);
            if (live && part == 0) {
                y = fmaf(dsk, xv, y);
                float z = to_float(xz[row * 2 * inner + inner + c]);
                y_out[row * inner + c] = from_float<T>(y * (z / (1.0f + expf(-z))));
            }
        }
    }
    if (!live) return;
#pragma unroll
    for (int i = 0; i < NL; ++i)
        if (n0 + i < N) S[n0 + i] = s[i];
    if (part == 0) {
        // the convolution's tail: the last taps - 1 inputs of (old tail, this step's inputs)
        const int L = taps - 1;
        float* tail = conv_state + (size_t)slot * L * inner;
        for (int i = 0; i < L; ++i) {
            int at = count + i;  // index into the old tail followed by the step's inputs
            float val = at < L ? tail[(size_t)at * inner + c]
                               : to_float(xz[(size_t)(first + at - L) * 2 * inner + c]);
            tail[(size_t)i * inner + c] = val;
        }
    }
}

}  // namespace nnis

using namespace nnis;

NNIS_API int nnis_conv_silu(const void* xz, const float* conv_w, const float* conv_b, const float* conv_state,
                            const int* token_pos, const int* token_seq, const int* seq_slots,
                            const int* seq_first_row, void* xc, int n_tokens, int inner, int taps, int dtype,
                            cudaStream_t stream) {
    if (n_tokens <= 0 || inner <= 0 || taps <= 0 || !xz || !conv_w || !conv_state || !xc) return NNIS_ERR_ARGUMENT;
    dim3 grid(n_tokens, (unsigned)min(64, (inner + 255) / 256));
    cudaError_t e;
    if (dtype == NNIS_DTYPE_F32)
        e = launch_dependent(conv_silu_kernel<float>, grid, 256, 0, stream, (const float*)xz, conv_w, conv_b,
                             conv_state, token_pos, token_seq, seq_slots, seq_first_row, (float*)xc, inner, taps);
    else if (dtype == NNIS_DTYPE_BF16)
        e = launch_dependent(conv_silu_kernel<bf16>, grid, 256, 0, stream, (const bf16*)xz, conv_w, conv_b,
                             conv_state, token_pos, token_seq, seq_slots, seq_first_row, (bf16*)xc, inner, taps);
    else
        return NNIS_ERR_UNSUPPORTED;
    return e == cudaSuccess ? NNIS_OK : (int)e;
}

// state: float32 [slots, inner, N]; conv_state: float32 [slots, taps - 1, inner]
NNIS_API int nnis_selective_scan(const void* xc, const void* xz, const float* dt_raw, const float* bc,
                                 const float* a_log, const float* dskip, float* state, float* conv_state,
                                 const int* token_pos, const int* token_seq, const int* seq_slots,
                                 const int* seq_first_row, const int* seq_count, void* y, int units, int inner,
                                 int N, int taps, int dtype, cudaStream_t stream) {
    if (units <= 0 || inner <= 0 || N <= 0 || taps <= 0 || !xc || !xz || !dt_raw || !bc || !a_log || !dskip ||
        !state || !conv_state || !y)
        return NNIS_ERR_ARGUMENT;
    if (N > 384) return NNIS_ERR_UNSUPPORTED;  // (a tile of B and C fits 48 KB of shared memory)
    // eight state values a thread where up to 32 threads cover N, else sixteen
    int NL = N <= 256 ? 8 : 16;
    int NS = 1;
    while (NS * NL < N) NS <<= 1;
    int per_cta = 128 / NS;
    unsigned tiles = (unsigned)((inner + per_cta - 1) / per_cta);
    if (tiles > 65535) return NNIS_ERR_UNSUPPORTED;
    dim3 grid(units, tiles);
    size_t smem = sizeof(float) * kScanTile * 2 * (size_t)N;
    cudaError_t e;
#define NNIS_SCAN_CASE(T, NLV) \
    e = launch_dependent(selective_scan_kernel<T, NLV>, grid, 128, smem, stream, (const T*)xc, (const T*)xz, dt_raw, \
                         bc, a_log, dskip, state, conv_state, token_pos, token_seq, seq_slots, seq_first_row, \
                         seq_count, (T*)y, inner, N, NS, taps)
    if (dtype == NNIS_DTYPE_F32) {
        if (NL == 8) NNIS_SCAN_CASE(float, 8);
        else NNIS_SCAN_CASE(float, 16);
    } else if (dtype == NNIS_DTYPE_BF16) {
        if (NL == 8) NNIS_SCAN_CASE(bf16, 8);
        else NNIS_SCAN_CASE(bf16, 16);
    } else {
        return NNIS_ERR_UNSUPPORTED;
    }
#undef NNIS_SCAN_CASE
    return e == cudaSuccess ? NNIS_OK : (int)e;
}
