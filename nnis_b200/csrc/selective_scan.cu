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
//                    16 at a time through shared memory (B, C, step sizes, inputs and gates
//                    of the tile); the threads that own a channel move its convolution state
//                    on when the step is over.  Long prompts: runs of tokens side by side in
//                    two passes with scan_prefix between them (see the kernel)
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
    if ((inner & 3) == 0) {  // four channels a thread: rows of xz and xc start on 8- or 16-byte borders
        for (int c = (blockIdx.y * 256 + threadIdx.x) * 4; c < inner; c += 1024 * gridDim.y) {
            float acc[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[e] = conv_b ? conv_b[c + e] : 0.f;
            for (int j = 0; j < taps; ++j) {
                const int back = L - j;  // tokens before this one
                const float4 in = n - back >= first ? load4(xz + (size_t)(n - back) * 2 * inner + c)
                                                    : load4(tail + (size_t)(L - (back - (n - first))) * inner + c);
                acc[0] = fmaf(conv_w[(size_t)c * taps + j], in.x, acc[0]);
                acc[1] = fmaf(conv_w[(size_t)(c + 1) * taps + j], in.y, acc[1]);
                acc[2] = fmaf(conv_w[(size_t)(c + 2) * taps + j], in.z, acc[2]);
                acc[3] = fmaf(conv_w[(size_t)(c + 3) * taps + j], in.w, acc[3]);
            }
            store4(xc + (size_t)n * inner + c, make_float4(acc[0] / (1.0f + expf(-acc[0])), acc[1] / (1.0f + expf(-acc[1])),
                                                           acc[2] / (1.0f + expf(-acc[2])), acc[3] / (1.0f + expf(-acc[3]))));
        }
        return;
    }
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

// exp of the recurrence: the library's in a float32 run, the fast one where operands are bfloat16
template <typename T> __device__ __forceinline__ float exp_for(float x) { return sizeof(T) == 4 ? expf(x) : __expf(x); }

constexpr int kScanTile = 16;

// NL: state values a thread holds; NS (a power of two up to 32) threads share a channel.
// dt_raw float32 [n, inner] (before softplus, bias added); bc float32 [n, 2 N] (B then C).
//
// PASS 0: a unit is a sequence of the step (or a row, in steps of single tokens): from the slot's
//         state to the slot's state, y written, the convolution's tail moved on.
// Long prompts are cut into runs of `seg_len` tokens that are worked side by side (the recurrence is
// linear in the state): a unit is then a run, (sequence, first token) in `segments`, and
// PASS 1: from a zero state; what the run adds to the state goes to seg_state[run], the sum of its
//         step sizes to seg_dt[run] (the state before the run decays by exp(A * that sum) over it);
//         scan_prefix_kernel then turns seg_state[run] into the state BEFORE each run and leaves
//         the slot's state as it is after the step;
// PASS 2: from seg_state[run], y written; a sequence's last run moves the convolution's tail on.
template <typename T, int NL, int PASS>
__global__ void __launch_bounds__(128)
selective_scan_kernel(const T* __restrict__ xc, const T* __restrict__ xz, const float* __restrict__ dt_raw,
                      const float* __restrict__ bc, const float* __restrict__ a_log, const float* __restrict__ dskip,
                      float* __restrict__ state, float* __restrict__ conv_state, const int* __restrict__ token_pos,
                      const int* __restrict__ token_seq, const int* __restrict__ seq_slots,
                      const int* __restrict__ seq_first_row, const int* __restrict__ seq_count,
                      const int* __restrict__ segments, int seg_len, float* __restrict__ seg_state,
                      float* __restrict__ seg_dt, T* __restrict__ y_out, int inner, int N, int NS, int taps) {
    extern __shared__ __align__(16) float smem[];  // [kScanTile][2 N] B and C, then [kScanTile][3][channels of the CTA]
    pdl_wait();
    pdl_launch_dependents();
    const int unit = blockIdx.x;
    int first, count, slot, seq_first = 0, seq_total = 0;
    bool last_run = true;
    if (PASS != 0) {
        const int seq = segments[2 * unit], t0 = segments[2 * unit + 1];
        seq_first = seq_first_row[seq];
        seq_total = seq_count[seq];
        first = seq_first + t0;
        count = min(seg_len, seq_total - t0);
        slot = seq_slots[seq];
        last_run = t0 + count == seq_total;
    } else if (seq_first_row) {
        first = seq_first_row[unit];
        count = seq_count[unit];
        slot = seq_slots[unit];
    } else {
        first = unit;
        count = token_pos[unit] < 0 ? 0 : 1;
        slot = seq_slots[token_seq[unit]];
    }
    if (PASS == 0) {
        seq_first = first;
        seq_total = count;
    }
    if (count <= 0) return;
    const int per_cta = 128 / NS;
    const int c_local = threadIdx.x / NS;
    const int c = blockIdx.y * per_cta + c_local;
    const int part = threadIdx.x % NS, n0 = part * NL;
    const bool live = c < inner;
    float* tile_bc = smem;
    float* tile_dt = smem + kScanTile * 2 * N;     // [kScanTile][per_cta], softplus taken
    float* tile_x = tile_dt + kScanTile * per_cta;
    float* tile_z = tile_x + kScanTile * per_cta;
    float s[NL], a[NL];
    float* S = PASS == 0 ? state + ((size_t)slot * inner + (live ? c : 0)) * N
                         : seg_state + ((size_t)unit * inner + (live ? c : 0)) * N;
#pragma unroll
    for (int i = 0; i < NL; ++i) {
        bool in = live && n0 + i < N;
        s[i] = (in && PASS != 1) ? S[n0 + i] : 0.f;
        a[i] = in ? -expf(a_log[(size_t)c * N + n0 + i]) : 0.f;
    }
    const float dsk = live ? dskip[c] : 0.f;
    float dt_sum = 0.f;
    const int c_base = blockIdx.y * per_cta;
    for (int t0 = 0; t0 < count; t0 += kScanTile) {
        const int tn = min(kScanTile, count - t0);
        __syncthreads();
        for (int i = threadIdx.x; i < tn * 2 * N; i += 128) tile_bc[i] = bc[(size_t)(first + t0) * 2 * N + i];
        for (int i = threadIdx.x; i < tn * per_cta; i += 128) {
            int t = i / per_cta, cl = i - t * per_cta, cc = c_base + cl;
            size_t row = (size_t)(first + t0 + t);
            bool in = cc < inner;
            tile_dt[i] = in ? softplus_f(dt_raw[row * inner + cc]) : 0.f;
            tile_x[i] = in ? to_float(xc[row * inner + cc]) : 0.f;
            if (PASS != 1) tile_z[i] = in ? to_float(xz[row * 2 * inner + inner + cc]) : 0.f;
        }
        __syncthreads();
        for (int t = 0; t < tn; ++t) {
            const float dt = tile_dt[t * per_cta + c_local];
            const float xv = tile_x[t * per_cta + c_local];
            const float* B = tile_bc + t * 2 * N + n0;
            const float* C = B + N;
            const float dx = dt * xv;
            float y = 0.f;
            if ((N & 3) == 0) {  // B and C four values a load (their rows start on 16-byte borders)
#pragma unroll
                for (int q = 0; q < NL / 4; ++q) {
                    if (n0 + 4 * q < N) {
                        const float4 b4 = reinterpret_cast<const float4*>(B)[q];
                        const float bv[4] = {b4.x, b4.y, b4.z, b4.w};
                        float cv[4] = {0.f, 0.f, 0.f, 0.f};
                        if (PASS != 1) {
                            const float4 c4 = reinterpret_cast<const float4*>(C)[q];
                            cv[0] = c4.x, cv[1] = c4.y, cv[2] = c4.z, cv[3] = c4.w;
                        }
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const int i = 4 * q + e;
                            s[i] = fmaf(exp_for<T>(dt * a[i]), s[i], dx * bv[e]);
                            if (PASS != 1) y = fmaf(s[i], cv[e], y);
                        }
                    }
                }
            } else {
#pragma unroll
                for (int i = 0; i < NL; ++i) {
                    if (n0 + i < N) {
                        s[i] = fmaf(exp_for<T>(dt * a[i]), s[i], dx * B[i]);
                        if (PASS != 1) y = fmaf(s[i], C[i], y);
                    }
                }
            }
            if (PASS == 1) {
                dt_sum += dt;
                continue;
            }
            for (int o = NS >> 1; o > 0; o >>= 1) y += __shfl_xor_sync(0xffffffffu, y, o);
            if (live && part == 0) {
                y = fmaf(dsk, xv, y);
                float z = tile_z[t * per_cta + c_local];
                y_out[(size_t)(first + t0 + t) * inner + c] = from_float<T>(y * (z / (1.0f + exp_for<T>(-z))));
            }
        }
    }
    if (!live) return;
    if (PASS != 2) {
#pragma unroll
        for (int i = 0; i < NL; ++i)
            if (n0 + i < N) S[n0 + i] = s[i];
    }
    if (PASS == 1 && part == 0) seg_dt[(size_t)unit * inner + c] = dt_sum;
    if (PASS != 1 && part == 0 && last_run) {
        // the convolution's tail: the last taps - 1 inputs of (old tail, this step's inputs)
        const int L = taps - 1;
        float* tail = conv_state + (size_t)slot * L * inner;
        for (int i = 0; i < L; ++i) {
            int at = seq_total + i;  // index into the old tail followed by the step's inputs
            float val = at < L ? tail[(size_t)at * inner + c]
                               : to_float(xz[(size_t)(seq_first + at - L) * 2 * inner + c]);
            tail[(size_t)i * inner + c] = val;
        }
    }
}

// Between the two passes over the runs: a thread per (sequence, channel, state index) walks the
// sequence's runs in order.  seg_state[run] (what the run added) becomes the state before the run;
// the slot's state becomes the state after the last run.
__global__ void __launch_bounds__(256)
scan_prefix_kernel(const float* __restrict__ a_log, float* __restrict__ state, const int* __restrict__ seq_slots,
                   const int* __restrict__ seq_first_segment, float* __restrict__ seg_state,
                   const float* __restrict__ seg_dt, int inner, int N) {
    pdl_wait();
    pdl_launch_dependents();
    const int seq = blockIdx.x;
    const int idx = blockIdx.y * 256 + threadIdx.x;
    if (idx >= inner * N) return;
    const int c = idx / N;
    const float a = -expf(a_log[idx]);
    float* S = state + (size_t)seq_slots[seq] * inner * N + idx;
    float carry = *S;
    const int last = seq_first_segment[seq + 1];
    const size_t per_run = (size_t)inner * N;
    // four runs' values are asked for together: the walk itself is a chain, its loads need not be
    for (int run = seq_first_segment[seq]; run < last; run += 4) {
        float added[4], dt[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const bool in = run + q < last;
            added[q] = in ? seg_state[(size_t)(run + q) * per_run + idx] : 0.f;
            dt[q] = in ? seg_dt[(size_t)(run + q) * inner + c] : 0.f;
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            if (run + q < last) {
                seg_state[(size_t)(run + q) * per_run + idx] = carry;
                carry = fmaf(expf(a * dt[q]), carry, added[q]);
            }
        }
    }
    *S = carry;
}

}  // namespace nnis

using namespace nnis;

NNIS_API int nnis_conv_silu(const void* xz, const float* conv_w, const float* conv_b, const float* conv_state,
                            const int* token_pos, const int* token_seq, const int* seq_slots,
                            const int* seq_first_row, void* xc, int n_tokens, int inner, int taps, int dtype,
                            cudaStream_t stream) {
    if (n_tokens <= 0 || inner <= 0 || taps <= 0 || !xz || !conv_w || !conv_state || !xc) return NNIS_ERR_ARGUMENT;
    dim3 grid(n_tokens, (unsigned)min(64, ((inner & 3) ? inner + 255 : inner / 4 + 255) / 256));
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

// state: float32 [slots, inner, N]; conv_state: float32 [slots, taps - 1, inner].  With `segments`
// (int32 [n_segments, 2] = (sequence, first token of the run), runs of seg_len tokens), the first
// run of every sequence in seq_first_segment [sequences + 1], and scratch seg_state float32
// [n_segments, inner, N] and seg_dt float32 [n_segments, inner], the runs are worked side by side.
NNIS_API int nnis_selective_scan(const void* xc, const void* xz, const float* dt_raw, const float* bc,
                                 const float* a_log, const float* dskip, float* state, float* conv_state,
                                 const int* token_pos, const int* token_seq, const int* seq_slots,
                                 const int* seq_first_row, const int* seq_count, const int* segments,
                                 int n_segments, const int* seq_first_segment, int seg_len, float* seg_state,
                                 float* seg_dt, void* y, int units, int inner, int N, int taps, int dtype,
                                 cudaStream_t stream) {
    if (units <= 0 || inner <= 0 || N <= 0 || taps <= 0 || !xc || !xz || !dt_raw || !bc || !a_log || !dskip ||
        !state || !conv_state || !y)
        return NNIS_ERR_ARGUMENT;
    if (segments && (!seq_first_row || !seq_first_segment || !seg_state || !seg_dt || seg_len <= 0 || n_segments <= 0))
        return NNIS_ERR_ARGUMENT;
    if (N > 256) return NNIS_ERR_UNSUPPORTED;
    // eight state values a thread, up to 32 threads a channel
    constexpr int NL = 8;
    int NS = 1;
    while (NS * NL < N) NS <<= 1;
    int per_cta = 128 / NS;
    unsigned tiles = (unsigned)((inner + per_cta - 1) / per_cta);
    if (tiles > 65535) return NNIS_ERR_UNSUPPORTED;
    size_t smem = sizeof(float) * kScanTile * (2 * (size_t)N + 3 * (size_t)per_cta);
    cudaError_t e = cudaSuccess;
#define NNIS_SCAN_PASS(T, PASS, UNITS) \
    e = launch_dependent(selective_scan_kernel<T, NL, PASS>, dim3(UNITS, tiles), 128, smem, stream, (const T*)xc, \
                         (const T*)xz, dt_raw, bc, a_log, dskip, state, conv_state, token_pos, token_seq, seq_slots, \
                         seq_first_row, seq_count, segments, seg_len, seg_state, seg_dt, (T*)y, inner, N, NS, taps)
#define NNIS_SCAN_ALL(T) \
    if (!segments) { \
        NNIS_SCAN_PASS(T, 0, units); \
    } else { \
        NNIS_SCAN_PASS(T, 1, n_segments); \
        if (e == cudaSuccess) \
            e = launch_dependent(scan_prefix_kernel, dim3(units, (unsigned)((inner * (size_t)N + 255) / 256)), 256, 0, \
                                 stream, a_log, state, seq_slots, seq_first_segment, seg_state, \
                                 (const float*)seg_dt, inner, N); \
        if (e == cudaSuccess) NNIS_SCAN_PASS(T, 2, n_segments); \
    }
    if (dtype == NNIS_DTYPE_F32) {
        NNIS_SCAN_ALL(float)
    } else if (dtype == NNIS_DTYPE_BF16) {
        NNIS_SCAN_ALL(bf16)
    } else {
        return NNIS_ERR_UNSUPPORTED;
    }
#undef NNIS_SCAN_ALL
#undef NNIS_SCAN_PASS
    return e == cudaSuccess ? NNIS_OK : (int)e;
}
