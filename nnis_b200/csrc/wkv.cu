// WKV time mixing: a recurrence with a decay per token, head and key channel, and a
// bonus for the current token.  Per head, with r, k, v of `dim` channels each and
// w = exp(-exp(d)) from the decay's projection d:
//
//     o_t = (S_{t-1} + diag(u) k_t v_t^T)^T r_t        S_t = diag(w_t) S_{t-1} + k_t v_t^T
//
// S [dim (key), dim (value)] is float32 in a per-sequence state area, and so is the
// previous token's input row, which the token shift needs; both are carried from step to
// step.  Everything between the projections and the gated output is float32.
//
//   wkv_mix      the token shift: mix_s = h + (h' - h) * mu_s for S streams (h' the row of
//                the token before: the row above, or the state's at a step's first token)
//   wkv_scan     a CTA per (sequence, head) walks the step's tokens in order, 16 (or fewer)
//                at a time through shared memory; a thread holds a run of key channels of
//                one value column of S in registers; partial outputs of the runs are added
//                up per tile of tokens.  Long prompts: runs of tokens side by side in two
//                passes with wkv_prefix between them (see the kernel)
//   wkv_finish   o / rms(o) per head, times the norm's weights, times silu(gate), rounded
//                once; the step's last row of every sequence becomes the state's h'
//
// A row whose position is -1 (padding) is skipped everywhere.
#include "async_copy.cuh"
#include "common.cuh"

namespace nnis {

// which sequence a row belongs to and whether it is that sequence's first row of the step
struct RowPlace {
    int slot, first, count;
};

__device__ __forceinline__ RowPlace place_of_row(int n, const int* token_pos, const int* token_seq,
                                                 const int* seq_slots, const int* seq_first_row,
                                                 const int* seq_count) {
    RowPlace p;
    int seq = token_seq[n];
    p.slot = seq_slots[seq];
    if (seq_first_row) {
        p.first = seq_first_row[seq];
        p.count = seq_count[seq];
    } else {
        p.first = n;
        p.count = 1;
    }
    return p;
}

// mixes [streams][n_tokens][width]; mu float32 [streams][width]; prev float32 [slots][width]
template <typename T>
__global__ void __launch_bounds__(256)
wkv_mix_kernel(const T* __restrict__ x, const float* __restrict__ mu, const float* __restrict__ prev,
               const int* __restrict__ token_pos, const int* __restrict__ token_seq,
               const int* __restrict__ seq_slots, const int* __restrict__ seq_first_row,
               const int* __restrict__ seq_count, T* __restrict__ mixes, int n_tokens, int width, int streams) {
    pdl_wait();
    pdl_launch_dependents();
    const int n = blockIdx.x;
    if (token_pos[n] < 0) return;
    RowPlace p = place_of_row(n, token_pos, token_seq, seq_slots, seq_first_row, seq_count);
    const T* h = x + (size_t)n * width;
    const float* before_state = prev + (size_t)p.slot * width;
    const bool above = n > p.first;
    for (int i = threadIdx.x; i < width; i += 256) {
        float cur = to_float(h[i]);
        float was = above ? to_float(h[i - width]) : before_state[i];
        float d = was - cur;
        for (int s = 0; s < streams; ++s)
            mixes[((size_t)s * n_tokens + n) * width + i] = from_float<T>(fmaf(d, mu[(size_t)s * width + i], cur));
    }
}

// KL: key channels a thread holds.  Threads: dim value columns x KS runs of KL key channels.
//
// PASS 0: a unit is a sequence of the step (or a row, in steps of single tokens): from the slot's
//         state to the slot's state, outputs written.
// Long prompts are cut into runs of `seg_len` tokens that are worked side by side (the recurrence is
// linear in the state): a unit is then a run, (sequence, first token) in `segments`, and
// PASS 1: from a zero state; what the run adds to the state goes to seg_state[run, head], the sum of
//         the logarithms of its decays per key channel to seg_logw[run, head] (the state before the
//         run decays by exp of that sum over it); wkv_prefix_kernel then turns seg_state[run] into
//         the state BEFORE each run and leaves the slot's state as it is after the step;
// PASS 2: from seg_state[run], outputs written.
template <typename T, int KL, int PASS>
__global__ void __launch_bounds__(1024, 1)
wkv_scan_kernel(const T* __restrict__ r, const T* __restrict__ k, const T* __restrict__ v,
                const float* __restrict__ d, const float* __restrict__ u, float* __restrict__ state,
                const int* __restrict__ token_pos, const int* __restrict__ token_seq,
                const int* __restrict__ seq_slots, const int* __restrict__ seq_first_row,
                const int* __restrict__ seq_count, const int* __restrict__ segments, int seg_len,
                float* __restrict__ seg_state, float* __restrict__ seg_logw, float* __restrict__ o_raw,
                int heads, int dim, int KS, int TT) {
    extern __shared__ __align__(16) float smem[];
    pdl_wait();
    pdl_launch_dependents();
    const int dimP = KS * KL;         // (a multiple of eight: the four arrays below start on 16-byte borders)
    float* rs = smem;                 // [TT][dimP]
    float* ks = rs + TT * dimP;       // [TT][dimP]
    float* ws = ks + TT * dimP;       // [TT][dimP]
    float* us = ws + TT * dimP;       // [dimP]
    float* vs = us + dimP;            // [TT][dim]
    float* part = vs + TT * dim;      // [TT][KS][dim]; PASS 1: [TT][dimP] logarithms of the decays
    const int unit = blockIdx.x, h = blockIdx.y;
    int first, count, slot;
    if (PASS != 0) {
        const int seq = segments[2 * unit], t0 = segments[2 * unit + 1];
        first = seq_first_row[seq] + t0;
        count = min(seg_len, seq_count[seq] - t0);
        slot = seq_slots[seq];
    } else if (seq_first_row) {
        first = seq_first_row[unit];
        count = seq_count[unit];
        slot = seq_slots[unit];
    } else {
        first = unit;
        count = token_pos[unit] < 0 ? 0 : 1;
        slot = seq_slots[token_seq[unit]];
    }
    if (count <= 0) return;
    const int threads = dim * KS;
    const int j = threadIdx.x % dim, run = threadIdx.x / dim, k0 = run * KL;
    const size_t row_len = (size_t)heads * dim;
    float* S = PASS == 0 ? state + ((size_t)slot * heads + h) * dim * dim
                         : seg_state + ((size_t)unit * heads + h) * dim * dim;
    float s[KL];
#pragma unroll
    for (int kk = 0; kk < KL; ++kk) s[kk] = (PASS != 1 && k0 + kk < dim) ? S[(size_t)(k0 + kk) * dim + j] : 0.f;
    for (int i = threadIdx.x; i < dimP; i += threads) us[i] = i < dim ? u[(size_t)h * dim + i] : 0.f;
    float logw = 0.f;  // PASS 1: thread i < dim adds up the logarithms of key channel i's decays
    for (int t0 = 0; t0 < count; t0 += TT) {
        const int tn = min(TT, count - t0);
        __syncthreads();  // the tile before has been added up and written
        for (int i = threadIdx.x; i < tn * dimP; i += threads) {
            int t = i / dimP, c = i - t * dimP;
            size_t at = (size_t)(first + t0 + t) * row_len + (size_t)h * dim + c;
            bool in = c < dim;
            float lw = in ? -expf(d[at]) : 0.f;
            if (PASS != 1) rs[i] = in ? to_float(r[at]) : 0.f;
            ks[i] = in ? to_float(k[at]) : 0.f;
            ws[i] = in ? expf(lw) : 0.f;
            if (PASS == 1) part[i] = lw;
            if (in) vs[t * dim + c] = to_float(v[at]);
        }
        __syncthreads();
        for (int t = 0; t < tn; ++t) {
            const float vj = vs[t * dim + j];
            // the tile's rows are read four values a load (every thread of a run reads the same ones)
            const float4* rt = reinterpret_cast<const float4*>(rs + t * dimP + k0);
            const float4* kt = reinterpret_cast<const float4*>(ks + t * dimP + k0);
            const float4* wt = reinterpret_cast<const float4*>(ws + t * dimP + k0);
            const float4* ut = reinterpret_cast<const float4*>(us + k0);
            float o = 0.f;
#pragma unroll
            for (int kq = 0; kq < KL / 4; ++kq) {
                const float4 k4 = kt[kq], w4 = wt[kq];
                const float kv[4] = {k4.x * vj, k4.y * vj, k4.z * vj, k4.w * vj};
                const float wv[4] = {w4.x, w4.y, w4.z, w4.w};
                if (PASS != 1) {
                    const float4 r4 = rt[kq], u4 = ut[kq];
                    const float rv[4] = {r4.x, r4.y, r4.z, r4.w}, uv[4] = {u4.x, u4.y, u4.z, u4.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) o = fmaf(rv[e], fmaf(uv[e], kv[e], s[kq * 4 + e]), o);
                }
#pragma unroll
                for (int e = 0; e < 4; ++e) s[kq * 4 + e] = fmaf(wv[e], s[kq * 4 + e], kv[e]);
            }
            if (PASS != 1) part[(t * KS + run) * dim + j] = o;
        }
        if (PASS == 1) {
            if (threadIdx.x < dim)
                for (int t = 0; t < tn; ++t) logw += part[t * dimP + threadIdx.x];
            continue;
        }
        __syncthreads();
        for (int i = threadIdx.x; i < tn * dim; i += threads) {
            int t = i / dim, c = i - t * dim;
            float o = 0.f;
            for (int q = 0; q < KS; ++q) o += part[(t * KS + q) * dim + c];
            o_raw[(size_t)(first + t0 + t) * row_len + (size_t)h * dim + c] = o;
        }
    }
    if (PASS != 2) {
#pragma unroll
        for (int kk = 0; kk < KL; ++kk)
            if (k0 + kk < dim) S[(size_t)(k0 + kk) * dim + j] = s[kk];
    }
    if (PASS == 1 && threadIdx.x < dim) seg_logw[((size_t)unit * heads + h) * dim + threadIdx.x] = logw;
}

// Between the two passes over the runs: a thread per (sequence, head, key channel, value channel)
// walks the sequence's runs in order.  seg_state[run] (what the run added) becomes the state before
// the run; the slot's state becomes the state after the last run.
__global__ void __launch_bounds__(256)
wkv_prefix_kernel(float* __restrict__ state, const int* __restrict__ seq_slots,
                  const int* __restrict__ seq_first_segment, float* __restrict__ seg_state,
                  const float* __restrict__ seg_logw, int heads, int dim) {
    pdl_wait();
    pdl_launch_dependents();
    const int seq = blockIdx.x;
    const size_t per_seq = (size_t)heads * dim * dim;
    const size_t idx = (size_t)blockIdx.y * 256 + threadIdx.x;
    if (idx >= per_seq) return;
    const size_t hk = idx / dim;  // head * dim + key channel
    float* S = state + (size_t)seq_slots[seq] * per_seq + idx;
    float carry = *S;
    const int last = seq_first_segment[seq + 1];
    // four runs' values are asked for together: the walk itself is a chain, its loads need not be
    for (int run = seq_first_segment[seq]; run < last; run += 4) {
        float added[4], decay[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const bool in = run + q < last;
            added[q] = in ? seg_state[(size_t)(run + q) * per_seq + idx] : 0.f;
            decay[q] = in ? seg_logw[(size_t)(run + q) * heads * dim + hk] : 0.f;
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            if (run + q < last) {
                seg_state[(size_t)(run + q) * per_seq + idx] = carry;
                carry = fmaf(expf(decay[q]), carry, added[q]);
            }
        }
    }
    *S = carry;
}

// a CTA per row; a warp per head in turn
template <typename T>
__global__ void __launch_bounds__(256)
wkv_finish_kernel(const float* __restrict__ o_raw, const T* __restrict__ gate, const float* __restrict__ norm_w,
                  const T* __restrict__ x, float* __restrict__ prev, const int* __restrict__ token_pos,
                  const int* __restrict__ token_seq, const int* __restrict__ seq_slots,
                  const int* __restrict__ seq_first_row, const int* __restrict__ seq_count,
                  T* __restrict__ out, int heads, int dim, int width, float eps) {
    pdl_wait();
    pdl_launch_dependents();
    const int n = blockIdx.x;
    if (token_pos[n] < 0) return;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const size_t row_len = (size_t)heads * dim;
    for (int h = warp; h < heads; h += 8) {
        const float* o = o_raw + (size_t)n * row_len + (size_t)h * dim;
        float ss = 0.f;
        for (int i = lane; i < dim; i += 32) ss = fmaf(o[i], o[i], ss);
        ss = warp_sum(ss);
        const float inv = 1.0f / sqrtf(ss / (float)dim + eps);
        for (int i = lane; i < dim; i += 32) {
            size_t at = (size_t)n * row_len + (size_t)h * dim + i;
            float g = to_float(gate[at]);
            float y = (o[i] * inv) * norm_w[(size_t)h * dim + i] * (g / (1.0f + expf(-g)));
            out[at] = from_float<T>(y);
        }
    }
    RowPlace p = place_of_row(n, token_pos, token_seq, seq_slots, seq_first_row, seq_count);
    if (n == p.first + p.count - 1) {
        const T* h = x + (size_t)n * width;
        float* keep = prev + (size_t)p.slot * width;
        for (int i = threadIdx.x; i < width; i += 256) keep[i] = to_float(h[i]);
    }
}

template <typename T>
static int wkv_launch(const void* x, const float* mu, float* prev, const int* token_pos, const int* token_seq,
                      const int* seq_slots, const int* seq_first_row, const int* seq_count, void* mixes,
                      int n_tokens, int width, int streams, cudaStream_t stream) {
    cudaError_t e = launch_dependent(wkv_mix_kernel<T>, (unsigned)n_tokens, 256, 0, stream, (const T*)x, mu,
                                     (const float*)prev, token_pos, token_seq, seq_slots, seq_first_row, seq_count,
                                     (T*)mixes, n_tokens, width, streams);
    return e == cudaSuccess ? NNIS_OK : (int)e;
}

template <typename T, int KL, int PASS>
static cudaError_t scan_launch(dim3 grid, int threads, size_t smem, cudaStream_t stream, const void* r,
                               const void* k, const void* v, const float* d, const float* u, float* state,
                               const int* token_pos, const int* token_seq, const int* seq_slots,
                               const int* seq_first_row, const int* seq_count, const int* segments, int seg_len,
                               float* seg_state, float* seg_logw, float* o_raw, int heads, int dim, int KS, int TT) {
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(wkv_scan_kernel<T, KL, PASS>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
    }
    return launch_dependent(wkv_scan_kernel<T, KL, PASS>, grid, threads, smem, stream, (const T*)r, (const T*)k,
                            (const T*)v, d, u, state, token_pos, token_seq, seq_slots, seq_first_row, seq_count,
                            segments, seg_len, seg_state, seg_logw, o_raw, heads, dim, KS, TT);
}

template <typename T, int KL>
static cudaError_t scan_passes(int units, int n_segments, int threads, size_t smem, cudaStream_t stream,
                               const void* r, const void* k, const void* v, const float* d, const float* u,
                               float* state, const int* token_pos, const int* token_seq, const int* seq_slots,
                               const int* seq_first_row, const int* seq_count, const int* segments,
                               const int* seq_first_segment, int seg_len, float* seg_state, float* seg_logw,
                               float* o_raw, int heads, int dim, int KS, int TT) {
#define NNIS_WKV_ARGS r, k, v, d, u, state, token_pos, token_seq, seq_slots, seq_first_row, seq_count, segments, \
                      seg_len, seg_state, seg_logw, o_raw, heads, dim, KS, TT
    if (!segments)
        return scan_launch<T, KL, 0>(dim3(units, heads), threads, smem, stream, NNIS_WKV_ARGS);
    cudaError_t e = scan_launch<T, KL, 1>(dim3(n_segments, heads), threads, smem, stream, NNIS_WKV_ARGS);
    if (e != cudaSuccess) return e;
    const size_t per_seq = (size_t)heads * dim * dim;
    e = launch_dependent(wkv_prefix_kernel, dim3(units, (unsigned)((per_seq + 255) / 256)), 256, 0, stream, state,
                         seq_slots, seq_first_segment, seg_state, (const float*)seg_logw, heads, dim);
    if (e != cudaSuccess) return e;
    return scan_launch<T, KL, 2>(dim3(n_segments, heads), threads, smem, stream, NNIS_WKV_ARGS);
#undef NNIS_WKV_ARGS
}

}  // namespace nnis

using namespace nnis;

NNIS_API int nnis_wkv_mix(const void* x, const float* mu, float* prev, const int* token_pos,
                          const int* token_seq, const int* seq_slots, const int* seq_first_row,
                          const int* seq_count, void* mixes, int n_tokens, int width, int streams, int dtype,
                          cudaStream_t stream) {
    if (n_tokens <= 0 || width <= 0 || streams <= 0 || !x || !mu || !prev || !mixes) return NNIS_ERR_ARGUMENT;
    if (dtype == NNIS_DTYPE_F32)
        return wkv_launch<float>(x, mu, prev, token_pos, token_seq, seq_slots, seq_first_row, seq_count, mixes,
                                 n_tokens, width, streams, stream);
    if (dtype == NNIS_DTYPE_BF16)
        return wkv_launch<bf16>(x, mu, prev, token_pos, token_seq, seq_slots, seq_first_row, seq_count, mixes,
                                n_tokens, width, streams, stream);
    return NNIS_ERR_UNSUPPORTED;
}

// r, k, v: operand dtype [n, heads * dim]; d: float32 [n, heads * dim] (the decay's projection,
// w = exp(-exp(d))); u: float32 [heads, dim]; state: float32 [slots, heads, dim, dim];
// o_raw: float32 [n, heads * dim].  `units`: sequences of the step (with seq_first_row) or rows.
// With `segments` (int32 [n_segments, 2] = (sequence, first token of the run), runs of seg_len
// tokens), seq_first_segment [sequences + 1] and scratch seg_state float32 [n_segments, heads, dim,
// dim] and seg_logw float32 [n_segments, heads, dim] the runs are worked side by side.
NNIS_API int nnis_wkv_scan(const void* r, const void* k, const void* v, const float* d, const float* u,
                           float* state, const int* token_pos, const int* token_seq, const int* seq_slots,
                           const int* seq_first_row, const int* seq_count, const int* segments, int n_segments,
                           const int* seq_first_segment, int seg_len, float* seg_state, float* seg_logw,
                           float* o_raw, int units, int heads, int dim, int dtype, cudaStream_t stream) {
    if (units <= 0 || heads <= 0 || dim <= 0 || !r || !k || !v || !d || !u || !state || !o_raw)
        return NNIS_ERR_ARGUMENT;
    if (segments && (!seq_first_row || !seq_first_segment || !seg_state || !seg_logw || seg_len <= 0 ||
                     n_segments <= 0))
        return NNIS_ERR_ARGUMENT;
    if (dim > 256 || heads > 65535) return NNIS_ERR_UNSUPPORTED;
    // as many runs of key channels as keep the CTA at 256 threads or more, at most 1,024
    int KL = dim <= 16 ? 8 : (dim <= 64 ? 16 : (dim <= 128 ? 32 : 64));
    int KS = (dim + KL - 1) / KL;
    int threads = dim * KS;
    if (threads > 1024) return NNIS_ERR_UNSUPPORTED;
    int dimP = KS * KL;
    int TT = seq_first_row ? 16 : 1;
    auto bytes = [&](int tt) {
        return sizeof(float) * ((size_t)tt * (3 * dimP + dim + (size_t)max(KS * dim, dimP)) + dimP);
    };
    while (TT > 1 && bytes(TT) > 96 * 1024) TT >>= 1;
    size_t smem = bytes(TT);
    cudaError_t e;
#define NNIS_WKV_CASE(T, KLV) \
    e = scan_passes<T, KLV>(units, n_segments, threads, smem, stream, r, k, v, d, u, state, token_pos, token_seq, \
                            seq_slots, seq_first_row, seq_count, segments, seq_first_segment, seg_len, seg_state, \
                            seg_logw, o_raw, heads, dim, KS, TT)
    if (dtype == NNIS_DTYPE_F32) {
        if (KL == 8) NNIS_WKV_CASE(float, 8);
        else if (KL == 16) NNIS_WKV_CASE(float, 16);
        else if (KL == 32) NNIS_WKV_CASE(float, 32);
        else NNIS_WKV_CASE(float, 64);
    } else if (dtype == NNIS_DTYPE_BF16) {
        if (KL == 8) NNIS_WKV_CASE(bf16, 8);
        else if (KL == 16) NNIS_WKV_CASE(bf16, 16);
        else if (KL == 32) NNIS_WKV_CASE(bf16, 32);
        else NNIS_WKV_CASE(bf16, 64);
    } else {
        return NNIS_ERR_UNSUPPORTED;
    }
#undef NNIS_WKV_CASE
    return e == cudaSuccess ? NNIS_OK : (int)e;
}

NNIS_API int nnis_wkv_finish(const float* o_raw, const void* gate, const float* norm_w, const void* x,
                             float* prev, const int* token_pos, const int* token_seq, const int* seq_slots,
                             const int* seq_first_row, const int* seq_count, void* out, int n_tokens, int heads,
                             int dim, int width, float eps, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0 || heads <= 0 || dim <= 0 || width <= 0 || !(eps > 0.f) || !o_raw || !gate || !norm_w ||
        !x || !prev || !out)
        return NNIS_ERR_ARGUMENT;
    cudaError_t e;
    if (dtype == NNIS_DTYPE_F32)
        e = launch_dependent(wkv_finish_kernel<float>, (unsigned)n_tokens, 256, 0, stream, o_raw, (const float*)gate,
                             norm_w, (const float*)x, prev, token_pos, token_seq, seq_slots, seq_first_row,
                             seq_count, (float*)out, heads, dim, width, eps);
    else if (dtype == NNIS_DTYPE_BF16)
        e = launch_dependent(wkv_finish_kernel<bf16>, (unsigned)n_tokens, 256, 0, stream, o_raw, (const bf16*)gate,
                             norm_w, (const bf16*)x, prev, token_pos, token_seq, seq_slots, seq_first_row,
                             seq_count, (bf16*)out, heads, dim, width, eps);
    else
        return NNIS_ERR_UNSUPPORTED;
    return e == cudaSuccess ? NNIS_OK : (int)e;
}
