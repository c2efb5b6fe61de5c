// Latent attention over the paged cache: every position keeps ONE row that all
// heads share, [c | kr]: the normed latent c (dv values) and the rotated key part
// kr (dk - dv values).  Queries come already carried into that space (per head
// [Wuk_h^T q_plain | q_rotated], dk values), so a head's score against a position is
// one dot product with the row, and its output is the softmax-weighted sum of the
// rows' first dv values; the heads' values are made from that sum afterwards.
//
//   latent_prep      the down-projection's float32 row [q latent | c raw | kr raw] ->
//                    normed q latent (operand dtype), normed c and rotated kr into
//                    the cache row of the token's position
//   attention_latent one warp per (query token, head) walks the visible rows 32 at a
//                    time with an online softmax in float32; prompts and single
//                    tokens, float32 and bfloat16 storage, any sizes; the key range
//                    may be split over several warps (records merged in order)
#include <float.h>

#include "attention_merge.cuh"
#include "common.cuh"

namespace nnis {

__device__ __forceinline__ float block_sum_128(float v, float* scratch) {
    v = warp_sum(v);
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    return scratch[0] + scratch[1] + scratch[2] + scratch[3];
}

template <typename T>
__global__ void __launch_bounds__(128)
latent_prep_kernel(const float* __restrict__ a, const float* __restrict__ wq,
                   const float* __restrict__ wkv, const float* __restrict__ freq,
                   const int* __restrict__ token_pos, const int* __restrict__ token_seq,
                   const int* __restrict__ page_table, int table_cols, T* __restrict__ cq,
                   T* __restrict__ cache, int q_rank, int kv_rank, int rot, int rot_dims,
                   int page_size, float eps) {
    __shared__ float scratch[4];
    pdl_wait();
    pdl_launch_dependents();
    int n = blockIdx.x;
    int pos = token_pos[n];
    if (pos < 0) return;  // a padding row
    const float* row = a + (size_t)n * (q_rank + kv_rank + rot);
    // the query's latent
    float ss = 0.f;
    for (int i = threadIdx.x; i < q_rank; i += 128) ss = fmaf(row[i], row[i], ss);
    float s = 1.0f / sqrtf(block_sum_128(ss, scratch) / (float)q_rank + eps);
    T* q_out = cq + (size_t)n * q_rank;
    for (int i = threadIdx.x; i < q_rank; i += 128) q_out[i] = from_float<T>((row[i] * s) * wq[i]);
    // the keys' and values' latent
    const float* c = row + q_rank;
    ss = 0.f;
    for (int i = threadIdx.x; i < kv_rank; i += 128) ss = fmaf(c[i], c[i], ss);
    s = 1.0f / sqrtf(block_sum_128(ss, scratch) / (float)kv_rank + eps);
    int page = page_table[(size_t)token_seq[n] * table_cols + pos / page_size];
    T* dst = cache + ((size_t)page * page_size + pos % page_size) * (size_t)(kv_rank + rot);
    for (int i = threadIdx.x; i < kv_rank; i += 128) dst[i] = from_float<T>((c[i] * s) * wkv[i]);
    // the rotated key part, shared by all heads
    const float* kr = c + kv_rank;
    int half = rot_dims >> 1;
    for (int j = threadIdx.x; j < rot - half; j += 128) {
        if (j < half) {
            float ang = (float)pos * freq[j];
            float cs = cosf(ang), sn = sinf(ang);
            float u = kr[j], v = kr[j + half];
            dst[kv_rank + j] = from_float<T>(u * cs - v * sn);
            dst[kv_rank + j + half] = from_float<T>(v * cs + u * sn);
        } else {
            dst[kv_rank + j + half] = from_float<T>(kr[j + half]);
        }
    }
}

// partial record per (token, head, split): [0] running max, [1] running sum,
// [2 .. 2+dv) unnormalised output
template <typename T, int R>
__global__ void __launch_bounds__(128)
latent_warp_kernel(const T* __restrict__ q, const T* __restrict__ cache,
                   const int* __restrict__ token_pos, const int* __restrict__ token_seq,
                   const int* __restrict__ page_table, int table_cols, T* __restrict__ out,
                   float* __restrict__ partial, int n_tokens, int heads, int dk, int dv,
                   int page_size, float scale, int n_splits) {
    extern __shared__ float q_smem[];
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int n = blockIdx.x * 4 + warp;
    if (n >= n_tokens) return;
    int h = blockIdx.y, split = blockIdx.z;
    int pos = token_pos[n];
    float* qs = q_smem + warp * dk;
    float m = -FLT_MAX, l = 0.f;
    float acc[R];
#pragma unroll
    for (int r = 0; r < R; ++r) acc[r] = 0.f;
    if (pos >= 0) {
        const T* qrow = q + ((size_t)n * heads + h) * dk;
        for (int i = lane; i < dk; i += 32) qs[i] = to_float(qrow[i]);
        __syncwarp();
        int hi = pos + 1;
        int per = (hi + n_splits - 1) / n_splits;
        per = (per + 31) & ~31;
        int start = split * per;
        int end = min(hi, start + per);
        const int* table = page_table + (size_t)token_seq[n] * table_cols;
        for (int c0 = start; c0 < end; c0 += 32) {
            int t = c0 + lane;
            bool valid = t < end;
            int row_index = 0;
            float s = -FLT_MAX;
            if (valid) {
                row_index = table[t / page_size] * page_size + (t % page_size);
                const T* krow = cache + (size_t)row_index * dk;
                float dot = 0.f;
                for (int i = 0; i < dk; ++i) dot = fmaf(qs[i], to_float(krow[i]), dot);
                s = dot * scale;
            }
            float m_new = fmaxf(m, warp_max(s));
            float p = valid ? expf(s - m_new) : 0.f;
            float alpha = l == 0.f ? 0.f : expf(m - m_new);
            l = l * alpha + warp_sum(p);
            m = m_new;
#pragma unroll
            for (int r = 0; r < R; ++r) acc[r] *= alpha;
            int count = min(32, end - c0);
            for (int j = 0; j < count; ++j) {
                float pj = __shfl_sync(0xffffffffu, p, j);
                int rj = __shfl_sync(0xffffffffu, row_index, j);
                const T* vrow = cache + (size_t)rj * dk;
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    int i = lane + 32 * r;
                    if (i < dv) acc[r] = fmaf(pj, to_float(vrow[i]), acc[r]);
                }
            }
        }
    }
    if (n_splits == 1) {
        float inv = l > 0.f ? 1.0f / l : 0.f;
        T* o = out + ((size_t)n * heads + h) * dv;
#pragma unroll
        for (int r = 0; r < R; ++r) {
            int i = lane + 32 * r;
            if (i < dv) o[i] = from_float<T>(acc[r] * inv);
        }
    } else {
        float* rec = partial + (((size_t)n * heads + h) * n_splits + split) * (size_t)(dv + 2);
        if (lane == 0) {
            rec[0] = m;
            rec[1] = l;
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
            int i = lane + 32 * r;
            if (i < dv) rec[2 + i] = acc[r];
        }
    }
}

template <typename T>
static int launch_latent(const void* q, const void* cache, const int* token_pos, const int* token_seq,
                         const int* page_table, int table_cols, void* out, float* partial,
                         int n_tokens, int heads, int dk, int dv, int page_size, float scale,
                         int n_splits, cudaStream_t stream) {
    dim3 grid((n_tokens + 3) / 4, heads, n_splits);
    size_t smem = 4 * (size_t)dk * sizeof(float);
#define NNIS_LATENT_CASE(R) \
    latent_warp_kernel<T, R><<<grid, 128, smem, stream>>>( \
        (const T*)q, (const T*)cache, token_pos, token_seq, page_table, table_cols, (T*)out, partial, \
        n_tokens, heads, dk, dv, page_size, scale, n_splits)
    if (dv <= 32) NNIS_LATENT_CASE(1);
    else if (dv <= 64) NNIS_LATENT_CASE(2);
    else if (dv <= 128) NNIS_LATENT_CASE(4);
    else if (dv <= 256) NNIS_LATENT_CASE(8);
    else NNIS_LATENT_CASE(16);
#undef NNIS_LATENT_CASE
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;
    if (n_splits > 1) {
        size_t rows = (size_t)n_tokens * heads;
        attn_merge_kernel<T><<<(unsigned)rows, 128, 0, stream>>>(partial, (T*)out, rows, dv,
                                                                             n_splits);
    }
    NNIS_RETURN_LAUNCH();
}

}  // namespace nnis

using namespace nnis;

NNIS_API int nnis_latent_prep(const float* a, const float* wq, const float* wkv, const float* freq,
                              const int* token_pos, const int* token_seq, const int* page_table,
                              int table_cols, void* cq, void* cache, int n_tokens, int q_rank,
                              int kv_rank, int rot, int rot_dims, int page_size, float eps, int dtype,
                              cudaStream_t stream) {
    if (n_tokens <= 0 || q_rank <= 0 || kv_rank <= 0 || rot < 0 || rot_dims < 0 || (rot_dims & 1) ||
        rot_dims > rot || page_size <= 0 || table_cols <= 0 || !(eps > 0.f) || !a || !wq || !wkv ||
        !freq || !cq || !cache)
        return NNIS_ERR_ARGUMENT;
    cudaError_t e;
    if (dtype == NNIS_DTYPE_F32)
        e = launch_dependent(latent_prep_kernel<float>, n_tokens, 128, 0, stream, a, wq, wkv, freq, token_pos,
                             token_seq, page_table, table_cols, (float*)cq, (float*)cache, q_rank, kv_rank, rot,
                             rot_dims, page_size, eps);
    else if (dtype == NNIS_DTYPE_BF16)
        e = launch_dependent(latent_prep_kernel<bf16>, n_tokens, 128, 0, stream, a, wq, wkv, freq, token_pos,
                             token_seq, page_table, table_cols, (bf16*)cq, (bf16*)cache, q_rank, kv_rank, rot,
                             rot_dims, page_size, eps);
    else
        return NNIS_ERR_UNSUPPORTED;
    return e == cudaSuccess ? NNIS_OK : (int)e;
}

// Scratch: `partial` needs n_tokens * heads * n_splits * (dv + 2) floats when
// n_splits > 1 and may be null otherwise.
NNIS_API int nnis_attention_latent(const void* q, const void* cache, const int* token_pos,
                                   const int* token_seq, const int* page_table, int table_cols,
                                   void* out, float* partial, int n_tokens, int heads, int dk, int dv,
                                   int page_size, float scale, int n_splits, int dtype,
                                   cudaStream_t stream) {
    if (n_tokens <= 0 || heads <= 0 || dk <= 0 || dv <= 0 || dv > dk || page_size <= 0 ||
        table_cols <= 0 || n_splits <= 0)
        return NNIS_ERR_ARGUMENT;
    if (dv > 512 || dk > 2048 || heads > 65535 || n_splits > 64) return NNIS_ERR_UNSUPPORTED;
    if (n_splits > 1 && !partial) return NNIS_ERR_ARGUMENT;
    if (dtype == NNIS_DTYPE_F32)
        return launch_latent<float>(q, cache, token_pos, token_seq, page_table, table_cols, out, partial,
                                    n_tokens, heads, dk, dv, page_size, scale, n_splits, stream);
    if (dtype == NNIS_DTYPE_BF16)
        return launch_latent<bf16>(q, cache, token_pos, token_seq, page_table, table_cols, out, partial,
                                   n_tokens, heads, dk, dv, page_size, scale, n_splits, stream);
    return NNIS_ERR_UNSUPPORTED;
}
