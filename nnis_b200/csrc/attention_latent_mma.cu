// Latent attention on the tensor cores (bfloat16): all heads of a token share the
// cached rows [c | kr], so the (token, head) pairs of a sequence are stacked into the
// rows of one matrix [tokens * heads, dk]: with 8 heads 64 rows are 8 query tokens, with
// 64 heads one.  A prompt, a later chunk and a single decoded token are the same case
// (one token gives `heads` rows).  A CTA of eight warps (two groups of four, a warp 16
// rows) walks the sequence's pages (64 positions) up to its last query; a page comes into
// swizzled shared memory once, by 16-byte cp.async copies, and serves both products:
// scores S = Q K^T over all dk values of the rows, and O += P V over their first dv
// values.  A group holds a run of NT * 8 output values per row in registers (128, or 256
// with the softmax taken 32 keys at a time so that S and P stay small).  Where one run
// covers dv, the two groups take 64 rows each (128 rows a CTA) and S is computed once;
// where dv needs more runs, both groups take the same 64 rows and a run each.  The online
// softmax between the products is float32 in registers.  Rows in shared memory are padded
// to a multiple of 64 values (zeros) so that the XOR swizzle stays inside a row.
//
// The key range may be cut into slices (blockIdx.z), for steps with few rows and long
// contexts: a slice leaves [max, sum, unnormalised output] per row and the merge kernel
// adds the slices up in order.
#include <float.h>

#include "attention_merge.cuh"
#include "mma_helpers.cuh"

namespace nnis {

constexpr int kLatRows = 64;   // rows of a warp group
constexpr int kLatPage = 64;

__device__ __forceinline__ int swz_rt(int row, int chunk, int width) {
    return row * width + (((chunk & ~7) | ((chunk & 7) ^ (row & 7))) << 3);
}

// NT: 8-value tiles of a group's run of the output (16 or 32); KH: keys per softmax step
// (64, or 32 with NT = 32); SPLIT_ROWS: the groups take 64 rows each and the same run.
template <int STAGES, int NT, bool SPLIT_ROWS>
__global__ void __launch_bounds__(256)
latent_mma_kernel(const bf16* __restrict__ q, const bf16* __restrict__ cache,
                  const int* __restrict__ tiles, const int* __restrict__ seq_first_row,
                  const int* __restrict__ seq_start, const int* __restrict__ seq_count,
                  const int* __restrict__ token_pos, const int* __restrict__ token_seq,
                  const int* __restrict__ page_table, int table_cols, bf16* __restrict__ out,
                  float* __restrict__ partial, int heads, int dk, int dv, int dkp, int tiles_per_token,
                  float scale, int n_splits) {
    constexpr int KH = NT == 16 ? 64 : 32, KB = KH / 8, RUN = NT * 8;
    constexpr int TILE = SPLIT_ROWS ? 2 * kLatRows : kLatRows;  // rows of the CTA
    extern __shared__ __align__(128) unsigned char smem_raw[];
    pdl_wait();
    pdl_launch_dependents();
    bf16* q_s = reinterpret_cast<bf16*>(smem_raw);       // [TILE, dkp] swizzled
    bf16* k_s = q_s + (size_t)TILE * dkp;                // stages x [64, dkp]
    const int lane = threadIdx.x & 31, warp = (threadIdx.x >> 5) & 3, group = threadIdx.x >> 7;
    const int tid = threadIdx.x;
    const int CH = dk >> 3, CHP = dkp >> 3;
    int seq, r0, count, start, first;
    if (tiles) {
        seq = tiles[2 * blockIdx.x];
        r0 = tiles[2 * blockIdx.x + 1];
        count = seq_count[seq];
        start = seq_start[seq];
        first = seq_first_row[seq];
    } else {  // one token per row of the step; a row without a sequence has position -1
        int n = blockIdx.x / tiles_per_token;
        r0 = (blockIdx.x - n * tiles_per_token) * TILE;
        start = token_pos[n];
        count = start < 0 ? 0 : 1;
        first = n;
        seq = token_seq[n];
    }
    const int total = count * heads;                 // stacked rows of this sequence's step
    const int rows = min(TILE, total - r0);          // valid rows of the tile
    const size_t row_base = (size_t)first * heads + r0;
    const int g_row = SPLIT_ROWS ? group * kLatRows : 0;                   // this group's first row
    const int run = SPLIT_ROWS ? (int)blockIdx.y : (int)blockIdx.y * 2 + group;  // ... and run of values
    const int c0 = run * NT;                         // the run's first 16-byte chunk
    // (<= 0: the group has no rows or no values of its own and only helps to copy)
    const int dv_here = g_row < rows ? min(RUN, dv - run * RUN) : 0;
    const int split = blockIdx.z;
    if (rows <= 0) {
        return;  // (a padding row: the merge and the projections after it read nothing of it)
    }
    const int hi = start + (r0 + rows - 1) / heads + 1;  // keys below this position may be seen
    const int all_pages = (hi - 1) / kLatPage + 1;
    const int per = (all_pages + n_splits - 1) / n_splits;
    const int first_page = split * per;
    const int n_pages = max(0, min(all_pages, first_page + per) - first_page);
    const int* table = page_table + (size_t)seq * table_cols;
    const size_t tile_elems = (size_t)kLatPage * dkp;

    // the padding columns of every buffer are zero and stay zero
    if (CHP > CH) {
        const int padc = CHP - CH;
        for (int c = tid; c < (TILE + STAGES * kLatPage) * padc; c += 256) {
            int row = c / padc, chunk = CH + c % padc;  // (the buffers lie one after another)
            *reinterpret_cast<uint4*>(q_s + swz_rt(row, chunk, dkp)) = make_uint4(0, 0, 0, 0);
        }
    }
    auto load_page = [&](int it) {
        if (it < n_pages) {
            int page = table[first_page + it];
            const bf16* src = cache + (size_t)page * kLatPage * dk;
            bf16* dst = k_s + (size_t)(it % STAGES) * tile_elems;
            for (int c = tid; c < kLatPage * CH; c += 256) {
                int row = c / CH, chunk = c - row * CH;
                cp_async16(dst + swz_rt(row, chunk, dkp), src + (size_t)c * 8);
            }
        }
        cp_async_commit();
    };
    for (int it = 0; it < STAGES - 1; ++it) load_page(it);
    for (int c = tid; c < TILE * CH; c += 256) {
        int row = c / CH, chunk = c - row * CH;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (row < rows) v = *reinterpret_cast<const uint4*>(q + (row_base + row) * dk + chunk * 8);
        *reinterpret_cast<uint4*>(q_s + swz_rt(row, chunk, dkp)) = v;
    }
    __syncthreads();

    const int r_lo = lane >> 2, c_lo = (lane & 3) * 2;
    int pos_r[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) pos_r[h] = start + (r0 + g_row + warp * 16 + r_lo + h * 8) / heads;
    const int warp_last_pos = start + (r0 + g_row + warp * 16 + 15) / heads;
    float o[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[j][e] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const float sc = scale * kLog2e;
    const int KS = dkp >> 4;

    for (int it = 0; it < n_pages; ++it) {
        cp_async_wait<STAGES - 2>();
        __syncthreads();
        load_page(it + STAGES - 1);
        const bf16* kt = k_s + (size_t)(it % STAGES) * tile_elems;
        const int t0 = (first_page + it) * kLatPage;
        if (t0 > warp_last_pos || dv_here <= 0) continue;  // none of this warp's rows sees the page

#pragma unroll
        for (int half = 0; half < kLatPage / KH; ++half) {
            const int tk = t0 + half * KH;  // first key of this softmax step
            if (tk > warp_last_pos) break;
            float s[KB][4];
#pragma unroll
            for (int j = 0; j < KB; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) s[j][e] = 0.f;
            for (int kk = 0; kk < KS; kk += 2) {
                uint32_t qa0[4], qa1[4];
                ldmatrix_x4(qa0, q_s + swz_rt(g_row + warp * 16 + (lane & 15), kk * 2 + (lane >> 4), dkp));
                ldmatrix_x4(qa1, q_s + swz_rt(g_row + warp * 16 + (lane & 15), kk * 2 + 2 + (lane >> 4), dkp));
#pragma unroll
                for (int j = 0; j < KB; ++j) {
                    uint32_t b[4];
                    ldmatrix_x4(b, kt + swz_rt(half * KH + j * 8 + (lane & 7), kk * 2 + (lane >> 3), dkp));
                    mma_bf16(s[j], qa0, b[0], b[1]);
                    mma_bf16(s[j], qa1, b[2], b[3]);
                }
            }
            uint32_t pa[KB / 2][4];
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int j = 0; j < KB; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    int key = tk + j * 8 + c_lo + (e & 1);
                    float v = key <= pos_r[e >> 1] ? s[j][e] * sc : -INFINITY;
                    s[j][e] = v;
                    mx[e >> 1] = fmaxf(mx[e >> 1], v);
                }
            float alpha[2], base[2];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
                float mn = fmaxf(m_run[r], mx[r]);
                base[r] = mn == -INFINITY ? 0.f : mn;
                alpha[r] = exp2f(m_run[r] - base[r]);
                m_run[r] = mn;
            }
            float psum[2] = {0.f, 0.f};
#pragma unroll
            for (int j = 0; j < KB; ++j) {
                float p0v = exp2f(s[j][0] - base[0]), p1v = exp2f(s[j][1] - base[0]);
                float p2v = exp2f(s[j][2] - base[1]), p3v = exp2f(s[j][3] - base[1]);
                psum[0] += p0v + p1v;
                psum[1] += p2v + p3v;
                pa[j >> 1][(j & 1) * 2] = pack_bf16(p0v, p1v);
                pa[j >> 1][(j & 1) * 2 + 1] = pack_bf16(p2v, p3v);
            }
#pragma unroll
            for (int r = 0; r < 2; ++r) l_run[r] = l_run[r] * alpha[r] + psum[r];
#pragma unroll
            for (int jn = 0; jn < NT; ++jn)
#pragma unroll
                for (int e = 0; e < 4; ++e) o[jn][e] *= alpha[e >> 1];
#pragma unroll
            for (int ks = 0; ks < KB / 2; ++ks) {
#pragma unroll
                for (int jn = 0; jn < NT; jn += 2) {
                    if (jn * 8 < dv_here) {
                        uint32_t b[4];
                        ldmatrix_x4_trans(b, kt + swz_rt(half * KH + ks * 16 + (lane & 15), c0 + jn + (lane >> 4), dkp));
                        mma_bf16(o[jn], pa[ks], b[0], b[1]);
                        mma_bf16(o[jn + 1], pa[ks], b[2], b[3]);
                    }
                }
            }
        }
    }
    cp_async_wait<0>();
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    }
    const int ra = g_row + warp * 16 + r_lo, rb = ra + 8;
    if (n_splits == 1) {
        const float inv_a = l_run[0] > 0.f ? 1.0f / l_run[0] : 0.f;
        const float inv_b = l_run[1] > 0.f ? 1.0f / l_run[1] : 0.f;
#pragma unroll
        for (int jn = 0; jn < NT; ++jn) {
            int col = jn * 8 + c_lo;
            if (col < dv_here) {
                int gc = run * RUN + col;
                if (ra < rows)
                    *reinterpret_cast<uint32_t*>(out + (row_base + ra) * dv + gc) =
                        pack_bf16(o[jn][0] * inv_a, o[jn][1] * inv_a);
                if (rb < rows)
                    *reinterpret_cast<uint32_t*>(out + (row_base + rb) * dv + gc) =
                        pack_bf16(o[jn][2] * inv_b, o[jn][3] * inv_b);
            }
        }
    } else {
        // records in natural-logarithm terms: o and l are relative to exp(m)
        const float ln2 = 0.6931471805599453f;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            int r = h ? rb : ra;
            if (r >= rows || dv_here <= 0) continue;
            float* rec = partial + ((row_base + r) * n_splits + split) * (size_t)(dv + 2);
            if (run == 0 && (lane & 3) == 0) {
                rec[0] = l_run[h] > 0.f ? m_run[h] * ln2 : 0.f;
                rec[1] = l_run[h];
            }
#pragma unroll
            for (int jn = 0; jn < NT; ++jn) {
                int col = jn * 8 + c_lo;
                if (col < dv_here) {
                    int gc = run * RUN + col;
                    rec[2 + gc] = o[jn][h * 2];
                    rec[2 + gc + 1] = o[jn][h * 2 + 1];
                }
            }
        }
    }
}

}  // namespace nnis

using namespace nnis;

// The launch shape for output rows of dv values: runs of 128 values (dv <= 128) or 256, the
// groups of a CTA 64 rows each where one run covers dv (128 rows a CTA), else a run each.
static int latent_run_values(int dv) { return dv <= 128 ? 128 : 256; }
static int latent_tile_rows(int dv) { return dv <= 256 ? 2 * kLatRows : kLatRows; }

// Shared memory of the kernel for rows of dk values with `stages` pages in flight.
static size_t latent_mma_smem(int dk, int dv, int stages) {
    int dkp = (dk + 63) / 64 * 64;
    return (size_t)(latent_tile_rows(dv) + stages * kLatPage) * dkp * sizeof(bf16);
}

// 1 if the tensor-core kernel takes these sizes (else the kernel for any sizes runs)
NNIS_API int nnis_attention_latent_mma_takes(int dk, int dv, int page_size) {
    return dk > 0 && dk % 8 == 0 && dv > 0 && dv % 16 == 0 && dv <= dk && page_size == kLatPage &&
           latent_mma_smem(dk, dv, 2) <= 227 * 1024;
}

// stacked (token, head) rows of a CTA for output rows of dv values
NNIS_API int nnis_attention_latent_mma_tile_rows(int dv) { return latent_tile_rows(dv); }

// `tiles`: int32 [n_tiles, 2] = (sequence of the batch, first stacked row of the tile among
// the sequence's tokens * heads rows of this step), nnis_attention_latent_mma_tile_rows(dv)
// rows per tile, with the per-sequence first packed row, first position and token count; or
// null, and then every row of the step is one token of a sequence of its own (n_tokens
// rows, ceil(heads / tile rows) tiles each).
// `partial`: float32 [n_tokens * heads * n_splits * (dv + 2)] when n_splits > 1.
NNIS_API int nnis_attention_latent_mma(const void* q, const void* cache, const int* tiles, int n_tiles,
                                       const int* seq_first_row, const int* seq_start,
                                       const int* seq_count, const int* token_pos, const int* token_seq,
                                       const int* page_table, int table_cols, void* out, float* partial,
                                       int n_tokens, int heads, int dk, int dv, int page_size,
                                       float scale, int n_splits, cudaStream_t stream) {
    if (n_tokens <= 0 || heads <= 0 || table_cols <= 0 || n_splits <= 0 || !q || !cache || !out ||
        !page_table)
        return NNIS_ERR_ARGUMENT;
    if (!nnis_attention_latent_mma_takes(dk, dv, page_size)) return NNIS_ERR_UNSUPPORTED;
    if (tiles ? (n_tiles <= 0 || !seq_first_row || !seq_start || !seq_count) : (!token_pos || !token_seq))
        return NNIS_ERR_ARGUMENT;
    if (n_splits > 1 && !partial) return NNIS_ERR_ARGUMENT;
    if (((uintptr_t)q | (uintptr_t)cache | (uintptr_t)out) % 16) return NNIS_ERR_ALIGNMENT;
    const int dkp = (dk + 63) / 64 * 64;
    const int tile_rows = latent_tile_rows(dv), run = latent_run_values(dv);
    const int tiles_per_token = (heads + tile_rows - 1) / tile_rows;
    const int runs = (dv + run - 1) / run;
    const bool split_rows = runs == 1;
    if (n_splits > 64) return NNIS_ERR_UNSUPPORTED;
    dim3 grid(tiles ? n_tiles : n_tokens * tiles_per_token, split_rows ? 1 : (runs + 1) / 2, n_splits);
    const int stages = latent_mma_smem(dk, dv, 3) <= 200 * 1024 ? 3 : 2;
    const size_t smem = latent_mma_smem(dk, dv, stages);
    using Kernel = void (*)(const bf16*, const bf16*, const int*, const int*, const int*, const int*, const int*,
                            const int*, const int*, int, bf16*, float*, int, int, int, int, int, float, int);
    Kernel kernel;
    if (run == 128) kernel = stages == 3 ? latent_mma_kernel<3, 16, true> : latent_mma_kernel<2, 16, true>;
    else if (split_rows) kernel = stages == 3 ? latent_mma_kernel<3, 32, true> : latent_mma_kernel<2, 32, true>;
    else kernel = stages == 3 ? latent_mma_kernel<3, 32, false> : latent_mma_kernel<2, 32, false>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    cudaError_t e = launch_dependent(kernel, grid, 256, smem, stream, (const bf16*)q, (const bf16*)cache, tiles,
                                     seq_first_row, seq_start, seq_count, token_pos, token_seq, page_table,
                                     table_cols, (bf16*)out, partial, heads, dk, dv, dkp, tiles_per_token, scale,
                                     n_splits);
    if (e != cudaSuccess) return (int)e;
    if (n_splits > 1) {
        size_t rows = (size_t)n_tokens * heads;
        e = launch_dependent(attn_merge_kernel<bf16>, (unsigned)rows, 128, 0, stream, (const float*)partial,
                             (bf16*)out, rows, dv, n_splits);
    }
    return e == cudaSuccess ? NNIS_OK : (int)e;
}
