// Products of one small matrix per head: C[b][M, N] = A[b][M, K] . W[b][N, K]^T for
// b = 0 .. batch - 1, where the heads' slices of A and C lie side by side in packed
// rows (row strides lda / ldc, head strides a_bs / c_bs in elements) and W[b] are
// consecutive [N, K] matrices.  Latent attention uses it twice: to carry the
// queries into the latent space (W = the keys' up-projection, transposed per head at
// load) and to carry the attention's latent output to the heads' values.
// Operands float32 or bfloat16, float32 accumulation with fmaf on the CUDA cores
// (the float32 path, and the bfloat16 path of shapes the tensor-core kernel refuses).
#include "async_copy.cuh"
#include "common.cuh"

namespace nnis {

template <typename T>
__global__ void __launch_bounds__(256)
batched_linear_kernel(const T* __restrict__ A, long long lda, long long a_bs,
                      const T* __restrict__ W, T* __restrict__ C, long long ldc, long long c_bs,
                      int M, int N, int K) {
    constexpr int BM = 64, BN = 64, BK = 16, PAD = 4;
    __shared__ __align__(16) float As[BK][BM + PAD];
    __shared__ __align__(16) float Ws[BK][BN + PAD];
    int b = blockIdx.z;
    A += (size_t)b * a_bs;
    C += (size_t)b * c_bs;
    W += (size_t)b * N * K;
    int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    int lr = tid >> 2, lk = (tid & 3) * 4;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            int gk = k0 + lk + i;
            As[lk + i][lr] = (m0 + lr < M && gk < K) ? to_float(A[(size_t)(m0 + lr) * lda + gk]) : 0.f;
            Ws[lk + i][lr] = (n0 + lr < N && gk < K) ? to_float(W[(size_t)(n0 + lr) * K + gk]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float4 av = *reinterpret_cast<const float4*>(&As[k][ty * 4]);
            float4 wv = *reinterpret_cast<const float4*>(&Ws[k][tx * 4]);
            float ar[4] = {av.x, av.y, av.z, av.w}, wr[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(ar[i], wr[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int n = n0 + tx * 4 + j;
            if (n < N) C[(size_t)m * ldc + n] = from_float<T>(acc[i][j]);
        }
    }
}

// Few rows (decoding): a warp per output column of a head, all rows of a tile of
// up to eight at once, so that a weight row is read once per tile.
template <typename T>
__global__ void __launch_bounds__(256)
batched_rows_kernel(const T* __restrict__ A, long long lda, long long a_bs, const T* __restrict__ W,
                    T* __restrict__ C, long long ldc, long long c_bs, int M, int N, int K) {
    pdl_wait();
    pdl_launch_dependents();
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int n = blockIdx.x * 8 + warp, b = blockIdx.z, m0 = blockIdx.y * 8;
    if (n >= N) return;
    const T* wrow = W + ((size_t)b * N + n) * K;
    const T* a = A + (size_t)b * a_bs;
    float acc[8] = {};
    if (sizeof(T) == 2 && K % 8 == 0 && lda % 8 == 0 && a_bs % 8 == 0 &&
        (((uintptr_t)A | (uintptr_t)W) & 15) == 0) {
        // bfloat16 rows on 16-byte boundaries: eight values a load
        for (int k = lane * 8; k < K; k += 256) {
            uint4 wv = *reinterpret_cast<const uint4*>(wrow + k);
            const uint32_t ws[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                if (m0 + i < M) {
                    uint4 xv = *reinterpret_cast<const uint4*>(a + (size_t)(m0 + i) * lda + k);
                    const uint32_t xs[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        acc[i] = fmaf(__uint_as_float(xs[j] << 16), __uint_as_float(ws[j] << 16), acc[i]);
                        acc[i] = fmaf(__uint_as_float(xs[j] & 0xffff0000u), __uint_as_float(ws[j] & 0xffff0000u), acc[i]);
                    }
                }
            }
        }
    } else {
        for (int k = lane; k < K; k += 32) {
            float w = to_float(wrow[k]);
#pragma unroll
            for (int i = 0; i < 8; ++i)
                if (m0 + i < M) acc[i] = fmaf(to_float(a[(size_t)(m0 + i) * lda + k]), w, acc[i]);
        }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        float v = warp_sum(acc[i]);
        if (lane == 0 && m0 + i < M) C[(size_t)(m0 + i) * ldc + (size_t)b * c_bs + n] = from_float<T>(v);
    }
}

template <typename T>
static int launch_batched(const void* A, long long lda, long long a_bs, const void* W, void* C,
                          long long ldc, long long c_bs, int batch, int M, int N, int K,
                          cudaStream_t stream) {
    if (M <= 16) {
        dim3 grid((N + 7) / 8, (M + 7) / 8, batch);
        cudaError_t e = launch_dependent(batched_rows_kernel<T>, grid, 256, 0, stream, (const T*)A, lda, a_bs,
                                         (const T*)W, (T*)C, ldc, c_bs, M, N, K);
        return e == cudaSuccess ? NNIS_OK : (int)e;
    } else {
        dim3 grid((N + 63) / 64, (M + 63) / 64, batch);
        if (grid.y > 65535u) return NNIS_ERR_UNSUPPORTED;
        batched_linear_kernel<T><<<grid, 256, 0, stream>>>((const T*)A, lda, a_bs, (const T*)W,
                                                           (T*)C, ldc, c_bs, M, N, K);
    }
    NNIS_RETURN_LAUNCH();
}

}  // namespace nnis

NNIS_API int nnis_batched_linear(const void* A, long long lda, long long a_bs, const void* W, void* C,
                                 long long ldc, long long c_bs, int batch, int M, int N, int K,
                                 int dtype, cudaStream_t stream) {
    if (!A || !W || !C || batch <= 0 || M <= 0 || N <= 0 || K <= 0 || batch > 65535)
        return NNIS_ERR_ARGUMENT;
    if (dtype == NNIS_DTYPE_F32)
        return nnis::launch_batched<float>(A, lda, a_bs, W, C, ldc, c_bs, batch, M, N, K, stream);
    if (dtype == NNIS_DTYPE_BF16)
        return nnis::launch_batched<nnis::bf16>(A, lda, a_bs, W, C, ldc, c_bs, batch, M, N, K, stream);
    return NNIS_ERR_UNSUPPORTED;
}
