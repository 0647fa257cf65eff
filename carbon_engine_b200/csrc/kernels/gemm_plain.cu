// y = x * W^T with float32 FMA arithmetic: the matrix product of the float32 path, and the plain
// twin (and odd-size fallback) of the tensor-core products.
//
// x is [M, K], W is [N, K] (a linear layer's weight as stored, src/model/layers.rs:441), both
// row-major.  Every output element is one thread's running sum over k = 0, 1, 2, ... in that order,
// so a token's result does not depend on M, on the tile it falls in, or on its neighbours.  No
// tensor-core instruction and no reduced-precision mode is involved.
//
// Epilogues: store (in the activation dtype or float32), add into the float32 residual stream, or
// SwiGLU, where W holds the gate rows [0, N) and the up rows [N, 2N) and the output is
// silu(gate) * up (src/model/layers.rs:625-648).
#include "common.cuh"

#define GP_BM 64
#define GP_BN 64
#define GP_BK 16

enum { GP_STORE = 0, GP_STORE_F32 = 1, GP_ACCUM_F32 = 2, GP_SWIGLU = 3 };

template <typename T, int MODE>
__global__ void __launch_bounds__(256) gemm_plain_kernel(const T* __restrict__ A, const T* __restrict__ W,
                                                         void* __restrict__ Cv, int M, int N, int K, int lda, int ldc) {
    ce_pdl_begin();
    constexpr int NW = MODE == GP_SWIGLU ? 2 : 1;
    __shared__ float As[GP_BK][GP_BM + 1];
    __shared__ float Ws[NW][GP_BK][GP_BN + 1];
    int tid = threadIdx.x;
    int m0 = blockIdx.y * GP_BM, n0 = blockIdx.x * GP_BN;
    int tm = (tid / 16) * 4, tn = (tid % 16) * 4;
    float acc[NW][4][4];
#pragma unroll
    for (int w = 0; w < NW; ++w)
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[w][i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += GP_BK) {
        for (int e = tid; e < GP_BM * GP_BK; e += 256) {
            int r = e / GP_BK, c = e % GP_BK;
            int gm = m0 + r, gk = k0 + c;
            As[c][r] = (gm < M && gk < K) ? CeType<T>::load(A + (size_t)gm * lda + gk) : 0.f;
            int gn = n0 + r;
#pragma unroll
            for (int w = 0; w < NW; ++w)
                Ws[w][c][r] = (gn < N && gk < K) ? CeType<T>::load(W + ((size_t)w * N + gn) * K + gk) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < GP_BK; ++kk) {
            float av[4], wv[NW][4];
#pragma unroll
            for (int i = 0; i < 4; ++i) av[i] = As[kk][tm + i];
#pragma unroll
            for (int w = 0; w < NW; ++w)
#pragma unroll
                for (int j = 0; j < 4; ++j) wv[w][j] = Ws[w][kk][tn + j];
#pragma unroll
            for (int w = 0; w < NW; ++w)
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) acc[w][i][j] = fmaf(av[i], wv[w][j], acc[w][i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        int gm = m0 + tm + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int gn = n0 + tn + j;
            if (gn >= N) continue;
            size_t o = (size_t)gm * ldc + gn;
            if (MODE == GP_STORE) {
                CeType<T>::store((T*)Cv + o, acc[0][i][j]);
            } else if (MODE == GP_STORE_F32) {
                ((float*)Cv)[o] = acc[0][i][j];
            } else if (MODE == GP_ACCUM_F32) {
                ((float*)Cv)[o] += acc[0][i][j];
            } else {
                float g = acc[0][i][j], u = acc[NW - 1][i][j];
                CeType<T>::store((T*)Cv + o, g / (1.0f + expf(-g)) * u);
            }
        }
    }
}

template <typename T>
static int launch_plain(const void* A, const void* W, void* C, int M, int N, int K, int lda, int ldc, int mode,
                        cudaStream_t stream) {
    dim3 grid((N + GP_BN - 1) / GP_BN, (M + GP_BM - 1) / GP_BM);
    switch (mode) {
        case GP_STORE: { ce_note("gemm_plain_kernel"); ce_launch(gemm_plain_kernel<T, GP_STORE>, grid, 256, 0, stream, (const T*)A, (const T*)W, C, M, N, K, lda, ldc); } break;
        case GP_STORE_F32: { ce_note("gemm_plain_kernel"); ce_launch(gemm_plain_kernel<T, GP_STORE_F32>, grid, 256, 0, stream, (const T*)A, (const T*)W, C, M, N, K, lda, ldc); } break;
        case GP_ACCUM_F32: { ce_note("gemm_plain_kernel"); ce_launch(gemm_plain_kernel<T, GP_ACCUM_F32>, grid, 256, 0, stream, (const T*)A, (const T*)W, C, M, N, K, lda, ldc); } break;
        case GP_SWIGLU: { ce_note("gemm_plain_kernel"); ce_launch(gemm_plain_kernel<T, GP_SWIGLU>, grid, 256, 0, stream, (const T*)A, (const T*)W, C, M, N, K, lda, ldc); } break;
        default: return ce_fail(CE_ERR_ARG, "ce_gemm_plain: unknown epilogue %d", mode);
    }
    return ce_check_launch("ce_gemm_plain");
}

// N is the number of output columns (for SwiGLU: the intermediate width, W having 2N rows).
extern "C" int ce_gemm_plain(const void* A, const void* W, void* C, int dtype, int M, int N, int K, int lda, int ldc,
                             int mode, cudaStream_t stream) {
    if (M == 0 || N == 0) return CE_OK;
    if (!A || !W || !C) return ce_fail(CE_ERR_ARG, "ce_gemm_plain: null pointer");
    if (K <= 0) return ce_fail(CE_ERR_SIZE, "ce_gemm_plain: K=%d", K);
    if ((M + GP_BM - 1) / GP_BM > 65535) return ce_fail(CE_ERR_SIZE, "ce_gemm_plain: M=%d is too large", M);
    if (dtype == CE_F32) return launch_plain<float>(A, W, C, M, N, K, lda, ldc, mode, stream);
    if (dtype == CE_BF16) return launch_plain<__nv_bfloat16>(A, W, C, M, N, K, lda, ldc, mode, stream);
    return ce_fail(CE_ERR_ARG, "ce_gemm_plain: unknown dtype %d", dtype);
}
