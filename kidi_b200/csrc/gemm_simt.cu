// y[M,N] = x[M,K] * W[N,K]^T with 32-bit multiply-add on the CUDA cores.
//
// This is the true 32-bit matrix product (no reduced-precision matrix mode) and the
// fallback for shapes the tensor-core kernels refuse. Every output element is one
// chain of fused multiply-adds over ascending k that starts from zero, so a row's
// result does not depend on how many other rows share the launch or on where the
// row falls in a tile. The reference's Linear is y = x W^T with W stored [out, in]
// (src/kidi/layers/linear.cpp:98-101,181-190).
#include "common.cuh"

namespace {
constexpr int TILE = 64;     // output tile is TILE x TILE
constexpr int TILE_K = 16;
constexpr int PAD = 4;

template <typename TX, typename TW, typename TY>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const TX* __restrict__ x, const TW* __restrict__ w, TY* __restrict__ y, int M, int N, int K,
                 long long ldx, long long ldw, long long ldy, const float* __restrict__ bias) {
    __shared__ float xs[TILE_K][TILE + PAD];
    __shared__ float ws[TILE_K][TILE + PAD];
    const int tx = threadIdx.x & 15;   // 4 output columns (n) each
    const int ty = threadIdx.x >> 4;   // 4 output rows (m) each
    const int m0 = blockIdx.y * TILE, n0 = blockIdx.x * TILE;
    const int load_row = threadIdx.x >> 2;         // 0..63
    const int load_k = (threadIdx.x & 3) * 4;      // 0,4,8,12
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += TILE_K) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int k = k0 + load_k + j;
            const int m = m0 + load_row, n = n0 + load_row;
            xs[load_k + j][load_row] = (m < M && k < K) ? to_float(x[m * ldx + k]) : 0.f;
            ws[load_k + j][load_row] = (n < N && k < K) ? to_float(w[n * ldw + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < TILE_K; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = xs[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n < N) y[m * ldy + n] = from_float<TY>(bias ? acc[i][j] + bias[n] : acc[i][j]);
        }
    }
}

template <typename TX, typename TW, typename TY>
int launch(const void* x, const void* w, void* y, int M, int N, int K, long long ldx, long long ldw, long long ldy,
           const float* bias, cudaStream_t stream) {
    dim3 grid((N + TILE - 1) / TILE, (M + TILE - 1) / TILE);
    return kidi_launch(gemm_simt_kernel<TX, TW, TY>, grid, 256, 0, stream, (const TX*)x, (const TW*)w, (TY*)y, M, N, K,
                       ldx, ldw, ldy, bias);
}
}  // namespace

// `bias` (float32 [N], or null) is added to every row after the chain of multiply-adds
// (the reference's Linear with bias, src/kidi/layers/linear.cpp:181-190).
KIDI_API int kidi_gemm_simt(const void* x, int x_dtype, const void* w, int w_dtype, void* y, int y_dtype, int M, int N,
                            int K, long long ldx, long long ldw, long long ldy, const float* bias, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || (M + TILE - 1) / TILE > 65535) return KIDI_REFUSED_SIZE;
#define KIDI_CASE(X, TX, W, TW, Y, TY)                                 \
    if (x_dtype == X && w_dtype == W && y_dtype == Y)                  \
        return launch<TX, TW, TY>(x, w, y, M, N, K, ldx, ldw, ldy, bias, stream);
    KIDI_CASE(KIDI_F32, float, KIDI_F32, float, KIDI_F32, float)
    KIDI_CASE(KIDI_F32, float, KIDI_F32, float, KIDI_BF16, bf16)
    KIDI_CASE(KIDI_F32, float, KIDI_BF16, bf16, KIDI_F32, float)
    KIDI_CASE(KIDI_F32, float, KIDI_BF16, bf16, KIDI_BF16, bf16)
    KIDI_CASE(KIDI_BF16, bf16, KIDI_F32, float, KIDI_F32, float)
    KIDI_CASE(KIDI_BF16, bf16, KIDI_F32, float, KIDI_BF16, bf16)
    KIDI_CASE(KIDI_BF16, bf16, KIDI_BF16, bf16, KIDI_F32, float)
    KIDI_CASE(KIDI_BF16, bf16, KIDI_BF16, bf16, KIDI_BF16, bf16)
#undef KIDI_CASE
    return KIDI_REFUSED_DTYPE;
}
