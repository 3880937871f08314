// y[M,N] = x[M,K] * W[N,K]^T in bfloat16 for few rows (M <= 64): the decode step's
// matrix products, which are bound by reading W once from HBM.
//
// The weight matrix is the "M" operand of the tensor-core instruction (16 weight rows
// per tile) and the batch is its "N" operand (8 batch rows per tile), so that no lane
// multiplies padding when the batch is small. Every lane loads 16 contiguous bytes of a
// weight row and 16 contiguous bytes of a batch row straight from global memory into
// the registers the instruction wants: within a 32-wide slice of k the four lanes of a
// quad hold k = 8t..8t+7 instead of the instruction's nominal {2t,2t+1,2t+8,2t+9};
// a dot product does not care in which order k runs as long as both operands agree.
// A block of eight warps owns one tile of weight rows; the warps split k between them
// and their partial sums are added in warp order through shared memory (a fixed order:
// the result does not depend on timing). Accumulation is 32-bit.
//
// Epilogues: plain store (bfloat16 or float32), or the SiLU gate of a fused
// [gate | up] projection, out = silu(gate) * up, for which a block reads the 16 gate
// rows and the 16 matching up rows.
#include "common.cuh"

namespace {

constexpr int WARPS = 8;

__device__ __forceinline__ uint4 load_streaming(const void* pointer) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(pointer));
    return v;
}

__device__ __forceinline__ void mma_bf16(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                         unsigned b0, unsigned b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// MT: tiles of 16 weight rows per block; NT: tiles of 8 batch rows; UNROLL: 32-wide k
// slices in flight per warp. GATED with MT == 2: tile 0 = 16 gate rows, tile 1 = the 16
// matching up rows. GATED with MT == 1: rows 0..7 of the tile are 8 gate rows and rows
// 8..15 the 8 matching up rows (twice the blocks, each with the deeper prefetch of the
// one-tile form: measured faster at one batch row).
template <int MT, int NT, int UNROLL, bool GATED, typename TY>
__global__ void __launch_bounds__(WARPS * 32)
gemm_skinny_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w, TY* __restrict__ y, int M, int N, int K,
                   long long ldx, long long ldw, long long ldy, const float* __restrict__ bias) {
    extern __shared__ float partial[];  // [WARPS][MT*16][NT*8]
    constexpr int ROWS = MT * 16, COLS = NT * 8;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    // Output features of this block: [n0, n0 + span). For the gated form N is the width
    // of the result (the weight has 2N rows: N gate rows, then N up rows).
    const int span = GATED ? (MT == 1 ? 8 : 16) : ROWS;
    const int n0 = blockIdx.x * span;

    const bf16* weight_row[MT][2];
    bool weight_ok[MT][2];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const bool up = GATED && (MT == 1 ? h == 1 : mt == 1);       // an up row: N rows further down
            const int local = GATED ? (MT == 1 ? g : g + 8 * h) : mt * 16 + g + 8 * h;
            const int feature = n0 + local;
            weight_ok[mt][h] = feature < N;
            const long long row = (up ? (long long)N : 0) + (weight_ok[mt][h] ? feature : 0);
            weight_row[mt][h] = w + row * ldw;
        }
    const bf16* batch_row[NT];
    bool batch_ok[NT];
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        const int m = j * 8 + g;
        batch_ok[j] = m < M;
        batch_row[j] = x + (long long)(batch_ok[j] ? m : 0) * ldx;
    }

    float acc[MT][NT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[mt][j][i] = 0.f;

    const int slices = (K + 31) >> 5;
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    uint4 a[UNROLL][MT][2], b[UNROLL][NT];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
        const int k = ((warp + u * WARPS) << 5) + 8 * t;
        const bool ok = k + 8 <= K;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int h = 0; h < 2; ++h)
                a[u][mt][h] = (ok && weight_ok[mt][h]) ? load_streaming(weight_row[mt][h] + k) : zero;
    }
    for (int first = warp; first < slices; first += WARPS * UNROLL) {
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int k = ((first + u * WARPS) << 5) + 8 * t;
            const bool ok = k + 8 <= K;  // also false for slices beyond the last
            if (first != warp) {
#pragma unroll
                for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                    for (int h = 0; h < 2; ++h)
                        a[u][mt][h] = (ok && weight_ok[mt][h]) ? load_streaming(weight_row[mt][h] + k) : zero;
            }
#pragma unroll
            for (int j = 0; j < NT; ++j)
                b[u][j] = (ok && batch_ok[j]) ? __ldg(reinterpret_cast<const uint4*>(batch_row[j] + k)) : zero;
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u)
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int j = 0; j < NT; ++j) {
                    mma_bf16(acc[mt][j], a[u][mt][0].x, a[u][mt][1].x, a[u][mt][0].y, a[u][mt][1].y, b[u][j].x,
                             b[u][j].y);
                    mma_bf16(acc[mt][j], a[u][mt][0].z, a[u][mt][1].z, a[u][mt][0].w, a[u][mt][1].w, b[u][j].z,
                             b[u][j].w);
                }
    }

    float* mine = partial + (long long)warp * ROWS * COLS;
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            const int col = j * 8 + 2 * t;
            mine[(mt * 16 + g) * COLS + col] = acc[mt][j][0];
            mine[(mt * 16 + g) * COLS + col + 1] = acc[mt][j][1];
            mine[(mt * 16 + g + 8) * COLS + col] = acc[mt][j][2];
            mine[(mt * 16 + g + 8) * COLS + col + 1] = acc[mt][j][3];
        }
    __syncthreads();

    // Thread i -> (batch row m, feature r): consecutive threads write consecutive features.
    for (int i = threadIdx.x; i < span * COLS; i += WARPS * 32) {
        const int m = i / span, r = i - m * span;
        if (m >= M || n0 + r >= N) continue;
        float sum = 0.f;
#pragma unroll
        for (int v = 0; v < WARPS; ++v) sum += partial[((long long)v * ROWS + r) * COLS + m];
        if (GATED) {
            float up = 0.f;
#pragma unroll
            for (int v = 0; v < WARPS; ++v) up += partial[((long long)v * ROWS + (MT == 1 ? 8 : 16) + r) * COLS + m];
            sum = sum / (1.0f + expf(-sum)) * up;
        } else if (bias) {
            sum += bias[n0 + r];
        }
        y[m * ldy + n0 + r] = from_float<TY>(sum);
    }
}

template <int MT, int NT, int UNROLL, bool GATED, typename TY>
int launch(const void* x, const void* w, void* y, int M, int N, int K, long long ldx, long long ldw, long long ldy,
           const float* bias, cudaStream_t stream) {
    const int span = GATED ? (MT == 1 ? 8 : 16) : MT * 16;
    const size_t shared = (size_t)WARPS * MT * 16 * NT * 8 * sizeof(float);
    auto kernel = gemm_skinny_kernel<MT, NT, UNROLL, GATED, TY>;
    if (shared > 48 * 1024) {
        cudaError_t status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
        if (status != cudaSuccess) return (int)status;
    }
    return kidi_launch(kernel, (N + span - 1) / span, WARPS * 32, shared, stream, (const bf16*)x, (const bf16*)w,
                       (TY*)y, M, N, K, ldx, ldw, ldy, bias);
}

template <int MT, bool GATED, typename TY>
int by_batch(const void* x, const void* w, void* y, int M, int N, int K, long long ldx, long long ldw, long long ldy,
             const float* bias, cudaStream_t stream) {
    if (M <= 8) return launch<MT, 1, (MT == 1 ? 8 : 4), GATED, TY>(x, w, y, M, N, K, ldx, ldw, ldy, bias, stream);
    if (M <= 16) return launch<MT, 2, (MT == 1 ? 8 : 4), GATED, TY>(x, w, y, M, N, K, ldx, ldw, ldy, bias, stream);
    if (M <= 32) return launch<MT, 4, (MT == 1 ? 4 : 2), GATED, TY>(x, w, y, M, N, K, ldx, ldw, ldy, bias, stream);
    return launch<MT, 8, 2, GATED, TY>(x, w, y, M, N, K, ldx, ldw, ldy, bias, stream);
}
}  // namespace

// Requirements (checked here; the caller falls back to another kernel otherwise):
// M in [1, 64]; K a multiple of 8; x, w rows 16-byte aligned (leading dimensions
// multiples of 8 and base pointers 16-byte aligned).
// gated != 0: w is [2N, K] (N gate rows then N up rows), y is [M, N] = silu(gate) * up.
// row_tiles: 1 or 2 tiles of 16 weight rows per block (the gated form uses 2).
// bias: float32 [N] added to every row, or null (not with the gate).
KIDI_API int kidi_gemm_skinny(const void* x, const void* w, void* y, int y_dtype, int M, int N, int K, long long ldx,
                              long long ldw, long long ldy, int gated, int row_tiles, const float* bias,
                              cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M > 64 || K <= 0 || (K & 7) || (ldx & 7) || (ldw & 7) || ((uintptr_t)x & 15) || ((uintptr_t)w & 15))
        return KIDI_REFUSED_SIZE;
    if (gated) {
        if (y_dtype != KIDI_BF16) return KIDI_REFUSED_DTYPE;
        if (bias) return KIDI_REFUSED_SIZE;
        // Up to seven batch rows: eight gate and eight up rows per tile (measured on the 201 MB
        // gate/up weight of the benchmark's model: 32.7 against 35.6 us at one row, 36.7 against
        // 38.1 at six, equal at eight); more rows: sixteen and sixteen.
        if (row_tiles == 1 || (M < 8 && row_tiles != 2))
            return by_batch<1, true, bf16>(x, w, y, M, N, K, ldx, ldw, ldy, bias, stream);
        return by_batch<2, true, bf16>(x, w, y, M, N, K, ldx, ldw, ldy, bias, stream);
    }
    if (y_dtype == KIDI_BF16)
        return row_tiles == 2 ? by_batch<2, false, bf16>(x, w, y, M, N, K, ldx, ldw, ldy, bias, stream)
                              : by_batch<1, false, bf16>(x, w, y, M, N, K, ldx, ldw, ldy, bias, stream);
    if (y_dtype == KIDI_F32)
        return row_tiles == 2 ? by_batch<2, false, float>(x, w, y, M, N, K, ldx, ldw, ldy, bias, stream)
                              : by_batch<1, false, float>(x, w, y, M, N, K, ldx, ldw, ldy, bias, stream);
    return KIDI_REFUSED_DTYPE;
}
