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
// Epilogues: plain store (bfloat16 or float32, with an optional bias), or the SiLU gate of
// a fused [gate | up] projection, out = silu(gate) * up, for which a block reads the 16
// gate rows and the 16 matching up rows.
//
// Two more epilogues take the RMSNorm between two products out of the step (a norm of its
// own is a launch that moves 64 KB). The product BEFORE a norm ("into the residual") does
// not store y: it adds y to the 32-bit residual stream in place, stores the new residual
// times the norm's weight in bfloat16 (not yet normalised) and, per batch row, the sum of
// squares of the new residual over the block's features. The product AFTER the norm
// ("row factors") multiplies each batch row of its result by 1 / sqrt(mean square + eps),
// for which it adds the row's parts up in block order: x W^T scaled by a factor per row is
// (factor * x) W^T. Sums, squares and factors are 32-bit; the order of every sum is fixed.
#include "common.cuh"

namespace {

constexpr int WARPS = 8;

struct Epilogue {
    const float* bias;            // [N] added to every row, or null (not with the gate)
    // Row factors (the product after a norm): parts[m * factor_stride + b], b < factor_count, are the
    // parts of row m's sum of squares; the row's result is multiplied by 1 / sqrt(sum / factor_width + eps).
    const float* factor_parts;    // null: no factors
    int factor_count, factor_stride, factor_width;
    float factor_eps;
    // Into the residual (the product before a norm; y is not stored): residual[m, n] += y[m, n] (+ bias),
    // normed[m, n] = residual[m, n] * norm_weight[n], parts_out[m * parts_stride + block] = the sum of
    // squares of the new residual[m, :] over this block's features.
    float* residual;              // null: the plain store
    long long ld_residual;
    const void* norm_weight;
    int norm_weight_is_float;
    bf16* normed;
    long long ld_normed;
    float* parts_out;
    int parts_stride;
};

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
// one-tile form: measured faster up to eight batch rows, 36.9 against 38.2 us for the
// 8B layer's gate and up at 8 rows).
// MODE (compile time, so that the plain product carries none of it): bit 0: row factors, bit 1: into
// the residual (see Epilogue).
// W: warps of a block (8, or 4: blocks half as heavy, of which twice as many fit an SM: for weights
// whose tiles are more than one round of 8-warp blocks and at most one of 4-warp blocks).
template <int MT, int NT, int UNROLL, bool GATED, typename TY, int MODE, int W>
__global__ void __launch_bounds__(W * 32)
gemm_skinny_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w, TY* __restrict__ y, int M, int N, int K,
                   long long ldx, long long ldw, long long ldy, const Epilogue e) {
    extern __shared__ float partial[];  // [W][MT*16][NT*8]
    __shared__ float row_factor[NT * 8];
    constexpr bool FACTORS = (MODE & 1) != 0, RESIDUAL = (MODE & 2) != 0 && !GATED;
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

    // This thread's element of the residual stream and its norm weight are asked for now, before
    // the weights are streamed, not at the block's end where nothing would hide the wait (the
    // first pass of the epilogue's loop; later passes, which only more than 16 batch rows have,
    // load late).
    float early_residual = 0.f, early_weight = 0.f;
    if (RESIDUAL && threadIdx.x < span * COLS) {
        const int m = threadIdx.x / span, r = threadIdx.x - m * span;
        if (m < M && n0 + r < N) {
            early_residual = e.residual[(long long)m * e.ld_residual + n0 + r];
            early_weight = e.norm_weight_is_float ? ((const float*)e.norm_weight)[n0 + r]
                                                  : to_float(((const bf16*)e.norm_weight)[n0 + r]);
        }
    }
    const int slices = (K + 31) >> 5;
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    uint4 a[UNROLL][MT][2], b[UNROLL][NT];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
        const int k = ((warp + u * W) << 5) + 8 * t;
        const bool ok = k + 8 <= K;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int h = 0; h < 2; ++h)
                a[u][mt][h] = (ok && weight_ok[mt][h]) ? load_streaming(weight_row[mt][h] + k) : zero;
    }
    if (FACTORS) {
        // Behind the first weight rows, which are on their way: a warp per batch row, lane l takes parts
        // l, l + 32, ... in order, eight loads in flight at a time (one trip to the L2 while the
        // weights come from further away), then the lanes' sums in a fixed tree.
        for (int m = warp; m < M; m += W) {
            const float* parts = e.factor_parts + (long long)m * e.factor_stride;
            float square = 0.f;
            for (int base = 0; base < e.factor_count; base += 8 * 32) {
                float part[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int b = base + i * 32 + lane;
                    part[i] = b < e.factor_count ? __ldcg(parts + b) : 0.f;
                }
#pragma unroll
                for (int i = 0; i < 8; ++i) square += part[i];
            }
            square = warp_sum(square);
            if (lane == 0) row_factor[m] = 1.0f / sqrtf(square / (float)e.factor_width + e.factor_eps);
        }
    }
    for (int first = warp; first < slices; first += W * UNROLL) {
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int k = ((first + u * W) << 5) + 8 * t;
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
    for (int i = threadIdx.x; i < span * COLS; i += W * 32) {
        const int m = i / span, r = i - m * span;
        const bool inside = m < M && n0 + r < N;
        float sum = 0.f;
#pragma unroll
        for (int v = 0; v < W; ++v) sum += partial[((long long)v * ROWS + r) * COLS + m];
        if (FACTORS && m < M) sum *= row_factor[m];
        if (GATED) {
            float up = 0.f;
#pragma unroll
            for (int v = 0; v < W; ++v) up += partial[((long long)v * ROWS + (MT == 1 ? 8 : 16) + r) * COLS + m];
            if (FACTORS && m < M) up *= row_factor[m];
            sum = sum / (1.0f + expf(-sum)) * up;
        } else if (e.bias && inside) {
            sum += e.bias[n0 + r];
        }
        if (RESIDUAL) {
            // span (16 or 32) consecutive lanes hold one batch row's features of this block.
            float value = 0.f;
            if (inside) {
                float* at = e.residual + (long long)m * e.ld_residual + n0 + r;
                const bool first = i == (int)threadIdx.x;            // loaded before the weights were streamed
                value = (first ? early_residual : *at) + sum;
                *at = value;
                const float weight = first ? early_weight
                                     : e.norm_weight_is_float ? ((const float*)e.norm_weight)[n0 + r]
                                                              : to_float(((const bf16*)e.norm_weight)[n0 + r]);
                e.normed[(long long)m * e.ld_normed + n0 + r] = from_float<bf16>(value * weight);
            }
            float square = value * value;
#pragma unroll
            for (int offset = span / 2; offset > 0; offset >>= 1) square += __shfl_xor_sync(0xffffffffu, square, offset);
            if (r == 0 && m < M) e.parts_out[(long long)m * e.parts_stride + blockIdx.x] = square;
        } else if (inside) {
            y[m * ldy + n0 + r] = from_float<TY>(sum);
        }
    }
}

template <int MT, int NT, int UNROLL, bool GATED, typename TY, int MODE = 0, int W = WARPS>
int launch(const void* x, const void* w, void* y, int M, int N, int K, long long ldx, long long ldw, long long ldy,
           const Epilogue& e, cudaStream_t stream) {
    const int span = GATED ? (MT == 1 ? 8 : 16) : MT * 16;
    const size_t shared = (size_t)W * MT * 16 * NT * 8 * sizeof(float);
    auto kernel = gemm_skinny_kernel<MT, NT, UNROLL, GATED, TY, MODE, W>;
    if (shared > 48 * 1024) {
        cudaError_t status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
        if (status != cudaSuccess) return (int)status;
    }
    return kidi_launch(kernel, (N + span - 1) / span, W * 32, shared, stream, (const bf16*)x, (const bf16*)w,
                       (TY*)y, M, N, K, ldx, ldw, ldy, e);
}

template <int MT, bool GATED, typename TY>
int by_batch(const void* x, const void* w, void* y, int M, int N, int K, long long ldx, long long ldw, long long ldy,
             const Epilogue& e, cudaStream_t stream) {
    if (M <= 8) return launch<MT, 1, (MT == 1 ? 8 : 4), GATED, TY>(x, w, y, M, N, K, ldx, ldw, ldy, e, stream);
    if (M <= 16) return launch<MT, 2, (MT == 1 ? 8 : 4), GATED, TY>(x, w, y, M, N, K, ldx, ldw, ldy, e, stream);
    if (M <= 32) return launch<MT, 4, (MT == 1 ? 4 : 2), GATED, TY>(x, w, y, M, N, K, ldx, ldw, ldy, e, stream);
    return launch<MT, 8, 2, GATED, TY>(x, w, y, M, N, K, ldx, ldw, ldy, e, stream);
}
}  // namespace

// Requirements (checked here; the caller falls back to another kernel otherwise):
// M in [1, 64]; K a multiple of 8; x, w rows 16-byte aligned (leading dimensions
// multiples of 8 and base pointers 16-byte aligned).
// gated != 0: w is [2N, K] (N gate rows then N up rows), y is [M, N] = silu(gate) * up.
// row_tiles: 1 or 2 tiles of 16 weight rows per block (the gated form uses 2); 4: one tile and four
// warps a block instead of eight (up to 8 batch rows, not gated).
// bias: float32 [N] added to every row, or null (not with the gate).
struct KidiSkinnyExtras {          // every pointer may be null: the plain product
    const float* factor_parts;     // row factors: see Epilogue
    int factor_count, factor_stride, factor_width;
    float factor_eps;
    float* residual;               // into the residual: see Epilogue (not gated; one tile of rows a block)
    long long ld_residual;
    const void* norm_weight;
    int norm_weight_is_float;
    void* normed;
    long long ld_normed;
    float* parts_out;
    int parts_stride;
};

// How many parts per row the product into the residual writes for N features.
KIDI_API int kidi_gemm_skinny_parts(int N) { return (N + 15) / 16; }

KIDI_API int kidi_gemm_skinny(const void* x, const void* w, void* y, int y_dtype, int M, int N, int K, long long ldx,
                              long long ldw, long long ldy, int gated, int row_tiles, const float* bias,
                              const KidiSkinnyExtras* extras, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M > 64 || K <= 0 || (K & 7) || (ldx & 7) || (ldw & 7) || ((uintptr_t)x & 15) || ((uintptr_t)w & 15))
        return KIDI_REFUSED_SIZE;
    Epilogue e = {};
    e.bias = bias;
    if (extras) {
        e.factor_parts = extras->factor_parts;
        e.factor_count = extras->factor_count;
        e.factor_stride = extras->factor_stride;
        e.factor_width = extras->factor_width;
        e.factor_eps = extras->factor_eps;
        e.residual = extras->residual;
        e.ld_residual = extras->ld_residual;
        e.norm_weight = extras->norm_weight;
        e.norm_weight_is_float = extras->norm_weight_is_float;
        e.normed = (bf16*)extras->normed;
        e.ld_normed = extras->ld_normed;
        e.parts_out = extras->parts_out;
        e.parts_stride = extras->parts_stride;
        if (e.factor_parts && (e.factor_count < 1 || e.factor_stride < e.factor_count || e.factor_width < 1))
            return KIDI_REFUSED_SIZE;
        if (e.residual && (gated || !e.norm_weight || !e.normed || !e.parts_out || e.parts_stride < (N + 15) / 16))
            return KIDI_REFUSED_SIZE;
        if (e.residual && row_tiles == 2) row_tiles = 1;      // the parts are per tile of 16 features
    }
    const int mode = (e.factor_parts ? 1 : 0) | (e.residual ? 2 : 0);
    if (mode) {
        // The forms with a norm folded in exist for the decode step's few rows and bfloat16 results.
        if (M > 8 || y_dtype != KIDI_BF16) return KIDI_REFUSED_SIZE;
        if (gated) {
            if (row_tiles != 2) return launch<1, 1, 8, true, bf16, 1>(x, w, y, M, N, K, ldx, ldw, ldy, e, stream);
            return launch<2, 1, 4, true, bf16, 1>(x, w, y, M, N, K, ldx, ldw, ldy, e, stream);
        }
        if (row_tiles == 4) {
            if (mode == 1) return launch<1, 1, 8, false, bf16, 1, 4>(x, w, y, M, N, K, ldx, ldw, ldy, e, stream);
            if (mode == 2) return launch<1, 1, 8, false, bf16, 2, 4>(x, w, y, M, N, K, ldx, ldw, ldy, e, stream);
            return launch<1, 1, 8, false, bf16, 3, 4>(x, w, y, M, N, K, ldx, ldw, ldy, e, stream);
        }
        if (mode == 1) return launch<1, 1, 8, false, bf16, 1>(x, w, y, M, N, K, ldx, ldw, ldy, e, stream);
        if (mode == 2) return launch<1, 1, 8, false, bf16, 2>(x, w, y, M, N, K, ldx, ldw, ldy, e, stream);
        return launch<1, 1, 8, false, bf16, 3>(x, w, y, M, N, K, ldx, ldw, ldy, e, stream);
    }
    if (gated) {
        if (y_dtype != KIDI_BF16) return KIDI_REFUSED_DTYPE;
        if (bias) return KIDI_REFUSED_SIZE;
        // Up to eight batch rows: eight gate and eight up rows per tile (twice the blocks, each with the
        // deeper prefetch of the one-tile form); more rows: sixteen and sixteen.
        if (row_tiles == 1 || (M <= 8 && row_tiles != 2))
            return by_batch<1, true, bf16>(x, w, y, M, N, K, ldx, ldw, ldy, e, stream);
        return by_batch<2, true, bf16>(x, w, y, M, N, K, ldx, ldw, ldy, e, stream);
    }
    if (row_tiles == 4 && M <= 8) {          // four warps a block
        if (y_dtype == KIDI_BF16) return launch<1, 1, 8, false, bf16, 0, 4>(x, w, y, M, N, K, ldx, ldw, ldy, e, stream);
        if (y_dtype == KIDI_F32) return launch<1, 1, 8, false, float, 0, 4>(x, w, y, M, N, K, ldx, ldw, ldy, e, stream);
        return KIDI_REFUSED_DTYPE;
    }
    if (y_dtype == KIDI_BF16)
        return row_tiles == 2 ? by_batch<2, false, bf16>(x, w, y, M, N, K, ldx, ldw, ldy, e, stream)
                              : by_batch<1, false, bf16>(x, w, y, M, N, K, ldx, ldw, ldy, e, stream);
    if (y_dtype == KIDI_F32)
        return row_tiles == 2 ? by_batch<2, false, float>(x, w, y, M, N, K, ldx, ldw, ldy, e, stream)
                              : by_batch<1, false, float>(x, w, y, M, N, K, ldx, ldw, ldy, e, stream);
    return KIDI_REFUSED_DTYPE;
}
