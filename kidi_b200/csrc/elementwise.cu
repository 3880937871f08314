// Embedding gather, residual-add + RMSNorm, the SiLU gate, and the bookkeeping kernel
// that advances a decode step.
//
// Formulas (reference): embedding row gather times a scalar scale
// (src/kidi/layers/gemma4.cpp:97-99,132-142); RMSNorm y = x * (1/sqrt(sum(x^2)/H + eps)) * w
// (src/kidi/runtime/mps/eager_kernels.metal:65-87); SiLU gate f = g / (1 + exp(-g)) * u
// (src/kidi/runtime/mps/eager_kernels.metal:129-137). The residual stream is kept in
// 32-bit in every engine dtype, and the sum of squares and the inverse root are 32-bit.
#include "common.cuh"


// Four consecutive elements of a row as 32-bit values, whatever the stored type.
__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const bf16* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(bf16* p, float4 v) {
    uint2 raw;
    *reinterpret_cast<__nv_bfloat162*>(&raw.x) = __floats2bfloat162_rn(v.x, v.y);
    *reinterpret_cast<__nv_bfloat162*>(&raw.y) = __floats2bfloat162_rn(v.z, v.w);
    *reinterpret_cast<uint2*>(p) = raw;
}

// ------------------------------------------------------------------ embedding
template <typename TW>
__global__ void embedding_kernel(float* __restrict__ out, const TW* __restrict__ table,
                                 const int* __restrict__ tokens, int hidden, int vocab, float scale) {
    const int row = blockIdx.x;
    const int token = tokens[row];
    float* destination = out + (long long)row * hidden;
    if (token < 0 || token >= vocab) {  // never read outside the table
        for (int c = threadIdx.x; c < hidden; c += blockDim.x) destination[c] = 0.f;
        return;
    }
    const TW* source = table + (long long)token * hidden;
    if (!(hidden & 3) && !((uintptr_t)table & 15) && !((uintptr_t)out & 15)) {   // four elements at a time
        for (int c = 4 * threadIdx.x; c < hidden; c += 4 * blockDim.x) {
            const float4 v = load4(source + c);
            store4(destination + c, make_float4(v.x * scale, v.y * scale, v.z * scale, v.w * scale));
        }
        return;
    }
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) destination[c] = to_float(source[c]) * scale;
}

KIDI_API int kidi_embedding(float* out, const void* table, int table_dtype, const int* tokens, int rows, int hidden,
                            int vocab, float scale, cudaStream_t stream) {
    if (rows <= 0) return 0;
    const int threads = hidden >= 1024 ? 256 : 128;
    if (table_dtype == KIDI_F32)
        return kidi_launch(embedding_kernel<float>, rows, threads, 0, stream, out, (const float*)table, tokens, hidden,
                           vocab, scale);
    if (table_dtype == KIDI_BF16)
        return kidi_launch(embedding_kernel<bf16>, rows, threads, 0, stream, out, (const bf16*)table, tokens, hidden,
                           vocab, scale);
    return KIDI_REFUSED_DTYPE;
}

// ------------------------------------------------------- residual add + RMSNorm
// One block per output row r. Source row s = row_index ? row_index[r] : r.
//   v = residual[s] + delta[s]   (delta optional)
//   if write_residual: residual[s] = v
//   y[r] = v * inv * w,  inv = 1 / sqrt(mean(v^2) + eps)
// The row is staged in shared memory so that it is read once.
template <typename TD, typename TW, typename TY, int THREADS>
__global__ void __launch_bounds__(THREADS)
add_rmsnorm_kernel(float* __restrict__ residual, const TD* __restrict__ delta, const TW* __restrict__ weight,
                   TY* __restrict__ y, const int* __restrict__ row_index, int hidden, float eps, int write_residual) {
    extern __shared__ float staged[];
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    const long long s = row_index ? row_index[r] : r;
    float* h = residual + s * hidden;
    float square = 0.f;
    for (int c = threadIdx.x; c < hidden; c += THREADS) {
        float value = h[c];
        if (delta) value += to_float(delta[s * hidden + c]);
        if (write_residual) h[c] = value;
        staged[c] = value;
        square = fmaf(value, value, square);
    }
    const float total = block_sum<THREADS>(square, scratch);
    const float inv = 1.0f / sqrtf(total / (float)hidden + eps);
    TY* out = y + (long long)r * hidden;
    for (int c = threadIdx.x; c < hidden; c += THREADS)
        out[c] = from_float<TY>(staged[c] * inv * to_float(weight[c]));
}

// The same for rows of exactly THREADS * 4 * CHUNKS elements: every thread keeps its
// CHUNKS groups of four elements in registers, all loads of a row are in flight at once,
// and nothing is staged in shared memory. (The sum of squares is added in this kernel's
// own fixed order; every step of an engine with such rows takes this kernel.)
template <typename TD, typename TW, typename TY, int THREADS, int CHUNKS>
__global__ void __launch_bounds__(THREADS)
add_rmsnorm_vector_kernel(float* __restrict__ residual, const TD* __restrict__ delta, const TW* __restrict__ weight,
                          TY* __restrict__ y, const int* __restrict__ row_index, float eps, int write_residual) {
    __shared__ float scratch[32];
    constexpr int hidden = THREADS * 4 * CHUNKS;
    const int r = blockIdx.x;
    const long long s = row_index ? row_index[r] : r;
    float* h = residual + s * hidden;
    float4 v[CHUNKS];
#pragma unroll
    for (int i = 0; i < CHUNKS; ++i) v[i] = load4(h + 4 * (threadIdx.x + THREADS * i));
    if (delta) {
        float4 d[CHUNKS];
#pragma unroll
        for (int i = 0; i < CHUNKS; ++i) d[i] = load4(delta + s * hidden + 4 * (threadIdx.x + THREADS * i));
#pragma unroll
        for (int i = 0; i < CHUNKS; ++i) {
            v[i].x += d[i].x; v[i].y += d[i].y; v[i].z += d[i].z; v[i].w += d[i].w;
        }
    }
    float4 w[CHUNKS];
#pragma unroll
    for (int i = 0; i < CHUNKS; ++i) w[i] = load4(weight + 4 * (threadIdx.x + THREADS * i));
    float square = 0.f;
#pragma unroll
    for (int i = 0; i < CHUNKS; ++i) {
        if (write_residual) store4(h + 4 * (threadIdx.x + THREADS * i), v[i]);
        square = fmaf(v[i].x, v[i].x, square);
        square = fmaf(v[i].y, v[i].y, square);
        square = fmaf(v[i].z, v[i].z, square);
        square = fmaf(v[i].w, v[i].w, square);
    }
    const float total = block_sum<THREADS>(square, scratch);
    const float inv = 1.0f / sqrtf(total / (float)hidden + eps);
    TY* out = y + (long long)r * hidden;
#pragma unroll
    for (int i = 0; i < CHUNKS; ++i)
        store4(out + 4 * (threadIdx.x + THREADS * i),
               make_float4(v[i].x * inv * w[i].x, v[i].y * inv * w[i].y, v[i].z * inv * w[i].z, v[i].w * inv * w[i].w));
}

template <typename TD, typename TW, typename TY>
static int launch_add_rmsnorm(float* residual, const void* delta, const void* weight, void* y, const int* row_index,
                              int rows, int hidden, float eps, int write_residual, cudaStream_t stream) {
    constexpr int THREADS = 256;
    const bool vectors = !((uintptr_t)residual & 15) && !((uintptr_t)delta & 15) && !((uintptr_t)weight & 15) &&
                         !((uintptr_t)y & 15);
#define KIDI_VECTOR_CASE(CHUNKS)                                                                              \
    if (vectors && hidden == THREADS * 4 * CHUNKS)                                                            \
        return kidi_launch(add_rmsnorm_vector_kernel<TD, TW, TY, THREADS, CHUNKS>, rows, THREADS, 0, stream, \
                           residual, (const TD*)delta, (const TW*)weight, (TY*)y, row_index, eps, write_residual);
    KIDI_VECTOR_CASE(1)     // every multiple of 1024 up to 8192 elements
    KIDI_VECTOR_CASE(2)
    KIDI_VECTOR_CASE(3)
    KIDI_VECTOR_CASE(4)
    KIDI_VECTOR_CASE(5)
    KIDI_VECTOR_CASE(6)
    KIDI_VECTOR_CASE(7)
    KIDI_VECTOR_CASE(8)
#undef KIDI_VECTOR_CASE
    const size_t shared = (size_t)hidden * sizeof(float);
    if (shared > 200 * 1024) return KIDI_REFUSED_SIZE;
    auto kernel = add_rmsnorm_kernel<TD, TW, TY, THREADS>;
    if (shared > 48 * 1024) {
        cudaError_t status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
        if (status != cudaSuccess) return (int)status;
    }
    return kidi_launch(kernel, rows, THREADS, shared, stream, residual, (const TD*)delta, (const TW*)weight, (TY*)y,
                       row_index, hidden, eps, write_residual);
}

// delta_dtype may be KIDI_NONE (no delta). The residual is always float.
KIDI_API int kidi_add_rmsnorm(float* residual, const void* delta, int delta_dtype, const void* weight,
                              int weight_dtype, void* y, int y_dtype, const int* row_index, int rows, int hidden,
                              float eps, int write_residual, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (delta_dtype == KIDI_NONE) { delta = nullptr; delta_dtype = KIDI_F32; }
#define KIDI_CASE(D, TD, W, TW, Y, TY)                                                                     \
    if (delta_dtype == D && weight_dtype == W && y_dtype == Y)                                             \
        return launch_add_rmsnorm<TD, TW, TY>(residual, delta, weight, y, row_index, rows, hidden, eps,    \
                                              write_residual, stream);
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

// ------------------------------------------------------- advancing a decode step
// After a decode step whose tokens were selected on the device: every live row takes
// its selected token as the next input and moves one position on. Rows whose
// row_seq is negative are padding and stay as they are.
__global__ void advance_decode_kernel(int* __restrict__ tokens, const int* __restrict__ selected,
                                      const int* __restrict__ row_seq, int* __restrict__ row_pos,
                                      int* __restrict__ seq_start, int* __restrict__ steps, int rows, int vocab) {
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= rows || row_seq[r] < 0) return;
    const int token = selected[r];
    tokens[r] = token >= 0 && token < vocab ? token : 0;
    row_pos[r] += 1;
    seq_start[row_seq[r]] += 1;
    steps[r] += 1;
}

KIDI_API int kidi_advance_decode(int* tokens, const int* selected, const int* row_seq, int* row_pos, int* seq_start,
                                 int* steps, int rows, int vocab, cudaStream_t stream) {
    if (rows <= 0) return 0;
    return kidi_launch(advance_decode_kernel, (rows + 127) / 128, 128, 0, stream, tokens, selected, row_seq, row_pos,
                       seq_start, steps, rows, vocab);
}

// ------------------------------------------------------------------ SiLU gate
// gate_up [rows, 2*inter] (gate = first inter columns, up = last inter) -> out [rows, inter]
template <typename T>
__global__ void silu_gate_kernel(const T* __restrict__ gate_up, T* __restrict__ out, long long total, int inter) {
    const long long index = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (index >= total) return;
    const long long row = index / inter;
    const int c = (int)(index - row * inter);
    const float gate = to_float(gate_up[row * 2 * inter + c]);
    const float up = to_float(gate_up[row * 2 * inter + inter + c]);
    out[index] = from_float<T>(gate / (1.0f + expf(-gate)) * up);
}

// The same for bfloat16 rows whose width is a multiple of 8: eight elements (16 bytes) per thread.
__global__ void silu_gate_bf16x8_kernel(const bf16* __restrict__ gate_up, bf16* __restrict__ out, long long groups,
                                        int inter) {
    const long long index = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (index >= groups) return;
    const int per_row = inter >> 3;
    const long long row = index / per_row;
    const int c = (int)(index - row * per_row) << 3;
    const uint4 gate = *reinterpret_cast<const uint4*>(gate_up + row * 2 * inter + c);
    const uint4 up = *reinterpret_cast<const uint4*>(gate_up + row * 2 * inter + inter + c);
    const __nv_bfloat162* g = reinterpret_cast<const __nv_bfloat162*>(&gate);
    const __nv_bfloat162* u = reinterpret_cast<const __nv_bfloat162*>(&up);
    uint4 result;
    __nv_bfloat162* r = reinterpret_cast<__nv_bfloat162*>(&result);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 gv = __bfloat1622float2(g[i]), uv = __bfloat1622float2(u[i]);
        r[i] = __floats2bfloat162_rn(gv.x / (1.0f + expf(-gv.x)) * uv.x, gv.y / (1.0f + expf(-gv.y)) * uv.y);
    }
    *reinterpret_cast<uint4*>(out + row * inter + c) = result;
}

KIDI_API int kidi_silu_gate(const void* gate_up, void* out, int dtype, int rows, int inter, cudaStream_t stream) {
    const long long total = (long long)rows * inter;
    if (total <= 0) return 0;
    const int threads = 256;
    const unsigned blocks = (unsigned)((total + threads - 1) / threads);
    if (dtype == KIDI_F32)
        return kidi_launch(silu_gate_kernel<float>, blocks, threads, 0, stream, (const float*)gate_up, (float*)out,
                           total, inter);
    if (dtype == KIDI_BF16) {
        if (!(inter & 7) && !((uintptr_t)gate_up & 15) && !((uintptr_t)out & 15)) {
            const long long groups = total >> 3;
            return kidi_launch(silu_gate_bf16x8_kernel, (unsigned)((groups + threads - 1) / threads), threads, 0, stream,
                               (const bf16*)gate_up, (bf16*)out, groups, inter);
        }
        return kidi_launch(silu_gate_kernel<bf16>, blocks, threads, 0, stream, (const bf16*)gate_up, (bf16*)out, total,
                           inter);
    }
    return KIDI_REFUSED_DTYPE;
}

// y[r, c] += bias[c]: the bias of a product that the vendor library computed (this package's
// own products add it in their epilogues).
template <typename T>
__global__ void add_bias_kernel(T* __restrict__ y, const float* __restrict__ bias, long long total, int features,
                                long long ldy) {
    const long long index = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (index >= total) return;
    const long long row = index / features;
    const int c = (int)(index - row * features);
    y[row * ldy + c] = from_float<T>(to_float(y[row * ldy + c]) + bias[c]);
}

KIDI_API int kidi_add_bias(void* y, int dtype, const float* bias, int rows, int features, long long ldy,
                           cudaStream_t stream) {
    const long long total = (long long)rows * features;
    if (total <= 0) return 0;
    const int threads = 256;
    const unsigned blocks = (unsigned)((total + threads - 1) / threads);
    if (dtype == KIDI_F32)
        return kidi_launch(add_bias_kernel<float>, blocks, threads, 0, stream, (float*)y, bias, total, features, ldy);
    if (dtype == KIDI_BF16)
        return kidi_launch(add_bias_kernel<bf16>, blocks, threads, 0, stream, (bf16*)y, bias, total, features, ldy);
    return KIDI_REFUSED_DTYPE;
}

// out[r, :] = values[r, :] * 1 / sqrt(sum(parts[r, :count]) / width + eps): rows that a product stored
// without their norm's factor (gemm_skinny.cu, "into the residual"), for a consumer that wants plain rows.
// The parts are added in the order the weight-streaming product adds them (a warp: lane l takes parts
// l, l + 32, ..., then the fixed tree), so both consumers see the same factor.
__global__ void __launch_bounds__(256)
apply_row_factors_kernel(const bf16* __restrict__ values, long long ld, const float* __restrict__ parts, int count,
                         int stride, int width, float eps, bf16* __restrict__ out, int hidden) {
    __shared__ float factor;
    const int r = blockIdx.x;
    if (threadIdx.x < 32) {
        float square = 0.f;
        for (int b = threadIdx.x; b < count; b += 32) square += parts[(long long)r * stride + b];   // ascending, as there
        square = warp_sum(square);
        if (threadIdx.x == 0) factor = 1.0f / sqrtf(square / (float)width + eps);
    }
    __syncthreads();
    for (int c = threadIdx.x; c < hidden; c += 256)
        out[(long long)r * hidden + c] = from_float<bf16>(to_float(values[r * ld + c]) * factor);
}

KIDI_API int kidi_apply_row_factors(const void* values, long long ld, const float* parts, int count, int stride,
                                    int width, float eps, void* out, int rows, int hidden, cudaStream_t stream) {
    if (rows <= 0 || hidden <= 0) return 0;
    if (count < 1 || stride < count || width < 1) return KIDI_REFUSED_SIZE;
    return kidi_launch(apply_row_factors_kernel, rows, 256, 0, stream, (const bf16*)values, ld, parts, count, stride,
                       width, eps, (bf16*)out, hidden);
}
