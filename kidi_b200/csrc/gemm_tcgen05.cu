// y[T, F] = x[T, K] * W[F, K]^T in bfloat16 on the 5th-generation tensor cores.
//
// The weight matrix is operand A of the instruction (a tile of 128 output features,
// K-major), the activations are operand B (a tile of BN tokens, K-major), and the
// 128 x BN accumulator lives in tensor memory (TMEM): TMEM lane = feature, TMEM column
// = token. Operand tiles of 64 k-elements (128 bytes per row) are brought in by TMA with
// the 128-byte swizzle, which is the canonical K-major layout the instruction's shared
// memory descriptors name; a ring of STAGES tiles is kept in flight with mbarriers.
// One thread issues the copies, one thread issues tcgen05.mma (four k=16 steps per
// tile, the descriptor's start address advanced by 32 bytes inside the swizzle atom),
// and four warps read the accumulator back with tcgen05.ld for the epilogue.
//
// With few tokens the product is bound by reading W once: a block then takes only a
// slice of K (split-K) so that every SM streams weights; blocks write their partial
// tiles to a workspace and the last one to arrive for a tile (an atomic counter) adds
// them in slice order, so the result does not depend on timing. Epilogues: store
// (bfloat16 or float32), or the SiLU gate of a fused [gate | up] projection, for which a
// tile is 64 gate rows and the 64 matching up rows.
//
// Every wait on an mbarrier is bounded: when the limit is reached the block records a
// code in `error`, waits (bounded) for its copies in flight, frees its tensor memory
// and returns.
#include <cuda.h>

#include "common.cuh"

namespace {

constexpr int BM = 128;          // features per tile (TMEM lanes)
constexpr int BK = 64;           // k-elements per stage: 128 bytes, one swizzle span
constexpr int UMMA_K = 16;
constexpr int THREADS = 192;     // warp 0: TMA, warp 1: MMA, warps 2-5: epilogue
constexpr unsigned SPIN_LIMIT = 1u << 24;

__device__ __forceinline__ unsigned smem_u32(const void* pointer) {
    return (unsigned)__cvta_generic_to_shared(pointer);
}

__device__ __forceinline__ void mbarrier_init(unsigned long long* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbarrier_expect_tx(unsigned long long* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbarrier_try_wait(unsigned long long* bar, unsigned parity) {
    unsigned done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return done != 0;
}
// Bounded wait: false when the limit was reached or another thread has given up.
__device__ __forceinline__ bool mbarrier_wait(unsigned long long* bar, unsigned parity, volatile int* gave_up) {
    for (unsigned spin = 0; spin < SPIN_LIMIT; ++spin) {
        if (mbarrier_try_wait(bar, parity)) return true;
        if ((spin & 1023u) == 1023u && *gave_up) return false;
    }
    return false;
}

__device__ __forceinline__ void tma_load_2d(void* smem, const CUtensorMap* map, unsigned long long* bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        :
        : "r"(smem_u32(smem)), "l"((unsigned long long)map), "r"(smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}

// Shared memory descriptor of a K-major tile with the 128-byte swizzle: rows are 128
// bytes apart, groups of eight rows 1024 bytes apart (the stride byte offset), version 1.
__device__ __forceinline__ unsigned long long make_smem_desc(const void* tile) {
    unsigned long long desc = 0;
    desc |= (unsigned long long)((smem_u32(tile) & 0x3FFFF) >> 4);   // start address, 16-byte units
    desc |= (unsigned long long)1 << 16;                              // leading byte offset (unused with a swizzle)
    desc |= (unsigned long long)(1024 >> 4) << 32;                    // stride byte offset
    desc |= (unsigned long long)1 << 46;                              // descriptor version of this architecture
    desc |= (unsigned long long)2 << 61;                              // layout type: 128-byte swizzle
    return desc;
}

// Instruction descriptor: D float32, A and B bfloat16, both K-major, M = 128, N = bn.
__host__ __device__ constexpr unsigned make_instr_desc(int bn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(bn >> 3) << 17) | ((unsigned)(BM >> 4) << 24);
}

__device__ __forceinline__ void umma_bf16(unsigned tmem_d, unsigned long long desc_a, unsigned long long desc_b,
                                          unsigned idesc, unsigned accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        :
        : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(unsigned long long* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void tmem_load_16(unsigned address, float (&v)[16]) {
    unsigned r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(address));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

struct Params {
    void* y;               // [tokens, ldy]
    float* workspace;      // [units][BM][BN] partial tiles (split-K only)
    int* counters;         // [feature tiles * token tiles], zero between calls (the kernel leaves them zero)
    int* error;            // set to a non-zero code when a bounded wait ran out
    const float* bias;     // [features] added to every token's row, or null (not with the gate)
    long long ldy;
    int tokens, features;  // features: width of y (for the gated form the weight has 2 * features rows)
    int k_blocks;          // ceil(K / 64)
    int splits;            // blocks that share one tile's K range
    int feature_tiles;
};

template <int BN, int STAGES, bool GATED, typename TY>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, Params p) {
    constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr int TMEM_COLUMNS = BN < 32 ? 32 : BN;
    constexpr int SPAN = GATED ? 64 : BM;                  // output features per tile
    extern __shared__ unsigned char raw[];
    unsigned char* tiles = (unsigned char*)(((uintptr_t)raw + 1023) & ~(uintptr_t)1023);
    __shared__ unsigned long long full_bar[STAGES], empty_bar[STAGES], done_bar;
    __shared__ unsigned tmem_base_slot;
    __shared__ int gave_up, is_last;
    // The gated epilogue passes the up rows of a 16-column chunk between warps (64 x 17
    // floats): in the first stage's tile, which is free once the accumulator is complete (a
    // buffer of its own would leave room for one block per SM instead of two).
    float* exchange = reinterpret_cast<float*>(tiles);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int feature_tile = blockIdx.x % p.feature_tiles, split = blockIdx.x / p.feature_tiles;
    const int token_tile = blockIdx.y;
    const int f0 = feature_tile * SPAN, t0 = token_tile * BN;
    // This block's slice of the k-blocks: slices differ by at most one block.
    const int base = p.k_blocks / p.splits, extra = p.k_blocks % p.splits;
    const int kb_first = split * base + min(split, extra);
    const int kb_count = base + (split < extra ? 1 : 0);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbarrier_init(&full_bar[s], 1);
            mbarrier_init(&empty_bar[s], 1);
        }
        mbarrier_init(&done_bar, 1);
        gave_up = 0;
        is_last = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {  // the whole warp allocates tensor memory
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)),
                     "r"(TMEM_COLUMNS));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const unsigned tmem_base = tmem_base_slot;
    volatile int* abort_flag = &gave_up;

    if (warp == 0 && lane == 0) {
        // ------------------------------------------------------------ producer
        int issued = 0;
        for (int i = 0; i < kb_count; ++i) {
            const int s = i % STAGES;
            if (i >= STAGES && !mbarrier_wait(&empty_bar[s], ((i / STAGES) - 1) & 1, abort_flag)) {
                if (!*abort_flag) { *abort_flag = 1; atomicExch(p.error, 1); }
                break;
            }
            unsigned char* stage = tiles + (size_t)s * STAGE_BYTES;
            mbarrier_expect_tx(&full_bar[s], STAGE_BYTES);
            const int k = (kb_first + i) * BK;
            if (GATED) {
                tma_load_2d(stage, &map_w, &full_bar[s], k, f0);                            // 64 gate rows
                tma_load_2d(stage + A_BYTES / 2, &map_w, &full_bar[s], k, p.features + f0);  // 64 up rows
            } else {
                tma_load_2d(stage, &map_w, &full_bar[s], k, f0);
            }
            tma_load_2d(stage + A_BYTES, &map_x, &full_bar[s], k, t0);
            ++issued;
        }
        if (*abort_flag) {  // let the copies in flight land before the block leaves
            for (int i = max(0, issued - STAGES); i < issued; ++i)
                for (unsigned spin = 0; spin < SPIN_LIMIT; ++spin)
                    if (mbarrier_try_wait(&full_bar[i % STAGES], (i / STAGES) & 1)) break;
        }
    } else if (warp == 1 && lane == 0) {
        // -------------------------------------------------------------- issuer
        constexpr unsigned idesc = make_instr_desc(BN);
        for (int i = 0; i < kb_count; ++i) {
            const int s = i % STAGES;
            if (!mbarrier_wait(&full_bar[s], (i / STAGES) & 1, abort_flag)) {
                if (!*abort_flag) { *abort_flag = 1; atomicExch(p.error, 2); }
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            unsigned char* stage = tiles + (size_t)s * STAGE_BYTES;
            const unsigned long long desc_a = make_smem_desc(stage), desc_b = make_smem_desc(stage + A_BYTES);
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k)  // 32 bytes further inside the swizzle span: +2 in 16-byte units
                umma_bf16(tmem_base, desc_a + 2 * k, desc_b + 2 * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
            umma_commit(&empty_bar[s]);  // arrives when these instructions have read the stage
        }
        umma_commit(&done_bar);          // arrives when the accumulator is complete
    } else if (warp >= 2) {
        // ------------------------------------------------------------ epilogue
        const int quarter = warp & 3;                     // TMEM lanes 32 * quarter .. + 31
        const int row = quarter * 32 + lane;              // row of the tile = TMEM lane
        bool ok = kb_count == 0 || mbarrier_wait(&done_bar, 0, abort_flag);
        if (!ok && !*abort_flag) { *abort_flag = 1; atomicExch(p.error, 3); }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const long long tile_index = (long long)token_tile * p.feature_tiles + feature_tile;
        bool reduce = false;
        if (p.splits > 1) {
            // Partial tile to the workspace; the last block to arrive adds all of them.
            float* mine = p.workspace + ((tile_index * p.splits + split) * BM + row) * BN;
#pragma unroll 1
            for (int c = 0; c < BN; c += 16) {
                float v[16];
                if (ok && kb_count > 0) tmem_load_16(tmem_base + ((unsigned)(quarter * 32) << 16) + c, v);
                else
#pragma unroll
                    for (int i = 0; i < 16; ++i) v[i] = 0.f;
#pragma unroll
                for (int i = 0; i < 16; i += 4)
                    *reinterpret_cast<float4*>(mine + c + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
            }
            __threadfence();
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (threadIdx.x == 64) is_last = atomicAdd(p.counters + tile_index, 1) == p.splits - 1;
            asm volatile("bar.sync 1, 128;" ::: "memory");
            reduce = is_last != 0;
            if (reduce) __threadfence();
        }
        if (p.splits == 1 || reduce) {
            TY* y = (TY*)p.y;
#pragma unroll 1
            for (int c = 0; c < BN; c += 16) {
                float v[16];
                if (p.splits == 1) {
                    if (ok && kb_count > 0) tmem_load_16(tmem_base + ((unsigned)(quarter * 32) << 16) + c, v);
                    else
#pragma unroll
                        for (int i = 0; i < 16; ++i) v[i] = 0.f;
                } else {
#pragma unroll
                    for (int i = 0; i < 16; ++i) v[i] = 0.f;
                    for (int s = 0; s < p.splits; ++s) {  // slice order: the sum does not depend on timing
                        const float* part = p.workspace + ((tile_index * p.splits + s) * BM + row) * BN + c;
#pragma unroll
                        for (int i = 0; i < 16; i += 4) {
                            const float4 q = __ldcg(reinterpret_cast<const float4*>(part + i));
                            v[i] += q.x; v[i + 1] += q.y; v[i + 2] += q.z; v[i + 3] += q.w;
                        }
                    }
                }
                if (GATED) {
                    // Rows 64..127 hold the up projection of the features in rows 0..63.
                    if (row >= 64)
#pragma unroll
                        for (int i = 0; i < 16; ++i) exchange[(row - 64) * 17 + i] = v[i];
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    if (row < 64 && f0 + row < p.features)
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            const int token = t0 + c + i;
                            const float gate = v[i], up = exchange[row * 17 + i];
                            if (token < p.tokens)
                                y[token * p.ldy + f0 + row] = from_float<TY>(gate / (1.0f + expf(-gate)) * up);
                        }
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                } else if (f0 + row < p.features) {
                    const float shift = p.bias ? p.bias[f0 + row] : 0.f;
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const int token = t0 + c + i;
                        if (token < p.tokens) y[token * p.ldy + f0 + row] = from_float<TY>(v[i] + shift);
                    }
                }
            }
            if (reduce && threadIdx.x == 64) p.counters[tile_index] = 0;  // ready for the next call
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLUMNS));
    }
}

typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encode_tiled() {
    static EncodeTiled function = nullptr;
    if (!function) {
        void* entry = nullptr;
        cudaDriverEntryPointQueryResult result;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &entry, cudaEnableDefault, &result) == cudaSuccess &&
            result == cudaDriverEntryPointSuccess)
            function = (EncodeTiled)entry;
    }
    return function;
}

// A map over a row-major bfloat16 matrix [rows, K] with leading dimension ld: boxes of
// 64 k-elements by box_rows rows, 128-byte swizzle, zeros outside the matrix.
int make_map(CUtensorMap* map, const void* base, long long rows, long long K, long long ld, int box_rows) {
    EncodeTiled encode = encode_tiled();
    if (!encode) return KIDI_REFUSED_SIZE;
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    const cuuint32_t box[2] = {BK, (cuuint32_t)box_rows};
    const cuuint32_t steps[2] = {1, 1};
    CUresult status = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box,
                             steps, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return status == CUDA_SUCCESS ? 0 : 1000 + (int)status;
}

template <int BN, int STAGES, bool GATED, typename TY>
int launch(const CUtensorMap& map_w, const CUtensorMap& map_x, const Params& p, int token_tiles, cudaStream_t stream) {
    constexpr size_t shared = (size_t)STAGES * (BM * BK * 2 + BN * BK * 2) + 1024;
    auto kernel = gemm_tcgen05_kernel<BN, STAGES, GATED, TY>;
    static bool configured = false;
    if (!configured) {
        cudaError_t status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
        if (status != cudaSuccess) return (int)status;
        configured = true;
    }
    dim3 grid(p.feature_tiles * p.splits, token_tiles);
    kernel<<<grid, THREADS, shared, stream>>>(map_w, map_x, p);
    return kidi_launch_status();
}

template <bool GATED, typename TY>
int by_tokens(int bn, const CUtensorMap& map_w, const CUtensorMap& map_x, const Params& p, int token_tiles,
              cudaStream_t stream) {
    switch (bn) {
        case 16: return launch<16, 6, GATED, TY>(map_w, map_x, p, token_tiles, stream);
        case 32: return launch<32, 5, GATED, TY>(map_w, map_x, p, token_tiles, stream);
        case 64: return launch<64, 4, GATED, TY>(map_w, map_x, p, token_tiles, stream);
        case 128: return launch<128, 6, GATED, TY>(map_w, map_x, p, token_tiles, stream);
        case 256: return launch<256, 4, GATED, TY>(map_w, map_x, p, token_tiles, stream);
    }
    return KIDI_REFUSED_SIZE;
}
}  // namespace

// The token tile that fits `tokens` rows.
KIDI_API int kidi_gemm_tcgen05_token_tile(int tokens) {
    return tokens <= 16 ? 16 : tokens <= 32 ? 32 : tokens <= 64 ? 64 : tokens <= 128 ? 128 : 256;
}

// Floats of workspace a call needs (0 without split-K) and the number of counters.
KIDI_API long long kidi_gemm_tcgen05_workspace(int tokens, int features, int splits, int gated) {
    const int bn = kidi_gemm_tcgen05_token_tile(tokens);
    const long long tiles = (long long)((features + (gated ? 64 : BM) - 1) / (gated ? 64 : BM)) * ((tokens + bn - 1) / bn);
    return splits > 1 ? tiles * splits * BM * bn : 0;
}

// x [tokens, K] and w [features (2 * features when gated), K] bfloat16, rows 16-byte
// aligned; y [tokens, features] bfloat16 or float32. `workspace`, `counters` (zeroed
// once by the caller; the kernel leaves them zero) and `error` are the caller's. `bias`
// (float32 [features], or null) is added to every row.
KIDI_API int kidi_gemm_tcgen05(const void* x, const void* w, void* y, int y_dtype, int tokens, int features, int K,
                               long long ldx, long long ldw, long long ldy, int gated, int splits, float* workspace,
                               int* counters, int* error, const float* bias, cudaStream_t stream) {
    if (tokens <= 0 || features <= 0) return 0;
    if (K <= 0 || (K & 7) || (ldx & 7) || (ldw & 7) || ((uintptr_t)x & 15) || ((uintptr_t)w & 15) || splits < 1)
        return KIDI_REFUSED_SIZE;
    const int bn = kidi_gemm_tcgen05_token_tile(tokens);
    const int span = gated ? 64 : BM;
    Params p;
    p.y = y;
    p.workspace = workspace;
    p.counters = counters;
    p.error = error;
    p.bias = bias;
    p.ldy = ldy;
    p.tokens = tokens;
    p.features = features;
    p.k_blocks = (K + BK - 1) / BK;
    p.splits = splits > p.k_blocks ? p.k_blocks : splits;
    p.feature_tiles = (features + span - 1) / span;
    if (p.splits > 1 && (!workspace || !counters)) return KIDI_REFUSED_SIZE;
    if (!error) return KIDI_REFUSED_SIZE;
    const int token_tiles = (tokens + bn - 1) / bn;
    if (token_tiles > 65535) return KIDI_REFUSED_SIZE;
    CUtensorMap map_w, map_x;
    int status = make_map(&map_w, w, gated ? 2LL * features : features, K, ldw, gated ? 64 : BM);
    if (status) return status;
    status = make_map(&map_x, x, tokens, K, ldx, bn);
    if (status) return status;
    if (gated) {
        if (y_dtype != KIDI_BF16) return KIDI_REFUSED_DTYPE;
        if (bias) return KIDI_REFUSED_SIZE;
        return by_tokens<true, bf16>(bn, map_w, map_x, p, token_tiles, stream);
    }
    if (y_dtype == KIDI_BF16) return by_tokens<false, bf16>(bn, map_w, map_x, p, token_tiles, stream);
    if (y_dtype == KIDI_F32) return by_tokens<false, float>(bn, map_w, map_x, p, token_tiles, stream);
    return KIDI_REFUSED_DTYPE;
}
