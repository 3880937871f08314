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
// and four warps read the accumulator back with tcgen05.ld for the epilogue. Blocks are
// persistent (one per SM, each walking its share of the tiles) and the accumulator is
// double-buffered in tensor memory, so that the epilogue of one tile runs under the
// products of the next and the ring of operand stages never drains between tiles.
//
// With fewer tiles than resident blocks (few tokens: the product is bound by reading W once) the
// tiles' k-blocks are dealt out evenly over the blocks, so that every SM streams weights (split-K).
// A block writes its part of a tile to a workspace and counts itself in; when all parts of the tile
// are there (the blocks are launched cooperatively, so they are resident together), the block that
// brought the i-th part adds the i-th share of the tile's token columns over all parts, in their
// order along k, so that the result does not depend on timing, and stores it: the sum and the
// stores are spread over the blocks. Epilogues: store (bfloat16 or float32), or the SiLU gate of a
// fused [gate | up] projection, for which a tile is 64 gate rows and the 64 matching up rows.
//
// Every wait on an mbarrier is bounded: when the limit is reached the block records a
// code in `error`, waits (bounded) for its copies in flight, frees its tensor memory
// and returns.
#include <cuda.h>

#include <atomic>
#include <string.h>

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
__device__ __forceinline__ void mbarrier_arrive(unsigned long long* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
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

// A tile of shared memory to global memory through a tensor map (clipped at the tensor's edges);
// the copies of a thread form groups that it can wait for.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* smem, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                 :
                 : "l"((unsigned long long)map), "r"(smem_u32(smem)), "r"(x), "r"(y)
                 : "memory");
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
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
    float* workspace;      // [2 * blocks][BM][BN] partial tiles
    int* counters;         // [2 * blocks]: parts arrived, parts read; zero between calls (the kernel leaves them zero)
    int* error;            // set to a non-zero code when a bounded wait ran out
    const float* bias;     // [features] added to every token's row, or null (not with the gate)
    long long ldy;
    int tokens, features;  // features: width of y (for the gated form the weight has 2 * features rows)
    int k_blocks;          // ceil(K / 64): the k-blocks of one tile
    int token_tiles;
    long long tiles;
    int rounds;            // whole tiles a block takes for itself: tiles b, b + blocks, ... (while there are)
    long long tail_first;  // the first tile of the tail
    int share, extra;      // of the tail's k-blocks a block takes `share`, the first `extra` blocks one more
    int staged;            // results leave through shared memory and TMA stores (bfloat16 y, 16-byte aligned rows)
};

// Tiles are numbered so that the blocks at work at one time share few weight tiles and few token
// tiles (see `locate`). With a tile for every block, block b takes whole tiles b,
// b + blocks, ... and writes their results to y. With fewer tiles than blocks (few tokens: the
// product is bound by reading the weights once) the tiles' k-blocks form one line, tile after
// tile, of which every block takes an equal, contiguous piece (split-K; a piece may end one tile
// and begin the next). A piece's parts of tiles go to the workspace; when all parts of a tile are
// there, every block that brought one adds its share of the tile's token columns over all parts,
// in their order along k, so the result does not depend on timing.
// A block keeps its ring of operand stages full across the borders of tiles, and the accumulator
// is double-buffered in tensor memory (2 x BN columns): while the four epilogue warps read one
// piece of work out, the tensor core is at the next.
template <int BN, int STAGES, bool GATED, typename TY>
__global__ void __launch_bounds__(THREADS, BN <= 64 ? 2 : 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                    const __grid_constant__ CUtensorMap map_y, Params p) {
    constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr int BUFFER_COLUMNS = BN < 32 ? 32 : BN;      // columns of one accumulator
    constexpr int TMEM_COLUMNS = 2 * BUFFER_COLUMNS;        // 64 .. 512, a power of two
    constexpr int SPAN = GATED ? 64 : BM;                  // output features per tile
    extern __shared__ unsigned char raw[];
    unsigned char* tiles = (unsigned char*)(((uintptr_t)raw + 1023) & ~(uintptr_t)1023);
    // The gated epilogue passes the up rows of a 16-column chunk between warps (64 x 17 floats).
    float* exchange = reinterpret_cast<float*>(tiles + (size_t)STAGES * STAGE_BYTES);
    // Results on their way out (p.staged): two buffers of 16 tokens x SPAN features, which TMA stores
    // write to y in whole lines (a thread holds one feature of 16 tokens: stored directly, every
    // token's 32 features of a warp would be a 64-byte piece of its own).
    bf16* staging = reinterpret_cast<bf16*>(tiles + (size_t)STAGES * STAGE_BYTES + 64 * 17 * sizeof(float));
    __shared__ unsigned long long full_bar[STAGES], empty_bar[STAGES], ready_bar[2], drained_bar[2];
    __shared__ unsigned tmem_base_slot;
    __shared__ int gave_up, is_last;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // Where block c's piece of the line begins, and which block holds k-block g of the line.
    auto begin_of = [&](long long c) -> long long { return c * p.share + (c < p.extra ? c : p.extra); };   // in the tail's line
    auto block_of = [&](long long g) -> int {
        const long long heavy = (long long)p.extra * (p.share + 1);
        return g < heavy ? (int)(g / (p.share + 1)) : (int)(p.extra + (g - heavy) / p.share);
    };
    const long long piece_begin = begin_of(blockIdx.x), piece_end = begin_of(blockIdx.x + 1);
    // Tiles are numbered in columns of eight token tiles: within a column token tile first, then
    // feature tile (the blocks at work at one time share few weight tiles and eight token tiles,
    // however long the prompt), column after column.
    const int feature_tiles = (int)(p.tiles / p.token_tiles);
    auto locate = [&](long long tile, int& token_tile, int& feature_tile) {
        const long long column = tile / (8LL * feature_tiles), within = tile - column * 8 * feature_tiles;
        const int wide = min(8, p.token_tiles - (int)column * 8);
        token_tile = (int)column * 8 + (int)(within % wide);
        feature_tile = (int)(within / wide);
    };

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbarrier_init(&full_bar[s], 1);
            mbarrier_init(&empty_bar[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbarrier_init(&ready_bar[b], 1);       // the tensor core has finished an accumulator
            mbarrier_init(&drained_bar[b], 128);   // every epilogue thread has read it out
        }
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
        int issued = 0;                                   // stages filled so far
        auto load = [&](long long tile, int kb_first, int kb_count) {
            int token_tile, feature_tile;
            locate(tile, token_tile, feature_tile);
            const int f0 = feature_tile * SPAN, t0 = token_tile * BN;
            for (int i = 0; i < kb_count; ++i, ++issued) {
                const int s = issued % STAGES;
                if (issued >= STAGES && !mbarrier_wait(&empty_bar[s], ((issued / STAGES) - 1) & 1, abort_flag)) {
                    if (!*abort_flag) { *abort_flag = 1; atomicExch(p.error, 1); }
                    return;
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
            }
        };
        for (int round = 0; round < p.rounds && !*abort_flag; ++round)
            if (blockIdx.x + (long long)round * gridDim.x < p.tail_first)
                load(blockIdx.x + (long long)round * gridDim.x, 0, p.k_blocks);
        for (long long g = piece_begin; g < piece_end && !*abort_flag;) {
            const long long tile = g / p.k_blocks;
            const int kb_first = (int)(g - tile * p.k_blocks);
            const int kb_count = (int)min((long long)(p.k_blocks - kb_first), piece_end - g);
            load(p.tail_first + tile, kb_first, kb_count);
            g += kb_count;
        }
        if (*abort_flag) {  // let the copies in flight land before the block leaves
            for (int i = max(0, issued - STAGES); i < issued; ++i)
                for (unsigned spin = 0; spin < SPIN_LIMIT; ++spin)
                    if (mbarrier_try_wait(&full_bar[i % STAGES], (i / STAGES) & 1)) break;
        }
    } else if (warp == 1 && lane == 0) {
        // -------------------------------------------------------------- issuer
        constexpr unsigned idesc = make_instr_desc(BN);
        int consumed = 0, done = 0;                        // stages read, accumulators finished
        auto multiply = [&](int kb_count) {
            const int buffer = done & 1;
            // The accumulator's last reader (two pieces of work ago) must have read it out.
            if (done >= 2 && !mbarrier_wait(&drained_bar[buffer], ((done >> 1) - 1) & 1, abort_flag)) {
                if (!*abort_flag) { *abort_flag = 1; atomicExch(p.error, 4); }
                return;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const unsigned accumulator = tmem_base + buffer * BUFFER_COLUMNS;
            for (int i = 0; i < kb_count; ++i, ++consumed) {
                const int s = consumed % STAGES;
                if (!mbarrier_wait(&full_bar[s], (consumed / STAGES) & 1, abort_flag)) {
                    if (!*abort_flag) { *abort_flag = 1; atomicExch(p.error, 2); }
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                unsigned char* stage = tiles + (size_t)s * STAGE_BYTES;
                const unsigned long long desc_a = make_smem_desc(stage), desc_b = make_smem_desc(stage + A_BYTES);
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; ++k)  // 32 bytes further inside the swizzle span: +2 in 16-byte units
                    umma_bf16(accumulator, desc_a + 2 * k, desc_b + 2 * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
                umma_commit(&empty_bar[s]);  // arrives when these instructions have read the stage
            }
            umma_commit(&ready_bar[buffer]);  // arrives when the accumulator is complete
            ++done;
        };
        for (int round = 0; round < p.rounds && !*abort_flag; ++round)
            if (blockIdx.x + (long long)round * gridDim.x < p.tail_first) multiply(p.k_blocks);
        for (long long g = piece_begin; g < piece_end && !*abort_flag;) {
            const int kb_first = (int)(g % p.k_blocks);
            const int kb_count = (int)min((long long)(p.k_blocks - kb_first), piece_end - g);
            multiply(kb_count);
            g += kb_count;
        }
    } else if (warp >= 2) {
        // ------------------------------------------------------------ epilogue
        const int quarter = warp & 3;                     // TMEM lanes 32 * quarter .. + 31
        const int row = quarter * 32 + lane;              // row of the tile = TMEM lane
        int done = 0, staged_chunks = 0;
        // The shared tiles this block has brought a part of (the second phase below).
        long long shared_tile[2];
        int shared_first[2], shared_count[2], shared_parts = 0;
        // `tail_tile` < 0: a whole tile of this block's own; else the tile's number within the tail, of
        // which this block brings k-blocks kb_first .. kb_first + kb_count - 1.
        auto finish = [&](long long tile, long long tail_tile, int kb_first, int kb_count) {
            int token_tile, feature_tile;
            locate(tile, token_tile, feature_tile);
            const int f0 = feature_tile * SPAN, t0 = token_tile * BN;
            const int buffer = done & 1;
            const unsigned accumulator = tmem_base + buffer * BUFFER_COLUMNS + ((unsigned)(quarter * 32) << 16);
            bool ok = !*abort_flag && mbarrier_wait(&ready_bar[buffer], (done >> 1) & 1, abort_flag);
            if (!ok && !*abort_flag) { *abort_flag = 1; atomicExch(p.error, 3); }
            ++done;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const bool whole = kb_count == p.k_blocks;    // the tile is this block's alone
            // A shared tile: the blocks that hold its first and last k-block, the parts between them.
            const int first_block = whole ? 0 : block_of(tail_tile * p.k_blocks);
            const int parts = whole ? 1 : block_of((tail_tile + 1) * p.k_blocks - 1) - first_block + 1;
            if (!whole) {
                // This part to the workspace (a block has at most two parts: the one its piece begins
                // with and the one it ends with), column by column so that a warp writes whole lines.
                const long long slot = 2LL * blockIdx.x + (kb_first > 0 || piece_begin == tail_tile * p.k_blocks ? 0 : 1);
                float* mine = p.workspace + slot * BM * BN + row;
#pragma unroll 1
                for (int c = 0; c < BN; c += 16) {
                    float v[16];
                    if (ok) tmem_load_16(accumulator + c, v);
                    else
#pragma unroll
                        for (int i = 0; i < 16; ++i) v[i] = 0.f;
#pragma unroll
                    for (int i = 0; i < 16; ++i) __stcg(mine + (long long)(c + i) * BM, v[i]);
                }
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                mbarrier_arrive(&drained_bar[buffer]);       // the tensor core may have the accumulator back
                __threadfence();
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (threadIdx.x == 64) atomicAdd(p.counters + first_block, 1);   // this part has arrived
                if (shared_parts < 2) {
                    shared_tile[shared_parts] = tile;
                    shared_first[shared_parts] = first_block;
                    shared_count[shared_parts] = parts;
                    ++shared_parts;
                }
                return;
            }
            {
                TY* y = (TY*)p.y;
#pragma unroll 1
                for (int c = 0; c < BN; c += 16) {
                    float v[16];
                    if (ok) tmem_load_16(accumulator + c, v);
                    else
#pragma unroll
                        for (int i = 0; i < 16; ++i) v[i] = 0.f;
                    bool mine = f0 + row < p.features;    // this thread has results of this chunk
                    if (GATED) {
                        // Rows 64..127 hold the up projection of the features in rows 0..63.
                        if (row >= 64)
#pragma unroll
                            for (int i = 0; i < 16; ++i) exchange[(row - 64) * 17 + i] = v[i];
                        asm volatile("bar.sync 1, 128;" ::: "memory");
                        mine = mine && row < 64;
                        if (row < 64)
#pragma unroll
                            for (int i = 0; i < 16; ++i) v[i] = v[i] / (1.0f + expf(-v[i])) * exchange[row * 17 + i];
                        asm volatile("bar.sync 1, 128;" ::: "memory");
                    } else if (p.bias && mine) {
                        const float shift = p.bias[f0 + row];
#pragma unroll
                        for (int i = 0; i < 16; ++i) v[i] += shift;
                    }
                    if (sizeof(TY) == 2 && p.staged) {
                        bf16* out = staging + (staged_chunks & 1) * (16 * SPAN);
                        // The copy that read this buffer two chunks ago must be through with it.
                        if (threadIdx.x == 64 && staged_chunks >= 2) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
                        asm volatile("bar.sync 1, 128;" ::: "memory");
                        if (row < SPAN)
#pragma unroll
                            for (int i = 0; i < 16; ++i) out[i * SPAN + row] = __float2bfloat16_rn(v[i]);
                        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the copy reads what these threads wrote
                        asm volatile("bar.sync 1, 128;" ::: "memory");
                        if (threadIdx.x == 64) tma_store_2d(&map_y, out, f0, t0 + c);
                        ++staged_chunks;
                    } else if (mine) {
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            const int token = t0 + c + i;
                            if (token < p.tokens) y[token * p.ldy + f0 + row] = from_float<TY>(v[i]);
                        }
                    }
                }
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                mbarrier_arrive(&drained_bar[buffer]);
            }
        };
        // A shared tile's second phase: when all its parts have arrived (the blocks of a call are
        // resident together: a cooperative launch), the block that brought the i-th part adds, in the
        // parts' order along k, the i-th share of the tile's token columns, and stores them.
        auto combine = [&](long long tile, int first_block, int parts) {
            int token_tile, feature_tile;
            locate(tile, token_tile, feature_tile);
            const int f0 = feature_tile * SPAN, t0 = token_tile * BN;
            const long long tail_tile = tile - p.tail_first;
            if (threadIdx.x == 64) {
                unsigned spin = 0;
                while (*abort_flag == 0) {
                    int arrived;
                    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(arrived) : "l"(p.counters + first_block) : "memory");
                    if (arrived >= parts) break;
                    if (++spin >= (SPIN_LIMIT >> 4)) { *abort_flag = 1; atomicExch(p.error, 5); }   // about a second
                }
                is_last = *abort_flag;                     // one reading of the flag for all (the barriers below)
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            const bool aborted = is_last != 0;
            __threadfence();
            TY* y = (TY*)p.y;
            const int share = (BN + parts - 1) / parts;
            const int first = (blockIdx.x - first_block) * share;
            const int count = aborted ? 0 : max(0, min(share, min(BN, p.tokens - t0) - first));
            const float shift = (!GATED && p.bias && f0 + row < p.features) ? p.bias[f0 + row] : 0.f;
#pragma unroll 1
            for (int j0 = 0; j0 < count; j0 += 16) {
                // Sixteen columns at a time and four parts' values asked for at once (64 loads in flight a
                // thread: the parts come from other SMs through the L2), added in the parts' order along k.
                float sum[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) sum[j] = 0.f;
#pragma unroll 1
                for (int part0 = 0; part0 < parts; part0 += 4) {
                    float v[4][16];
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const long long holder = first_block + min(part0 + q, parts - 1);
                        const long long slot = 2 * holder + (begin_of(holder) >= tail_tile * p.k_blocks ? 0 : 1);
                        const float* from = p.workspace + slot * BM * BN + (long long)(first + j0) * BM + row;
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            v[q][j] = (part0 + q < parts && j0 + j < count) ? __ldcg(from + j * BM) : 0.f;
                    }
#pragma unroll
                    for (int q = 0; q < 4; ++q)
#pragma unroll
                        for (int j = 0; j < 16; ++j) sum[j] += v[q][j];
                }
                if (GATED) {
                    // Rows 64..127 hold the up projection of the features in rows 0..63.
                    if (row >= 64)
#pragma unroll
                        for (int j = 0; j < 16; ++j) exchange[(row - 64) * 17 + j] = sum[j];
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    if (row < 64 && f0 + row < p.features)
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (j0 + j < count)
                                y[(long long)(t0 + first + j0 + j) * p.ldy + f0 + row] =
                                    from_float<TY>(sum[j] / (1.0f + expf(-sum[j])) * exchange[row * 17 + j]);
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                } else if (f0 + row < p.features) {
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        if (j0 + j < count)
                            y[(long long)(t0 + first + j0 + j) * p.ldy + f0 + row] = from_float<TY>(sum[j] + shift);
                }
            }
            // The last block to have read the parts leaves the tile's counters at zero for the next call.
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (threadIdx.x == 64 && atomicAdd(p.counters + gridDim.x + first_block, 1) == parts - 1) {
                p.counters[first_block] = 0;
                p.counters[gridDim.x + first_block] = 0;
            }
        };
        for (int round = 0; round < p.rounds; ++round)
            if (blockIdx.x + (long long)round * gridDim.x < p.tail_first)
                finish(blockIdx.x + (long long)round * gridDim.x, -1, 0, p.k_blocks);
        for (long long g = piece_begin; g < piece_end;) {
            const long long tail_tile = g / p.k_blocks;
            const int kb_first = (int)(g - tail_tile * p.k_blocks);
            const int kb_count = (int)min((long long)(p.k_blocks - kb_first), piece_end - g);
            finish(p.tail_first + tail_tile, tail_tile, kb_first, kb_count);
            g += kb_count;
        }
        for (int i = 0; i < shared_parts; ++i) combine(shared_tile[i], shared_first[i], shared_count[i]);
        if (threadIdx.x == 64) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");   // the last stores have left
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

int sm_count_of_current_device() {
    static int cached[64] = {0};
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return 1;
    if (!cached[device]) {
        int count = 0;
        if (cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || count < 1) return 1;
        cached[device] = count;
    }
    return cached[device];
}

// A map over y [tokens, features] (bfloat16, leading dimension ld) for stores of 16 tokens x `span` features.
int make_store_map(CUtensorMap* map, void* base, long long tokens, long long features, long long ld, int span) {
    EncodeTiled encode = encode_tiled();
    if (!encode) return KIDI_REFUSED_SIZE;
    const cuuint64_t dims[2] = {(cuuint64_t)features, (cuuint64_t)tokens};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    const cuuint32_t box[2] = {(cuuint32_t)span, 16};
    const cuuint32_t steps[2] = {1, 1};
    CUresult status = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, dims, strides, box, steps,
                             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                             CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return status == CUDA_SUCCESS ? 0 : 1000 + (int)status;
}

// Shared memory of a block: the stages, a kilobyte to align them, the gated epilogue's exchange
// buffer and two buffers of results on their way out.
template <int BN, int STAGES>
constexpr size_t shared_bytes() {
    return (size_t)STAGES * (BM * BK * 2 + BN * BK * 2) + 1024 + 64 * 17 * sizeof(float) + 2 * 16 * BM * sizeof(bf16);
}

// Sets the kernel up (once) and returns how many of its blocks the device promises to hold on an SM
// at a time, which bounds a cooperative launch (0: the set-up failed). For a kernel that allocates
// tensor memory the device reports one, whatever its other needs; two such blocks do run on an SM
// together where shared memory and tensor memory allow (measured), which launches whose blocks do not
// wait for each other make use of.
template <int BN, int STAGES, bool GATED, typename TY>
int blocks_per_sm() {
    constexpr size_t shared = shared_bytes<BN, STAGES>();
    static_assert(shared <= (BN <= 64 ? 113 : 227) * 1024, "the stages fit an SM's shared memory (twice for small tiles)");
    static std::atomic<int> known_by_device[64];         // 0: not asked yet; else the answer + 1
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return 0;
    std::atomic<int>& known = known_by_device[device];
    int value = known.load(std::memory_order_acquire) - 1;
    if (value < 0) {
        auto kernel = gemm_tcgen05_kernel<BN, STAGES, GATED, TY>;
        value = 0;
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared) == cudaSuccess &&
            cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared) ==
                cudaSuccess) {
            int found = 0;
            cudaError_t status = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&found, kernel, THREADS, shared);
            if (status == cudaSuccess)
                value = found > 2 ? 2 : found;             // tensor memory: two accumulator pairs an SM at most anyway
        }
        known.store(value + 1, std::memory_order_release);
    }
    return value;
}

template <int BN, int STAGES, bool GATED, typename TY>
int launch(const CUtensorMap& map_w, const CUtensorMap& map_x, const CUtensorMap& map_y, const Params& p, int blocks,
           cudaStream_t stream) {
    constexpr size_t shared = shared_bytes<BN, STAGES>();
    auto kernel = gemm_tcgen05_kernel<BN, STAGES, GATED, TY>;
    const int per_sm = blocks_per_sm<BN, STAGES, GATED, TY>();
    if (per_sm <= 0) return KIDI_REFUSED_SIZE;
    if (p.rounds > 0) {
        kernel<<<blocks, THREADS, shared, stream>>>(map_w, map_x, map_y, p);
        return kidi_launch_status();
    }
    // Shared tiles: blocks wait for each other's parts, so they must be resident together.
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(blocks, 1, 1);
    config.blockDim = dim3(THREADS, 1, 1);
    config.dynamicSmemBytes = shared;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeCooperative;
    attribute[0].val.cooperative = 1;
    config.attrs = attribute;
    config.numAttrs = 1;
    cudaError_t status = cudaLaunchKernelEx(&config, kernel, map_w, map_x, map_y, p);
    return status != cudaSuccess ? (int)status : kidi_launch_status();
}

template <bool GATED, typename TY>
int by_tokens(int bn, const CUtensorMap& map_w, const CUtensorMap& map_x, const CUtensorMap& map_y, const Params& p,
              int blocks, cudaStream_t stream) {
    switch (bn) {   // stages of 16 KB of weights + 128 bytes a token: two blocks an SM up to 64 tokens, one above
        case 16: return launch<16, 5, GATED, TY>(map_w, map_x, map_y, p, blocks, stream);
        case 32: return launch<32, 4, GATED, TY>(map_w, map_x, map_y, p, blocks, stream);
        case 64: return launch<64, 4, GATED, TY>(map_w, map_x, map_y, p, blocks, stream);
        case 128: return launch<128, 6, GATED, TY>(map_w, map_x, map_y, p, blocks, stream);
        case 256: return launch<256, 4, GATED, TY>(map_w, map_x, map_y, p, blocks, stream);
    }
    return KIDI_REFUSED_SIZE;
}
}  // namespace

// The token tile that fits `tokens` rows.
KIDI_API int kidi_gemm_tcgen05_token_tile(int tokens) {
    return tokens <= 16 ? 16 : tokens <= 32 ? 32 : tokens <= 64 ? 64 : tokens <= 128 ? 128 : 256;
}

namespace {
template <bool GATED>
int blocks_per_sm_of(int bn) {
    switch (bn) {
        case 16: return blocks_per_sm<16, 5, GATED, bf16>();
        case 32: return blocks_per_sm<32, 4, GATED, bf16>();
        case 64: return blocks_per_sm<64, 4, GATED, bf16>();
        case 128: return blocks_per_sm<128, 6, GATED, bf16>();
        case 256: return blocks_per_sm<256, 4, GATED, bf16>();
    }
    return 0;
}
}  // namespace

// Blocks of the kernel for `tokens` rows that are surely resident on an SM together (as the device
// reports it: the bound of a cooperative launch).
KIDI_API int kidi_gemm_tcgen05_blocks_per_sm(int tokens, int gated) {
    const int bn = kidi_gemm_tcgen05_token_tile(tokens);
    return gated ? blocks_per_sm_of<true>(bn) : blocks_per_sm_of<false>(bn);
}

// How many blocks a call launches. With at least as many tiles as blocks that are surely resident
// together, blocks take whole tiles: one each, up to what the SMs hold at a time (two per SM up to 64
// tokens, one above), and rounds of tiles beyond that. With fewer tiles the tiles are shared: as many
// blocks as are surely resident together and get at least four k-blocks each (`splits` > 0 asks
// for that many blocks per tile instead).
KIDI_API int kidi_gemm_tcgen05_blocks(int tokens, int features, int K, int gated, int splits) {
    const int bn = kidi_gemm_tcgen05_token_tile(tokens);
    const long long tiles = (long long)((features + (gated ? 64 : BM) - 1) / (gated ? 64 : BM)) * ((tokens + bn - 1) / bn);
    const int k_blocks = (K + BK - 1) / BK;
    const int per_sm = kidi_gemm_tcgen05_blocks_per_sm(tokens, gated);
    const long long sms = sm_count_of_current_device();
    const long long together = sms * (per_sm > 0 ? per_sm : 1), at_a_time = sms * (bn <= 64 ? 2 : 1);
    if (tiles >= together) return (int)(tiles < at_a_time ? tiles : at_a_time);
    if (splits > 0) {
        long long per_tile = together / tiles;
        if (splits < per_tile) per_tile = splits;
        if (per_tile > k_blocks) per_tile = k_blocks;
        return (int)(tiles * (per_tile < 1 ? 1 : per_tile));
    }
    if (bn >= 128) {
        // Wide tiles: a part's trip through the workspace is long, so a tile is shared only by whole
        // multiples of blocks (measured at 512 rows: 53 us with the k-blocks dealt out evenly over all
        // SMs against 32 us with a block per tile on two thirds of them).
        long long per_tile = together / tiles;
        if (per_tile > k_blocks / 4) per_tile = k_blocks / 4;
        return (int)(tiles * (per_tile < 1 ? 1 : per_tile));
    }
    // The tiles' k-blocks dealt out evenly, a block's piece being at least four of them.
    long long blocks = tiles * k_blocks / 4;
    if (blocks > together) blocks = together;
    return (int)(blocks < tiles ? tiles : blocks);
}

// Floats of workspace a call needs (two partial tiles a block) and, in counters, its number of blocks.
KIDI_API long long kidi_gemm_tcgen05_workspace(int tokens, int features, int K, int gated, int splits) {
    const int bn = kidi_gemm_tcgen05_token_tile(tokens);
    return 2LL * kidi_gemm_tcgen05_blocks(tokens, features, K, gated, splits) * BM * bn;
}

// x [tokens, K] and w [features (2 * features when gated), K] bfloat16, rows 16-byte
// aligned; y [tokens, features] bfloat16 or float32. `workspace` (kidi_gemm_tcgen05_workspace
// floats), `counters` (two per block; zeroed once by the caller; the kernel leaves them zero) and
// `error` are the caller's. `bias` (float32 [features], or null) is added to every row.
KIDI_API int kidi_gemm_tcgen05(const void* x, const void* w, void* y, int y_dtype, int tokens, int features, int K,
                               long long ldx, long long ldw, long long ldy, int gated, int splits, float* workspace,
                               int* counters, int* error, const float* bias, cudaStream_t stream) {
    if (tokens <= 0 || features <= 0) return 0;
    if (K <= 0 || (K & 7) || (ldx & 7) || (ldw & 7) || ((uintptr_t)x & 15) || ((uintptr_t)w & 15) || splits < 0)
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
    p.token_tiles = (tokens + bn - 1) / bn;
    const long long tiles = (long long)((features + span - 1) / span) * p.token_tiles;
    const int blocks = kidi_gemm_tcgen05_blocks(tokens, features, K, gated, splits);
    if (tiles / blocks > 0x7fffffffLL) return KIDI_REFUSED_SIZE;
    p.tiles = tiles;
    // A tile for every block: whole tiles only, block b takes b, b + blocks, ... (sharing the tiles of
    // the last, partly filled round out in k-blocks was measured slower: the parts' trip through the
    // workspace costs more than the idle SMs). Fewer tiles than blocks: all of it is tail.
    p.rounds = tiles >= blocks ? (int)((tiles + blocks - 1) / blocks) : 0;
    p.tail_first = tiles >= blocks ? tiles : 0;
    const long long tail = (tiles - p.tail_first) * p.k_blocks;   // dealt out in k-blocks
    p.share = (int)(tail / blocks);
    p.extra = (int)(tail % blocks);
    if (!workspace || !counters || !error) return KIDI_REFUSED_SIZE;
    CUtensorMap map_w, map_x;
    int status = make_map(&map_w, w, gated ? 2LL * features : features, K, ldw, gated ? 64 : BM);
    if (status) return status;
    status = make_map(&map_x, x, tokens, K, ldx, bn);
    if (status) return status;
    // bfloat16 results whose rows 16-byte copies can write leave through shared memory and TMA stores.
    CUtensorMap map_y;
    memset(&map_y, 0, sizeof(map_y));
    p.staged = y_dtype == KIDI_BF16 && !(ldy & 7) && !((uintptr_t)y & 15);
    if (p.staged) {
        status = make_store_map(&map_y, y, tokens, features, ldy, span);
        if (status) return status;
    }
    if (gated) {
        if (y_dtype != KIDI_BF16) return KIDI_REFUSED_DTYPE;
        if (bias) return KIDI_REFUSED_SIZE;
        return by_tokens<true, bf16>(bn, map_w, map_x, map_y, p, blocks, stream);
    }
    if (y_dtype == KIDI_BF16) return by_tokens<false, bf16>(bn, map_w, map_x, map_y, p, blocks, stream);
    if (y_dtype == KIDI_F32) return by_tokens<false, float>(bn, map_w, map_x, map_y, p, blocks, stream);
    return KIDI_REFUSED_DTYPE;
}
