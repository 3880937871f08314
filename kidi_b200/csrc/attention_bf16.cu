// Causal grouped-query attention in bfloat16 on the tensor cores, compiled for one
// head width (-DKIDI_HEAD_DIM=..., a multiple of 16 up to 256):
//
//  * kidi_attention_prefill: every row of a step (whole prompts, or chunks that
//    continue a cached prefix) against its sequence's keys. A block owns 64 query
//    rows of one (sequence, head) and walks the keys in tiles of 64 aligned to
//    absolute positions; keys of the step's own rows come from the packed qkv rows,
//    earlier ones from the paged cache.
//  * kidi_attention_decode: one query row per sequence against the cache only. A
//    block owns one (sequence, key/value head, split of the key range): the query heads
//    that share the key/value head are the rows of one tensor-core tile, the four
//    warps split each 64-key page, and splits are merged by kidi_attention_combine in
//    split order. Partial results live in a caller-provided workspace.
//
// Scores are (q . k) * scale in 32-bit, the softmax (running maximum, exponentials,
// denominator) is 32-bit, probabilities are rounded to bfloat16 for the product with
// V, which accumulates in 32-bit. Formulas: src/kidi/layers/qwen3.cpp:53-54,
// src/kidi/runtime/vulkan/attention.comp:32-101; causal rule
// src/kidi/model/gemma4.cpp:736-740.
#include <atomic>
#include <cstddef>

#include <cooperative_groups.h>
#include <cuda.h>

#include "common.cuh"
#include "attention_no_alloc.h"


#ifndef KIDI_HEAD_DIM
#error "compile with -DKIDI_HEAD_DIM=<head width>"
#endif

namespace {

constexpr int D = KIDI_HEAD_DIM;
static_assert(D % 16 == 0 && D >= 16 && D <= 256, "head width must be a multiple of 16 up to 256");
constexpr int PITCH = D + 8;            // elements; rows shift by 4 banks, ldmatrix is conflict-free
constexpr int TILE = 64;                // keys per tile = cache page size
constexpr int CHUNKS = D / 8;           // 16-byte chunks per row
constexpr int THREADS = 128;
constexpr float LOG2E = 1.4426950408889634f;
// Shared memory of a decode block: the query rows and two key and two value tiles (or, once
// they are consumed, the warps' partial results).
constexpr size_t DECODE_TILES = (size_t)(16 + 4 * TILE) * PITCH * sizeof(bf16);
constexpr size_t DECODE_MERGE =
    (size_t)16 * PITCH * sizeof(bf16) + (size_t)(4 * 16 * D + 4 * 16 * 2 + 2 * 8 * 32 + 8) * sizeof(float);
constexpr size_t DECODE_SHARED = DECODE_TILES > DECODE_MERGE ? DECODE_TILES : DECODE_MERGE;
// The kernel for at most eight query heads a key/value head keeps eight query rows, and
// behind its tiles what the other blocks of a cluster send it: [splits][share] partial
// values and [8 splits][8 heads] maxima and denominators. Three blocks of head width 128
// fit an SM.
constexpr int NARROW_RECV_OUT_FLOATS = 8 * D + 8 * 4;    // [splits][share], share rounded up to four
constexpr int NARROW_RECV_FLOATS = NARROW_RECV_OUT_FLOATS + 8 * 8 * 2;
constexpr size_t NARROW_TILES = (size_t)(8 + 4 * TILE) * PITCH * sizeof(bf16);
constexpr size_t NARROW_MERGE =
    (size_t)8 * PITCH * sizeof(bf16) + (size_t)(4 * 8 * (D + 4) + 4 * 8 * 2 + 2 * 8 * 32 + 8) * sizeof(float);
constexpr size_t NARROW_TILE_BYTES = ((NARROW_TILES > NARROW_MERGE ? NARROW_TILES : NARROW_MERGE) + 15) / 16 * 16;
constexpr size_t NARROW_SHARED = NARROW_TILE_BYTES + NARROW_RECV_FLOATS * sizeof(float);
// The swizzled form: four unpadded tiles on a 1024-byte boundary, then the query rows (the
// warps' partial results reuse the tiles).
constexpr size_t SWIZZLED_TILE_BYTES = ((size_t)(4 * TILE * D + 8 * PITCH) * sizeof(bf16) + 15) / 16 * 16;
constexpr size_t SWIZZLED_SHARED = 1024 + SWIZZLED_TILE_BYTES + NARROW_RECV_FLOATS * sizeof(float);
// The ring form of it: three tiles.
constexpr size_t RING_TILE_BYTES = ((size_t)(3 * TILE * D + 8 * PITCH) * sizeof(bf16) + 15) / 16 * 16;
constexpr size_t RING_SHARED = 1024 + RING_TILE_BYTES + NARROW_RECV_FLOATS * sizeof(float);
static_assert((size_t)(4 * 8 * (D + 4) + 4 * 8 * 2 + 2 * 8 * 32 + 8) * sizeof(float) <= (size_t)3 * TILE * D * sizeof(bf16) || D % 64,
              "the warps' partial results fit the tiles");

__device__ __forceinline__ unsigned smem_address(const void* pointer) {
    return (unsigned)__cvta_generic_to_shared(pointer);
}

__device__ __forceinline__ void copy_async_16(void* shared, const void* global, bool valid) {
    const int bytes = valid ? 16 : 0;  // 0: the destination is filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_address(shared)), "l"(global), "r"(bytes));
}
__device__ __forceinline__ void copy_async_commit() { asm volatile("cp.async.commit_group;"); }
template <int N> __device__ __forceinline__ void copy_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* shared) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(smem_address(shared)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], const void* shared) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(smem_address(shared)));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float low, float high) {
    __nv_bfloat162 pair = __floats2bfloat162_rn(low, high);
    return *reinterpret_cast<unsigned*>(&pair);
}

struct Args {
    const bf16* q;        // [rows, ldq], head h at h*D
    long long ldq;
    const bf16* k_step;   // this step's keys [rows, ldkv], kv head g at g*D (prefill only; may be null)
    const bf16* v_step;
    long long ldkv;
    const bf16* k_cache;  // [pages, kv_heads, 64, D]
    const bf16* v_cache;
    CacheGeometry cache;
    bf16* out;            // [rows, ldo]
    long long ldo;
    const int* row_seq;   // [rows]; -1: padding row
    const int* row_pos;   // [rows]
    const int* seq_slot;  // [seqs]
    const int* seq_start; // [seqs] tokens cached before this step
    const int* seq_len;   // [seqs] tokens this step brings
    const int* seq_row0;  // [seqs] first packed row
    int rows, seqs, heads, kv_heads, window;  // window 0: none
    float scale;
    // decode only
    float* partial_out;   // [rows, heads, splits, D]
    float* partial_stat;  // [rows, heads, splits, 2]  (maximum in log2 units, denominator)
    int splits;
    int* counters;        // [rows, kv_heads], zero between calls: the last block of a (row, kv head) merges its splits
    // decode with eight query heads a key/value head at most: the step's rows come as the
    // projection left them (q at `q`, the new key and value rows at k_step and v_step), and
    // the kernel normalises and rotates them itself and writes the new key and value to
    // the cache (src/kidi/layers/qwen3.cpp:46-57: norm, then rotation, then attention).
    int fuse;             // bit 0: normalise and rotate q and the new k; bit 1: write the new k and v to the cache
    int norm_is_float;    // the norm weights are float32 (else bfloat16)
    const void* q_norm;   // [D] or null
    const void* k_norm;
    const float* cos_table;   // [positions, rotary_dim / 2] or null
    const float* sin_table;
    int rotary_dim;
    float eps;
    long long cache_rows;     // rows of head width in k_cache and in v_cache (pages * kv_heads * 64); 0: not told
};

// Loads one 64 x D tile of keys (or values) for absolute key positions [tile*64, tile*64+64)
// of a sequence into padded shared memory. Positions >= step_from come from the step's
// packed rows, earlier ones from the cache; positions > last are zero-filled.
__device__ __forceinline__ void load_tile(bf16* shared, const bf16* step, long long ld_step, int row0, int step_from,
                                          const bf16* cache, const CacheGeometry& geometry, int slot, int kv_head,
                                          int tile, int last) {
    const int base = tile * TILE;
    // Cache address of the tile's first row (rows of a page are contiguous).
    const bf16* page = nullptr;
    if (cache && base < step_from) page = cache + cache_row_offset(geometry, slot, base, kv_head);
    for (int chunk = threadIdx.x; chunk < TILE * CHUNKS; chunk += THREADS) {
        const int r = chunk / CHUNKS, c = chunk - r * CHUNKS;
        const int u = base + r;
        const bf16* source = step ? step : cache;
        bool valid = u <= last;
        if (valid) {
            if (u >= step_from) source = step + (long long)(row0 + u - step_from) * ld_step + (long long)kv_head * D + c * 8;
            else source = page + (long long)r * D + c * 8;
        }
        copy_async_16(shared + r * PITCH + c * 8, source, valid);
    }
}

// Online-softmax update of one warp's 16 x (NT*8) score tile `s` (already in log2
// units and masked with -inf) followed by P*V. Rows g and g+8 of the tile.
template <int NT>
__device__ __forceinline__ void softmax_and_weighted_sum(float (&s)[NT][4], float (&best)[2], float (&denom)[2],
                                                        float (&o)[D / 8][4], const bf16* v_tile, int first_key,
                                                        int lane) {
    float top[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        top[0] = fmaxf(top[0], fmaxf(s[j][0], s[j][1]));
        top[1] = fmaxf(top[1], fmaxf(s[j][2], s[j][3]));
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        top[i] = fmaxf(top[i], __shfl_xor_sync(0xffffffffu, top[i], 1));
        top[i] = fmaxf(top[i], __shfl_xor_sync(0xffffffffu, top[i], 2));
    }
    float keep[2], use[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const float next = fmaxf(best[i], top[i]);
        use[i] = next == -INFINITY ? 0.f : next;  // a row that has seen no key yet
        keep[i] = exp2f(best[i] - use[i]);
        best[i] = next;
    }
    float sum[2] = {0.f, 0.f};
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        s[j][0] = exp2f(s[j][0] - use[0]);
        s[j][1] = exp2f(s[j][1] - use[0]);
        s[j][2] = exp2f(s[j][2] - use[1]);
        s[j][3] = exp2f(s[j][3] - use[1]);
        sum[0] += s[j][0] + s[j][1];
        sum[1] += s[j][2] + s[j][3];
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        sum[i] += __shfl_xor_sync(0xffffffffu, sum[i], 1);
        sum[i] += __shfl_xor_sync(0xffffffffu, sum[i], 2);
        denom[i] = denom[i] * keep[i] + sum[i];
    }
#pragma unroll
    for (int n = 0; n < D / 8; ++n) {
        o[n][0] *= keep[0];
        o[n][1] *= keep[0];
        o[n][2] *= keep[1];
        o[n][3] *= keep[1];
    }
    // P (bf16) times V: 16 keys per k-step = two score tiles.
    const int matrix = lane >> 3, within = lane & 7;
#pragma unroll
    for (int kk = 0; kk < NT / 2; ++kk) {
        unsigned p[4] = {pack_bf16(s[2 * kk][0], s[2 * kk][1]), pack_bf16(s[2 * kk][2], s[2 * kk][3]),
                         pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]), pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3])};
        const int key = first_key + kk * 16 + within + (matrix & 1) * 8;
#pragma unroll
        for (int n = 0; n < D / 16; ++n) {
            unsigned v[4];
            ldmatrix_x4_trans(v, v_tile + key * PITCH + n * 16 + (matrix >> 1) * 8);
            mma_bf16(o[2 * n], p, v[0], v[1]);
            mma_bf16(o[2 * n + 1], p, v[2], v[3]);
        }
    }
}

// Scores of one warp: 16 query rows (A from q_tile rows [q_row, q_row+16)) against
// NT*8 keys starting at `first_key` of k_tile, times scale_log2.
template <int NT>
__device__ __forceinline__ void scores(float (&s)[NT][4], const bf16* q_tile, int q_row, const bf16* k_tile,
                                       int first_key, float scale_log2, int lane) {
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) s[j][i] = 0.f;
    const int matrix = lane >> 3, within = lane & 7;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
        unsigned a[4];
        ldmatrix_x4(a, q_tile + (q_row + within + (matrix & 1) * 8) * PITCH + kk * 16 + (matrix >> 1) * 8);
#pragma unroll
        for (int jj = 0; jj < NT / 2; ++jj) {
            unsigned b[4];
            ldmatrix_x4(b, k_tile + (first_key + jj * 16 + within + (matrix >> 1) * 8) * PITCH + kk * 16 + (matrix & 1) * 8);
            mma_bf16(s[2 * jj], a, b[0], b[1]);
            mma_bf16(s[2 * jj + 1], a, b[2], b[3]);
        }
    }
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) s[j][i] *= scale_log2;
}

// ------------------------------------------------------------------- prefill
__global__ void __launch_bounds__(THREADS) attention_prefill_kernel(Args a) {
    extern __shared__ __align__(16) unsigned char raw[];
    bf16* q_tile = reinterpret_cast<bf16*>(raw);            // [64][PITCH]
    bf16* k_tiles = q_tile + TILE * PITCH;                  // [2][64][PITCH]
    bf16* v_tiles = k_tiles + 2 * TILE * PITCH;             // [2][64][PITCH]
    const int seq = blockIdx.y, head = blockIdx.z;
    const int q0 = blockIdx.x * TILE;
    const int count = a.seq_len[seq];
    if (q0 >= count) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int start = a.seq_start[seq], row0 = a.seq_row0[seq], slot = a.seq_slot[seq];
    const int kv_head = head / (a.heads / a.kv_heads);
    const int q_rows = min(TILE, count - q0);
    const int last = start + count - 1;                     // last key position that exists
    const int step_from = a.k_step ? start : 0x7fffffff;
    const int high = start + q0 + q_rows - 1;               // largest query position of the block
    const int low = a.window > 0 ? max(0, start + q0 - a.window + 1) : 0;
    const int tile_low = low / TILE, tile_high = high / TILE;

    for (int chunk = threadIdx.x; chunk < TILE * CHUNKS; chunk += THREADS) {
        const int r = chunk / CHUNKS, c = chunk - r * CHUNKS;
        const bool valid = r < q_rows;
        const bf16* source = a.q + (long long)(row0 + q0 + (valid ? r : 0)) * a.ldq + (long long)head * D + c * 8;
        copy_async_16(q_tile + r * PITCH + c * 8, source, valid);
    }
    load_tile(k_tiles, a.k_step, a.ldkv, row0, step_from, a.k_cache, a.cache, slot, kv_head, tile_low, last);
    load_tile(v_tiles, a.v_step, a.ldkv, row0, step_from, a.v_cache, a.cache, slot, kv_head, tile_low, last);
    copy_async_commit();

    float best[2] = {-INFINITY, -INFINITY}, denom[2] = {0.f, 0.f};
    float o[D / 8][4];
#pragma unroll
    for (int n = 0; n < D / 8; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) o[n][i] = 0.f;
    const float scale_log2 = a.scale * LOG2E;
    const int position0 = start + q0 + warp * 16 + g;       // query position of accumulator rows 0,1 (and +8 for 2,3)

    for (int tile = tile_low; tile <= tile_high; ++tile) {
        const int buffer = (tile - tile_low) & 1;
        if (tile < tile_high) {
            load_tile(k_tiles + (buffer ^ 1) * TILE * PITCH, a.k_step, a.ldkv, row0, step_from, a.k_cache, a.cache,
                      slot, kv_head, tile + 1, last);
            load_tile(v_tiles + (buffer ^ 1) * TILE * PITCH, a.v_step, a.ldkv, row0, step_from, a.v_cache, a.cache,
                      slot, kv_head, tile + 1, last);
            copy_async_commit();
            copy_async_wait<1>();
        } else {
            copy_async_wait<0>();
        }
        __syncthreads();
        // Warps whose 16 query rows do not exist, or lie wholly before this tile, have nothing to do.
        const bool active = warp * 16 < q_rows && start + q0 + warp * 16 + 15 >= tile * TILE;
        if (active) {
            float s[8][4];
            scores<8>(s, q_tile, warp * 16, k_tiles + buffer * TILE * PITCH, 0, scale_log2, lane);
#pragma unroll
            for (int j = 0; j < 8; ++j)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int u = tile * TILE + j * 8 + 2 * t + (i & 1);
                    const int p = position0 + (i >> 1) * 8;
                    const bool visible = u <= p && (a.window <= 0 || u > p - a.window);
                    if (!visible) s[j][i] = -INFINITY;
                }
            softmax_and_weighted_sum<8>(s, best, denom, o, v_tiles + buffer * TILE * PITCH, 0, lane);
        }
        __syncthreads();
    }

#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int r = warp * 16 + g + half * 8;
        if (r >= q_rows) continue;
        const float inverse = 1.0f / denom[half];
        bf16* out = a.out + (long long)(row0 + q0 + r) * a.ldo + (long long)head * D;
#pragma unroll
        for (int n = 0; n < D / 8; ++n) {
            const unsigned pair = pack_bf16(o[n][half * 2] * inverse, o[n][half * 2 + 1] * inverse);
            *reinterpret_cast<unsigned*>(out + n * 8 + 2 * t) = pair;
        }
    }
}

// -------------------------------------------------------------------- decode
// grid (splits, kv_heads, rows). The `group` query heads of a key/value head are rows
// 0..group-1 of a 16-row tile (group <= 16); warp w takes keys 16w..16w+15 of each page.
__global__ void __launch_bounds__(THREADS) attention_decode_kernel(Args a) {
    extern __shared__ __align__(16) unsigned char raw[];
    bf16* q_tile = reinterpret_cast<bf16*>(raw);            // [16][PITCH]
    bf16* k_tiles = q_tile + 16 * PITCH;                    // [2][64][PITCH]
    bf16* v_tiles = k_tiles + 2 * TILE * PITCH;             // [2][64][PITCH]
    const int split = blockIdx.x, kv_head = blockIdx.y, row = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int group = a.heads / a.kv_heads;
    const int seq = a.row_seq[row];
    const int head0 = kv_head * group;
    float* merged_out = a.partial_out;   // set below when splits > 1
    float best[2] = {-INFINITY, -INFINITY}, denom[2] = {0.f, 0.f};
    float o[D / 8][4];
#pragma unroll
    for (int n = 0; n < D / 8; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) o[n][i] = 0.f;

    int tiles = 0, tile_first = 0, position = 0, low = 0, slot = 0;
    if (seq >= 0) {
        position = a.row_pos[row];
        slot = a.seq_slot[seq];
        low = a.window > 0 ? max(0, position - a.window + 1) : 0;
        const int tile_low = low / TILE, tile_high = position / TILE;
        const int all = tile_high - tile_low + 1;
        const int per_split = (all + a.splits - 1) / a.splits;
        tile_first = tile_low + split * per_split;
        tiles = max(0, min(per_split, tile_high + 1 - tile_first));
    }
    // The pages of this block do not depend on the kernel before this one, except for the
    // newest token's row: they are asked into L2 before the wait for that kernel; the loads
    // into shared memory, and the query, come after it.
#ifndef KIDI_ATTN_PREFETCH
#define KIDI_ATTN_PREFETCH 0
#endif
    for (int line = threadIdx.x; KIDI_ATTN_PREFETCH && line < tiles * (TILE * D * 2 / 128); line += THREADS) {
        const int index = line / (TILE * D * 2 / 128), within = line - index * (TILE * D * 2 / 128);
        const long long offset = cache_row_offset(a.cache, slot, (tile_first + index) * TILE, kv_head) + within * 64;
        prefetch_l2(a.k_cache + offset);
        prefetch_l2(a.v_cache + offset);
    }
    if (tiles > 0) {
        for (int chunk = threadIdx.x; chunk < 16 * CHUNKS; chunk += THREADS) {
            const int r = chunk / CHUNKS, c = chunk - r * CHUNKS;
            const bool valid = r < group;
            const bf16* source = a.q + (long long)row * a.ldq + (long long)(head0 + (valid ? r : 0)) * D + c * 8;
            copy_async_16(q_tile + r * PITCH + c * 8, source, valid);
        }
        load_tile(k_tiles, nullptr, 0, 0, 0x7fffffff, a.k_cache, a.cache, slot, kv_head, tile_first, position);
        load_tile(v_tiles, nullptr, 0, 0, 0x7fffffff, a.v_cache, a.cache, slot, kv_head, tile_first, position);
        copy_async_commit();
        const float scale_log2 = a.scale * LOG2E;
        for (int index = 0; index < tiles; ++index) {
            const int tile = tile_first + index, buffer = index & 1;
            if (index + 1 < tiles) {
                load_tile(k_tiles + (buffer ^ 1) * TILE * PITCH, nullptr, 0, 0, 0x7fffffff, a.k_cache, a.cache, slot,
                          kv_head, tile + 1, position);
                load_tile(v_tiles + (buffer ^ 1) * TILE * PITCH, nullptr, 0, 0, 0x7fffffff, a.v_cache, a.cache, slot,
                          kv_head, tile + 1, position);
                copy_async_commit();
                copy_async_wait<1>();
            } else {
                copy_async_wait<0>();
            }
            __syncthreads();
            const int first_key = warp * 16;
            if (tile * TILE + first_key <= position && tile * TILE + first_key + 15 >= low) {
                float s[2][4];
                scores<2>(s, q_tile, 0, k_tiles + buffer * TILE * PITCH, first_key, scale_log2, lane);
#pragma unroll
                for (int j = 0; j < 2; ++j)
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int u = tile * TILE + first_key + j * 8 + 2 * t + (i & 1);
                        if (u > position || u < low) s[j][i] = -INFINITY;
                    }
                softmax_and_weighted_sum<2>(s, best, denom, o, v_tiles + buffer * TILE * PITCH, first_key, lane);
            }
            __syncthreads();
        }
    }

    // Merge the four warps in warp order through shared memory (the tiles are free now).
    float* merge_out = reinterpret_cast<float*>(k_tiles);                // [4][16][D]
    float* merge_stat = merge_out + 4 * 16 * D;                          // [4][16][2]
    __syncthreads();
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int r = g + half * 8;
#pragma unroll
        for (int n = 0; n < D / 8; ++n) {
            merge_out[(warp * 16 + r) * D + n * 8 + 2 * t] = o[n][half * 2];
            merge_out[(warp * 16 + r) * D + n * 8 + 2 * t + 1] = o[n][half * 2 + 1];
        }
        if (t == 0) {
            merge_stat[(warp * 16 + r) * 2] = best[half];
            merge_stat[(warp * 16 + r) * 2 + 1] = denom[half];
        }
    }
    __syncthreads();
    for (int item = threadIdx.x; item < group * D; item += THREADS) {
        const int r = item / D, c = item - r * D;
        float top = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) top = fmaxf(top, merge_stat[(w * 16 + r) * 2]);
        float total = 0.f, value = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float m = merge_stat[(w * 16 + r) * 2];
            const float factor = m == -INFINITY ? 0.f : exp2f(m - top);
            total += merge_stat[(w * 16 + r) * 2 + 1] * factor;
            value += merge_out[(w * 16 + r) * D + c] * factor;
        }
        const int head = head0 + r;
        if (a.splits == 1) {
            a.out[(long long)row * a.ldo + (long long)head * D + c] =
                from_float<bf16>(total > 0.f ? value / total : 0.f);
        } else {
            const long long where = ((long long)row * a.heads + head) * a.splits + split;
            merged_out[where * D + c] = value;
            if (c == 0) {
                a.partial_stat[where * 2] = top;
                a.partial_stat[where * 2 + 1] = total;
            }
        }
    }
}

// The same for at most eight query heads per key/value head, in the transposed form that
// needs half the tensor-core instructions and half the accumulator registers: the keys
// are the rows of the score tile, S^T = K Q^T (16 keys x 8 heads per warp), and the
// output is accumulated transposed, O^T = V^T P^T (head_dim x 8 heads). P^T reaches the
// layout of a B operand through two 8x8 register transposes (movmatrix).
__device__ int kidi_attention_timeout = 0;  // set when a bounded wait for a tile ran out

__device__ __forceinline__ void bulk_copy_row(void* shared, const void* global, unsigned bytes,
                                              unsigned long long* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_address(shared)),
                 "l"(global), "r"(bytes), "r"(smem_address(bar))
                 : "memory");
}

__device__ __forceinline__ void tensor_copy_2d(void* shared, const CUtensorMap* map, unsigned long long* bar, int x,
                                               int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        :
        : "r"(smem_address(shared)), "l"((unsigned long long)map), "r"(smem_address(bar)), "r"(x), "r"(y)
        : "memory");
}

// One 64-row tile of keys and one of values, a bulk copy per row (rows are contiguous in
// the cache and padded in shared memory): threads 0..63 bring key rows, 64..127 value
// rows, thread 0 tells the barrier how many bytes to expect. Rows beyond `rows_valid`
// are left as they are (their scores are masked; the caller keeps their values finite).
__device__ __forceinline__ void issue_tile(bf16* k_tile, bf16* v_tile, const bf16* k_cache, const bf16* v_cache,
                                           const CacheGeometry& geometry, int slot, int kv_head, int tile,
                                           int rows_valid, unsigned long long* bar) {
    const long long page = cache_row_offset(geometry, slot, tile * TILE, kv_head);
    const int r = threadIdx.x & 63;
    if (threadIdx.x == 0)
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_address(bar)),
                     "r"((unsigned)(rows_valid * D * 2 * 2))
                     : "memory");
    if (r < rows_valid) {
        if (threadIdx.x < 64) bulk_copy_row(k_tile + r * PITCH, k_cache + page + (long long)r * D, D * 2, bar);
        else bulk_copy_row(v_tile + r * PITCH, v_cache + page + (long long)r * D, D * 2, bar);
    }
}

__device__ __forceinline__ void wait_tile(unsigned long long* bar, unsigned parity) {
    for (unsigned spin = 0; spin < (1u << 24); ++spin) {
        unsigned done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(smem_address(bar)), "r"(parity)
            : "memory");
        if (done) return;
    }
    kidi_attention_timeout = 1;
}

__device__ __forceinline__ unsigned transpose_8x8(unsigned packed) {
    unsigned out;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(out) : "r"(packed));
    return out;
}

// Eight elements c0..c0+7 of a head, normalised and rotated as the separate kernel does it
// (rope_store_bf16_kernel: the same operations in the same order, in 32-bit): `own` holds
// them as the projection left them, `partner` the eight elements half a rotation away,
// `square_sum` the sum of squares over the whole head.
__device__ __forceinline__ uint4 normalise_rotate(uint4 own, uint4 partner, float square_sum, const Args& a,
                                                  const void* weight, int c0, int position) {
    const __nv_bfloat162* mine = reinterpret_cast<const __nv_bfloat162*>(&own);
    const __nv_bfloat162* theirs = reinterpret_cast<const __nv_bfloat162*>(&partner);
    float v[8], other[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 x = __bfloat1622float2(mine[i]), y = __bfloat1622float2(theirs[i]);
        v[2 * i] = x.x; v[2 * i + 1] = x.y;
        other[2 * i] = y.x; other[2 * i + 1] = y.y;
    }
    const int half = a.rotary_dim / 2;
    const bool low = c0 < half;
    const int partner_c0 = low ? c0 + half : c0 - half;
    if (weight) {
        const float inv = 1.0f / sqrtf(square_sum / (float)D + a.eps);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float w = a.norm_is_float ? ((const float*)weight)[c0 + i] : to_float(((const bf16*)weight)[c0 + i]);
            v[i] = v[i] * inv * w;
        }
        if (a.cos_table && c0 < a.rotary_dim) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float w = a.norm_is_float ? ((const float*)weight)[partner_c0 + i]
                                                : to_float(((const bf16*)weight)[partner_c0 + i]);
                other[i] = other[i] * inv * w;
            }
        }
    }
    if (a.cos_table && c0 < a.rotary_dim) {
        const int j = low ? c0 : c0 - half;
        const float4* cosine = reinterpret_cast<const float4*>(a.cos_table + (long long)position * half + j);
        const float4* sine = reinterpret_cast<const float4*>(a.sin_table + (long long)position * half + j);
        const float4 ca = cosine[0], cb = cosine[1], sa = sine[0], sb = sine[1];
        const float c8[8] = {ca.x, ca.y, ca.z, ca.w, cb.x, cb.y, cb.z, cb.w};
        const float s8[8] = {sa.x, sa.y, sa.z, sa.w, sb.x, sb.y, sb.z, sb.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = v[i] * c8[i] + (low ? -other[i] : other[i]) * s8[i];
    }
    uint4 packed;
    __nv_bfloat162* out = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
    for (int i = 0; i < 4; ++i) out[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    return packed;
}

// The sum of squares of a head of which lane l holds elements 8l..8l+7 (lanes past the
// head hold zeros), added in the order of the separate kernel.
__device__ __forceinline__ float head_square_sum(uint4 own) {
    const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(&own);
    float square = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 two = __bfloat1622float2(pairs[i]);
        square = fmaf(two.x, two.x, square);
        square = fmaf(two.y, two.y, square);
    }
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) square += __shfl_xor_sync(0xffffffffu, square, offset);
    return square;
}

// CLUSTER: the blocks that share a (row, key/value head), one per split, form a thread-block
// cluster and merge their partial results through distributed shared memory (no trip
// through global memory, no second kernel); at most 8 splits.
// SWIZZLED (head widths that are multiples of 64): a page of keys or values comes as one
// TMA tensor copy per 64 columns with the 128-byte swizzle, into rows without padding, and
// ldmatrix reads it through the same swizzle. Measured on a B200 at batch 64 the 128 small
// row copies per tile of the other form hold the stream at 4.6 TB/s where page copies
// reach 5.7 TB/s. A page is copied whole: rows past the sequence's end hold what the
// cache held before (zeros or an earlier sequence's finite values), and their weights
// are exact zeros.
template <bool CLUSTER, int FORM>
__global__ void __launch_bounds__(THREADS, 4)     // four blocks an SM where shared memory allows (the ring form; narrow heads)
attention_decode_narrow_kernel(const __grid_constant__ CUtensorMap k_map, const __grid_constant__ CUtensorMap v_map,
                               Args a) {
    constexpr bool SWIZZLED = FORM != 0, RING = FORM == 2;
    constexpr int BUFFERS = RING ? 3 : 4;
    extern __shared__ __align__(16) unsigned char raw_unaligned[];
    // Swizzled tiles want 1024-byte boundaries and come first; the query rows follow them.
    unsigned char* raw = SWIZZLED ? (unsigned char*)(((uintptr_t)raw_unaligned + 1023) & ~(uintptr_t)1023) : raw_unaligned;
    constexpr int TP = SWIZZLED ? D : PITCH;               // elements between rows of a key or value tile
    bf16* q_tile = reinterpret_cast<bf16*>(raw) + (SWIZZLED ? BUFFERS * TILE * TP : 0);   // [8][PITCH]
    bf16* k_tiles = SWIZZLED ? reinterpret_cast<bf16*>(raw) : q_tile + 8 * PITCH;   // [2][64][TP]
    bf16* v_tiles = k_tiles + 2 * TILE * TP;                                        // [2][64][TP]
    // Where the eight elements from column `col` (a multiple of 8) of row `r` of a tile lie.
    auto tile_at = [](bf16* tile, int r, int col) -> bf16* {
        if (SWIZZLED) return tile + (col >> 6) * (TILE * 64) + r * 64 + ((((col & 63) >> 3) ^ (r & 7)) << 3);
        return tile + r * PITCH + col;
    };
    const int split = blockIdx.x, kv_head = blockIdx.y, row = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int matrix = lane >> 3, within = lane & 7;
    const int group = a.heads / a.kv_heads;                 // <= 8
    const int seq = a.row_seq[row];
    const int head0 = kv_head * group;
    // Lane (g, t) keeps heads 2t and 2t+1: running maximum, its own share of the
    // denominator, and O^T[dims g / g+8 of each 16-dim tile][heads 2t, 2t+1].
    float best[2] = {-INFINITY, -INFINITY}, denom[2] = {0.f, 0.f};
    float o[D / 16][4];
#pragma unroll
    for (int n = 0; n < D / 16; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) o[n][i] = 0.f;

    // A step of one token per sequence has row b for sequence b: the position and the slot are asked
    // for together with the row's sequence instead of after it (one trip instead of two).
    const int guess = row < a.seqs ? row : 0;
    const int position_ahead = a.row_pos[row], slot_ahead = a.seq_slot[guess];
    int tiles = 0, tile_first = 0, position = 0, low = 0, slot = 0;
    if (seq >= 0) {
        position = position_ahead;
        slot = seq == guess ? slot_ahead : a.seq_slot[seq];
        low = a.window > 0 ? max(0, position - a.window + 1) : 0;
        const int tile_low = low / TILE, tile_high = position / TILE;
        const int all = tile_high - tile_low + 1;
        const int per_split = (all + a.splits - 1) / a.splits;
        tile_first = tile_low + split * per_split;
        tiles = max(0, min(per_split, tile_high + 1 - tile_first));
    }
    __shared__ unsigned long long tile_bar[3];
    constexpr int PAGES_AHEAD = 16;                          // (four blocks of the ring form fill an SM to 200 bytes)
    __shared__ int page_of[PAGES_AHEAD];                     // the pages of the block's first tiles
    if (tiles > 0) {
        if (SWIZZLED && threadIdx.x < min(tiles, PAGES_AHEAD)) {   // all at once, not one look-up before each copy
            int page_index = tile_first + threadIdx.x;
            if (a.cache.ring_pages) page_index %= a.cache.ring_pages;
            page_of[threadIdx.x] = a.cache.table[(long long)slot * a.cache.pages_per_seq + page_index];
        }
        if (threadIdx.x == 0) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_address(&tile_bar[0])));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_address(&tile_bar[1])));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_address(&tile_bar[2])));
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
        __syncthreads();
        // With the rotation fused the step's own key and value are not in the cache yet: the
        // block whose last tile holds position `position` computes them, puts them into its
        // tile and (bit 1) into the cache; the copies leave that row out.
        const int new_tile = position / TILE;
        const bool has_new = a.fuse != 0 && tile_first + tiles - 1 == new_tile;
        auto rows_to_copy = [&](int tile) {
            return min(TILE, position - tile * TILE + 1) - (a.fuse != 0 && tile == new_tile ? 1 : 0);
        };
        // The first row of the block's tile `index` in the cache seen as [rows, D] (pages of 64 rows).
        auto page_row_of = [&](int index) -> int {
            if (index < PAGES_AHEAD) return (page_of[index] * a.cache.kv_heads + kv_head) * TILE;
            return (int)(cache_row_offset(a.cache, slot, (tile_first + index) * TILE, kv_head) / D);
        };
        // The first two tiles are asked for before anything else: the kernel's time is the
        // time its keys and values take to arrive.
        auto issue = [&](int tile, int buffer) {
            if (SWIZZLED) {
                if (threadIdx.x == 0) {         // one copy per 64 columns of the key page and of the value page
                    const int page_row = page_row_of(tile - tile_first);
                    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(
                                     smem_address(&tile_bar[buffer])),
                                 "r"((unsigned)(2 * TILE * D * 2))
                                 : "memory");
                    for (int span = 0; span < D / 64; ++span) {
                        tensor_copy_2d(k_tiles + buffer * TILE * TP + span * TILE * 64, &k_map, &tile_bar[buffer],
                                       span * 64, page_row);
                        tensor_copy_2d(v_tiles + buffer * TILE * TP + span * TILE * 64, &v_map, &tile_bar[buffer],
                                       span * 64, page_row);
                    }
                }
            } else {
                issue_tile(k_tiles + buffer * TILE * TP, v_tiles + buffer * TILE * TP, a.k_cache, a.v_cache, a.cache,
                           slot, kv_head, tile, rows_to_copy(tile), &tile_bar[buffer]);
            }
        };
        // The ring: three buffers that take, in turn, the keys of the block's tile 0, its values,
        // the keys of tile 1, ... (load 2i: keys of tile i, load 2i + 1: its values), each on the
        // barrier of its buffer. Two loads are on their way while a third is read; a block
        // holds 3 instead of 4 tiles, so that four blocks of head width 128 fit an SM.
        auto issue_load = [&](int load) {
            if (threadIdx.x == 0) {
                const int buffer = load % 3;
                const int page_row = page_row_of(load >> 1);
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(
                                 smem_address(&tile_bar[buffer])),
                             "r"((unsigned)(TILE * D * 2))
                             : "memory");
                for (int span = 0; span < D / 64; ++span)
                    tensor_copy_2d(k_tiles + buffer * TILE * TP + span * TILE * 64, (load & 1) ? &v_map : &k_map,
                                   &tile_bar[buffer], span * 64, page_row);
            }
        };
        if (RING) {
            issue_load(0);
            issue_load(1);
            if (tiles > 1) issue_load(2);
        } else {
            issue(tile_first, 0);
            if (tiles > 1) issue(tile_first + 1, 1);
        }
        uint4 new_raw = make_uint4(0u, 0u, 0u, 0u);          // warp 0: the new key row's chunk, warp 1: the value's
        if (has_new && warp < 2 && lane < CHUNKS)
            new_raw = *reinterpret_cast<const uint4*>((warp == 0 ? a.k_step : a.v_step) + (long long)row * a.ldkv +
                                                      (long long)kv_head * D + lane * 8);
        // Value rows that no copy writes must be finite (their weights are exact zeros; a
        // masked score is replaced whatever its key row holds). Only the sequence's last tile
        // can be short, and only while a buffer has not yet held a whole tile can its rows be
        // unwritten: the rows past the end of the block's first two tiles are zeroed (the
        // copies write other rows).
        for (int index = 0; !SWIZZLED && index < 2 && index < tiles; ++index) {
            const int valid = min(TILE, position - (tile_first + index) * TILE + 1);
            for (int chunk = threadIdx.x; chunk < (TILE - valid) * CHUNKS; chunk += THREADS) {
                const int r = valid + chunk / CHUNKS, c = chunk % CHUNKS;
                *reinterpret_cast<uint4*>(v_tiles + (index * TILE + r) * PITCH + c * 8) = make_uint4(0u, 0u, 0u, 0u);
            }
        }
        for (int chunk = threadIdx.x; chunk < 8 * CHUNKS; chunk += THREADS) {
            const int r = chunk / CHUNKS, c = chunk - r * CHUNKS;
            const bool valid = r < group;
            const bf16* source = a.q + (long long)row * a.ldq + (long long)(head0 + (valid ? r : 0)) * D + c * 8;
            copy_async_16(q_tile + r * PITCH + c * 8, source, valid);
        }
        copy_async_commit();
        const float scale_log2 = a.scale * LOG2E;
        unsigned q_frag[D / 16][2];                         // Q^T as B operand: (dims, head g)
        for (int index = 0; index < tiles; ++index) {
            const int tile = tile_first + index, buffer = index & 1;
            const int k_load = 2 * index, v_load = 2 * index + 1;                 // the ring's loads of this tile
            const bool newest = has_new && tile == new_tile;
            if (RING) {
                wait_tile(&tile_bar[k_load % 3], (k_load / 3) & 1);
                if (newest) wait_tile(&tile_bar[v_load % 3], (v_load / 3) & 1);   // the step's value goes into the value tile
            } else {
                wait_tile(&tile_bar[buffer], (index >> 1) & 1);
            }
            if (index == 0) {
                copy_async_wait<0>();
                // The rows zeroed above will be overwritten by later copies: order the two kinds of write.
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncthreads();
                if (a.fuse & 1) {                           // q as the projection left it: norm, then rotation
                    const int half_lanes = a.rotary_dim / 16;
                    const int partner_lane = (lane * 8 < a.rotary_dim / 2 ? lane + half_lanes : lane - half_lanes) & 31;
                    for (int r = warp; r < group; r += 4) {
                        uint4 own = make_uint4(0u, 0u, 0u, 0u);
                        if (lane < CHUNKS) own = *reinterpret_cast<const uint4*>(q_tile + r * PITCH + lane * 8);
                        const float square = head_square_sum(own);
                        uint4 partner;
                        partner.x = __shfl_sync(0xffffffffu, own.x, partner_lane);
                        partner.y = __shfl_sync(0xffffffffu, own.y, partner_lane);
                        partner.z = __shfl_sync(0xffffffffu, own.z, partner_lane);
                        partner.w = __shfl_sync(0xffffffffu, own.w, partner_lane);
                        if (lane < CHUNKS)
                            *reinterpret_cast<uint4*>(q_tile + r * PITCH + lane * 8) =
                                normalise_rotate(own, partner, square, a, a.q_norm, lane * 8, position);
                    }
                    __syncthreads();
                }
#pragma unroll
                for (int kk = 0; kk < D / 32; ++kk) {       // two 16-dim steps per load
                    unsigned r4[4];
                    ldmatrix_x4(r4, q_tile + within * PITCH + kk * 32 + matrix * 8);
                    q_frag[2 * kk][0] = r4[0]; q_frag[2 * kk][1] = r4[1];
                    q_frag[2 * kk + 1][0] = r4[2]; q_frag[2 * kk + 1][1] = r4[3];
                }
                if (D % 32) {                                // an odd number of 16-dim steps: the last one alone
                    unsigned r4[4];
                    ldmatrix_x4(r4, q_tile + within * PITCH + (D / 32) * 32 + (matrix & 1) * 8);
                    q_frag[D / 16 - 1][0] = r4[0]; q_frag[D / 16 - 1][1] = r4[1];
                }
            }
            const int first_key = warp * 16;
            bf16* k_tile = k_tiles + (RING ? k_load % 3 : buffer) * TILE * TP;
            bf16* v_tile = RING ? k_tiles + (v_load % 3) * TILE * TP : v_tiles + buffer * TILE * TP;
            if (newest) {                                   // the step's own key (warp 0) and value (warp 1)
                const int r_new = position - tile * TILE;
                if (warp < 2) {
                    uint4 fresh = new_raw;
                    if (warp == 0 && (a.fuse & 1)) {
                        const int half_lanes = a.rotary_dim / 16;
                        const int partner_lane = (lane * 8 < a.rotary_dim / 2 ? lane + half_lanes : lane - half_lanes) & 31;
                        const float square = head_square_sum(new_raw);
                        uint4 partner;
                        partner.x = __shfl_sync(0xffffffffu, new_raw.x, partner_lane);
                        partner.y = __shfl_sync(0xffffffffu, new_raw.y, partner_lane);
                        partner.z = __shfl_sync(0xffffffffu, new_raw.z, partner_lane);
                        partner.w = __shfl_sync(0xffffffffu, new_raw.w, partner_lane);
                        if (lane < CHUNKS)     // lanes past the head have no weights to read
                            fresh = normalise_rotate(new_raw, partner, square, a, a.k_norm, lane * 8, position);
                    }
                    if (lane < CHUNKS) {
                        *reinterpret_cast<uint4*>(tile_at(warp == 0 ? k_tile : v_tile, r_new, lane * 8)) = fresh;
                        if (a.fuse & 2) {
                            bf16* cache = const_cast<bf16*>(warp == 0 ? a.k_cache : a.v_cache);
                            *reinterpret_cast<uint4*>(cache + cache_row_offset(a.cache, slot, position, kv_head) + lane * 8) =
                                fresh;
                        }
                    }
                }
                __syncthreads();
            }
            const bool active = tile * TILE + first_key <= position && tile * TILE + first_key + 15 >= low;
            unsigned p0 = 0u, p1 = 0u;
            if (active) {
                float s[4] = {0.f, 0.f, 0.f, 0.f};          // keys g (0,1) and g+8 (2,3) x heads 2t, 2t+1
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    unsigned k_frag[4];
                    ldmatrix_x4(k_frag, tile_at(k_tile, first_key + within + (matrix & 1) * 8, kk * 16 + (matrix >> 1) * 8));
                    mma_bf16(s, k_frag, q_frag[kk][0], q_frag[kk][1]);
                }
                const int u0 = tile * TILE + first_key + g, u1 = u0 + 8;
                const bool see0 = u0 <= position && u0 >= low, see1 = u1 <= position && u1 >= low;
                s[0] = see0 ? s[0] * scale_log2 : -INFINITY;
                s[1] = see0 ? s[1] * scale_log2 : -INFINITY;
                s[2] = see1 ? s[2] * scale_log2 : -INFINITY;
                s[3] = see1 ? s[3] * scale_log2 : -INFINITY;
                float top[2] = {fmaxf(s[0], s[2]), fmaxf(s[1], s[3])};
#pragma unroll
                for (int i = 0; i < 2; ++i) {               // over the eight lanes that share t
                    top[i] = fmaxf(top[i], __shfl_xor_sync(0xffffffffu, top[i], 4));
                    top[i] = fmaxf(top[i], __shfl_xor_sync(0xffffffffu, top[i], 8));
                    top[i] = fmaxf(top[i], __shfl_xor_sync(0xffffffffu, top[i], 16));
                }
                float keep[2], use[2];
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    const float next = fmaxf(best[i], top[i]);
                    use[i] = next == -INFINITY ? 0.f : next;
                    keep[i] = exp2f(best[i] - use[i]);
                    best[i] = next;
                }
                s[0] = exp2f(s[0] - use[0]);
                s[1] = exp2f(s[1] - use[1]);
                s[2] = exp2f(s[2] - use[0]);
                s[3] = exp2f(s[3] - use[1]);
                denom[0] = denom[0] * keep[0] + s[0] + s[2];
                denom[1] = denom[1] * keep[1] + s[1] + s[3];
#pragma unroll
                for (int n = 0; n < D / 16; ++n) {
                    o[n][0] *= keep[0]; o[n][1] *= keep[1]; o[n][2] *= keep[0]; o[n][3] *= keep[1];
                }
                p0 = transpose_8x8(pack_bf16(s[0], s[1]));   // keys 2t, 2t+1 of head g
                p1 = transpose_8x8(pack_bf16(s[2], s[3]));   // keys 2t+8, 2t+9
            }
            if (RING) {
                __syncthreads();                            // the keys are read: their buffer takes the next values
                if (v_load + 2 < 2 * tiles) issue_load(v_load + 2);
                wait_tile(&tile_bar[v_load % 3], (v_load / 3) & 1);
            }
            if (active) {
#pragma unroll
                for (int n = 0; n < D / 16; ++n) {          // V^T as A operand: 16 dims x 16 keys
                    unsigned v_frag[4];
                    ldmatrix_x4_trans(v_frag, tile_at(v_tile, first_key + within + (matrix >> 1) * 8, n * 16 + (matrix & 1) * 8));
                    mma_bf16(o[n], v_frag, p0, p1);
                }
            }
            __syncthreads();
            if (RING) {
                if (k_load + 4 < 2 * tiles) issue_load(k_load + 4);   // the values are read: the keys of the tile after next
            } else if (index + 2 < tiles) {
                issue(tile + 2, buffer);                     // the buffer that was just read takes the tile after next
            }
        }
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {                           // the lanes' shares of the denominator
        denom[i] += __shfl_xor_sync(0xffffffffu, denom[i], 4);
        denom[i] += __shfl_xor_sync(0xffffffffu, denom[i], 8);
        denom[i] += __shfl_xor_sync(0xffffffffu, denom[i], 16);
    }

    // Merge the four warps in warp order through shared memory (the tiles are free now). Rows of
    // the partial results are padded by four floats: the 32 lanes of a store hit 32 banks.
    constexpr int MP = D + 4;
    float* merge_out = reinterpret_cast<float*>(k_tiles);                // [4][8][MP]
    float* merge_stat = merge_out + 4 * 8 * MP;                          // [4][8][2]
    // What the other blocks of a cluster send (never used for anything else: a block that is
    // ahead may send while this one still works on its tiles).
    float* recv_out = reinterpret_cast<float*>(raw + (RING ? RING_TILE_BYTES : SWIZZLED ? SWIZZLED_TILE_BYTES : NARROW_TILE_BYTES));   // [splits][share]
    float* recv_stat = recv_out + NARROW_RECV_OUT_FLOATS;                // [8 splits][8 heads][2]
    cooperative_groups::cluster_group cluster = cooperative_groups::this_cluster();
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 2; ++i) {                                        // heads 2t and 2t + 1 of this lane
        const int head = 2 * t + i;
        if (head < group) {
            float* mine = merge_out + (warp * 8 + head) * MP;
#pragma unroll
            for (int n = 0; n < D / 16; ++n) {
                mine[n * 16 + g] = o[n][i];
                mine[n * 16 + g + 8] = o[n][2 + i];
            }
            if (g == 0) {
                merge_stat[(warp * 8 + head) * 2] = best[i];
                merge_stat[(warp * 8 + head) * 2 + 1] = denom[i];
            }
        }
    }
    __syncthreads();
    // Per head: the block's maximum and denominator and each warp's weight in the merge, by the
    // lanes of one warp (lane = 8 * warp of the partial + head; the sums run through a fixed tree
    // of shuffles, so their order does not depend on timing).
    float* merge_weight = merge_stat + 4 * 8 * 2;                        // [4][8], then [8][2]: maximum, denominator
    if (warp == 0) {
        const int source = lane >> 3, r = lane & 7;
        const bool real = r < group;
        const float m = real ? merge_stat[(source * 8 + r) * 2] : -INFINITY;
        const float d = real ? merge_stat[(source * 8 + r) * 2 + 1] : 0.f;
        float top = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 8));
        top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, 16));
        const float factor = m == -INFINITY ? 0.f : exp2f(m - top);
        float total = d * factor;
        total += __shfl_xor_sync(0xffffffffu, total, 8);
        total += __shfl_xor_sync(0xffffffffu, total, 16);
        merge_weight[source * 8 + r] = factor;
        if (source == 0) {
            merge_weight[32 + r * 2] = top;
            merge_weight[32 + r * 2 + 1] = total;
        }
        if (CLUSTER && a.splits > 1) {                                   // every block of the cluster needs them
            for (int base = 0; base < a.splits * group; base += 32) {    // the whole warp shuffles together
                const int i = base + lane;
                const bool sends = i < a.splits * group;
                const int target = sends ? i / group : 0, head = sends ? i - target * group : 0;
                const float head_top = __shfl_sync(0xffffffffu, top, head), head_total = __shfl_sync(0xffffffffu, total, head);
                if (sends)
                    *reinterpret_cast<float2*>(cluster.map_shared_rank(recv_stat, target) + (split * 8 + head) * 2) =
                        make_float2(head_top, head_total);
            }
        }
    }
    __syncthreads();
    // Four elements a thread: the weighted sum of the four warps' partial results, then to where
    // the splits are merged. A cluster's blocks share the output elements in pieces of `share`
    // elements (a multiple of four), and each sends its partial values to the block that merges
    // them (distributed shared memory, 16 bytes a store).
    const int share = CLUSTER ? ((group * D + a.splits - 1) / a.splits + 3) & ~3 : 0;
    for (int item = threadIdx.x * 4; item < group * D; item += THREADS * 4) {
        const int r = item / D, c = item - r * D;
        float4 value = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float4 part = *reinterpret_cast<const float4*>(merge_out + (w * 8 + r) * MP + c);
            const float weight = merge_weight[w * 8 + r];
            value.x += part.x * weight; value.y += part.y * weight; value.z += part.z * weight; value.w += part.w * weight;
        }
        const int head = head0 + r;
        if (a.splits == 1) {
            const float total = merge_weight[32 + r * 2 + 1];
            const float scale = total > 0.f ? 1.0f / total : 0.f;
            bf16* out = a.out + (long long)row * a.ldo + (long long)head * D + c;
            *reinterpret_cast<__nv_bfloat162*>(out) = __floats2bfloat162_rn(value.x * scale, value.y * scale);
            *reinterpret_cast<__nv_bfloat162*>(out + 2) = __floats2bfloat162_rn(value.z * scale, value.w * scale);
        } else if (CLUSTER) {
            const int target = item / share;
            *reinterpret_cast<float4*>(cluster.map_shared_rank(recv_out, target) + split * share + item - target * share) = value;
        } else {
            const long long where = ((long long)row * a.heads + head) * a.splits + split;
            *reinterpret_cast<float4*>(a.partial_out + where * D + c) = value;
            if (c == 0) {
                a.partial_stat[where * 2] = merge_weight[32 + r * 2];
                a.partial_stat[where * 2 + 1] = merge_weight[32 + r * 2 + 1];
            }
        }
    }
    if (CLUSTER && a.splits > 1) {
        // One barrier: after it every block holds, for its share of the output elements, the
        // partial values of all splits, and merges them in split order (so the result does not
        // depend on timing). Nothing is read from another block after the barrier, so a block
        // may leave as soon as it has written its share.
        cluster.sync();
        const int splits = a.splits;                   // == the cluster's size, <= 8
        const int begin = split * share, count = min(group * D, begin + share) - begin;
        for (int i = threadIdx.x * 4; i < count; i += THREADS * 4) {
            const int r = (begin + i) / D, c = begin + i - r * D;
            float top = -INFINITY;
            for (int sp = 0; sp < splits; ++sp) top = fmaxf(top, recv_stat[(sp * 8 + r) * 2]);
            float total = 0.f;
            float4 value = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int sp = 0; sp < splits; ++sp) {
                const float m = recv_stat[(sp * 8 + r) * 2];
                const float factor = m == -INFINITY ? 0.f : exp2f(m - top);
                total += recv_stat[(sp * 8 + r) * 2 + 1] * factor;
                const float4 part = *reinterpret_cast<const float4*>(recv_out + sp * share + i);
                value.x += part.x * factor; value.y += part.y * factor; value.z += part.z * factor; value.w += part.w * factor;
            }
            const float scale = total > 0.f ? 1.0f / total : 0.f;
            bf16* out = a.out + (long long)row * a.ldo + (long long)(head0 + r) * D + c;
            *reinterpret_cast<__nv_bfloat162*>(out) = __floats2bfloat162_rn(value.x * scale, value.y * scale);
            *reinterpret_cast<__nv_bfloat162*>(out + 2) = __floats2bfloat162_rn(value.z * scale, value.w * scale);
        }
        return;
    }
    if (a.splits > 1 && a.counters) {
        // The block that finishes last for this (row, key/value head) merges the splits: in
        // split order whichever block it is, so the result does not depend on timing. All the
        // partial maxima and denominators are fetched at once, then every thread adds the
        // partial outputs of its elements with the loads of a few splits in flight together.
        __shared__ int last_block;
        float* stat_max = merge_stat;                  // [group][splits]
        float* stat_factor = merge_stat + 8 * 32;      // [group][splits]; then [group] 1 / denominator
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0)
            last_block = atomicAdd(a.counters + (long long)row * a.kv_heads + kv_head, 1) == a.splits - 1;
        __syncthreads();
        if (!last_block) return;
        __threadfence();
        const int splits = a.splits;                   // <= 32
        for (int i = threadIdx.x; i < group * splits; i += THREADS) {
            const int r = i / splits, sp = i - r * splits;
            const long long where = ((long long)row * a.heads + head0 + r) * splits + sp;
            stat_max[r * 32 + sp] = __ldcg(a.partial_stat + where * 2);
            stat_factor[r * 32 + sp] = __ldcg(a.partial_stat + where * 2 + 1);
        }
        __syncthreads();
        if (threadIdx.x < group) {
            const int r = threadIdx.x;
            float top = -INFINITY, total = 0.f;
            for (int sp = 0; sp < splits; ++sp) top = fmaxf(top, stat_max[r * 32 + sp]);
            for (int sp = 0; sp < splits; ++sp) {
                const float m = stat_max[r * 32 + sp];
                const float factor = m == -INFINITY ? 0.f : exp2f(m - top);
                total += stat_factor[r * 32 + sp] * factor;
                stat_factor[r * 32 + sp] = factor;
            }
            stat_factor[8 * 32 + r] = total > 0.f ? 1.0f / total : 0.f;
        }
        __syncthreads();
        for (int item = threadIdx.x; item < group * D; item += THREADS) {
            const int r = item / D, c = item - r * D;
            const int head = head0 + r;
            const float* part = a.partial_out + ((long long)row * a.heads + head) * splits * D + c;
            float value = 0.f;
            int sp = 0;
            for (; sp + 4 <= splits; sp += 4) {
                const float v0 = __ldcg(part + (long long)sp * D), v1 = __ldcg(part + (long long)(sp + 1) * D);
                const float v2 = __ldcg(part + (long long)(sp + 2) * D), v3 = __ldcg(part + (long long)(sp + 3) * D);
                value += v0 * stat_factor[r * 32 + sp];
                value += v1 * stat_factor[r * 32 + sp + 1];
                value += v2 * stat_factor[r * 32 + sp + 2];
                value += v3 * stat_factor[r * 32 + sp + 3];
            }
            for (; sp < splits; ++sp) value += __ldcg(part + (long long)sp * D) * stat_factor[r * 32 + sp];
            a.out[(long long)row * a.ldo + (long long)head * D + c] = from_float<bf16>(value * stat_factor[8 * 32 + r]);
        }
        if (threadIdx.x == 0) a.counters[(long long)row * a.kv_heads + kv_head] = 0;
    }
}

// grid (heads, rows): merges the splits of one (row, head) in split order.
__global__ void attention_combine_kernel(Args a) {
    const int head = blockIdx.x, row = blockIdx.y;
    const long long where = ((long long)row * a.heads + head) * a.splits;
    float top = -INFINITY;
    for (int s = 0; s < a.splits; ++s) top = fmaxf(top, a.partial_stat[(where + s) * 2]);
    for (int c = threadIdx.x; c < D; c += blockDim.x) {
        float total = 0.f, value = 0.f;
        for (int s = 0; s < a.splits; ++s) {
            const float m = a.partial_stat[(where + s) * 2];
            const float factor = m == -INFINITY ? 0.f : exp2f(m - top);
            total += a.partial_stat[(where + s) * 2 + 1] * factor;
            value += a.partial_out[(where + s) * D + c] * factor;
        }
        a.out[(long long)row * a.ldo + (long long)head * D + c] = from_float<bf16>(total > 0.f ? value / total : 0.f);
    }
}

constexpr size_t PREFILL_SHARED = (size_t)(TILE + 4 * TILE) * PITCH * sizeof(bf16);
int kidi_decode_ring = 1;

typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// A map over a cache [rows, D] of bfloat16: boxes of 64 columns by 64 rows (a page of one
// key/value head), 128-byte swizzle.
int page_map(CUtensorMap* map, const void* base, long long rows) {
    static EncodeTiled encode = nullptr;
    if (!encode) {
        void* entry = nullptr;
        cudaDriverEntryPointQueryResult result;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &entry, cudaEnableDefault, &result) != cudaSuccess ||
            result != cudaDriverEntryPointSuccess)
            return KIDI_REFUSED_SIZE;
        encode = (EncodeTiled)entry;
    }
    const cuuint64_t dims[2] = {(cuuint64_t)D, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)D * 2};
    const cuuint32_t box[2] = {64, 64};
    const cuuint32_t steps[2] = {1, 1};
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, steps,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS
               ? 0
               : KIDI_REFUSED_SIZE;
}

bool aligned(const Args& a) {
    return !((uintptr_t)a.q & 15) && !((uintptr_t)a.k_step & 15) && !((uintptr_t)a.v_step & 15) &&
           !((uintptr_t)a.k_cache & 15) && !((uintptr_t)a.v_cache & 15) && !((uintptr_t)a.out & 3) && !(a.ldq & 7) &&
           !(a.ldkv & 7) && !(a.ldo & 1);
}
}  // namespace

KIDI_API int kidi_attention_head_dim() { return D; }

// 0: the decode kernel copies pages row by row into padded tiles whatever the head width.

// 0: the page-copying decode kernel keeps two key and two value tiles (three blocks of head
// width 128 an SM) instead of a ring of three tiles (four blocks).
KIDI_API void kidi_attention_decode_ring(int enabled) { kidi_decode_ring = enabled; }

// Decode blocks of the kernel for up to eight query heads a key/value head that fit an SM
// by shared memory (`swizzled`: the cache is one contiguous array and pages are copied whole).
KIDI_API int kidi_attention_decode_blocks_per_sm(int swizzled) {
    const size_t block = (swizzled && D % 64 == 0)
                             ? (kidi_decode_ring ? RING_SHARED : SWIZZLED_SHARED) : NARROW_SHARED;
    const int fitting = (int)((228 * 1024) / (block + 1024));       // a kilobyte a block is the system's
    return fitting < 1 ? 1 : fitting > 4 ? 4 : fitting;             // four by registers
}

// Whether a bounded wait for a tile ever ran out in this process (reads the flag back; synchronises).
KIDI_API int kidi_attention_timeout_flag() {
    int flag = 0;
    if (cudaMemcpyFromSymbol(&flag, kidi_attention_timeout, sizeof(int)) != cudaSuccess) return -1;
    return flag;
}

// max_new: the longest seq_len of the step (sizes the grid).
KIDI_API int kidi_attention_prefill(const Args* args, int max_new, cudaStream_t stream) {
    const Args& a = *args;
    if (a.rows <= 0 || a.seqs <= 0 || max_new <= 0) return 0;
    if (a.cache.head_dim != D || a.heads % a.kv_heads || a.heads > 65535 || a.seqs > 65535 || !aligned(a) ||
        (a.cache.table && a.cache.page_shift != 6))
        return KIDI_REFUSED_SIZE;
    static std::atomic<bool> configured{false};      // setting the attribute twice is harmless
    if (!configured.load(std::memory_order_acquire)) {
        cudaError_t status = cudaFuncSetAttribute(attention_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                  (int)PREFILL_SHARED);
        if (status != cudaSuccess) return (int)status;
        configured.store(true, std::memory_order_release);
    }
    dim3 grid((max_new + TILE - 1) / TILE, a.seqs, a.heads);
    return kidi_launch(attention_prefill_kernel, grid, THREADS, PREFILL_SHARED, stream, a);
}

// One query row per sequence; every key comes from the cache. With splits > 1 the
// workspace pointers must hold rows*heads*splits*(D + 2) floats.
KIDI_API int kidi_attention_decode(const Args* args, cudaStream_t stream) {
    const Args& a = *args;
    if (a.rows <= 0) return 0;
    const int group = a.kv_heads > 0 ? a.heads / a.kv_heads : 0;
    if (a.cache.head_dim != D || a.heads % a.kv_heads || group > 16 || a.kv_heads > 65535 || a.rows > 65535 ||
        !aligned(a) || a.cache.page_shift != 6 || a.splits < 1 || a.splits > 65535 || (a.counters && a.splits > 32))
        return KIDI_REFUSED_SIZE;
    if (a.fuse) {   // the rotation inside the kernel: the narrow kernel, vectors of eight elements
        if (group > 8 || !a.k_step || !a.v_step || (a.ldkv & 7) || (a.rotary_dim & 15) || a.rotary_dim > D ||
            a.rotary_dim < 0 || ((uintptr_t)a.cos_table & 15) || ((uintptr_t)a.sin_table & 15) ||
            ((a.fuse & 1) && a.cos_table && !a.sin_table))
            return KIDI_REFUSED_SIZE;
    }
    // Without a workspace the splits merge inside a thread-block cluster.
    const bool clustered = a.splits > 1 && !a.partial_out && !a.partial_stat;
    if (clustered && (group > 8 || a.splits > 8)) return KIDI_REFUSED_SIZE;
    if (a.splits > 1 && !clustered && (!a.partial_out || !a.partial_stat)) return KIDI_REFUSED_SIZE;
    // Head widths that are multiples of 64 take whole pages by TMA tensor copies.
    const bool swizzled = group <= 8 && D % 64 == 0 && a.cache_rows > 0;
    CUtensorMap k_map, v_map;
    memset(&k_map, 0, sizeof(k_map));
    memset(&v_map, 0, sizeof(v_map));
    if (swizzled) {
        int status = page_map(&k_map, a.k_cache, a.cache_rows);
        if (!status) status = page_map(&v_map, a.v_cache, a.cache_rows);
        if (status) return status;
    }
    static std::atomic<bool> configured{false};      // setting the attributes twice is harmless
    if (!configured.load(std::memory_order_acquire)) {
        cudaError_t status = cudaFuncSetAttribute(attention_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                  (int)DECODE_SHARED);
        const void* narrow[6] = {(const void*)attention_decode_narrow_kernel<false, 0>,
                                 (const void*)attention_decode_narrow_kernel<true, 0>,
                                 (const void*)attention_decode_narrow_kernel<false, 1>,
                                 (const void*)attention_decode_narrow_kernel<true, 1>,
                                 (const void*)attention_decode_narrow_kernel<false, 2>,
                                 (const void*)attention_decode_narrow_kernel<true, 2>};
        const size_t sizes[3] = {NARROW_SHARED, SWIZZLED_SHARED, RING_SHARED};
        for (int i = 0; i < 6 && status == cudaSuccess; ++i)
            status = cudaFuncSetAttribute(narrow[i], cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizes[i >> 1]);
        if (status != cudaSuccess) return (int)status;
        configured.store(true, std::memory_order_release);
    }
    dim3 grid(a.splits, a.kv_heads, a.rows);
    const int form = !swizzled ? 0 : kidi_decode_ring ? 2 : 1;
    const size_t narrow_shared = form == 2 ? RING_SHARED : form == 1 ? SWIZZLED_SHARED : NARROW_SHARED;
    if (clustered) {
        const unsigned cluster = (unsigned)a.splits;
        if (form == 2)
            return kidi_launch_clusters(attention_decode_narrow_kernel<true, 2>, grid, THREADS, narrow_shared, stream,
                                        cluster, k_map, v_map, a);
        if (form == 1)
            return kidi_launch_clusters(attention_decode_narrow_kernel<true, 1>, grid, THREADS, narrow_shared, stream,
                                        cluster, k_map, v_map, a);
        return kidi_launch_clusters(attention_decode_narrow_kernel<true, 0>, grid, THREADS, narrow_shared, stream, cluster,
                                    k_map, v_map, a);
    }
    int status;
    if (group > 8) status = kidi_launch(attention_decode_kernel, grid, THREADS, DECODE_SHARED, stream, a);
    else if (form == 2)
        status = kidi_launch(attention_decode_narrow_kernel<false, 2>, grid, THREADS, narrow_shared, stream, k_map, v_map, a);
    else if (form == 1)
        status = kidi_launch(attention_decode_narrow_kernel<false, 1>, grid, THREADS, narrow_shared, stream, k_map, v_map, a);
    else
        status = kidi_launch(attention_decode_narrow_kernel<false, 0>, grid, THREADS, narrow_shared, stream, k_map, v_map, a);
    if (status || a.splits == 1 || (group <= 8 && a.counters)) return status;
    dim3 combine(a.heads, a.rows);
    return kidi_launch(attention_combine_kernel, combine, D >= 128 ? 128 : 64, 0, stream, a);
}

// ---------------------------------------------------------------------------
// The variant that allocates nothing (attention_no_alloc.h). Its workspace is this
// array; the host code below never uses the array's name as an address: it asks the
// runtime for the device address once per device and passes that to the kernels.
static __device__ __align__(256) float kidi_static_scratch[KIDI_STATIC_SCRATCH_FLOATS];

// The published argument block is the kernels' own, field for field.
static_assert(sizeof(KidiAttentionArgs) == sizeof(Args) && sizeof(KidiCacheGeometry) == sizeof(CacheGeometry) &&
                  offsetof(KidiAttentionArgs, out) == offsetof(Args, out) &&
                  offsetof(KidiAttentionArgs, splits) == offsetof(Args, splits) &&
                  offsetof(KidiAttentionArgs, cache_rows) == offsetof(Args, cache_rows),
              "attention_no_alloc.h and the kernels disagree about the argument block");

// Floats of workspace a call needs; -1 when rows, heads or splits lie outside the bounds
// (checked before the product is formed, so that it cannot overflow).
KIDI_API long long kidi_attention_decode_static_need(int rows, int heads, int splits) {
    if (rows < 0 || heads < 0 || splits < 1 || rows > KIDI_STATIC_MAX_ROWS || heads > KIDI_STATIC_MAX_HEADS ||
        splits > KIDI_STATIC_MAX_SPLITS)
        return -1;
    return splits > 1 ? (long long)rows * heads * splits * (D + 2) : 0;
}

KIDI_API int kidi_attention_decode_static(const KidiAttentionArgs* args, cudaStream_t stream) {
    constexpr int MAX_DEVICES = 64;
    static std::atomic<float*> scratch_of_device[MAX_DEVICES];      // zero-initialised
    Args a = *reinterpret_cast<const Args*>(args);
    if (a.rows <= 0) return 0;
    const long long need = kidi_attention_decode_static_need(a.rows, a.heads, a.splits);
    if (need < 0 || a.heads <= 0) return KIDI_REFUSED_SIZE;
    if (need > KIDI_STATIC_SCRATCH_FLOATS) return KIDI_REFUSED_SIZE;  // more splits than the fixed workspace holds
    int device = -1;
    cudaError_t status = cudaGetDevice(&device);
    if (status != cudaSuccess) return (int)status;
    if (device < 0 || device >= MAX_DEVICES) return KIDI_REFUSED_SIZE;
    float* scratch = scratch_of_device[device].load(std::memory_order_acquire);
    if (!scratch) {  // set-up, once per device, with that device current (threads that race here find the same address)
        status = cudaGetSymbolAddress((void**)&scratch, kidi_static_scratch);
        if (status != cudaSuccess) return (int)status;
        scratch_of_device[device].store(scratch, std::memory_order_release);
    }
    a.partial_out = scratch;
    a.partial_stat = scratch + (long long)a.rows * a.heads * a.splits * D;
    a.counters = nullptr;  // the splits are merged by the second kernel
    return kidi_attention_decode(&a, stream);
}
