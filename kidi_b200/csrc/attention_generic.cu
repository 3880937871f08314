// Per-head RMSNorm + rotary encoding + cache write, and attention over the cache
// for any element type, head size and number of heads.
//
// Formulas (reference):
//  * fused per-head norm and rotation, norm before rotation, half-split pairing:
//      n_c = x_c * (1/sqrt(sum(x^2)/d + eps)) * w_c
//      out_c = n_c * cos[pos, c mod half] + r_c * sin[pos, c mod half],
//      r_c = -n_{c+half} for c < half, n_{c-half} otherwise
//    (src/kidi/layers/qwen3.cpp:37-48, src/kidi/ops/context.cpp:1051-1065,
//     src/kidi/runtime/mps/eager_kernels.metal:87-97)
//  * scores s = (q . k) * scale, key head = query head / (heads / kv_heads), softmax
//    over the visible keys, output = sum p_u v_u
//    (src/kidi/layers/qwen3.cpp:53-54, src/kidi/runtime/vulkan/attention.comp:32-101)
//  * the causal rule is the generic causal path's: key u is visible to the query at
//    position p when u <= p (src/kidi/model/gemma4.cpp:736-740); with a window W,
//    when also u > p - W.
// Norm sums, rotation, scores, softmax and the weighted sum are 32-bit.
#include "common.cuh"

struct RopeStoreArgs {
    void* qkv;                 // [rows, ld] : q heads, then k heads, then v heads, each head_dim wide
    long long ld;
    const void* q_norm;        // [head_dim] or null
    const void* k_norm;        // [head_dim] or null
    const float* cos_table;    // [positions, rotary_dim/2] or null (no rotation)
    const float* sin_table;
    const int* row_seq;        // [rows]  (-1: padding row, skipped)
    const int* row_pos;        // [rows]
    const int* seq_slot;       // [seqs]
    const int* seq_start;      // [seqs]
    const int* seq_len;        // [seqs]
    void* k_cache;             // storage of this schedule entry, or null (no write)
    void* v_cache;
    CacheGeometry cache;
    int rows, heads, kv_heads, head_dim, rotary_dim;
    float eps;
    int transform;             // 0: only copy the k and v heads, as they are, to the cache
};

// One warp per (row, head) over heads + 2*kv_heads heads.
template <typename T, typename TW>
__global__ void __launch_bounds__(128) rope_store_kernel(RopeStoreArgs a) {
    __shared__ float normed[4][256];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int total_heads = a.heads + 2 * a.kv_heads;
    const long long item = (long long)blockIdx.x * 4 + warp;
    if (item >= (long long)a.rows * total_heads) return;
    const int row = (int)(item / total_heads);
    const int head = (int)(item - (long long)row * total_heads);
    const int seq = a.row_seq[row];
    if (seq < 0) return;
    const int position = a.row_pos[row];
    const int d = a.head_dim;
    T* vector = (T*)a.qkv + row * a.ld + (long long)head * d;

    // Where this head goes in the cache, if anywhere.
    T* cached = nullptr;
    if (head >= a.heads && a.k_cache) {
        bool keep = true;
        if (a.cache.ring_pages) {  // a ring keeps the last ring_tokens tokens of the step only
            const int ring_tokens = a.cache.ring_pages << a.cache.page_shift;
            keep = position >= a.seq_start[seq] + a.seq_len[seq] - ring_tokens;
        }
        if (keep) {
            const bool is_key = head < a.heads + a.kv_heads;
            const int kv_head = is_key ? head - a.heads : head - a.heads - a.kv_heads;
            cached = (T*)(is_key ? a.k_cache : a.v_cache) +
                     cache_row_offset(a.cache, a.seq_slot[seq], position, kv_head);
        }
    }

    if (head >= a.heads + a.kv_heads || !a.transform) {  // a value head, or copy only
        if (cached)
            for (int c = lane; c < d; c += 32) cached[c] = vector[c];
        return;
    }

    const TW* weight = (const TW*)(head < a.heads ? a.q_norm : a.k_norm);
    float values[8];
    float square = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int c = lane + 32 * i;
        values[i] = c < d ? to_float(vector[c]) : 0.f;
        square = fmaf(values[i], values[i], square);
    }
    float inv = 1.f;
    if (weight) inv = 1.0f / sqrtf(warp_sum(square) / (float)d + a.eps);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int c = lane + 32 * i;
        if (c < d) {
            if (weight) values[i] = values[i] * inv * to_float(weight[c]);
            normed[warp][c] = values[i];
        }
    }
    __syncwarp();
    const int half = a.rotary_dim / 2;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int c = lane + 32 * i;
        if (c >= d) continue;
        float out = values[i];
        if (a.cos_table && c < a.rotary_dim) {
            const int j = c < half ? c : c - half;
            const float cosine = a.cos_table[(long long)position * half + j];
            const float sine = a.sin_table[(long long)position * half + j];
            const float rotated = c < half ? -normed[warp][c + half] : normed[warp][c - half];
            out = values[i] * cosine + rotated * sine;
        }
        const T stored = from_float<T>(out);
        vector[c] = stored;
        if (cached) cached[c] = stored;
    }
}

// Eight consecutive norm weights as 32-bit values (the address is 16-byte aligned: the head
// width is a multiple of eight).
__device__ __forceinline__ void load8(const float* p, float (&w)[8]) {
    const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
    w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w; w[4] = b.x; w[5] = b.y; w[6] = b.z; w[7] = b.w;
}
__device__ __forceinline__ void load8(const bf16* p, float (&w)[8]) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 two = __bfloat1622float2(pairs[i]);
        w[2 * i] = two.x;
        w[2 * i + 1] = two.y;
    }
}

// The same for bfloat16 rows in 16-byte vectors. A (row, head) is handled by a group of
// L lanes (L the power of two that covers head_dim / 8: 16 lanes for a head of 128), so a
// warp takes 32 / L of them; lane l of a group owns elements 8l..8l+7 of the head, and its
// rotation partners are the eight elements of lane l +- half/8, fetched with shuffles.
// Needs head_dim and rotary_dim/2 to be multiples of 8 and 16-byte aligned rows.
template <typename TW>
__global__ void __launch_bounds__(128) rope_store_bf16_kernel(RopeStoreArgs a, int group_lanes) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int total_heads = a.heads + 2 * a.kv_heads;
    const int per_warp = 32 / group_lanes;
    const int group = lane / group_lanes, l = lane - group * group_lanes;
    const int item = (blockIdx.x * 4 + warp) * per_warp + group;   // the launcher keeps the count below 2^31
    // Every lane stays to the end (the shuffles are warp-wide); `alive` says whether the
    // group has a (row, head) to work on.
    bool alive = item < a.rows * total_heads;
    const int row = alive ? item / total_heads : 0;
    const int head = alive ? item - row * total_heads : 0;
    const int d = a.head_dim, c0 = 8 * l;
    bf16* vector = (bf16*)a.qkv + (long long)row * a.ld + head * d;
    // The row's elements are asked for together with its sequence and position (a padding
    // row's elements are there to be read; nothing of it is stored).
    uint4 raw = make_uint4(0u, 0u, 0u, 0u);
    if (alive && c0 < d) raw = *reinterpret_cast<const uint4*>(vector + c0);
    const int seq = a.row_seq[row];
    const int position = a.row_pos[row];
    alive = alive && seq >= 0;
    const bool mine = alive && c0 < d;

    bf16* cached = nullptr;
    if (alive && head >= a.heads && a.k_cache) {
        bool keep = true;
        if (a.cache.ring_pages) {
            const int ring_tokens = a.cache.ring_pages << a.cache.page_shift;
            keep = position >= a.seq_start[seq] + a.seq_len[seq] - ring_tokens;
        }
        if (keep) {
            const bool is_key = head < a.heads + a.kv_heads;
            const int kv_head = is_key ? head - a.heads : head - a.heads - a.kv_heads;
            cached = (bf16*)(is_key ? a.k_cache : a.v_cache) +
                     cache_row_offset(a.cache, a.seq_slot[seq], position, kv_head);
        }
    }
    if (!mine) raw = make_uint4(0u, 0u, 0u, 0u);
    const bool plain = head >= a.heads + a.kv_heads || !a.transform;  // a value head, or copy only
    if (plain && cached && mine) *reinterpret_cast<uint4*>(cached + c0) = raw;
    const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(&raw);
    float v[8];
    float square = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 two = __bfloat1622float2(pairs[i]);
        v[2 * i] = two.x;
        v[2 * i + 1] = two.y;
        square = fmaf(two.x, two.x, square);
        square = fmaf(two.y, two.y, square);
    }
    const TW* weight = (const TW*)(head < a.heads ? a.q_norm : a.k_norm);
    if (a.q_norm || a.k_norm) {      // the same for the whole launch: the shuffles stay warp-wide
        for (int offset = group_lanes >> 1; offset > 0; offset >>= 1)
            square += __shfl_xor_sync(0xffffffffu, square, offset);
        if (weight && mine && !plain) {
            const float inv = 1.0f / sqrtf(square / (float)d + a.eps);
            float w[8];
            load8(weight + c0, w);
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = v[i] * inv * w[i];
        }
    }
    if (a.cos_table) {
        const int half = a.rotary_dim / 2;
        const bool low = c0 < half;
        const int partner = group * group_lanes + ((low ? l + half / 8 : l - half / 8) & (group_lanes - 1));
        float other[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) other[i] = __shfl_sync(0xffffffffu, v[i], partner);
        if (mine && !plain && c0 < a.rotary_dim) {
            const int j = low ? c0 : c0 - half;
            const float4* cosine = reinterpret_cast<const float4*>(a.cos_table + (long long)position * half + j);
            const float4* sine = reinterpret_cast<const float4*>(a.sin_table + (long long)position * half + j);
            const float4 ca = cosine[0], cb = cosine[1], sa = sine[0], sb = sine[1];
            const float c8[8] = {ca.x, ca.y, ca.z, ca.w, cb.x, cb.y, cb.z, cb.w};
            const float s8[8] = {sa.x, sa.y, sa.z, sa.w, sb.x, sb.y, sb.z, sb.w};
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = v[i] * c8[i] + (low ? -other[i] : other[i]) * s8[i];
        }
    }
    if (mine && !plain) {
        uint4 packed;
        __nv_bfloat162* out = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
        for (int i = 0; i < 4; ++i) out[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        *reinterpret_cast<uint4*>(vector + c0) = packed;
        if (cached) *reinterpret_cast<uint4*>(cached + c0) = packed;
    }
}

KIDI_API int kidi_rope_store(const RopeStoreArgs* args, int dtype, int norm_dtype, cudaStream_t stream) {
    const RopeStoreArgs& a = *args;
    if (a.rows <= 0) return 0;
    if (a.head_dim > 256 || a.head_dim <= 0 || a.rotary_dim > a.head_dim || (a.rotary_dim & 1)) return KIDI_REFUSED_SIZE;
    const long long items = (long long)a.rows * (a.heads + 2 * a.kv_heads);
    const unsigned blocks = (unsigned)((items + 3) / 4);
    const bool vectors = dtype == KIDI_BF16 && items < (1LL << 30) && !((uintptr_t)a.q_norm & 15) &&
                         !((uintptr_t)a.k_norm & 15) && !(a.head_dim & 7) && !(a.ld & 7) && !((uintptr_t)a.qkv & 15) &&
                         !((uintptr_t)a.k_cache & 15) && !((uintptr_t)a.v_cache & 15) &&
                         (!a.cos_table || (!(a.rotary_dim & 15) && !((uintptr_t)a.cos_table & 15) &&
                                           !((uintptr_t)a.sin_table & 15)));
    if (vectors) {
        int group_lanes = 1;                    // lanes that cover a head in 16-byte vectors
        while (group_lanes * 8 < a.head_dim) group_lanes <<= 1;
        const long long per_block = 4 * (32 / group_lanes);
        const unsigned vector_blocks = (unsigned)((items + per_block - 1) / per_block);
        if (norm_dtype == KIDI_F32)
            return kidi_launch(rope_store_bf16_kernel<float>, vector_blocks, 128, 0, stream, a, group_lanes);
        if (norm_dtype == KIDI_BF16)
            return kidi_launch(rope_store_bf16_kernel<bf16>, vector_blocks, 128, 0, stream, a, group_lanes);
    }
    if (dtype == KIDI_F32 && norm_dtype == KIDI_F32) return kidi_launch(rope_store_kernel<float, float>, blocks, 128, 0, stream, a);
    if (dtype == KIDI_F32 && norm_dtype == KIDI_BF16) return kidi_launch(rope_store_kernel<float, bf16>, blocks, 128, 0, stream, a);
    if (dtype == KIDI_BF16 && norm_dtype == KIDI_F32) return kidi_launch(rope_store_kernel<bf16, float>, blocks, 128, 0, stream, a);
    if (dtype == KIDI_BF16 && norm_dtype == KIDI_BF16) return kidi_launch(rope_store_kernel<bf16, bf16>, blocks, 128, 0, stream, a);
    return KIDI_REFUSED_DTYPE;
}

// ---------------------------------------------------------------------------
struct AttentionArgs {
    const void* q;        // [rows, ldq], head h at h*head_dim
    long long ldq;
    const void* k_step;   // keys of this step's rows [rows, ldkv], kv head g at g*head_dim; null: read the cache only
    const void* v_step;
    long long ldkv;
    const void* k_cache;  // storage of this schedule entry (may be null when every key is in the step)
    const void* v_cache;
    CacheGeometry cache;
    void* out;            // [rows, ldo]
    long long ldo;
    const int* row_seq;   // [rows] (-1: padding row: output zeros)
    const int* row_pos;
    const int* seq_slot;
    const int* seq_start; // tokens in the cache before this step
    const int* seq_row0;  // first packed row of the sequence
    int rows, heads, kv_heads, head_dim, window;  // window 0: every earlier key is visible
    float scale;
    float softcap;        // > 0: a score s becomes softcap * tanh(s / softcap)
    const float* slopes;  // [heads] or null: head h adds slopes[h] * (key position - query position) to a score
};

// One block of 4 warps per (row, head). Warp w takes keys lo+w, lo+w+4, ... in
// ascending order with an online softmax; the four partial results are merged in
// warp order. The order depends on the row's position and window only, so a row's
// result is the same in every batch and under every cut of the work.
template <typename T>
__global__ void __launch_bounds__(128) attention_generic_kernel(AttentionArgs a) {
    __shared__ float query[256];
    __shared__ float part_acc[4][256];
    __shared__ float part_max[4], part_sum[4];
    const int row = blockIdx.x, head = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int d = a.head_dim;
    T* out = (T*)a.out + row * a.ldo + (long long)head * d;
    const int seq = a.row_seq[row];
    if (seq < 0) {
        for (int c = threadIdx.x; c < d; c += 128) out[c] = from_float<T>(0.f);
        return;
    }
    const int position = a.row_pos[row];
    const int first = a.window > 0 ? max(0, position - a.window + 1) : 0;
    const int kv_head = head / (a.heads / a.kv_heads);
    const int slot = a.seq_slot[seq];
    const int start = a.k_step ? a.seq_start[seq] : 0x7fffffff;  // keys >= start come from the step
    const int row0 = a.seq_row0[seq];
    const T* q = (const T*)a.q + row * a.ldq + (long long)head * d;
    for (int c = threadIdx.x; c < d; c += 128) query[c] = to_float(q[c]);
    __syncthreads();

    float best = -INFINITY, denom = 0.f;
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    for (int u = first + warp; u <= position; u += 4) {
        const T *key, *value;
        if (u >= start) {
            const long long offset = (long long)(row0 + u - start) * a.ldkv + (long long)kv_head * d;
            key = (const T*)a.k_step + offset;
            value = (const T*)a.v_step + offset;
        } else {
            const long long offset = cache_row_offset(a.cache, slot, u, kv_head);
            key = (const T*)a.k_cache + offset;
            value = (const T*)a.v_cache + offset;
        }
        float dot = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int c = lane + 32 * i;
            if (c < d) dot = fmaf(query[c], to_float(key[c]), dot);
        }
        float score = warp_sum(dot) * a.scale;
        if (a.softcap > 0.f) score = a.softcap * tanhf(score / a.softcap);
        if (a.slopes) score += a.slopes[head] * (float)(u - position);
        const float next = fmaxf(best, score);
        const float keep = expf(best - next);  // 0 on the first key (best = -inf)
        const float weight = expf(score - next);
        denom = denom * keep + weight;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int c = lane + 32 * i;
            if (c < d) acc[i] = acc[i] * keep + weight * to_float(value[c]);
        }
        best = next;
    }
    if (lane == 0) { part_max[warp] = best; part_sum[warp] = denom; }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int c = lane + 32 * i;
        if (c < d) part_acc[warp][c] = acc[i];
    }
    __syncthreads();
    float top = part_max[0];
#pragma unroll
    for (int w = 1; w < 4; ++w) top = fmaxf(top, part_max[w]);
    float total = 0.f, factor[4];
#pragma unroll
    for (int w = 0; w < 4; ++w) {
        factor[w] = part_max[w] == -INFINITY ? 0.f : expf(part_max[w] - top);
        total += part_sum[w] * factor[w];
    }
    for (int c = threadIdx.x; c < d; c += 128) {
        float value = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) value += part_acc[w][c] * factor[w];
        out[c] = from_float<T>(value / total);
    }
}

KIDI_API int kidi_attention_generic(const AttentionArgs* args, int dtype, cudaStream_t stream) {
    const AttentionArgs& a = *args;
    if (a.rows <= 0) return 0;
    if (a.head_dim > 256 || a.head_dim <= 0 || a.heads % a.kv_heads || a.heads > 65535) return KIDI_REFUSED_SIZE;
    dim3 grid(a.rows, a.heads);
    if (dtype == KIDI_F32) return kidi_launch(attention_generic_kernel<float>, grid, 128, 0, stream, a);
    if (dtype == KIDI_BF16) return kidi_launch(attention_generic_kernel<bf16>, grid, 128, 0, stream, a);
    return KIDI_REFUSED_DTYPE;
}
