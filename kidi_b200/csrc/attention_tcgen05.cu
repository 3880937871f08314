// Causal grouped-query attention for prompts on the 5th-generation tensor cores,
// compiled for one head width (-DKIDI_HEAD_DIM=64 or 128).
//
// A block owns 128 query rows of one (sequence, head) and walks the sequence's keys in
// tiles of 128. Every key of the step is one of the step's own rows (the sequences start
// at position 0), so queries, keys and values are tiles of the packed qkv matrix and
// arrive by TMA with the 128-byte swizzle. Per key tile:
//   S = Q K^T      tcgen05.mma, 128 x 128 x head width, accumulator in tensor memory;
//   softmax        a query row is one TMEM lane; the four warps that may read a lane
//                  quarter each take a share of the tile's keys (16 softmax warps in all),
//                  so that each SM scheduler has several warps to switch between. A thread
//                  loads its share of the row's scores, the row's warps combine their
//                  maxima through shared memory, then each computes its exponentials and
//                  its part of the row sum, all in 32-bit; P is rounded to bfloat16 and
//                  written to shared memory in the swizzled K-major layout of an A operand;
//   O += P V       tcgen05.mma with V as an MN-major B operand (V rows are keys, the
//                  contraction runs over keys), accumulating in a second TMEM region over
//                  all key tiles. The exponentials are taken against a reference maximum
//                  that is raised only when the row's maximum has grown by more than 2^8
//                  since (then the warp multiplies its rows of O and the row sums by the
//                  ratio); P stays below 2^8, and the final division by the row sum makes
//                  the result independent of the reference.
// One thread issues all copies and matrix instructions; mbarriers order it with the
// softmax warps. A softmax thread reads its scores of S into registers and releases S at
// once, so that the next tile's Q K^T and this tile's P V run while the exponentials are
// computed; K, V and P are double-buffered. Every wait is bounded: a block that gives up
// records it in kidi_attention_timeout and leaves without storing.
//
// Formulas: src/kidi/layers/qwen3.cpp:53-54, src/kidi/runtime/vulkan/attention.comp:32-101;
// causal rule src/kidi/model/gemma4.cpp:736-740.
#include <cuda.h>

#include "common.cuh"

KIDI_DEFINE_PDL_FLAG()

#ifndef KIDI_HEAD_DIM
#error "compile with -DKIDI_HEAD_DIM=64 or 128"
#endif

namespace {

constexpr int D = KIDI_HEAD_DIM;
static_assert(D == 64 || D == 128, "the tensor-memory attention kernel takes head widths 64 and 128");
constexpr int BM = 128, BN = 128;                 // queries per block, keys per tile
constexpr int SPANS = D / 64;                     // 128-byte swizzle spans per row of Q, K, V
constexpr int SPAN_BYTES = 128 * 128;             // 128 rows x 128 bytes
constexpr int QKV_TILE = SPANS * SPAN_BYTES;      // bytes of a Q, K or V tile
constexpr int P_TILE = 2 * SPAN_BYTES;            // P: 128 rows x 128 keys (two of them)
#ifndef KIDI_SOFTMAX_GROUPS
#define KIDI_SOFTMAX_GROUPS 4
#endif
constexpr int GROUPS = KIDI_SOFTMAX_GROUPS;       // warps that share a query row's keys of a tile
static_assert(GROUPS == 1 || GROUPS == 2 || GROUPS == 4, "1, 2 or 4 warps share a row");
constexpr int SHARE = BN / GROUPS;                // keys of a tile per softmax thread
constexpr int SOFTMAX_THREADS = 128 * GROUPS;
constexpr int THREADS = 32 + SOFTMAX_THREADS;     // warp 0: control; then GROUPS x 4 softmax warps
constexpr unsigned SPIN_LIMIT = 1u << 24;
constexpr float LOG2E = 1.4426950408889634f;
constexpr float RAISE_AFTER = 8.0f;               // the reference maximum follows after a growth of 2^8
constexpr int TMEM_COLUMNS = 512;                 // S of even tiles: columns 0..127, O: 128..128+D-1, S of odd tiles: 256..383

__device__ int kidi_attention_timeout = 0;

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
__device__ __forceinline__ bool mbarrier_wait(unsigned long long* bar, unsigned parity, volatile int* gave_up) {
    for (unsigned spin = 0; spin < SPIN_LIMIT; ++spin) {
        unsigned done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(smem_u32(bar)), "r"(parity)
            : "memory");
        if (done) return true;
        if ((spin & 1023u) == 1023u && *gave_up) return false;
    }
    *gave_up = 1;
    kidi_attention_timeout = 1;
    return false;
}
__device__ __forceinline__ void tma_load_2d(void* smem, const CUtensorMap* map, unsigned long long* bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        :
        : "r"(smem_u32(smem)), "l"((unsigned long long)map), "r"(smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}
// K-major operand tile with the 128-byte swizzle (rows 128 bytes apart, groups of eight
// rows 1024 bytes apart).
__device__ __forceinline__ unsigned long long desc_k_major(const void* tile) {
    unsigned long long desc = (unsigned long long)((smem_u32(tile) & 0x3FFFF) >> 4);
    desc |= (unsigned long long)1 << 16;
    desc |= (unsigned long long)(1024 >> 4) << 32;
    desc |= (unsigned long long)1 << 46;
    desc |= (unsigned long long)2 << 61;
    return desc;
}
// MN-major operand tile with the 128-byte swizzle: 64 MN-elements are contiguous in a
// 128-byte row, consecutive rows are consecutive k; groups of eight k are 1024 bytes apart
// (stride byte offset), the next 64 MN-elements start `mn_atom_bytes` further (leading
// byte offset).
__device__ __forceinline__ unsigned long long desc_mn_major(const void* tile, unsigned mn_atom_bytes) {
    unsigned long long desc = (unsigned long long)((smem_u32(tile) & 0x3FFFF) >> 4);
    desc |= (unsigned long long)(mn_atom_bytes >> 4) << 16;
    desc |= (unsigned long long)(1024 >> 4) << 32;
    desc |= (unsigned long long)1 << 46;
    desc |= (unsigned long long)2 << 61;
    return desc;
}
__host__ __device__ constexpr unsigned instr_desc(int n, bool b_mn_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn_major ? 1u : 0u) << 16) | ((unsigned)(n >> 3) << 17) |
           ((unsigned)(BM >> 4) << 24);
}
__device__ __forceinline__ void umma(unsigned tmem_d, unsigned long long a, unsigned long long b, unsigned idesc,
                                     unsigned accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        :
        : "r"(tmem_d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(unsigned long long* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ float exp2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ void tmem_store_32(unsigned address, const float (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
        "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        :
        : "r"(address), "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]), "f"(v[4]), "f"(v[5]), "f"(v[6]), "f"(v[7]),
          "f"(v[8]), "f"(v[9]), "f"(v[10]), "f"(v[11]), "f"(v[12]), "f"(v[13]), "f"(v[14]), "f"(v[15]), "f"(v[16]),
          "f"(v[17]), "f"(v[18]), "f"(v[19]), "f"(v[20]), "f"(v[21]), "f"(v[22]), "f"(v[23]), "f"(v[24]), "f"(v[25]),
          "f"(v[26]), "f"(v[27]), "f"(v[28]), "f"(v[29]), "f"(v[30]), "f"(v[31])
        : "memory");
}
// Issues the load of 32 columns; the values may be used after tmem_load_wait().
__device__ __forceinline__ void tmem_load_32_issue(unsigned address, float* v) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3]), "=f"(v[4]), "=f"(v[5]), "=f"(v[6]), "=f"(v[7]), "=f"(v[8]),
          "=f"(v[9]), "=f"(v[10]), "=f"(v[11]), "=f"(v[12]), "=f"(v[13]), "=f"(v[14]), "=f"(v[15]), "=f"(v[16]),
          "=f"(v[17]), "=f"(v[18]), "=f"(v[19]), "=f"(v[20]), "=f"(v[21]), "=f"(v[22]), "=f"(v[23]), "=f"(v[24]),
          "=f"(v[25]), "=f"(v[26]), "=f"(v[27]), "=f"(v[28]), "=f"(v[29]), "=f"(v[30]), "=f"(v[31])
        : "r"(address)
        : "memory");
}
__device__ __forceinline__ void tmem_load_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_load_32(unsigned address, float (&v)[32]) {
    unsigned r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(address));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// The maxima that the warps of a row exchange only fix the reference of the exponentials,
// which cancels in the result: with four warps a row they are exchanged as bfloat16 to fit
// the shared memory left beside the tiles.
template <int N> struct ExchangeType { typedef float type; };
template <> struct ExchangeType<4> { typedef bf16 type; };
typedef ExchangeType<GROUPS>::type Exchange;

struct Control {
    Exchange row_part[2][BM][GROUPS];   // per tile parity: each warp's maximum of a row
    unsigned long long q_full, k_full[2], v_full[2], k_free[2], v_free[2], s_ready[2], s_free[2], p_ready[2];
    unsigned long long row_shared[4];   // the warps of a row quarter have written their part
    unsigned tmem_slot;
    int gave_up;
};

struct Params {
    bf16* out;              // [rows, ldo]
    long long ldo;
    const int* seq_len;     // [seqs] tokens of each sequence (all of them in this step)
    const int* seq_row0;    // [seqs] first packed row
    int heads, kv_heads, window;
    float scale;
};

// One softmax thread holds SHARE raw scores of a query row: the keys first..last (relative
// to the thread's first key) are the ones the row may see. Returns their maximum, scaled
// to base-2 exponents.
template <bool MASKED>
__device__ __forceinline__ float share_maximum(const float (&s)[SHARE], float scale_log2, int first, int last) {
    float top[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
    for (int i = 0; i < SHARE; ++i)
        if (!MASKED || (i >= first && i <= last)) top[i & 3] = fmaxf(top[i & 3], s[i]);
    return fmaxf(fmaxf(top[0], top[1]), fmaxf(top[2], top[3])) * scale_log2;
}

// Writes P = exp2(s * scale - reference) as bfloat16 into the swizzled K-major tile
// (`key` is the thread's first key within the tile) and returns the sum.
template <bool MASKED>
__device__ __forceinline__ float write_probabilities(const float (&s)[SHARE], float scale_log2, float reference,
                                                     int first, int last, unsigned char* p_tile, int r, int key) {
    float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
    for (int c = 0; c < SHARE; c += 8) {        // one 16-byte chunk of eight keys
        unsigned packed[4];
#pragma unroll
        for (int i = 0; i < 8; i += 2) {
            float p0 = exp2_approx(fmaf(s[c + i], scale_log2, -reference));
            float p1 = exp2_approx(fmaf(s[c + i + 1], scale_log2, -reference));
            if (MASKED) {
                if (c + i < first || c + i > last) p0 = 0.f;
                if (c + i + 1 < first || c + i + 1 > last) p1 = 0.f;
            }
            sum0 += p0;
            sum1 += p1;
            __nv_bfloat162 pair = __floats2bfloat162_rn(p0, p1);
            packed[i >> 1] = *reinterpret_cast<unsigned*>(&pair);
        }
        const int at = key + c;
        const int chunk = (at & 63) >> 3;
        *reinterpret_cast<uint4*>(p_tile + (at >> 6) * SPAN_BYTES + r * 128 + ((chunk ^ (r & 7)) << 4)) =
            make_uint4(packed[0], packed[1], packed[2], packed[3]);
    }
    return sum0 + sum1;
}

__global__ void __launch_bounds__(THREADS, 1)
attention_prefill_tcgen05_kernel(const __grid_constant__ CUtensorMap map, Params p) {
    // All shared memory is dynamic and laid out here; the tiles come first because the
    // 128-byte swizzle wants them on 1024-byte boundaries.
    extern __shared__ __align__(1024) unsigned char base[];
    unsigned char* q_tile = base;                          // [SPANS][128][128 B]
    unsigned char* k_tiles = q_tile + QKV_TILE;            // 2 buffers
    unsigned char* v_tiles = k_tiles + 2 * QKV_TILE;       // 2 buffers
    unsigned char* p_tiles = v_tiles + 2 * QKV_TILE;       // 2 buffers of [2][128][128 B]
    Control& ctl = *reinterpret_cast<Control*>(p_tiles + 2 * P_TILE);
    unsigned long long& q_full = ctl.q_full;
    unsigned long long(&k_full)[2] = ctl.k_full, (&v_full)[2] = ctl.v_full, (&k_free)[2] = ctl.k_free,
                      (&v_free)[2] = ctl.v_free, (&s_ready)[2] = ctl.s_ready, (&s_free)[2] = ctl.s_free, (&p_ready)[2] = ctl.p_ready,
                      (&row_shared)[4] = ctl.row_shared;
    unsigned& tmem_slot = ctl.tmem_slot;
    int& gave_up = ctl.gave_up;
    if (smem_u32(base) & 1023u) {                          // never seen; a wrong result would be worse than none
        if (threadIdx.x == 0) kidi_attention_timeout = 2;
        return;
    }

    // Long blocks first: a block's number of key tiles grows with its query tile, and blocks
    // start in the order of their linear index, of which z is the slowest part.
    const int q_index = gridDim.z - 1 - blockIdx.z;
    const int seq = blockIdx.y, head = blockIdx.x;
    const int count = p.seq_len[seq];
    const int q0 = q_index * BM;
    if (q0 >= count) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row0 = p.seq_row0[seq];
    const int kv_head = head / (p.heads / p.kv_heads);
    const int q_rows = min(BM, count - q0);
    const int high = q0 + q_rows - 1;                                     // last query position of the block
    const int low = p.window > 0 ? max(0, q0 - p.window + 1) : 0;        // first key any of its queries sees
    const int tile_low = low / BN, tile_high = high / BN;
    const int tiles = tile_high - tile_low + 1;
    const int q_col = head * D, k_col = (p.heads + kv_head) * D, v_col = (p.heads + p.kv_heads + kv_head) * D;

    if (threadIdx.x == 0) {
        mbarrier_init(&q_full, 1);
        for (int i = 0; i < 2; ++i) {
            mbarrier_init(&k_full[i], 1);
            mbarrier_init(&v_full[i], 1);
            mbarrier_init(&k_free[i], 1);
            mbarrier_init(&v_free[i], 1);
            mbarrier_init(&s_ready[i], 1);
            mbarrier_init(&s_free[i], SOFTMAX_THREADS);
            mbarrier_init(&p_ready[i], SOFTMAX_THREADS);
        }
        for (int i = 0; i < 4; ++i) mbarrier_init(&row_shared[i], 32 * GROUPS);
        gave_up = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)),
                     "r"(TMEM_COLUMNS));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const unsigned tmem = tmem_slot;
    const unsigned tmem_o = tmem + 128;
    volatile int* abort_flag = &gave_up;
    // Tile j: S in TMEM buffer j & 1, K, V and P in shared buffers j & 1; the barriers of a
    // buffer complete once per use, so tile j waits for parity (j >> 1) & 1. A barrier counts
    // arrivals without knowing which tile they belong to: every barrier here is one that a
    // thread cannot reach for tile j+2 before all threads have arrived for tile j.

    if (warp == 0) {
        if (lane == 0) {
            // ----------------------------------------------------------- control
            constexpr unsigned idesc_s = instr_desc(BN, false), idesc_o = instr_desc(D, true);
            auto load_tile = [&](unsigned char* tile, unsigned long long* bar, int column, int row) {
                mbarrier_expect_tx(bar, QKV_TILE);
                for (int s = 0; s < SPANS; ++s) tma_load_2d(tile + s * SPAN_BYTES, &map, bar, column + 64 * s, row);
            };
            auto load_k = [&](int j) { load_tile(k_tiles + (j & 1) * QKV_TILE, &k_full[j & 1], k_col, row0 + (tile_low + j) * BN); };
            auto load_v = [&](int j) { load_tile(v_tiles + (j & 1) * QKV_TILE, &v_full[j & 1], v_col, row0 + (tile_low + j) * BN); };
            auto scores = [&](int j) {      // S_j = Q K_j^T
                const unsigned char* k_tile = k_tiles + (j & 1) * QKV_TILE;
                const unsigned tmem_s = tmem + (j & 1) * 256;
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const int offset = (kk >> 2) * SPAN_BYTES + (kk & 3) * 32;
                    umma(tmem_s, desc_k_major(q_tile + offset), desc_k_major(k_tile + offset), idesc_s, kk > 0);
                }
                umma_commit(&s_ready[j & 1]);
                umma_commit(&k_free[j & 1]);
            };
            load_tile(q_tile, &q_full, q_col, row0 + q0);
            load_k(0);
            load_v(0);
            if (tiles > 1) {
                load_k(1);
                load_v(1);
            }
            // The scores run three tiles ahead of the products with V: tile t's scores need the S
            // buffer that the softmax warps emptied of tile t-2 and the K buffer that tile t-2's
            // scores have read.
            auto full = [&](unsigned long long (&bars)[2], int t) { return mbarrier_wait(&bars[t & 1], (t >> 1) & 1, abort_flag); };
            bool ok = mbarrier_wait(&q_full, 0, abort_flag) && full(k_full, 0);
            if (ok) scores(0);
            if (ok && tiles > 1) ok = full(k_full, 1);
            if (ok && tiles > 1) scores(1);
            for (int t = 2; t < 4 && t < tiles && ok; ++t) {
                ok = full(k_free, t - 2);
                if (ok) load_k(t);
            }
            if (ok && tiles > 2) {
                ok = full(k_full, 2) && full(s_free, 0);
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                if (ok) scores(2);
            }
            for (int j = 0; j < tiles && ok; ++j) {
                const int b = j & 1;
                if (j + 4 < tiles) {        // K_{j+2} has been multiplied: its buffer takes K_{j+4}
                    ok = full(k_free, j + 2);
                    if (!ok) break;
                    load_k(j + 4);
                }
                if (j >= 1 && j + 1 < tiles) {  // P_{j-1} V_{j-1} is done: its buffer takes V_{j+1}
                    ok = full(v_free, j - 1);
                    if (!ok) break;
                    load_v(j + 1);
                }
                ok = full(v_full, j) && full(p_ready, j);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const unsigned char* v_tile = v_tiles + b * QKV_TILE;
                const unsigned char* p_tile = p_tiles + b * P_TILE;
#pragma unroll
                for (int kk = 0; kk < BN / 16; ++kk) {
                    const unsigned long long a = desc_k_major(p_tile + (kk >> 2) * SPAN_BYTES + (kk & 3) * 32);
                    const unsigned long long v = desc_mn_major(v_tile + kk * 2048, SPAN_BYTES);
                    umma(tmem_o, a, v, idesc_o, (j > 0 || kk > 0) ? 1u : 0u);
                }
                umma_commit(&v_free[b]);
                if (j + 3 < tiles) {        // the softmax warps have just taken S_{j+1} into registers
                    ok = full(k_full, j + 3) && full(s_free, j + 1);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    scores(j + 3);
                }
            }
        }
    } else {
        // ------------------------------------------------------------- softmax
        const int quarter = warp & 3;                           // TMEM lanes 32*quarter .. +31
        const int group = (warp - 1) >> 2;                      // which share of a tile's keys
        const int r = quarter * 32 + lane;                      // query row of this thread
        const int key = group * SHARE;                          // its first key within a tile
        const int position = q0 + r;
        const unsigned lane_bits = (unsigned)(quarter * 32) << 16;
        const float scale_log2 = p.scale * LOG2E;
        float reference = -INFINITY;                            // what the exponentials are taken against
        float denom = 0.f;                                      // this thread's part of the row sum
        unsigned exchanges = 0;                                 // uses of row_shared so far
        bool ok = true;
        // The warps of a row share values: each writes its part and arrives; later it waits for
        // the others and reads all parts. The parts are double-buffered by the use's parity.
        auto row_post = [&]() { mbarrier_arrive(&row_shared[quarter]); };
        auto row_wait = [&]() {
            ok = mbarrier_wait(&row_shared[quarter], exchanges & 1, abort_flag);
            ++exchanges;
        };
        // Which keys of tile j this thread's share may see, and whether the tile needs a mask at all.
        auto bounds = [&](int j, int& first, int& last) -> bool {
            const int key0 = (tile_low + j) * BN;
            last = position - key0 - key;
            first = p.window > 0 ? position - p.window + 1 - key0 - key : 0;
            return key0 + BN - 1 > q0 || (p.window > 0 && q0 + BM - p.window > key0);   // the same for the block
        };
        // Loads this thread's scores of tile j (the values may be used after tmem_load_wait()).
        auto load_scores = [&](int j, float* s) {
            ok = mbarrier_wait(&s_ready[j & 1], (j >> 1) & 1, abort_flag);
            if (!ok) return;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
            for (int c = 0; c < SHARE; c += 32) tmem_load_32_issue(tmem + (j & 1) * 256 + lane_bits + key + c, s + c);
        };
        // Scores are in registers: the S buffer is free, and the row's warps post their maxima.
        auto release_and_post = [&](int j, const float (&s)[SHARE]) {
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            mbarrier_arrive(&s_free[j & 1]);
            int first, last;
            const bool masked = bounds(j, first, last);
            const float mine = masked ? share_maximum<true>(s, scale_log2, first, last)
                                      : share_maximum<false>(s, scale_log2, first, last);
            if (GROUPS > 1) {
                ctl.row_part[exchanges & 1][r][group] = (Exchange)mine;
                row_post();
            }
            return mine;
        };
        float s_even[SHARE], s_odd[SHARE];                      // scores of even and of odd tiles
        float mine = 0.f;
        // One tile: `s` holds its scores and `mine` this thread's maximum of them, already posted.
        auto tile = [&](int j, float (&s)[SHARE], float (&s_next)[SHARE]) {
            // The next tile's scores start coming while this tile's exponentials are computed.
            if (j + 1 < tiles) load_scores(j + 1, s_next);
            if (!ok) return;
            float top = mine;
            if (GROUPS > 1) {
                const Exchange(&parts)[GROUPS] = ctl.row_part[exchanges & 1][r];
                row_wait();
                if (!ok) return;
                top = (float)parts[0];
#pragma unroll
                for (int g = 1; g < GROUPS; ++g) top = fmaxf(top, (float)parts[g]);
            }
            // Raise the reference when a row of the warp has outgrown it; the warp then scales
            // its columns of O (TMEM loads and stores are warp-wide instructions). The warps
            // that share a row see the same maxima and decide alike.
            const bool raise = top > reference + RAISE_AFTER || (reference == -INFINITY && top > -INFINITY);
            if (__any_sync(0xffffffffu, raise)) {
                const float next = raise ? top : reference;
                const float ratio = reference == -INFINITY ? 0.f : exp2_approx(reference - next);
                reference = next;
                denom *= ratio;
                if (j > 0) {   // O holds the tiles before this one once P_{j-1} V_{j-1} is done
                    ok = mbarrier_wait(&v_free[(j - 1) & 1], ((j - 1) >> 1) & 1, abort_flag);
                    if (!ok) return;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    if (j + 1 < tiles) tmem_load_wait();   // the scores on their way come first
#pragma unroll 1
                    for (int c = 32 * group; c < D; c += 32 * GROUPS) {
                        float o[32];
                        tmem_load_32(tmem_o + lane_bits + c, o);
#pragma unroll
                        for (int i = 0; i < 32; ++i) o[i] *= ratio;
                        tmem_store_32(tmem_o + lane_bits + c, o);
                    }
                    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                }
            }
            if (j >= 2) {      // the P buffer was read by P_{j-2} V_{j-2}
                ok = mbarrier_wait(&v_free[j & 1], ((j - 2) >> 1) & 1, abort_flag);
                if (!ok) return;
            }
            const float against = reference == -INFINITY ? 0.f : reference;
            unsigned char* p_tile = p_tiles + (j & 1) * P_TILE;
            int first, last;
            const bool masked = bounds(j, first, last);
            denom += masked ? write_probabilities<true>(s, scale_log2, against, first, last, p_tile, r, key)
                            : write_probabilities<false>(s, scale_log2, against, first, last, p_tile, r, key);
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // P is read by the tensor core
            mbarrier_arrive(&p_ready[j & 1]);
            if (j + 1 < tiles) {
                tmem_load_wait();
                mine = release_and_post(j + 1, s_next);
            }
        };
        load_scores(0, s_even);
        tmem_load_wait();
        if (ok) mine = release_and_post(0, s_even);
        for (int j = 0; j < tiles && ok; j += 2) {
            tile(j, s_even, s_odd);
            if (j + 1 < tiles && ok) tile(j + 1, s_odd, s_even);
        }
        float total = denom;
        if (ok) ok = mbarrier_wait(&v_free[(tiles - 1) & 1], ((tiles - 1) >> 1) & 1, abort_flag);
        if (ok && GROUPS > 1) {   // every product is done: a P tile holds the parts of the row sums
            float* parts = reinterpret_cast<float*>(p_tiles) + r * GROUPS;
            parts[group] = denom;
            row_post();
            row_wait();
            total = parts[0];
#pragma unroll
            for (int g = 1; g < GROUPS; ++g) total += parts[g];
        }
        if (ok) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const float inverse = 1.0f / total;
            bf16* out = p.out + (long long)(row0 + q0 + r) * p.ldo + (long long)head * D;
#pragma unroll 1
            for (int c = 32 * group; c < D; c += 32 * GROUPS) {
                float o[32];
                tmem_load_32(tmem_o + lane_bits + c, o);
                if (r < q_rows) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        uint4 packed;
                        __nv_bfloat162* pairs = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
                        for (int t = 0; t < 4; ++t)
                            pairs[t] = __floats2bfloat162_rn(o[i + 2 * t] * inverse, o[i + 2 * t + 1] * inverse);
                        *reinterpret_cast<uint4*>(out + c + i) = packed;
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        if (lane == 0 && *abort_flag) {  // let the copies in flight land before the block leaves
            unsigned long long* loads[4] = {&k_full[0], &k_full[1], &v_full[0], &v_full[1]};
            for (int b = 0; b < 4; ++b)
                for (unsigned spin = 0; spin < (1u << 20); ++spin) {
                    unsigned done;
                    asm volatile(
                        "{\n\t.reg .pred p;\n\t"
                        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                        "selp.u32 %0, 1, 0, p;\n\t}"
                        : "=r"(done)
                        : "r"(smem_u32(loads[b])), "r"(0u)
                        : "memory");
                    if (done) break;
                }
        }
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLUMNS));
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

constexpr size_t SHARED_BYTES = (size_t)QKV_TILE * 5 + 2 * P_TILE + sizeof(Control);
}  // namespace

KIDI_API int kidi_attention_tcgen05_head_dim() { return D; }

KIDI_API int kidi_attention_tcgen05_timeout_flag() {
    int flag = 0;
    if (cudaMemcpyFromSymbol(&flag, kidi_attention_timeout, sizeof(int)) != cudaSuccess) return -1;
    return flag;
}

// Attention of every row of a step whose sequences all start at position 0.
// qkv [rows, ld]: heads query heads, then kv_heads key heads, then kv_heads value heads,
// each D wide, bfloat16, 16-byte aligned rows. out [rows, ldo] bfloat16.
KIDI_API int kidi_attention_prefill_tcgen05(const void* qkv, long long ld, int rows, void* out, long long ldo,
                                            const int* seq_len, const int* seq_row0, int seqs, int max_new, int heads,
                                            int kv_heads, int window, float scale, cudaStream_t stream) {
    if (rows <= 0 || seqs <= 0 || max_new <= 0) return 0;
    if (!(scale > 0.f) || heads % kv_heads || (max_new + BM - 1) / BM > 65535 || seqs > 65535 || (ld & 7) || (ldo & 7) || ((uintptr_t)qkv & 15) ||
        ((uintptr_t)out & 15))
        return KIDI_REFUSED_SIZE;
    EncodeTiled encode = encode_tiled();
    if (!encode) return KIDI_REFUSED_SIZE;
    CUtensorMap map;
    const cuuint64_t dims[2] = {(cuuint64_t)(heads + 2 * kv_heads) * D, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    const cuuint32_t box[2] = {64, 128};
    const cuuint32_t steps[2] = {1, 1};
    if (encode(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(qkv), dims, strides, box, steps,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return KIDI_REFUSED_SIZE;
    static bool configured = false;
    if (!configured) {
        cudaError_t status = cudaFuncSetAttribute(attention_prefill_tcgen05_kernel,
                                                  cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SHARED_BYTES);
        if (status != cudaSuccess) return (int)status;
        configured = true;
    }
    Params p;
    p.out = (bf16*)out;
    p.ldo = ldo;
    p.seq_len = seq_len;
    p.seq_row0 = seq_row0;
    p.heads = heads;
    p.kv_heads = kv_heads;
    p.window = window;
    p.scale = scale;
    dim3 grid(heads, seqs, (max_new + BM - 1) / BM);
    attention_prefill_tcgen05_kernel<<<grid, THREADS, SHARED_BYTES, stream>>>(map, p);
    return kidi_launch_status();
}
