// Causal grouped-query attention for prompts on the 5th-generation tensor cores,
// compiled for one head width (-DKIDI_HEAD_DIM=64 or 128).
//
// A block owns 128 query rows of one sequence for two query heads that share a key/value
// head, and walks the sequence's keys in tiles of 128. Every key of the step is one of the
// step's own rows (the sequences start at position 0), so queries, keys and values are
// tiles of the packed qkv matrix and arrive by TMA with the 128-byte swizzle; a K/V tile is
// loaded once and used by both heads. Per key tile and head:
//   S = Q K^T      tcgen05.mma, 128 x 128 x head width, accumulator in tensor memory;
//   softmax        a head has a team of eight warps; a query row is one TMEM lane, and the
//                  team's two warps that may read a lane quarter each take half of the
//                  tile's keys. A thread loads its share of the row's scores and releases
//                  S at once (the head's scores of the next tile are computed meanwhile),
//                  the row's warps combine their maxima through shared memory, then each
//                  computes its exponentials and its part of the row sum, all in 32-bit;
//                  P is rounded to bfloat16, kept in registers until the product of the
//                  tile before has read its P, and then written to shared memory in the
//                  swizzled K-major layout of an A operand;
//   O += P V       tcgen05.mma with V as an MN-major B operand (V rows are keys, the
//                  contraction runs over keys), accumulating in the head's TMEM region
//                  over all key tiles. The exponentials are taken against a reference
//                  maximum that is raised only when the row's maximum has grown by more
//                  than 2^8 since (then the warp multiplies its rows of O and the row sums
//                  by the ratio); P stays below 2^8, and the final division by the row sum
//                  makes the result independent of the reference.
// One thread a head issues its matrix instructions and another thread the copies; mbarriers
// order them with the softmax teams. The two heads run independently of each other beyond
// sharing K and V. Measured on a B200 the matrix instructions, whose operands all come
// from shared memory, keep its 128 bytes a cycle busy most of the time, and the
// exponentials the special-function unit about half of it. Every wait is bounded: a block
// that gives up records it in kidi_attention_timeout and leaves without storing.
//
// Formulas: src/kidi/layers/qwen3.cpp:53-54, src/kidi/runtime/vulkan/attention.comp:32-101;
// causal rule src/kidi/model/gemma4.cpp:736-740.
#include <cuda.h>

#include "common.cuh"


#ifndef KIDI_HEAD_DIM
#error "compile with -DKIDI_HEAD_DIM=64 or 128"
#endif

namespace {

constexpr int D = KIDI_HEAD_DIM;
static_assert(D == 64 || D == 128, "the tensor-memory attention kernel takes head widths 64 and 128");
constexpr int BM = 128, BN = 128;                 // queries per block and head, keys per tile
constexpr int HEADS = 2;                          // query heads of a block (they share K and V)
constexpr int SPANS = D / 64;                     // 128-byte swizzle spans per row of Q, K, V
constexpr int SPAN_BYTES = 128 * 128;             // 128 rows x 128 bytes
constexpr int QKV_TILE = SPANS * SPAN_BYTES;      // bytes of a Q, K or V tile
constexpr int P_TILE = 2 * SPAN_BYTES;            // P: 128 rows x 128 keys
constexpr int GROUPS = 2;                         // warps that share a query row's keys of a tile
constexpr int SHARE = BN / GROUPS;                // keys of a tile per softmax thread
constexpr int TEAM_THREADS = 128 * GROUPS;        // the softmax warps of one head
// Warps 0..3 are the control warpgroup (a warp per head for its matrix instructions, one for
// the copies, one idle); then a team of GROUPS x 4 softmax warps per head.
constexpr int CONTROL_WARPS = 4;
constexpr int THREADS = 32 * CONTROL_WARPS + HEADS * TEAM_THREADS;
// Registers move from the control warps, which need few, to the softmax warps, which hold a
// row's 64 scores (setmaxnreg works on warpgroups of four warps).
constexpr int CONTROL_REGISTERS = 32, SOFTMAX_REGISTERS = 112;
constexpr unsigned SPIN_LIMIT = 1u << 24;
constexpr float LOG2E = 1.4426950408889634f;
constexpr float RAISE_AFTER = 8.0f;               // the reference maximum follows after a growth of 2^8
constexpr int TMEM_COLUMNS = 512;                 // S of head h: columns 128 h ..; O of head h: 256 + 128 h ..

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
// The instruction is ordered with the barriers around it by tcgen05.commit and the
// tcgen05 fences, which carry the memory clobbers.
__device__ __forceinline__ void umma(unsigned tmem_d, unsigned long long a, unsigned long long b, unsigned idesc,
                                     bool accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        :
        : "r"(tmem_d), "l"(a), "l"(b), "r"(idesc), "r"((unsigned)accumulate));
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
// Eight columns at a time, for code that has few registers to spare.
__device__ __forceinline__ void tmem_load_8(unsigned address, float (&v)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3]), "=f"(v[4]), "=f"(v[5]), "=f"(v[6]), "=f"(v[7])
                 : "r"(address)
                 : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_store_8(unsigned address, const float (&v)[8]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
                 :
                 : "r"(address), "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]), "f"(v[4]), "f"(v[5]), "f"(v[6]), "f"(v[7])
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
// which cancels in the result: they are exchanged as bfloat16 to fit the shared memory left
// beside the tiles.
typedef bf16 Exchange;

struct Control {
    Exchange row_part[HEADS][2][BM][GROUPS];   // by head and the exchange's parity: each warp's maximum of a row
    unsigned long long q_full, k_full, k_free, v_full[2], v_free[2];
    unsigned long long s_ready[HEADS], s_free[HEADS], p_ready[HEADS], pv_done[HEADS];
    unsigned long long row_shared[HEADS][4];   // the warps of a head's row quarter have written their part
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
    // Prompts that continue sequences whose earlier tokens are in the cache (from_cache): every
    // key and value, the step's own included, is read from the cache's pages (the step's rows
    // were written there before this kernel), two 64-token pages per tile.
    int from_cache;
    const int* seq_start;   // [seqs] tokens in the cache before this step
    const int* seq_slot;    // [seqs]
    CacheGeometry cache;
};

// Where a block works: its sequence, query rows, heads and key tiles.
struct Place {
    int count, q0, row0, q_rows, tile_low, tiles, kv_head, head0, heads_here, start, slot;
    __device__ __forceinline__ explicit Place(const Params& p) {
        // Long blocks first: a block's number of key tiles grows with its query tile, and blocks
        // start in the order of their linear index, of which z is the slowest part.
        const int q_index = gridDim.z - 1 - blockIdx.z;
        const int seq = blockIdx.y;
        const int group_size = p.heads / p.kv_heads;
        const int pairs = (group_size + HEADS - 1) / HEADS;
        kv_head = blockIdx.x / pairs;
        head0 = kv_head * group_size + (blockIdx.x % pairs) * HEADS;     // the block's first query head
        heads_here = min(HEADS, (kv_head + 1) * group_size - head0);
        count = p.seq_len[seq];
        q0 = q_index * BM;
        row0 = p.seq_row0[seq];
        start = p.from_cache ? p.seq_start[seq] : 0;
        slot = p.from_cache ? p.seq_slot[seq] : 0;
        q_rows = min(BM, count - q0);
        const int high = start + q0 + q_rows - 1;                          // last query position of the block
        const int low = p.window > 0 ? max(0, start + q0 - p.window + 1) : 0;   // first key any of its queries sees
        tile_low = low / BN;
        tiles = high / BN - tile_low + 1;
    }
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

// P = exp2(s * scale - reference), rounded to bfloat16 and packed in pairs; returns the sum.
template <bool MASKED>
__device__ __forceinline__ float probabilities(const float (&s)[SHARE], float scale_log2, float reference, int first,
                                               int last, unsigned (&packed)[SHARE / 2]) {
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < SHARE; i += 2) {
        float p0 = exp2_approx(fmaf(s[i], scale_log2, -reference));
        float p1 = exp2_approx(fmaf(s[i + 1], scale_log2, -reference));
        if (MASKED) {
            if (i < first || i > last) p0 = 0.f;
            if (i + 1 < first || i + 1 > last) p1 = 0.f;
        }
        sum += p0 + p1;
        __nv_bfloat162 pair = __floats2bfloat162_rn(p0, p1);
        packed[i >> 1] = *reinterpret_cast<unsigned*>(&pair);
    }
    return sum;
}

// Writes a thread's packed P into the swizzled K-major tile. `p_row` is the shared-memory
// address of the thread's row in the tile's first 64-key span, `key` its first key.
__device__ __forceinline__ void store_probabilities(const unsigned (&packed)[SHARE / 2], unsigned p_row, int r,
                                                    int key) {
#pragma unroll
    for (int c = 0; c < SHARE; c += 8) {        // one 16-byte chunk of eight keys
        const int at = key + c;                 // SHARE divides 64 or is a multiple of it
        const unsigned address = p_row + (at >> 6) * SPAN_BYTES + ((((at & 63) >> 3) ^ (r & 7)) << 4);
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(address), "r"(packed[c / 2]),
                     "r"(packed[c / 2 + 1]), "r"(packed[c / 2 + 2]), "r"(packed[c / 2 + 3])
                     : "memory");
    }
}

__global__ void __launch_bounds__(THREADS, 1)
attention_prefill_tcgen05_kernel(const __grid_constant__ CUtensorMap map, const __grid_constant__ CUtensorMap k_map,
                                 const __grid_constant__ CUtensorMap v_map, Params p) {
    // All shared memory is dynamic and laid out here; the tiles come first because the
    // 128-byte swizzle wants them on 1024-byte boundaries.
    extern __shared__ __align__(1024) unsigned char base[];
    unsigned char* q_tiles = base;                         // HEADS tiles of [SPANS][128][128 B]
    unsigned char* k_tile = q_tiles + HEADS * QKV_TILE;    // 1 buffer
    unsigned char* v_tiles = k_tile + QKV_TILE;            // 2 buffers
    unsigned char* p_tiles = v_tiles + 2 * QKV_TILE;       // HEADS tiles of [2][128][128 B]
    Control& ctl = *reinterpret_cast<Control*>(p_tiles + HEADS * P_TILE);
    if (smem_u32(base) & 1023u) {                          // never seen; a wrong result would be worse than none
        if (threadIdx.x == 0) kidi_attention_timeout = 2;
        return;
    }

    // Each role works out the block's place itself, after it has taken or given registers:
    // what is computed before that point would have to live in the smaller register set.
    const Place first_look(p);
    if (first_look.q0 >= first_look.count) return;
    const int heads_here = first_look.heads_here;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        mbarrier_init(&ctl.q_full, 1);
        mbarrier_init(&ctl.k_full, 1);
        mbarrier_init(&ctl.k_free, heads_here);            // each head's thread commits its scores
        for (int i = 0; i < 2; ++i) {
            mbarrier_init(&ctl.v_full[i], 1);
            mbarrier_init(&ctl.v_free[i], heads_here);
        }
        for (int h = 0; h < HEADS; ++h) {
            mbarrier_init(&ctl.s_ready[h], 1);
            mbarrier_init(&ctl.s_free[h], TEAM_THREADS);
            mbarrier_init(&ctl.p_ready[h], TEAM_THREADS);
            for (int i = 0; i < 4; ++i) mbarrier_init(&ctl.row_shared[h][i], 32 * GROUPS);
            mbarrier_init(&ctl.pv_done[h], 1);
        }
        ctl.gave_up = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&ctl.tmem_slot)),
                     "r"(TMEM_COLUMNS));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const unsigned tmem = ctl.tmem_slot;
    volatile int* abort_flag = &ctl.gave_up;
    // The barriers of a head (s_ready, s_free, p_ready, pv_done) and of K complete once per
    // key tile: tile j waits for parity j & 1. V has two buffers: tile j uses buffer j & 1 and
    // waits for parity (j >> 1) & 1. (K's one buffer is refilled a tile ahead, when both heads'
    // scores have read it; V's copy would lie on the path from one tile's products to the next.)
    // A barrier counts arrivals without knowing which tile they belong to: every barrier here
    // is one that a thread cannot reach for its next use before all threads have arrived for
    // this one.

    // (One if/else holds both register changes and the roles under them, so that the compiler
    // sees which register count each role's code runs with.)
    if (warp < CONTROL_WARPS) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(CONTROL_REGISTERS));
        if (warp < HEADS) {
            const int h = warp;
            if (lane == 0 && h < heads_here) {
                const Place at(p);
                const int tiles = at.tiles;
                // ------------------------------ matrix instructions of head h (one thread a head)
                // The operand descriptors are built once; a step along k adds to the address field
                // (16-byte units; a shared-memory address never carries out of its 14 bits).
                constexpr unsigned idesc_s = instr_desc(BN, false), idesc_o = instr_desc(D, true);
                const unsigned long long q_desc = desc_k_major(q_tiles + h * QKV_TILE), k_desc = desc_k_major(k_tile);
                const unsigned long long p_desc = desc_k_major(p_tiles + h * P_TILE);
                const unsigned tmem_s = tmem + h * 128, tmem_o = tmem + 256 + h * 128;
                // (The loops over k stay rolled: this thread runs with few registers, and an
                // instruction takes longer to be accepted than its operands to be computed.)
                auto scores = [&]() {                   // S_h = Q_h K^T
#pragma unroll 1
                    for (int kk = 0; kk < D / 16; ++kk) {
                        const unsigned offset = (kk >> 2) * (SPAN_BYTES >> 4) + (kk & 3) * 2;
                        umma(tmem_s, q_desc + offset, k_desc + offset, idesc_s, kk > 0);
                    }
                    umma_commit(&ctl.s_ready[h]);
                    umma_commit(&ctl.k_free);
                };
                bool ok = mbarrier_wait(&ctl.q_full, 0, abort_flag) && mbarrier_wait(&ctl.k_full, 0, abort_flag);
                if (ok) scores();
                for (int j = 0; j < tiles && ok; ++j) {
                    if (j + 1 < tiles) {             // the head's next scores, as soon as the softmax warps hold these
                        ok = mbarrier_wait(&ctl.k_full, (j + 1) & 1, abort_flag) &&
                             mbarrier_wait(&ctl.s_free[h], j & 1, abort_flag);
                        if (!ok) break;
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        scores();
                    }
                    ok = mbarrier_wait(&ctl.v_full[j & 1], (j >> 1) & 1, abort_flag);
                    ok = ok && mbarrier_wait(&ctl.p_ready[h], j & 1, abort_flag);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const unsigned long long v_desc = desc_mn_major(v_tiles + (j & 1) * QKV_TILE, SPAN_BYTES);
#pragma unroll 1
                    for (int kk = 0; kk < BN / 16; ++kk) {
                        const unsigned a_offset = (kk >> 2) * (SPAN_BYTES >> 4) + (kk & 3) * 2;
                        umma(tmem_o, p_desc + a_offset, v_desc + kk * (2048 >> 4), idesc_o, j > 0 || kk > 0);
                    }
                    umma_commit(&ctl.pv_done[h]);
                    umma_commit(&ctl.v_free[j & 1]);
                }
            }
        } else if (warp == HEADS) {
            if (lane == 0) {
                // -------------------------------------------------------------- copies
                const Place at(p);
                const int tiles = at.tiles, tile_low = at.tile_low, row0 = at.row0, q0 = at.q0, head0 = at.head0;
                const int k_col = (p.heads + at.kv_head) * D, v_col = (p.heads + p.kv_heads + at.kv_head) * D;
                auto load_tile = [&](unsigned char* tile, unsigned long long* bar, int column, int row) {
                    for (int s = 0; s < SPANS; ++s) tma_load_2d(tile + s * SPAN_BYTES, &map, bar, column + 64 * s, row);
                };
                // From the cache a tile is two pages (64 rows each) of the sequence's row of the block
                // table; a page past the sequence's last one is replaced by the last one (masked).
                const int last_page = (at.start + at.count - 1) >> 6;
                auto load_pages = [&](unsigned char* tile, unsigned long long* bar, const CUtensorMap* pages, int j) {
                    for (int half = 0; half < 2; ++half) {
                        const int page_index = min((tile_low + j) * 2 + half, last_page);
                        const int page = p.cache.table[(long long)at.slot * p.cache.pages_per_seq + page_index];
                        const int page_row = (page * p.cache.kv_heads + at.kv_head) * 64;
                        for (int s = 0; s < SPANS; ++s)
                            tma_load_2d(tile + s * SPAN_BYTES + half * (64 * 128), pages, bar, 64 * s, page_row);
                    }
                };
                auto load_k = [&](int j) {
                    mbarrier_expect_tx(&ctl.k_full, QKV_TILE);
                    if (p.from_cache) load_pages(k_tile, &ctl.k_full, &k_map, j);
                    else load_tile(k_tile, &ctl.k_full, k_col, row0 + (tile_low + j) * BN);
                };
                auto load_v = [&](int j) {
                    mbarrier_expect_tx(&ctl.v_full[j & 1], QKV_TILE);
                    if (p.from_cache) load_pages(v_tiles + (j & 1) * QKV_TILE, &ctl.v_full[j & 1], &v_map, j);
                    else load_tile(v_tiles + (j & 1) * QKV_TILE, &ctl.v_full[j & 1], v_col, row0 + (tile_low + j) * BN);
                };
                mbarrier_expect_tx(&ctl.q_full, heads_here * QKV_TILE);
                for (int h = 0; h < heads_here; ++h)
                    load_tile(q_tiles + h * QKV_TILE, &ctl.q_full, (head0 + h) * D, row0 + q0);
                load_k(0);
                load_v(0);
                if (tiles > 1) load_v(1);
                bool ok = true;
                for (int j = 0; j + 1 < tiles && ok; ++j) {
                    // Both heads' scores of tile j are done (they were issued a tile ago): K_{j+1} follows.
                    ok = mbarrier_wait(&ctl.k_free, j & 1, abort_flag);
                    if (!ok) break;
                    load_k(j + 1);
                    if (j >= 1) {                    // both heads' P V_{j-1} are done: the buffer takes V_{j+1}
                        ok = mbarrier_wait(&ctl.v_free[(j - 1) & 1], ((j - 1) >> 1) & 1, abort_flag);
                        if (!ok) break;
                        load_v(j + 1);
                    }
                }
            }
        }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(SOFTMAX_REGISTERS));
        if ((warp - CONTROL_WARPS) / (4 * GROUPS) < heads_here) {
            // ------------------------------------------- softmax: a team of warps per head
            const Place at(p);
            const int tiles = at.tiles, tile_low = at.tile_low, row0 = at.row0, q0 = at.q0, head0 = at.head0,
                      q_rows = at.q_rows;
            const int h = (warp - CONTROL_WARPS) / (4 * GROUPS);    // the team's head
            const int quarter = warp & 3;                           // TMEM lanes 32*quarter .. +31
            const int group = ((warp - CONTROL_WARPS) >> 2) % GROUPS;   // which share of a tile's keys
            const int r = quarter * 32 + lane;                      // query row of this thread
            const int key = group * SHARE;                          // its first key within a tile
            const int position = at.start + q0 + r;
            const unsigned lane_bits = (unsigned)(quarter * 32) << 16;
            const unsigned tmem_s = tmem + h * 128 + lane_bits + key, tmem_o = tmem + 256 + h * 128 + lane_bits;
            unsigned char* p_tile = p_tiles + h * P_TILE;
            const unsigned p_row = smem_u32(p_tile) + r * 128;
            const float scale_log2 = p.scale * LOG2E;
            float reference = -INFINITY;                            // what the exponentials are taken against
            float denom = 0.f;                                      // this thread's part of the row sum
            unsigned exchanges = 0;                                 // uses of row_shared so far
            bool ok = true;
            // The warps of a row share values: each writes its part and arrives, waits for the
            // others and reads all parts. The parts are double-buffered by the use's parity.
            auto row_exchange = [&]() {
                mbarrier_arrive(&ctl.row_shared[h][quarter]);
                ok = mbarrier_wait(&ctl.row_shared[h][quarter], exchanges & 1, abort_flag);
                ++exchanges;
            };
            for (int j = 0; j < tiles && ok; ++j) {
                // The keys of this thread's share that the row may see: first..last; whether the
                // tile needs a mask at all is the same for the whole block.
                const int key0 = (tile_low + j) * BN;
                const int last = position - key0 - key;
                const int first = p.window > 0 ? position - p.window + 1 - key0 - key : 0;
                const bool masked =
                    key0 + BN - 1 > at.start + q0 || (p.window > 0 && at.start + q0 + BM - p.window > key0);
                ok = mbarrier_wait(&ctl.s_ready[h], j & 1, abort_flag);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                float s[SHARE];
#pragma unroll
                for (int c = 0; c < SHARE; c += 32) tmem_load_32_issue(tmem_s + c, s + c);
                tmem_load_wait();
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                mbarrier_arrive(&ctl.s_free[h]);
                const float mine = masked ? share_maximum<true>(s, scale_log2, first, last)
                                          : share_maximum<false>(s, scale_log2, first, last);
                Exchange(&parts)[GROUPS] = ctl.row_part[h][exchanges & 1][r];
                parts[group] = (Exchange)mine;
                row_exchange();
                if (!ok) break;
                float top = (float)parts[0];
#pragma unroll
                for (int g = 1; g < GROUPS; ++g) top = fmaxf(top, (float)parts[g]);
                // Raise the reference when a row of the warp has outgrown it; the warp then scales
                // its columns of O (TMEM loads and stores are warp-wide instructions), for which the
                // product of the tile before must be done. The warps that share a row see the same
                // maxima and decide alike.
                const bool raise = top > reference + RAISE_AFTER || (reference == -INFINITY && top > -INFINITY);
                bool rested = j == 0;                                   // O is at rest and the P tile is free
                if (__any_sync(0xffffffffu, raise)) {
                    const float next = raise ? top : reference;
                    const float ratio = reference == -INFINITY ? 0.f : exp2_approx(reference - next);
                    reference = next;
                    denom *= ratio;
                    if (j > 0) {
                        ok = mbarrier_wait(&ctl.pv_done[h], (j - 1) & 1, abort_flag);
                        if (!ok) break;
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        rested = true;
#pragma unroll 1
                        for (int c = (D / GROUPS) * group; c < (D / GROUPS) * (group + 1); c += 8) {
                            float o[8];      // the scores are alive: few registers to spare
                            tmem_load_8(tmem_o + c, o);
#pragma unroll
                            for (int i = 0; i < 8; ++i) o[i] *= ratio;
                            tmem_store_8(tmem_o + c, o);
                        }
                        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                    }
                }
                // The exponentials stay in registers until the product of the tile before has read
                // its P from the tile in shared memory: they are computed while that product runs.
                const float against = reference == -INFINITY ? 0.f : reference;
                unsigned packed[SHARE / 2];
                denom += masked ? probabilities<true>(s, scale_log2, against, first, last, packed)
                                : probabilities<false>(s, scale_log2, against, first, last, packed);
                if (!rested) {
                    ok = mbarrier_wait(&ctl.pv_done[h], (j - 1) & 1, abort_flag);
                    if (!ok) break;
                }
                store_probabilities(packed, p_row, r, key);
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // P is read by the tensor core
                mbarrier_arrive(&ctl.p_ready[h]);
            }
            if (ok) ok = mbarrier_wait(&ctl.pv_done[h], (tiles - 1) & 1, abort_flag);
            if (ok) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                // The head's products are done: its P tile holds the parts of the row sums.
                float* parts = reinterpret_cast<float*>(p_tile) + r * GROUPS;
                parts[group] = denom;
                row_exchange();
                float total = parts[0];
#pragma unroll
                for (int g = 1; g < GROUPS; ++g) total += parts[g];
                const float inverse = 1.0f / total;
                bf16* out = p.out + (long long)(row0 + q0 + r) * p.ldo + (long long)(head0 + h) * D;
#pragma unroll 1
                for (int c = 32 * group; c < D && ok; c += 32 * GROUPS) {
                    float o[32];
                    tmem_load_32(tmem_o + c, o);
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
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        if (lane == 0 && *abort_flag) {  // let the copies in flight land before the block leaves
            unsigned long long* loads[4] = {&ctl.q_full, &ctl.k_full, &ctl.v_full[0], &ctl.v_full[1]};
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

constexpr size_t SHARED_BYTES = (size_t)QKV_TILE * (HEADS + 3) + HEADS * P_TILE + sizeof(Control);
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
struct KidiPromptCache {     // where the keys and values lie when prompts continue cached sequences
    const void* keys;        // [pages, kv_heads, 64, D] bfloat16
    const void* values;
    long long rows;          // pages * kv_heads * 64
    const int* table;        // [slots, pages_per_seq]
    int pages_per_seq;
    const int* seq_start;    // [seqs]
    const int* seq_slot;     // [seqs]
};

// `cache` null: every sequence starts at position 0 and its keys are rows of qkv. Else every
// key and value is read from the cache (64-token pages; no ring), into which the step's own
// rows have been written already.
KIDI_API int kidi_attention_prefill_tcgen05(const void* qkv, long long ld, int rows, void* out, long long ldo,
                                            const int* seq_len, const int* seq_row0, int seqs, int max_new, int heads,
                                            int kv_heads, int window, float scale, const KidiPromptCache* cache,
                                            cudaStream_t stream) {
    if (rows <= 0 || seqs <= 0 || max_new <= 0) return 0;
    if (!(scale > 0.f) || heads % kv_heads || (max_new + BM - 1) / BM > 65535 || seqs > 65535 || (ld & 7) ||
        (ldo & 7) || ((uintptr_t)qkv & 15) ||
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
    static bool configured[64] = {};        // per device: the kernel may use this much shared memory
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return KIDI_REFUSED_SIZE;
    if (!configured[device]) {
        cudaError_t status = cudaFuncSetAttribute(attention_prefill_tcgen05_kernel,
                                                  cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SHARED_BYTES);
        if (status != cudaSuccess) return (int)status;
        configured[device] = true;
    }
    CUtensorMap k_map, v_map;
    memset(&k_map, 0, sizeof(k_map));
    memset(&v_map, 0, sizeof(v_map));
    Params p;
    memset(&p, 0, sizeof(p));
    if (cache) {
        if (!cache->keys || !cache->values || cache->rows <= 0 || !cache->table || !cache->seq_start ||
            !cache->seq_slot || ((uintptr_t)cache->keys & 15) || ((uintptr_t)cache->values & 15))
            return KIDI_REFUSED_SIZE;
        const cuuint64_t page_dims[2] = {(cuuint64_t)D, (cuuint64_t)cache->rows};
        const cuuint64_t page_strides[1] = {(cuuint64_t)D * 2};
        const cuuint32_t page_box[2] = {64, 64};
        const void* bases[2] = {cache->keys, cache->values};
        CUtensorMap* maps[2] = {&k_map, &v_map};
        for (int i = 0; i < 2; ++i)
            if (encode(maps[i], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(bases[i]), page_dims,
                       page_strides, page_box, steps, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                       CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
                return KIDI_REFUSED_SIZE;
        p.from_cache = 1;
        p.seq_start = cache->seq_start;
        p.seq_slot = cache->seq_slot;
        p.cache.table = cache->table;
        p.cache.pages_per_seq = cache->pages_per_seq;
        p.cache.page_shift = 6;
        p.cache.kv_heads = kv_heads;
        p.cache.head_dim = D;
    }
    p.out = (bf16*)out;
    p.ldo = ldo;
    p.seq_len = seq_len;
    p.seq_row0 = seq_row0;
    p.heads = heads;
    p.kv_heads = kv_heads;
    p.window = window;
    p.scale = scale;
    const int group_size = heads / kv_heads;
    dim3 grid(kv_heads * ((group_size + HEADS - 1) / HEADS), seqs, (max_new + BM - 1) / BM);
    attention_prefill_tcgen05_kernel<<<grid, THREADS, SHARED_BYTES, stream>>>(map, k_map, v_map, p);
    return kidi_launch_status();
}
