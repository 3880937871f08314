// kidi_attention_decode_static: split-key decode attention for callers that must not
// allocate device memory.
//
// This entry point has no counterpart in the reference; it exists for users of this
// library's C interface.
//
// kidi_attention_decode merges the partial results of its key splits through a
// workspace that the caller allocates (rows * heads * splits * (head width + 2) floats).
// Some callers cannot provide one: a host program that drives the shared object through
// its exported C symbols has no tensor allocator, and a serving loop that has handed all
// device memory to its own pool at start-up must never reach cudaMalloc afterwards
// (cudaMalloc synchronises the whole device and may fail once the pool holds everything).
// For them this variant keeps the workspace in a file-scope device array of fixed size
// inside the library, KIDI_STATIC_SCRATCH_FLOATS floats (8 MiB), which every GPU that
// loads the library holds until the process exits. Inputs and outputs are still the
// caller's; the partial_out and partial_stat fields of the arguments are ignored.
//
// * It allocates nothing: no cudaMalloc, cudaFree or allocating library routine.
// * A call whose splits need more than KIDI_STATIC_SCRATCH_FLOATS floats, or whose rows,
//   heads or splits exceed KIDI_STATIC_MAX_ROWS / _HEADS / _SPLITS, is refused with
//   KIDI_REFUSED_SIZE (-3) and launches nothing.
// * The first call on a device looks up the device address of the array (with that
//   device current: the device is taken from cudaGetDevice, not from the stream) and keeps
//   it; make that first call before any stream capture. First calls from several host
//   threads at once are safe (the look-up gives every thread the same address).
// * Every call uses the same array, which keeps the contents of the last call. Nothing
//   in it has to start at zero: every block writes its own partial result before the
//   merge reads it. Two calls that overlap on the GPU (different streams) race on it;
//   issue them on one stream, or order them with events.
#pragma once

#include <cuda_runtime.h>

#define KIDI_STATIC_SCRATCH_FLOATS (2 * 1024 * 1024)

// Where the cached keys and values of a sequence lie: its pages are found through its row of
// the block table [slots, pages_per_seq]; a page holds 64 tokens (page_shift 6).
struct KidiCacheGeometry {
    const int* table;
    int pages_per_seq;
    int page_shift;
    int ring_pages;       // 0: every page of a sequence is kept; else the pages of a windowed ring
    int kv_heads;
    int head_dim;
};

// The argument block of kidi_attention_decode and of kidi_attention_decode_static, field by
// field what the library's own launcher fills in (all pointers are device pointers; bfloat16
// elements unless said otherwise). One query row per sequence; every key comes from the cache.
struct KidiAttentionArgs {
    const void* q;                 // [rows, ldq] bfloat16, head h at h * head width
    long long ldq;
    const void* k_step;            // with `fuse`: the step's new key and value rows [rows, ldkv]; else null
    const void* v_step;
    long long ldkv;
    const void* k_cache;           // [pages, kv_heads, 64, head width]
    const void* v_cache;
    struct KidiCacheGeometry cache;
    void* out;                     // [rows, ldo] bfloat16
    long long ldo;
    const int* row_seq;            // [rows]: the row's sequence; -1: a padding row (nothing is read or written)
    const int* row_pos;            // [rows]: the row's position in its sequence
    const int* seq_slot;           // [seqs]: the sequence's row of the block table
    const int* seq_start;          // [seqs]: tokens cached before this step
    const int* seq_len;            // [seqs]: tokens this step brings (1)
    const int* seq_row0;           // [seqs]: the sequence's first row
    int rows, seqs, heads, kv_heads, window;   // window 0: every earlier key is seen
    float scale;
    float* partial_out;            // the caller's workspace (ignored by the static entry point)
    float* partial_stat;
    int splits;                    // blocks that share a sequence's keys
    int* counters;                 // ignored by the static entry point
    int fuse;                      // bit 0: normalise and rotate q and the new key; bit 1: write the new key and value
    int norm_is_float;
    const void* q_norm;            // [head width] or null
    const void* k_norm;
    const float* cos_table;        // [positions, rotary_dim / 2] or null
    const float* sin_table;
    int rotary_dim;
    float eps;
    long long cache_rows;          // pages * kv_heads * 64 when k_cache and v_cache are contiguous (pages are then
                                   // copied whole by TMA where the head width allows), else 0
};

// Bounds the static entry point checks before it forms the size of the workspace.
#define KIDI_STATIC_MAX_ROWS 65535
#define KIDI_STATIC_MAX_HEADS 1024
#define KIDI_STATIC_MAX_SPLITS 256

extern "C" int kidi_attention_decode_static(const KidiAttentionArgs* args, cudaStream_t stream);

// The number of floats a call would need; at most KIDI_STATIC_SCRATCH_FLOATS is accepted.
extern "C" long long kidi_attention_decode_static_need(int rows, int heads, int splits);
