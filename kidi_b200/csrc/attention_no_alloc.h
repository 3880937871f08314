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
// * A call whose splits need more than KIDI_STATIC_SCRATCH_FLOATS floats is refused
//   with KIDI_REFUSED_SIZE (-3) and launches nothing.
// * The first call on a device looks up the device address of the array (with that
//   device current) and keeps it; make that first call before any stream capture.
// * Every call uses the same array, which keeps the contents of the last call. Nothing
//   in it has to start at zero: every block writes its own partial result before the
//   merge reads it. Two calls that overlap on the GPU (different streams) race on it;
//   issue them on one stream, or order them with events.
#pragma once

#include <cuda_runtime.h>

#define KIDI_STATIC_SCRATCH_FLOATS (2 * 1024 * 1024)

struct KidiAttentionArgs;  // the argument block of kidi_attention_decode (attention_bf16.cu: Args)

extern "C" int kidi_attention_decode_static(const KidiAttentionArgs* args, cudaStream_t stream);

// The number of floats a call would need; at most KIDI_STATIC_SCRATCH_FLOATS is accepted.
extern "C" long long kidi_attention_decode_static_need(int rows, int heads, int splits);
