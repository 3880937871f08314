// Token selection on the device: greedy argmax and temperature sampling.
//
// Greedy follows the reference's rules: the largest logit wins, ties go to the lowest
// index, and a row that holds a NaN or +infinity, or no finite value at all, selects
// -1, which the generation loop rejects (ARCHITECTURE.md:612-616,
// src/kidi/runtime/mps/eager_kernels.metal:30-50, src/kidi/inference/decoder.cpp:72-78).
// Temperature sampling is this library's own (the reference samples text greedily
// only): p = softmax(logits / T) in 32-bit, then the inverse of the cumulative
// distribution in index order at a uniform number u that depends on (seed, sequence
// key, step) only, so a sequence draws the same tokens in any batch.
#include "common.cuh"

namespace {
constexpr int THREADS = 256;

struct Best {
    float value;
    int index;
};

__device__ __forceinline__ Best better(Best a, Best b) {
    if (b.value > a.value || (b.value == a.value && b.index < a.index)) return b;
    return a;
}

// Returns the row's argmax to every thread; index -1 for an invalid row.
__device__ Best block_argmax(const float* row, int vocab, float inverse_temperature, Best* scratch, int* invalid) {
    Best best{-INFINITY, 0x7fffffff};
    bool bad = false;
    for (int c = threadIdx.x; c < vocab; c += THREADS) {
        const float value = row[c];
        bad |= isnan(value) || value == INFINITY;
        if (value > best.value) best = Best{value, c};  // ascending c: the first maximum stays
    }
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
        Best other{__shfl_xor_sync(0xffffffffu, best.value, offset), __shfl_xor_sync(0xffffffffu, best.index, offset)};
        best = better(best, other);
    }
    if (threadIdx.x == 0) *invalid = 0;
    __syncthreads();
    if (bad) atomicOr(invalid, 1);
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = best;
    __syncthreads();
    best = scratch[0];
#pragma unroll
    for (int w = 1; w < THREADS / 32; ++w) best = better(best, scratch[w]);
    if (*invalid || best.value == -INFINITY) best.index = -1;
    (void)inverse_temperature;
    return best;
}

__global__ void __launch_bounds__(THREADS) argmax_kernel(const float* __restrict__ logits, int* __restrict__ out,
                                                         int vocab) {
    __shared__ Best scratch[THREADS / 32];
    __shared__ int invalid;
    const Best best = block_argmax(logits + (long long)blockIdx.x * vocab, vocab, 1.f, scratch, &invalid);
    if (threadIdx.x == 0) out[blockIdx.x] = best.index;
}

// Greedy selection in two stages, so that a row's vocabulary is scanned by many blocks:
// stage one reduces a slice of the row per block, stage two the slices of a row.
// index -2 marks a slice that holds a NaN or +infinity.
__global__ void __launch_bounds__(THREADS)
argmax_slices_kernel(const float* __restrict__ logits, float* __restrict__ slice_value, int* __restrict__ slice_index,
                     int vocab, int slices) {
    __shared__ Best scratch[THREADS / 32];
    __shared__ int invalid;
    const int slice = blockIdx.x, row = blockIdx.y;
    const int width = (vocab + slices - 1) / slices;
    const int begin = min(vocab, slice * width), count = min(vocab, begin + width) - begin;
    Best best = block_argmax(logits + (long long)row * vocab + begin, count, 1.f, scratch, &invalid);
    if (threadIdx.x == 0) {
        const bool bad = invalid != 0;
        slice_value[row * slices + slice] = best.value;
        slice_index[row * slices + slice] = bad ? -2 : (best.index >= 0 ? best.index + begin : -1);
    }
}

__global__ void argmax_merge_kernel(const float* __restrict__ slice_value, const int* __restrict__ slice_index,
                                    int* __restrict__ out, int slices) {
    const int row = blockIdx.x;
    if (threadIdx.x != 0) return;
    Best best{-INFINITY, -1};
    bool bad = false;
    for (int s = 0; s < slices; ++s) {  // ascending slices: the first maximum stays
        const int index = slice_index[row * slices + s];
        bad |= index == -2;
        if (index >= 0 && slice_value[row * slices + s] > best.value) best = Best{slice_value[row * slices + s], index};
    }
    out[row] = bad ? -1 : best.index;
}

// 64-bit mix (splitmix64 finaliser) of the three keys; 24 random bits -> u in [0, 1).
__device__ __forceinline__ float uniform_from(unsigned long long seed, unsigned long long key,
                                              unsigned long long step) {
    unsigned long long z = seed * 0x9E3779B97F4A7C15ull + key * 0xBF58476D1CE4E5B9ull + step * 0x94D049BB133111EBull +
                           0x2545F4914F6CDD1Dull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z = z ^ (z >> 31);
    return (float)(z >> 40) * (1.0f / 16777216.0f);
}

// One block per row. Thread t owns the contiguous chunk [t*chunk, (t+1)*chunk) of the
// vocabulary, so that the cumulative sum runs in index order.
__global__ void __launch_bounds__(THREADS)
sample_kernel(const float* __restrict__ logits, int* __restrict__ out, int vocab, const float* __restrict__ temperature,
              unsigned long long seed, const long long* __restrict__ keys, const int* __restrict__ steps) {
    __shared__ float sums[THREADS];
    __shared__ float reduce[32];
    const int r = blockIdx.x;
    const float* row = logits + (long long)r * vocab;
    // out[r] holds the row's argmax already (the two greedy stages ran before this kernel).
    const float t = temperature[r];
    const int top = out[r];
    if (top < 0 || !(t > 0.f)) return;  // greedy, or nothing to draw from
    const Best best{row[top], top};
    const float inverse = 1.0f / t;
    const int chunk = (vocab + THREADS - 1) / THREADS;
    const int begin = min(vocab, (int)threadIdx.x * chunk), end = min(vocab, begin + chunk);
    float mine = 0.f;
    for (int c = begin; c < end; ++c) mine += expf((row[c] - best.value) * inverse);
    sums[threadIdx.x] = mine;
    const float total = block_sum<THREADS>(mine, reduce);
    const float target = uniform_from(seed, (unsigned long long)keys[r], (unsigned long long)steps[r]) * total;
    __syncthreads();
    // The owner of the target: the first thread whose inclusive prefix exceeds it.
    if (threadIdx.x == 0) {
        float before = 0.f;
        int owner = THREADS - 1;
        for (int w = 0; w < THREADS; ++w) {
            if (before + sums[w] > target) { owner = w; break; }
            before += sums[w];
        }
        // Walk the owner's chunk.
        const int first = min(vocab, owner * chunk), last = min(vocab, first + chunk);
        int chosen = -1;
        float running = before;
        for (int c = first; c < last; ++c) {
            const float p = expf((row[c] - best.value) * inverse);
            running += p;
            if (p > 0.f) chosen = c;          // the last token with mass, should rounding leave the target beyond
            if (running > target) { chosen = c; break; }
        }
        out[r] = chosen >= 0 ? chosen : best.index;
    }
}
}  // namespace

// The number of slices a row is cut into, and the floats of scratch a call needs
// (rows * slices values, then rows * slices indices).
KIDI_API int kidi_argmax_slices(int vocab) { return vocab >= 65536 ? 32 : vocab >= 8192 ? 8 : 1; }

KIDI_API int kidi_argmax(const float* logits, int* out, int rows, int vocab, float* scratch, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (vocab <= 0 || rows > 65535) return KIDI_REFUSED_SIZE;
    const int slices = kidi_argmax_slices(vocab);
    if (slices == 1 || !scratch) return kidi_launch(argmax_kernel, rows, THREADS, 0, stream, logits, out, vocab);
    float* values = scratch;
    int* indices = reinterpret_cast<int*>(scratch + (long long)rows * slices);
    int status = kidi_launch(argmax_slices_kernel, dim3(slices, rows), THREADS, 0, stream, logits, values, indices,
                             vocab, slices);
    if (status) return status;
    return kidi_launch(argmax_merge_kernel, rows, 32, 0, stream, (const float*)values, (const int*)indices, out, slices);
}

// Greedy rows (temperature 0) are final after the argmax stages; the others are drawn.
KIDI_API int kidi_sample(const float* logits, int* out, int rows, int vocab, const float* temperature,
                         unsigned long long seed, const long long* keys, const int* steps, float* scratch,
                         cudaStream_t stream) {
    int status = kidi_argmax(logits, out, rows, vocab, scratch, stream);
    if (status || rows <= 0) return status;
    return kidi_launch(sample_kernel, rows, THREADS, 0, stream, logits, out, vocab, temperature, seed, keys, steps);
}
