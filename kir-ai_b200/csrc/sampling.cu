// Sampling over the full vocabulary, one block per row of logits [rows, vocab].
//
// Greedy: the greatest logit, the lowest index on ties
// (crates/llm-sampler/src/lib.rs:160-179 of the reference).
// Nucleus: p = softmax(logits / temperature) in 32-bit; order the entries by
// probability descending, ties to the lower index; the nucleus is the shortest
// prefix whose sum reaches top_p; threshold = draw * nucleus_total; the first
// entry whose running sum reaches the threshold is taken
// (crates/llm-sampler/src/lib.rs:39-108,110-158).  The reference sorts; here the
// two prefix searches are bisections over the probability value: for a value v,
// G(v) = sum of the probabilities greater than v is found by a block reduction,
// the boundary value is the smallest v with G(v) < target, and ties at that
// value are taken in index order.  Sums are formed in another order than a
// sequential walk, so a draw within rounding of a boundary may fall on the
// neighbouring entry.  The draw in [0, 1) is the caller's (one per row and token).
#include "common.cuh"

#define SAMPLE_THREADS 1024

__device__ __forceinline__ void argmax_combine(float& best, int& best_index, float other, int other_index) {
    if (other > best || (other == best && other_index < best_index)) {
        best = other;
        best_index = other_index;
    }
}

// Block-wide argmax with the lowest index on ties; every thread gets the result.  A row in which nothing is
// greater than -infinity (all NaN, all -inf) has no maximum: the result is then -1, for the caller to handle.
__device__ int block_argmax(const float* __restrict__ row, int vocab, float inv_temperature, float* out_max) {
    __shared__ float s_val[32];
    __shared__ int s_idx[32];
    float best = -INFINITY;
    int best_index = 0x7fffffff;
    // four loads in flight per thread; they are compared in ascending index order, so strict >
    // keeps the lowest index among equal values
    const int stride = blockDim.x;
    for (int i = threadIdx.x; i < vocab; i += 4 * stride) {
        float v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) v[u] = (i + u * stride < vocab) ? row[i + u * stride] * inv_temperature : -INFINITY;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            if (v[u] > best) {
                best = v[u];
                best_index = i + u * stride;
            }
        }
    }
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
        const float other = __shfl_xor_sync(0xffffffffu, best, offset);
        const int other_index = __shfl_xor_sync(0xffffffffu, best_index, offset);
        argmax_combine(best, best_index, other, other_index);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) {
        s_val[warp] = best;
        s_idx[warp] = best_index;
    }
    __syncthreads();
    const int warps = (blockDim.x + 31) >> 5;
    best = lane < warps ? s_val[lane] : -INFINITY;
    best_index = lane < warps ? s_idx[lane] : 0x7fffffff;
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
        const float other = __shfl_xor_sync(0xffffffffu, best, offset);
        const int other_index = __shfl_xor_sync(0xffffffffu, best_index, offset);
        argmax_combine(best, best_index, other, other_index);
    }
    if (out_max) *out_max = best;
    return best_index == 0x7fffffff ? -1 : best_index;
}

// A row without a maximum: token 0 is written (an index inside the vocabulary) and the device error word set.
__device__ __forceinline__ void no_maximum(int* __restrict__ out, int r, int* __restrict__ error_flag) {
    if (threadIdx.x == 0) {
        out[r] = 0;
        if (error_flag) atomicExch(error_flag, KIRAI_FLAG_NO_MAXIMUM);
    }
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
argmax_rows_kernel(const float* __restrict__ logits, int* __restrict__ out, int vocab, int* __restrict__ error_flag) {
    pdl_launch_dependents();
    pdl_wait();
    const float* row = logits + (size_t)blockIdx.x * vocab;
    const int best = block_argmax(row, vocab, 1.0f, nullptr);
    if (best < 0) return no_maximum(out, blockIdx.x, error_flag);
    if (threadIdx.x == 0) out[blockIdx.x] = best;
}

KIRAI_EXPORT int kirai_argmax_rows(const float* logits, int* out, int rows, int vocab, int* error_flag, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (vocab <= 0) return KIRAI_ERR_BAD_SIZE;
    const int pdl_status = launch_pdl(argmax_rows_kernel, dim3(rows), dim3(SAMPLE_THREADS), 0, stream, 1u, logits, out, vocab, error_flag);
    return pdl_status;
}

// Sum of the probabilities greater than `value` (and how many equal it).
__device__ float sum_greater(const float* __restrict__ probs, int vocab, float value, float* scratch) {
    float acc = 0.0f;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float p = probs[i];
        if (p > value) acc += p;
    }
    return block_sum(acc, scratch);
}

// Smallest probability value v (as a bit pattern in [0, hi_bits]) with sum_greater(v) < target.
// Positive floats order like their bit patterns.  Requires sum_greater(hi) < target.
__device__ float boundary_value(const float* __restrict__ probs, int vocab, float target, unsigned hi_bits,
                                float* scratch) {
    unsigned lo = 0u, hi = hi_bits;  // invariant: G(hi) < target
    while (lo < hi) {
        const unsigned mid = lo + ((hi - lo) >> 1);
        const float g = sum_greater(probs, vocab, __uint_as_float(mid), scratch);
        if (g < target) hi = mid;
        else lo = mid + 1;
    }
    return __uint_as_float(hi);
}

// Index of the n-th (1-based) entry equal to `value`, in index order; -1 if fewer exist.
__device__ int nth_equal(const float* __restrict__ probs, int vocab, float value, int n, int* s_counts) {
    const int chunk = (vocab + blockDim.x - 1) / blockDim.x;
    const int begin = threadIdx.x * chunk;
    const int end = min(vocab, begin + chunk);
    int count = 0;
    for (int i = begin; i < end; ++i) count += (probs[i] == value);
    __syncthreads();
    s_counts[threadIdx.x] = count;
    __syncthreads();
    __shared__ int s_found;
    if (threadIdx.x == 0) {
        s_found = -1;
        int before = 0;
        for (int t = 0; t < (int)blockDim.x; ++t) {
            if (before + s_counts[t] >= n) {
                s_found = t;
                s_counts[0] = before;  // matches before that thread's chunk
                break;
            }
            before += s_counts[t];
        }
    }
    __syncthreads();
    const int owner = s_found;
    const int before = s_counts[0];
    __shared__ int s_result;
    if (threadIdx.x == 0) s_result = -1;
    __syncthreads();
    if (owner >= 0 && (int)threadIdx.x == owner) {
        int seen = before;
        for (int i = begin; i < end; ++i) {
            if (probs[i] == value && ++seen == n) {
                s_result = i;
                break;
            }
        }
    }
    __syncthreads();
    return s_result;
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_rows_kernel(const float* __restrict__ logits, float* __restrict__ probs_scratch,
                   const float* __restrict__ temperature, const float* __restrict__ top_p,
                   const float* __restrict__ draw, int* __restrict__ out, int vocab, int* __restrict__ error_flag) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scratch[32];
    __shared__ int s_counts[SAMPLE_THREADS];
    const int r = blockIdx.x;
    const float* row = logits + (size_t)r * vocab;
    const float temp = temperature[r];
    const int best = block_argmax(row, vocab, 1.0f, nullptr);
    if (best < 0) return no_maximum(out, r, error_flag);  // before anything is read at that index
    if (!(temp > 0.0f)) {  // greedy
        if (threadIdx.x == 0) out[r] = best;
        return;
    }
    float* probs = probs_scratch + (size_t)r * vocab;
    float max_scaled;
    max_scaled = row[best] / temp;
    float acc = 0.0f;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float e = expf(row[i] / temp - max_scaled);
        probs[i] = e;
        acc += e;
    }
    const float total = block_sum(acc, scratch);
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) probs[i] = probs[i] / total;
    __syncthreads();
    const float p_max = probs[best];
    const unsigned hi_bits = __float_as_uint(p_max);  // nothing is greater than the maximum: G = 0

    // nucleus: boundary value, how many ties at it belong, and the nucleus total
    const float want = top_p[r];
    float nucleus_total;
    float nucleus_value = 0.0f;  // smallest probability inside the nucleus
    int nucleus_ties = 0x7fffffff;
    const float all = sum_greater(probs, vocab, -1.0f, scratch);
    if (want >= 1.0f || all < want) {
        nucleus_total = all;  // the whole vocabulary is the nucleus
    } else {
        nucleus_value = boundary_value(probs, vocab, want, hi_bits, scratch);
        const float above = sum_greater(probs, vocab, nucleus_value, scratch);
        float running = above;
        int n = 0;
        do {  // ties enter one by one, as a sequential walk would add them
            running += nucleus_value;
            ++n;
        } while (running < want && n < vocab);
        nucleus_ties = n;
        nucleus_total = running;
    }

    const float threshold = draw[r] * nucleus_total;
    int chosen;
    if (!(threshold > 0.0f)) {
        chosen = best;  // the first entry of the order already reaches a zero threshold
    } else {
        float value = boundary_value(probs, vocab, threshold, hi_bits, scratch);
        int n;
        if (value < nucleus_value) {  // rounding pushed the threshold past the nucleus: its last entry
            value = nucleus_value;
            n = nucleus_ties;
        } else {
            const float above = sum_greater(probs, vocab, value, scratch);
            float running = above;
            n = 0;
            do {
                running += value;
                ++n;
            } while (running < threshold && n < vocab);
            if (value == nucleus_value && n > nucleus_ties) n = nucleus_ties;
        }
        chosen = nth_equal(probs, vocab, value, n, s_counts);
        if (chosen < 0) {  // fewer ties than counted (rounding): the last of them
            int have = 0;
            for (int i = threadIdx.x; i < vocab; i += blockDim.x) have += (probs[i] == value);
            __syncthreads();
            s_counts[threadIdx.x] = have;
            __syncthreads();
            if (threadIdx.x == 0) {
                int sum = 0;
                for (int t = 0; t < (int)blockDim.x; ++t) sum += s_counts[t];
                s_counts[0] = sum;
            }
            __syncthreads();
            const int total_ties = s_counts[0];
            __syncthreads();
            chosen = total_ties > 0 ? nth_equal(probs, vocab, value, total_ties, s_counts) : best;
        }
    }
    if (threadIdx.x == 0) out[r] = chosen;
}

// probs_scratch: [rows, vocab] floats, overwritten.  temperature <= 0 means greedy for that row.
KIRAI_EXPORT int kirai_sample_rows(const float* logits, float* probs_scratch, const float* temperature,
                                   const float* top_p, const float* draw, int* out, int rows, int vocab,
                                   int* error_flag, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (vocab <= 0) return KIRAI_ERR_BAD_SIZE;
    const int pdl_status = launch_pdl(sample_rows_kernel, dim3(rows), dim3(SAMPLE_THREADS), 0, stream, 1u, logits, probs_scratch, temperature, top_p, draw, out, vocab, error_flag);
    return pdl_status;
}
