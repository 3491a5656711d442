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

// ------------------------------------------------------------------ one row over a cluster of eight CTAs
// The same arithmetic with a row's vocabulary cut into eight contiguous slices, one per CTA of a thread-block
// cluster.  A CTA keeps its slice of the probabilities in shared memory, so the passes of the two searches read no
// global memory (one block per row read its 600 KB row from L2 in every one of up to 62 passes: 0.9 to 1.6 ms a step
// for rows with a temperature), and the CTAs exchange their partial results through distributed shared memory: each
// leaves its numbers in a slot of its own, the cluster synchronises, and every CTA adds the eight slots in rank order,
// so all of them hold the same bits and take the same branches.  Each search step tries seven values at once.
#define SC_CTAS 8
#define SC_THREADS 1024

#define SC_TRIES 7  // values that a search step tries at once: the candidates shrink to an eighth a step

struct SampleExchange {
    float f[2][8];  // this CTA's contribution to the reduction in flight; two in turn, so that one cluster barrier a
    int i[2][2];    // reduction is enough (a slot is written again only after the barrier that follows its reading)
};

__device__ __forceinline__ uint32_t sc_rank() {
    uint32_t rank;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    return rank;
}
__device__ __forceinline__ void sc_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t sc_remote(const void* local, uint32_t rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"((uint32_t)__cvta_generic_to_shared(local)), "r"(rank));
    return remote;
}
__device__ __forceinline__ float sc_load_f32(const float* local, uint32_t rank) {
    float value;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(value) : "r"(sc_remote(local, rank)) : "memory");
    return value;
}
__device__ __forceinline__ int sc_load_s32(const int* local, uint32_t rank) {
    int value;
    asm volatile("ld.shared::cluster.s32 %0, [%1];" : "=r"(value) : "r"(sc_remote(local, rank)) : "memory");
    return value;
}

// Block-wide sums of COUNT numbers at once (two block barriers for all of them); every thread gets the results, and
// the order of the additions depends only on the block size.  scratch: 32 * COUNT floats of shared memory.
template <int COUNT>
__device__ __forceinline__ void sc_block_sums(float (&values)[COUNT], float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int j = 0; j < COUNT; ++j) values[j] = warp_sum(values[j]);
    __syncthreads();
    if (lane == 0) {
#pragma unroll
        for (int j = 0; j < COUNT; ++j) scratch[warp * COUNT + j] = values[j];
    }
    __syncthreads();
    const int warps = (blockDim.x + 31) >> 5;
#pragma unroll
    for (int j = 0; j < COUNT; ++j) values[j] = warp_sum(lane < warps ? scratch[lane * COUNT + j] : 0.0f);
}

// Sums over the cluster of numbers that every thread of this CTA holds (its CTA's partial results), in rank order.
// One thread per number reads the eight slots (every thread doing so was 57,000 remote loads a CTA and step) and
// hands the totals on through `totals` (8 floats of shared memory).
template <int COUNT>
__device__ __forceinline__ void sc_cluster_sum(float (&values)[COUNT], SampleExchange* ex, int& turn, float* totals) {
    if (threadIdx.x == 0) {
#pragma unroll
        for (int j = 0; j < COUNT; ++j) ex->f[turn][j] = values[j];
    }
    sc_sync();
    if (threadIdx.x < COUNT) {
        float total = 0.0f;
        for (uint32_t q = 0; q < SC_CTAS; ++q) total += sc_load_f32(&ex->f[turn][threadIdx.x], q);
        totals[threadIdx.x] = total;
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < COUNT; ++j) values[j] = totals[j];
    turn ^= 1;  // (totals is written again only behind the next cluster barrier, which every thread reaches after this)
}

// G(v) = sum of the row's probabilities greater than v, for COUNT values at once.
template <int COUNT>
__device__ __forceinline__ void sc_sums_greater(const float* probs_s, int count, const float (&v)[COUNT], float (&g)[COUNT],
                                                float* scratch, SampleExchange* ex, int& turn) {
#pragma unroll
    for (int j = 0; j < COUNT; ++j) g[j] = 0.0f;
    for (int i = threadIdx.x; i < count; i += blockDim.x) {
        const float p = probs_s[i];
#pragma unroll
        for (int j = 0; j < COUNT; ++j)
            if (p > v[j]) g[j] += p;
    }
    sc_block_sums<COUNT>(g, scratch);
    sc_cluster_sum<COUNT>(g, ex, turn, scratch + 32 * COUNT);
}
__device__ __forceinline__ float sc_sum_greater(const float* probs_s, int count, float value, float* scratch,
                                                SampleExchange* ex, int& turn) {
    const float v[1] = {value};
    float g[1];
    sc_sums_greater<1>(probs_s, count, v, g, scratch, ex, turn);
    return g[0];
}

// Smallest probability value v (a bit pattern in [0, hi_bits]) with G(v) < target; requires G(hi_bits) < target.
// G does not grow with v, so SC_TRIES values cut the candidates [lo, hi] into SC_TRIES + 1 parts a step: everything
// up to the last value that fails is out, the first value that passes is the new upper end.
__device__ float sc_boundary_value(const float* probs_s, int count, float target, unsigned hi_bits, float* scratch,
                                   SampleExchange* ex, int& turn) {
    unsigned lo = 0u, hi = hi_bits;
    while (lo < hi) {
        unsigned m[SC_TRIES];
        float v[SC_TRIES], g[SC_TRIES];
#pragma unroll
        for (int j = 0; j < SC_TRIES; ++j) {
            m[j] = lo + (unsigned)(((unsigned long long)(hi - lo) * (unsigned)(j + 1)) / (SC_TRIES + 1));
            v[j] = __uint_as_float(m[j]);
        }
        sc_sums_greater<SC_TRIES>(probs_s, count, v, g, scratch, ex, turn);
        unsigned new_lo = lo, new_hi = hi;
        bool passed = false;
#pragma unroll
        for (int j = 0; j < SC_TRIES; ++j) {
            if (!passed) {
                if (g[j] < target) new_hi = m[j], passed = true;
                else new_lo = m[j] + 1u;
            }
        }
        lo = new_lo, hi = new_hi;
    }
    return __uint_as_float(hi);
}

// Index (in the row) of the n-th entry equal to `value` in index order, -1 if there are fewer; the slices lie in
// rank order, so the CTA that holds the n-th entry is found from the CTAs' counts.  Every CTA returns the same.
__device__ int sc_nth_equal(const float* probs_s, int count, int first, float value, int n, int* s_counts,
                            float* scratch, SampleExchange* ex, int& turn) {
    int mine = 0;
    for (int i = threadIdx.x; i < count; i += blockDim.x) mine += (probs_s[i] == value);
    const int in_slice = (int)(block_sum((float)mine, scratch) + 0.5f);  // a slice has fewer than 2^24 entries
    if (threadIdx.x == 0) ex->i[turn][0] = in_slice;
    sc_sync();
    int before = 0, owner = -1;
    for (uint32_t q = 0; q < SC_CTAS; ++q) {
        const int have = sc_load_s32(&ex->i[turn][0], q);
        if (owner < 0 && before + have >= n) owner = (int)q;
        if (owner < 0) before += have;
    }
    turn ^= 1;
    int found = -1;
    if (owner == (int)sc_rank()) found = nth_equal(probs_s, count, value, n - before, s_counts);  // the block's own search
    if (threadIdx.x == 0) ex->i[turn][0] = found < 0 ? -1 : first + found;
    sc_sync();
    const int result = owner < 0 ? -1 : sc_load_s32(&ex->i[turn][0], (uint32_t)owner);
    turn ^= 1;
    return result;
}

__global__ void __launch_bounds__(SC_THREADS)
sample_rows_cluster_kernel(const float* __restrict__ logits, const float* __restrict__ temperature,
                           const float* __restrict__ top_p, const float* __restrict__ draw, int* __restrict__ out,
                           int vocab, int per, int* __restrict__ error_flag) {
    pdl_launch_dependents();
    extern __shared__ float probs_s[];  // [per] this CTA's slice: logits first, then probabilities
    __shared__ float scratch[32 * 8 + 8];  // block sums of up to 8 numbers, then the cluster's totals
    __shared__ int s_counts[SC_THREADS];
    __shared__ SampleExchange ex;
    const int r = blockIdx.y;
    const uint32_t rank = sc_rank();
    const int first = (int)rank * per;
    const int count = max(0, min(per, vocab - first));
    const float* row = logits + (size_t)r * vocab + first;
    int turn = 0;
    pdl_wait();
    const float temp = temperature[r];
    // the slice into shared memory, and its greatest logit (lowest index on ties)
    float best = -INFINITY;
    int best_index = 0x7fffffff;
    for (int i = threadIdx.x; i < count; i += blockDim.x) {
        const float v = row[i];
        probs_s[i] = v;
        if (v > best) best = v, best_index = first + i;
    }
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
        const float other = __shfl_xor_sync(0xffffffffu, best, offset);
        const int other_index = __shfl_xor_sync(0xffffffffu, best_index, offset);
        argmax_combine(best, best_index, other, other_index);
    }
    {
        __shared__ float s_val[32];
        __shared__ int s_idx[32];
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
        if (lane == 0) s_val[warp] = best, s_idx[warp] = best_index;
        __syncthreads();
        if (threadIdx.x == 0) {
            for (int w = 1; w < SC_THREADS / 32; ++w) argmax_combine(best, best_index, s_val[w], s_idx[w]);
            ex.f[turn][0] = best, ex.i[turn][0] = best_index;
        }
    }
    sc_sync();
    best = -INFINITY, best_index = 0x7fffffff;
    for (uint32_t q = 0; q < SC_CTAS; ++q)
        argmax_combine(best, best_index, sc_load_f32(&ex.f[turn][0], q), sc_load_s32(&ex.i[turn][0], q));
    turn ^= 1;
    const bool greedy = !(temp > 0.0f);
    if (best_index == 0x7fffffff || greedy) {
        if (rank == 0) {
            if (best_index == 0x7fffffff) no_maximum(out, r, error_flag);
            else if (threadIdx.x == 0) out[r] = best_index;
        }
        sc_sync();  // nobody leaves while its slot may still be read
        return;
    }
    const float max_scaled = best / temp;
    float acc = 0.0f;
    for (int i = threadIdx.x; i < count; i += blockDim.x) {
        const float e = expf(probs_s[i] / temp - max_scaled);
        probs_s[i] = e;
        acc += e;
    }
    float sums[1] = {block_sum(acc, scratch)};
    sc_cluster_sum<1>(sums, &ex, turn, scratch + 32 * 8);
    const float total = sums[0];
    for (int i = threadIdx.x; i < count; i += blockDim.x) probs_s[i] = probs_s[i] / total;
    __syncthreads();
    const float p_max = 1.0f / total;  // exp(0) / total: the probability of the greatest logit, nothing is greater
    const unsigned hi_bits = __float_as_uint(p_max);

    const float want = top_p[r];
    float nucleus_total;
    float nucleus_value = 0.0f;
    int nucleus_ties = 0x7fffffff;
    const float all = sc_sum_greater(probs_s, count, -1.0f, scratch, &ex, turn);
    if (want >= 1.0f || all < want) {
        nucleus_total = all;
    } else {
        nucleus_value = sc_boundary_value(probs_s, count, want, hi_bits, scratch, &ex, turn);
        const float above = sc_sum_greater(probs_s, count, nucleus_value, scratch, &ex, turn);
        float running = above;
        int n = 0;
        do {
            running += nucleus_value;
            ++n;
        } while (running < want && n < vocab);
        nucleus_ties = n;
        nucleus_total = running;
    }
    const float threshold = draw[r] * nucleus_total;
    int chosen;
    if (!(threshold > 0.0f)) {
        chosen = best_index;
    } else {
        float value = sc_boundary_value(probs_s, count, threshold, hi_bits, scratch, &ex, turn);
        int n;
        if (value < nucleus_value) {
            value = nucleus_value;
            n = nucleus_ties;
        } else {
            const float above = sc_sum_greater(probs_s, count, value, scratch, &ex, turn);
            float running = above;
            n = 0;
            do {
                running += value;
                ++n;
            } while (running < threshold && n < vocab);
            if (value == nucleus_value && n > nucleus_ties) n = nucleus_ties;
        }
        chosen = sc_nth_equal(probs_s, count, first, value, n, s_counts, scratch, &ex, turn);
        if (chosen < 0) {  // fewer ties than counted (rounding): the last of them
            int mine = 0;
            for (int i = threadIdx.x; i < count; i += blockDim.x) mine += (probs_s[i] == value);
            float ties[1] = {block_sum((float)mine, scratch)};
            sc_cluster_sum<1>(ties, &ex, turn, scratch + 32 * 8);
            const int total_ties = (int)(ties[0] + 0.5f);
            chosen = total_ties > 0 ? sc_nth_equal(probs_s, count, first, value, total_ties, s_counts, scratch, &ex, turn) : best_index;
        }
    }
    if (rank == 0 && threadIdx.x == 0) out[r] = chosen;
    sc_sync();  // nobody leaves while its slots may still be read
}

// Whether a row of `vocab` logits goes over a cluster of eight CTAs: an eighth of it fits a CTA's shared memory beside
// a second CTA's, and every CTA has something to do.  Otherwise one block takes the row and reads it from global
// memory in every pass, which needs the scratch rows.
static bool sample_rows_over_a_cluster(int rows, int vocab, int* per_out) {
    const int per = (((vocab + SC_CTAS - 1) / SC_CTAS) + 3) & ~3;
    if (per_out) *per_out = per;
    return (size_t)per * sizeof(float) <= 100 * 1024 && rows <= 65535 && vocab >= SC_CTAS * 32;
}
KIRAI_EXPORT int kirai_sample_rows_needs_scratch(int rows, int vocab) { return sample_rows_over_a_cluster(rows, vocab, nullptr) ? 0 : 1; }

// probs_scratch: [rows, vocab] floats, overwritten (may be null where kirai_sample_rows_needs_scratch says 0).
// temperature <= 0 means greedy for that row.
KIRAI_EXPORT int kirai_sample_rows(const float* logits, float* probs_scratch, const float* temperature,
                                   const float* top_p, const float* draw, int* out, int rows, int vocab,
                                   int* error_flag, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (vocab <= 0) return KIRAI_ERR_BAD_SIZE;
    int per = 0;
    if (sample_rows_over_a_cluster(rows, vocab, &per)) {
        const size_t slice_bytes = (size_t)per * sizeof(float);
        cudaError_t err = cudaFuncSetAttribute(sample_rows_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)slice_bytes);
        if (err != cudaSuccess) return (int)err;
        return launch_pdl_clusters(sample_rows_cluster_kernel, dim3(SC_CTAS, rows), dim3(SC_THREADS), slice_bytes, stream,
                                   dim3(SC_CTAS, 1, 1), logits, temperature, top_p, draw, out, vocab, per, error_flag);
    }
    if (!probs_scratch) return KIRAI_ERR_BAD_SIZE;
    const int pdl_status = launch_pdl(sample_rows_kernel, dim3(rows), dim3(SAMPLE_THREADS), 0, stream, 1u, logits, probs_scratch, temperature, top_p, draw, out, vocab, error_flag);
    return pdl_status;
}
