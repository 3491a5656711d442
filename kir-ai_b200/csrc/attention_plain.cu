// Plain causal grouped-query attention over the paged cache: one block per
// (token, query head), keys walked in position order, scores, softmax and the
// weighted sum in 32-bit.  It serves the true 32-bit path and is the reference
// beside the tensor-core attention kernels.
//
// Token t of request r at absolute position pos reads the keys at positions
// [lo, pos] of r, lo = max(0, pos - window + 1) with a window, else 0
// (crates/llm-backend/src/core/native_attention.rs:731-764 scores and weighted sum,
// :827-841 the d^-1/2 scale; crates/llm-kv-cache/src/layer.rs:765-805 the window as a
// ring of the last W rows).  The keys of the step's own tokens are already in the
// cache when this runs; later positions of the same portion are masked by j <= pos.
// Query head h reads kv head h / (q_heads / kv_heads).  Any head_dim <= 512.
#include "common.cuh"

#define ATT_WARPS 4
#define ATT_MAX_PER_LANE 16

template <typename T>
__global__ void __launch_bounds__(ATT_WARPS * 32)
paged_attention_plain_kernel(const T* __restrict__ q, const T* __restrict__ cache, T* __restrict__ out,
                             const int* __restrict__ block_table, const int* __restrict__ request_of_token,
                             const int* __restrict__ positions, int q_heads, int kv_heads, int head_dim,
                             long q_row_stride, int page_size, int table_width, int num_pages, int window, float scale,
                             int* __restrict__ error_flag) {
    extern __shared__ float smem[];
    float* q_s = smem;                       // [head_dim]
    float* o_s = smem + head_dim;            // [ATT_WARPS][head_dim]
    float* m_s = o_s + ATT_WARPS * head_dim; // [ATT_WARPS]
    float* l_s = m_s + ATT_WARPS;            // [ATT_WARPS]

    const int token = blockIdx.x, head = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int kv_head = head / (q_heads / kv_heads);
    const int pos = positions[token];
    const int* table = block_table + (long)request_of_token[token] * table_width;
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;

    const T* q_row = q + (size_t)token * q_row_stride + (size_t)head * head_dim;
    for (int i = threadIdx.x; i < head_dim; i += blockDim.x) q_s[i] = to_f32<T>(q_row[i]);
    __syncthreads();

    float m = -INFINITY, l = 0.0f;
    float o[ATT_MAX_PER_LANE];
#pragma unroll
    for (int n = 0; n < ATT_MAX_PER_LANE; ++n) o[n] = 0.0f;

    for (int j = lo + warp; j <= pos; j += ATT_WARPS) {
        const int logical = j / page_size;
        const int page = logical < table_width ? table[logical] : -1;
        if (page < 0 || page >= num_pages) {
            if (lane == 0) atomicExch(error_flag, 3);
            continue;
        }
        const long base = ((((long)page * 2) * kv_heads + kv_head) * page_size + (j % page_size)) * (long)head_dim;
        const T* k_row = cache + base;
        const T* v_row = cache + base + (long)kv_heads * page_size * head_dim;
        float dot = 0.0f;
        for (int i = lane; i < head_dim; i += 32) dot = fmaf(q_s[i], to_f32<T>(k_row[i]), dot);
        dot = warp_sum(dot) * scale;
        const float m_new = fmaxf(m, dot);
        const float corr = expf(m - m_new);  // 0 on the first key (m = -inf)
        const float p = expf(dot - m_new);
        l = l * corr + p;
#pragma unroll
        for (int n = 0; n < ATT_MAX_PER_LANE; ++n) {
            const int i = lane + 32 * n;
            if (i < head_dim) o[n] = o[n] * corr + p * to_f32<T>(v_row[i]);
        }
        m = m_new;
    }
#pragma unroll
    for (int n = 0; n < ATT_MAX_PER_LANE; ++n) {
        const int i = lane + 32 * n;
        if (i < head_dim) o_s[warp * head_dim + i] = o[n];
    }
    if (lane == 0) {
        m_s[warp] = m;
        l_s[warp] = l;
    }
    __syncthreads();
    float m_all = -INFINITY;
#pragma unroll
    for (int w = 0; w < ATT_WARPS; ++w) m_all = fmaxf(m_all, m_s[w]);
    float l_all = 0.0f;
    float weight[ATT_WARPS];
#pragma unroll
    for (int w = 0; w < ATT_WARPS; ++w) {
        weight[w] = (m_s[w] == -INFINITY) ? 0.0f : expf(m_s[w] - m_all);
        l_all += l_s[w] * weight[w];
    }
    T* out_row = out + ((size_t)token * q_heads + head) * head_dim;
    for (int i = threadIdx.x; i < head_dim; i += blockDim.x) {
        float acc = 0.0f;
#pragma unroll
        for (int w = 0; w < ATT_WARPS; ++w) acc += o_s[w * head_dim + i] * weight[w];
        out_row[i] = from_f32<T>(l_all > 0.0f ? acc / l_all : 0.0f);
    }
}

template <typename T>
static int paged_attention_plain_launch(const void* q, const void* cache, void* out, const int* block_table,
                                        const int* request_of_token, const int* positions, int tokens, int q_heads,
                                        int kv_heads, int head_dim, long q_row_stride, int page_size, int table_width,
                                        int num_pages, int window, float scale, int* error_flag, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (head_dim > 32 * ATT_MAX_PER_LANE || head_dim <= 0) return KIRAI_ERR_BAD_SIZE;
    if (kv_heads <= 0 || q_heads % kv_heads != 0) return KIRAI_ERR_BAD_SIZE;
    if (q_heads > 65535) return KIRAI_ERR_BAD_SIZE;
    const size_t smem = (size_t)(head_dim * (1 + ATT_WARPS) + 2 * ATT_WARPS) * sizeof(float);
    dim3 grid(tokens, q_heads);
    paged_attention_plain_kernel<T><<<grid, ATT_WARPS * 32, smem, stream>>>(
        (const T*)q, (const T*)cache, (T*)out, block_table, request_of_token, positions, q_heads, kv_heads, head_dim,
        q_row_stride, page_size, table_width, num_pages, window, scale, error_flag);
    return launch_status();
}

KIRAI_EXPORT int kirai_paged_attention_plain_f32(const void* q, const void* cache, void* out, const int* block_table,
                                                 const int* request_of_token, const int* positions, int tokens,
                                                 int q_heads, int kv_heads, int head_dim, long q_row_stride,
                                                 int page_size, int table_width, int num_pages, int window,
                                                 float scale, int* error_flag, cudaStream_t stream) {
    return paged_attention_plain_launch<float>(q, cache, out, block_table, request_of_token, positions, tokens, q_heads,
                                               kv_heads, head_dim, q_row_stride, page_size, table_width, num_pages,
                                               window, scale, error_flag, stream);
}
KIRAI_EXPORT int kirai_paged_attention_plain_bf16(const void* q, const void* cache, void* out, const int* block_table,
                                                  const int* request_of_token, const int* positions, int tokens,
                                                  int q_heads, int kv_heads, int head_dim, long q_row_stride,
                                                  int page_size, int table_width, int num_pages, int window,
                                                  float scale, int* error_flag, cudaStream_t stream) {
    return paged_attention_plain_launch<bf16>(q, cache, out, block_table, request_of_token, positions, tokens, q_heads,
                                              kv_heads, head_dim, q_row_stride, page_size, table_width, num_pages,
                                              window, scale, error_flag, stream);
}
