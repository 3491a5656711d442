// Row-wise kernels of the forward pass: embedding gather, RMSNorm with the
// residual add fused in, per-head RMSNorm, rotary embedding, SwiGLU, the paged
// key/value write, and the fusion of per-head norm + rotation + cache write.
// Each is a template over the activation type (float for the true 32-bit path,
// bf16 for serving); statistics, angles and the residual stream are 32-bit in
// both.  Formulas: crates/llm-backend/src/core/math.rs:73-113 (RMSNorm),
// :223-225 (SiLU), :515-529 (rotary, half-split pairs) of the reference.
#include "common.cuh"

// ----------------------------------------------------------------- embedding
template <typename T>
__global__ void embedding_kernel(const T* __restrict__ table, const int* __restrict__ ids, float* __restrict__ out,
                                 int hidden, int vocab, int* __restrict__ error_flag) {
    pdl_launch_dependents();
    pdl_wait();
    const int token = blockIdx.x;
    const int id = ids[token];
    if (id < 0 || id >= vocab) {
        if (threadIdx.x == 0) atomicExch(error_flag, 1);
        return;
    }
    const T* row = table + (size_t)id * hidden;
    float* dst = out + (size_t)token * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = to_f32<T>(row[i]);
}

template <typename T>
static int embedding_launch(const void* table, const int* ids, float* out, int tokens, int hidden, int vocab,
                            int* error_flag, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    const int pdl_status = launch_pdl(embedding_kernel<T>, dim3(tokens), dim3(256), 0, stream, 1u, (const T*)table, ids, out, hidden, vocab, error_flag);
    return pdl_status;
}

KIRAI_EXPORT int kirai_embedding_f32(const void* table, const int* ids, float* out, int tokens, int hidden, int vocab,
                                     int* error_flag, cudaStream_t stream) {
    return embedding_launch<float>(table, ids, out, tokens, hidden, vocab, error_flag, stream);
}
KIRAI_EXPORT int kirai_embedding_bf16(const void* table, const int* ids, float* out, int tokens, int hidden, int vocab,
                                      int* error_flag, cudaStream_t stream) {
    return embedding_launch<bf16>(table, ids, out, tokens, hidden, vocab, error_flag, stream);
}

// The same gather from a bf16 table kept in the tensor-core product's box layout (boxes of 128 rows x 64
// columns under the 128-byte swizzle, box (row tile, k block) at row_tile * k_blocks + k_block): the 16-byte
// chunk c of row r of a box lies at byte r * 128 + (c ^ (r % 8)) * 16.
__global__ void embedding_tiled_kernel(const uint4* __restrict__ boxes, const int* __restrict__ ids, float* __restrict__ out,
                                       int hidden, int vocab, int* __restrict__ error_flag) {
    pdl_launch_dependents();
    pdl_wait();
    const int token = blockIdx.x;
    const int id = ids[token];
    if (id < 0 || id >= vocab) {
        if (threadIdx.x == 0) atomicExch(error_flag, 1);
        return;
    }
    const int k_blocks = (hidden + 63) / 64, r = id % 128;
    const uint4* tile = boxes + (size_t)(id / 128) * k_blocks * 1024;  // 1,024 chunks of 16 bytes per box
    float* dst = out + (size_t)token * hidden;
    for (int chunk = threadIdx.x; chunk * 8 < hidden; chunk += blockDim.x) {
        const uint4 raw = tile[(size_t)(chunk / 8) * 1024 + r * 8 + ((chunk % 8) ^ (r % 8))];
        const bf16* values = reinterpret_cast<const bf16*>(&raw);
        if (chunk * 8 + 8 <= hidden && (((uintptr_t)(dst + chunk * 8)) & 15) == 0) {
            float4* wide = reinterpret_cast<float4*>(dst + chunk * 8);
            wide[0] = make_float4(to_f32<bf16>(values[0]), to_f32<bf16>(values[1]), to_f32<bf16>(values[2]), to_f32<bf16>(values[3]));
            wide[1] = make_float4(to_f32<bf16>(values[4]), to_f32<bf16>(values[5]), to_f32<bf16>(values[6]), to_f32<bf16>(values[7]));
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j)
                if (chunk * 8 + j < hidden) dst[chunk * 8 + j] = to_f32<bf16>(values[j]);
        }
    }
}

KIRAI_EXPORT int kirai_embedding_tiled_bf16(const void* boxes, const int* ids, float* out, int tokens, int hidden, int vocab,
                                            int* error_flag, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    return launch_pdl(embedding_tiled_kernel, dim3(tokens), dim3(256), 0, stream, 1u, (const uint4*)boxes, ids, out, hidden,
                      vocab, error_flag);
}

// ------------------------------------------------------- residual add + RMSNorm
// resid (32-bit, in place) += delta; out = resid * 1/sqrt(mean(resid^2) + eps) * weight.
// With row_index != nullptr, output row r reads residual row row_index[r] and
// leaves the residual stream untouched (the sum goes to resid_out instead).
template <typename T>
__global__ void add_rmsnorm_kernel(float* __restrict__ resid, const T* __restrict__ delta,
                                   const float* __restrict__ weight, T* __restrict__ out,
                                   const int* __restrict__ row_index, float* __restrict__ resid_out, int hidden,
                                   float eps) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scratch[32];
    const int row = blockIdx.x;
    const int src = row_index ? row_index[row] : row;
    const float* x = resid + (size_t)src * hidden;
    const T* d = delta ? delta + (size_t)src * hidden : nullptr;
    float* sum_dst = row_index ? resid_out + (size_t)row * hidden : resid + (size_t)src * hidden;
    float acc = 0.0f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        float v = x[i];
        if (d) {
            v += to_f32<T>(d[i]);
            sum_dst[i] = v;
        } else if (row_index) {
            sum_dst[i] = v;
        }
        acc = fmaf(v, v, acc);
    }
    const float total = block_sum(acc, scratch);
    const float variance = total / (float)hidden + eps;
    const float scale = variance == 0.0f ? 0.0f : 1.0f / sqrtf(variance);
    T* y = out + (size_t)row * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        // each thread re-reads what it wrote itself above
        y[i] = from_f32<T>(sum_dst[i] * scale * weight[i]);
    }
}

// The same, for rows whose width is a multiple of 4 and fits 4 * VEC * blockDim values: 16-byte
// loads, and the summed row stays in registers between the statistics and the scaling.
template <typename T>
struct Vec4 {};
template <>
struct Vec4<float> {
    typedef float4 type;
    static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
    static __device__ __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <>
struct Vec4<bf16> {
    typedef uint2 type;
    static __device__ __forceinline__ float4 load(const bf16* p) {
        const uint2 raw = *reinterpret_cast<const uint2*>(p);
        const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
        const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
        return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
    }
    static __device__ __forceinline__ void store(bf16* p, float4 v) {
        __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
        uint2 raw;
        raw.x = *reinterpret_cast<uint32_t*>(&a);
        raw.y = *reinterpret_cast<uint32_t*>(&b);
        *reinterpret_cast<uint2*>(p) = raw;
    }
};

template <typename T, int VEC>
__global__ void add_rmsnorm_vec_kernel(float* __restrict__ resid, const T* __restrict__ delta,
                                       const float* __restrict__ weight, T* __restrict__ out,
                                       const int* __restrict__ row_index, float* __restrict__ resid_out, int hidden,
                                       float eps) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scratch[32];
    const int row = blockIdx.x;
    const int src = row_index ? row_index[row] : row;
    const float* x = resid + (size_t)src * hidden;
    const T* d = delta ? delta + (size_t)src * hidden : nullptr;
    float* sum_dst = row_index ? resid_out + (size_t)row * hidden : resid + (size_t)src * hidden;
    float4 v[VEC];
    float acc = 0.0f;
#pragma unroll
    for (int n = 0; n < VEC; ++n) {
        const int i = (n * blockDim.x + threadIdx.x) * 4;
        v[n] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (i < hidden) {
            v[n] = Vec4<float>::load(x + i);
            if (d) {
                const float4 dv = Vec4<T>::load(d + i);
                v[n].x += dv.x; v[n].y += dv.y; v[n].z += dv.z; v[n].w += dv.w;
            }
            if (d || row_index) Vec4<float>::store(sum_dst + i, v[n]);
            acc = fmaf(v[n].x, v[n].x, acc);
            acc = fmaf(v[n].y, v[n].y, acc);
            acc = fmaf(v[n].z, v[n].z, acc);
            acc = fmaf(v[n].w, v[n].w, acc);
        }
    }
    const float total = block_sum(acc, scratch);
    const float variance = total / (float)hidden + eps;
    const float scale = variance == 0.0f ? 0.0f : 1.0f / sqrtf(variance);
    T* y = out + (size_t)row * hidden;
#pragma unroll
    for (int n = 0; n < VEC; ++n) {
        const int i = (n * blockDim.x + threadIdx.x) * 4;
        if (i < hidden) {
            const float4 w = Vec4<float>::load(weight + i);
            Vec4<T>::store(y + i, make_float4(v[n].x * scale * w.x, v[n].y * scale * w.y, v[n].z * scale * w.z, v[n].w * scale * w.w));
        }
    }
}

template <typename T>
static int add_rmsnorm_launch(float* resid, const void* delta, const float* weight, void* out, const int* row_index,
                              float* resid_out, int rows, int hidden, float eps, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (row_index && !resid_out) return KIRAI_ERR_BAD_SIZE;
    const bool aligned = hidden % 4 == 0 && (((uintptr_t)resid | (uintptr_t)delta | (uintptr_t)weight | (uintptr_t)out |
                                              (uintptr_t)resid_out) & 15) == 0;
    if (aligned && hidden <= 4 * 4 * 512) {
        const int threads = hidden <= 4 * 4 * 128 ? 128 : (hidden <= 4 * 4 * 256 ? 256 : 512);
        return launch_pdl(add_rmsnorm_vec_kernel<T, 4>, dim3(rows), dim3(threads), 0, stream, 1u, resid, (const T*)delta,
                          weight, (T*)out, row_index, resid_out, hidden, eps);
    }
    const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
    const int pdl_status = launch_pdl(add_rmsnorm_kernel<T>, dim3(rows), dim3(threads), 0, stream, 1u, resid, (const T*)delta, weight, (T*)out, row_index, resid_out,
                                                        hidden, eps);
    return pdl_status;
}

KIRAI_EXPORT int kirai_add_rmsnorm_f32(float* resid, const void* delta, const float* weight, void* out,
                                       const int* row_index, float* resid_out, int rows, int hidden, float eps,
                                       cudaStream_t stream) {
    return add_rmsnorm_launch<float>(resid, delta, weight, out, row_index, resid_out, rows, hidden, eps, stream);
}
KIRAI_EXPORT int kirai_add_rmsnorm_bf16(float* resid, const void* delta, const float* weight, void* out,
                                        const int* row_index, float* resid_out, int rows, int hidden, float eps,
                                        cudaStream_t stream) {
    return add_rmsnorm_launch<bf16>(resid, delta, weight, out, row_index, resid_out, rows, hidden, eps, stream);
}

// ------------------------------------------------------------- per-head RMSNorm
// x is [rows, heads, width] with a row stride (in elements); one warp per head.
template <typename T>
__global__ void head_rmsnorm_kernel(T* __restrict__ x, const float* __restrict__ weight, int rows, int heads, int width,
                                    long row_stride, float eps) {
    pdl_launch_dependents();
    pdl_wait();
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (warp >= rows * heads) return;
    T* head = x + (size_t)(warp / heads) * row_stride + (size_t)(warp % heads) * width;
    float acc = 0.0f;
    for (int i = lane; i < width; i += 32) {
        const float v = to_f32<T>(head[i]);
        acc = fmaf(v, v, acc);
    }
    acc = warp_sum(acc);
    const float variance = acc / (float)width + eps;
    const float scale = variance == 0.0f ? 0.0f : 1.0f / sqrtf(variance);
    for (int i = lane; i < width; i += 32) head[i] = from_f32<T>(to_f32<T>(head[i]) * scale * weight[i]);
}

template <typename T>
static int head_rmsnorm_launch(void* x, const float* weight, int rows, int heads, int width, long row_stride, float eps,
                               cudaStream_t stream) {
    const long warps = (long)rows * heads;
    if (warps <= 0) return 0;
    const int threads = 128;
    const long blocks = (warps * 32 + threads - 1) / threads;
    const int pdl_status = launch_pdl(head_rmsnorm_kernel<T>, dim3((unsigned)blocks), dim3(threads), 0, stream, 1u, (T*)x, weight, rows, heads, width, row_stride, eps);
    return pdl_status;
}
KIRAI_EXPORT int kirai_head_rmsnorm_f32(void* x, const float* weight, int rows, int heads, int width, long row_stride,
                                        float eps, cudaStream_t stream) {
    return head_rmsnorm_launch<float>(x, weight, rows, heads, width, row_stride, eps, stream);
}
KIRAI_EXPORT int kirai_head_rmsnorm_bf16(void* x, const float* weight, int rows, int heads, int width, long row_stride,
                                         float eps, cudaStream_t stream) {
    return head_rmsnorm_launch<bf16>(x, weight, rows, heads, width, row_stride, eps, stream);
}

// ------------------------------------------------------------------------ rotary
// x is [rows, heads, width] with a row stride; pairs (i, i + rotary_dim/2), angle
// = float(position) * inv_freq[i], all in 32-bit.
template <typename T>
__global__ void rope_kernel(T* __restrict__ x, const int* __restrict__ positions, const float* __restrict__ inv_freq,
                            int rows, int heads, int width, int rotary_dim, long row_stride) {
    pdl_launch_dependents();
    pdl_wait();
    const int half = rotary_dim >> 1;
    const long total = (long)rows * heads * half;
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int i = (int)(idx % half);
    const int head = (int)((idx / half) % heads);
    const int row = (int)(idx / ((long)half * heads));
    T* base = x + (size_t)row * row_stride + (size_t)head * width;
    const float angle = (float)positions[row] * inv_freq[i];
    float s, c;
    sincosf(angle, &s, &c);
    const float first = to_f32<T>(base[i]);
    const float second = to_f32<T>(base[i + half]);
    base[i] = from_f32<T>(first * c - second * s);
    base[i + half] = from_f32<T>(second * c + first * s);
}

template <typename T>
static int rope_launch(void* x, const int* positions, const float* inv_freq, int rows, int heads, int width,
                       int rotary_dim, long row_stride, cudaStream_t stream) {
    if (rotary_dim <= 0 || (rotary_dim & 1) || rotary_dim > width) return KIRAI_ERR_BAD_SIZE;
    const long total = (long)rows * heads * (rotary_dim / 2);
    if (total <= 0) return 0;
    const int threads = 256;
    const int pdl_status = launch_pdl(rope_kernel<T>, dim3((unsigned)((total + threads - 1) / threads)), dim3(threads), 0, stream, 1u, (T*)x, positions, inv_freq, rows,
                                                                                      heads, width, rotary_dim,
                                                                                      row_stride);
    return pdl_status;
}
KIRAI_EXPORT int kirai_rope_f32(void* x, const int* positions, const float* inv_freq, int rows, int heads, int width,
                                int rotary_dim, long row_stride, cudaStream_t stream) {
    return rope_launch<float>(x, positions, inv_freq, rows, heads, width, rotary_dim, row_stride, stream);
}
KIRAI_EXPORT int kirai_rope_bf16(void* x, const int* positions, const float* inv_freq, int rows, int heads, int width,
                                 int rotary_dim, long row_stride, cudaStream_t stream) {
    return rope_launch<bf16>(x, positions, inv_freq, rows, heads, width, rotary_dim, row_stride, stream);
}

// ---------------------------------------------------------------- paged KV write
// One cache layer is [num_pages, 2, kv_heads, page_size, head_dim]; key rows at
// index 0 and value rows at index 1 of the second axis.  The row of a token is
// found through its request's block table: page = table[request, pos / page_size].
__device__ __forceinline__ long kv_row_offset(int page, int which, int kv_head, int slot, int kv_heads, int page_size,
                                              int head_dim) {
    return ((((long)page * 2 + which) * kv_heads + kv_head) * page_size + slot) * (long)head_dim;
}

template <typename T>
__global__ void kv_write_kernel(const T* __restrict__ k, const T* __restrict__ v, T* __restrict__ cache,
                                const int* __restrict__ block_table, const int* __restrict__ request_of_token,
                                const int* __restrict__ positions, int rows, int kv_heads, int head_dim,
                                long k_row_stride, long v_row_stride, int page_size, int table_width, int num_pages,
                                int* __restrict__ error_flag) {
    pdl_launch_dependents();
    pdl_wait();
    const long total = (long)rows * kv_heads * head_dim;
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int i = (int)(idx % head_dim);
    const int head = (int)((idx / head_dim) % kv_heads);
    const int row = (int)(idx / ((long)head_dim * kv_heads));
    const int pos = positions[row];
    const int logical = pos / page_size;
    const int page = logical < table_width ? block_table[(long)request_of_token[row] * table_width + logical] : -1;
    if (page < 0 || page >= num_pages) {
        atomicExch(error_flag, 2);
        return;
    }
    const int slot = pos % page_size;
    cache[kv_row_offset(page, 0, head, slot, kv_heads, page_size, head_dim) + i] =
        k[(size_t)row * k_row_stride + (size_t)head * head_dim + i];
    cache[kv_row_offset(page, 1, head, slot, kv_heads, page_size, head_dim) + i] =
        v[(size_t)row * v_row_stride + (size_t)head * head_dim + i];
}

template <typename T>
static int kv_write_launch(const void* k, const void* v, void* cache, const int* block_table,
                           const int* request_of_token, const int* positions, int rows, int kv_heads, int head_dim,
                           long k_row_stride, long v_row_stride, int page_size, int table_width, int num_pages,
                           int* error_flag, cudaStream_t stream) {
    const long total = (long)rows * kv_heads * head_dim;
    if (total <= 0) return 0;
    const int threads = 256;
    const int pdl_status = launch_pdl(kv_write_kernel<T>, dim3((unsigned)((total + threads - 1) / threads)), dim3(threads), 0, stream, 1u, 
        (const T*)k, (const T*)v, (T*)cache, block_table, request_of_token, positions, rows, kv_heads, head_dim,
        k_row_stride, v_row_stride, page_size, table_width, num_pages, error_flag);
    return pdl_status;
}
KIRAI_EXPORT int kirai_kv_write_f32(const void* k, const void* v, void* cache, const int* block_table,
                                    const int* request_of_token, const int* positions, int rows, int kv_heads,
                                    int head_dim, long k_row_stride, long v_row_stride, int page_size, int table_width,
                                    int num_pages, int* error_flag, cudaStream_t stream) {
    return kv_write_launch<float>(k, v, cache, block_table, request_of_token, positions, rows, kv_heads, head_dim,
                                  k_row_stride, v_row_stride, page_size, table_width, num_pages, error_flag, stream);
}
KIRAI_EXPORT int kirai_kv_write_bf16(const void* k, const void* v, void* cache, const int* block_table,
                                     const int* request_of_token, const int* positions, int rows, int kv_heads,
                                     int head_dim, long k_row_stride, long v_row_stride, int page_size, int table_width,
                                     int num_pages, int* error_flag, cudaStream_t stream) {
    return kv_write_launch<bf16>(k, v, cache, block_table, request_of_token, positions, rows, kv_heads, head_dim,
                                 k_row_stride, v_row_stride, page_size, table_width, num_pages, error_flag, stream);
}

// ------------------------------------ fused per-head norm + rotary + cache write
// qkv is [rows, (q_heads + 2 kv_heads) * head_dim]: query heads, then key heads,
// then value heads.  One warp per (row, head): query heads are normed and
// rotated in place; key heads are normed, rotated and written to the cache page
// (and back in place); value heads are copied to the cache.  With norm weights
// absent (nullptr) the norm is skipped; with inv_freq absent the rotation is.
// head_dim <= 512 (16 values per lane).
#define FUSED_MAX_PAIRS 8
#define FUSED_WARPS 4
// One block per token: the rotation's sines and cosines depend on the token's position only, so
// they are computed once into shared memory; then the block's warps take the token's heads in
// turn, one warp per head, each lane holding pairs (i, i + head_dim / 2).
template <typename T>
__global__ void __launch_bounds__(FUSED_WARPS * 32)
qk_norm_rope_kv_write_kernel(T* __restrict__ qkv, const float* __restrict__ q_weight,
                                             const float* __restrict__ k_weight, const float* __restrict__ inv_freq,
                                             T* __restrict__ cache, const int* __restrict__ block_table,
                                             const int* __restrict__ request_of_token,
                                             const int* __restrict__ positions, int rows, int q_heads, int kv_heads,
                                             int head_dim, int rotary_dim, float eps, int page_size, int table_width,
                                             int num_pages, int write_cache, int* __restrict__ error_flag) {
    pdl_launch_dependents();
    // positions, the request of each token and the block tables are constant during a step: the angles and the
    // page are worked out before the kernel before this one (the q, k, v product) has finished
    __shared__ float cos_s[32 * FUSED_MAX_PAIRS], sin_s[32 * FUSED_MAX_PAIRS];
    const int heads_total = q_heads + 2 * kv_heads;
    const int row = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int pos = positions[row];
    const int half_dim = head_dim >> 1;  // values are held as (i, i + head_dim/2) so that the norm sees all of them
    if (inv_freq) {
        for (int i = threadIdx.x; i < half_dim; i += blockDim.x) sincosf((float)pos * inv_freq[i], &sin_s[i], &cos_s[i]);
        __syncthreads();
    }
    int page = -1;
    if (write_cache) {
        const int logical = pos / page_size;
        page = logical < table_width ? block_table[(long)request_of_token[row] * table_width + logical] : -1;
        if (page < 0 || page >= num_pages) {
            if (threadIdx.x == 0) atomicExch(error_flag, 2);
            page = -1;
        }
    }
    pdl_wait();
    // with few tokens the heads are spread over gridDim.y blocks, so that enough blocks run at once
    for (int head = blockIdx.y * FUSED_WARPS + warp; head < heads_total; head += gridDim.y * FUSED_WARPS) {
        T* x = qkv + (size_t)row * heads_total * head_dim + (size_t)head * head_dim;
        const bool is_q = head < q_heads;
        const bool is_k = !is_q && head < q_heads + kv_heads;
        const int kv_head = is_q ? 0 : (is_k ? head - q_heads : head - q_heads - kv_heads);
        T* dst = nullptr;
        if (!is_q && write_cache) {
            if (page < 0) continue;
            dst = cache + kv_row_offset(page, is_k ? 0 : 1, kv_head, pos % page_size, kv_heads, page_size, head_dim);
        }
        if (!is_q && !is_k) {  // value head: plain copy
            if (dst)
                for (int i = lane; i < head_dim; i += 32) dst[i] = x[i];
            continue;
        }
        float lo[FUSED_MAX_PAIRS], hi[FUSED_MAX_PAIRS];
        float acc = 0.0f;
#pragma unroll
        for (int j = 0; j < FUSED_MAX_PAIRS; ++j) {
            const int i = lane + 32 * j;
            lo[j] = hi[j] = 0.0f;
            if (i < half_dim) {
                lo[j] = to_f32<T>(x[i]);
                hi[j] = to_f32<T>(x[i + half_dim]);
                acc = fmaf(lo[j], lo[j], acc);
                acc = fmaf(hi[j], hi[j], acc);
            }
        }
        const float* weight = is_q ? q_weight : k_weight;
        float scale = 1.0f;
        if (weight) {
            acc = warp_sum(acc);
            const float variance = acc / (float)head_dim + eps;
            scale = variance == 0.0f ? 0.0f : 1.0f / sqrtf(variance);
        }
#pragma unroll
        for (int j = 0; j < FUSED_MAX_PAIRS; ++j) {
            const int i = lane + 32 * j;
            if (i < half_dim) {
                float a = lo[j], b = hi[j];
                if (weight) {
                    a = a * scale * weight[i];
                    b = b * scale * weight[i + half_dim];
                }
                if (inv_freq) {  // rotary_dim == head_dim: the pairs are the (lo, hi) held here
                    const float c = cos_s[i], sn = sin_s[i];
                    const float ra = a * c - b * sn, rb = b * c + a * sn;
                    a = ra;
                    b = rb;
                }
                const T ta = from_f32<T>(a), tb = from_f32<T>(b);
                x[i] = ta;
                x[i + half_dim] = tb;
                if (dst) {
                    dst[i] = ta;
                    dst[i + half_dim] = tb;
                }
            }
        }
    }
}

// The same work for head sizes that are multiples of 4, which is every size in steps of 16: each lane holds
// adjacent pairs (2i, 2i + 1) of both halves, so that loads and stores are 4 bytes wide in bf16 (8 in float), and a
// warp has the loads of four heads in flight before it computes the first.  Many tokens make this kernel a
// pure stream over q, k, v and the cache rows; with 2-byte accesses and one head at a time it ran at a quarter
// of the memory rate.
template <typename T> struct Pair;
template <> struct Pair<float> {
    using type = float2;
    static __device__ __forceinline__ float2 widen(float2 v) { return v; }
    static __device__ __forceinline__ float2 narrow(float a, float b) { return make_float2(a, b); }
};
template <> struct Pair<bf16> {
    using type = __nv_bfloat162;
    static __device__ __forceinline__ float2 widen(__nv_bfloat162 v) { return __bfloat1622float2(v); }
    static __device__ __forceinline__ __nv_bfloat162 narrow(float a, float b) { return __floats2bfloat162_rn(a, b); }
};
#define FUSED_UNROLL 4

// SLOTS: pairs per lane and half, 1 for head sizes up to 128, 2 up to 256, 4 up to 512 (the loops are unrolled over it).
template <typename T, int SLOTS>
__global__ void __launch_bounds__(FUSED_WARPS * 32)
qk_norm_rope_kv_write_vec_kernel(T* __restrict__ qkv, const float* __restrict__ q_weight,
                                 const float* __restrict__ k_weight, const float* __restrict__ inv_freq,
                                 T* __restrict__ cache, const int* __restrict__ block_table,
                                 const int* __restrict__ request_of_token, const int* __restrict__ positions, int rows,
                                 int q_heads, int kv_heads, int head_dim, float eps, int page_size, int table_width,
                                 int num_pages, int write_cache, int* __restrict__ error_flag) {
    using P = typename Pair<T>::type;
    pdl_launch_dependents();
    // positions, the request of each token and the block tables are constant during a step: the angles and the
    // page are worked out before the kernel before this one (the q, k, v product) has finished
    __shared__ float cos_s[32 * FUSED_MAX_PAIRS], sin_s[32 * FUSED_MAX_PAIRS];
    const int heads_total = q_heads + 2 * kv_heads;
    const int row = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int pos = positions[row];
    const int half_dim = head_dim >> 1, half_pairs = head_dim >> 2;  // pairs of adjacent values in one half
    if (inv_freq) {
        for (int i = threadIdx.x; i < half_dim; i += blockDim.x) sincosf((float)pos * inv_freq[i], &sin_s[i], &cos_s[i]);
        __syncthreads();
    }
    int page = -1;
    if (write_cache) {
        const int logical = pos / page_size;
        page = logical < table_width ? block_table[(long)request_of_token[row] * table_width + logical] : -1;
        if (page < 0 || page >= num_pages) {
            if (threadIdx.x == 0) atomicExch(error_flag, 2);
            page = -1;
        }
    }
    pdl_wait();
    const int slot_in_page = pos % page_size;
    const int stride = gridDim.y * FUSED_WARPS;  // warps that share this token's heads
    for (int base = blockIdx.y * FUSED_WARPS + warp; base < heads_total; base += stride * FUSED_UNROLL) {
        P lo[FUSED_UNROLL][SLOTS], hi[FUSED_UNROLL][SLOTS];
#pragma unroll
        for (int u = 0; u < FUSED_UNROLL; ++u) {
            const int head = base + u * stride;
            if (head >= heads_total) break;
            const P* x = reinterpret_cast<const P*>(qkv + (size_t)row * heads_total * head_dim + (size_t)head * head_dim);
#pragma unroll
            for (int j = 0; j < SLOTS; ++j) {
                const int i = lane + 32 * j;
                if (i < half_pairs) {
                    lo[u][j] = x[i];
                    hi[u][j] = x[i + half_pairs];
                }
            }
        }
#pragma unroll
        for (int u = 0; u < FUSED_UNROLL; ++u) {
            const int head = base + u * stride;
            if (head >= heads_total) break;
            P* x = reinterpret_cast<P*>(qkv + (size_t)row * heads_total * head_dim + (size_t)head * head_dim);
            const bool is_q = head < q_heads;
            const bool is_k = !is_q && head < q_heads + kv_heads;
            const int kv_head = is_q ? 0 : (is_k ? head - q_heads : head - q_heads - kv_heads);
            P* dst = nullptr;
            if (!is_q && write_cache) {
                if (page < 0) continue;
                dst = reinterpret_cast<P*>(cache + kv_row_offset(page, is_k ? 0 : 1, kv_head, slot_in_page, kv_heads, page_size, head_dim));
            }
            if (!is_q && !is_k) {  // value head: plain copy
                if (dst) {
#pragma unroll
                    for (int j = 0; j < SLOTS; ++j) {
                        const int i = lane + 32 * j;
                        if (i < half_pairs) {
                            dst[i] = lo[u][j];
                            dst[i + half_pairs] = hi[u][j];
                        }
                    }
                }
                continue;
            }
            float2 a[SLOTS], b[SLOTS];
            float acc = 0.0f;
#pragma unroll
            for (int j = 0; j < SLOTS; ++j) {
                a[j] = b[j] = make_float2(0.0f, 0.0f);
                if (lane + 32 * j < half_pairs) {
                    a[j] = Pair<T>::widen(lo[u][j]);
                    b[j] = Pair<T>::widen(hi[u][j]);
                    acc = fmaf(a[j].x, a[j].x, acc);
                    acc = fmaf(b[j].x, b[j].x, acc);
                    acc = fmaf(a[j].y, a[j].y, acc);
                    acc = fmaf(b[j].y, b[j].y, acc);
                }
            }
            const float* weight = is_q ? q_weight : k_weight;
            float scale = 1.0f;
            if (weight) {
                acc = warp_sum(acc);
                const float variance = acc / (float)head_dim + eps;
                scale = variance == 0.0f ? 0.0f : 1.0f / sqrtf(variance);
            }
#pragma unroll
            for (int j = 0; j < SLOTS; ++j) {
                const int i = lane + 32 * j;
                if (i < half_pairs) {
                    float2 va = a[j], vb = b[j];
                    if (weight) {
                        const float2 wa = *reinterpret_cast<const float2*>(weight + 2 * i);
                        const float2 wb = *reinterpret_cast<const float2*>(weight + 2 * i + half_dim);
                        va.x = va.x * scale * wa.x, va.y = va.y * scale * wa.y;
                        vb.x = vb.x * scale * wb.x, vb.y = vb.y * scale * wb.y;
                    }
                    if (inv_freq) {  // the rotation pairs value e of the first half with e + head_dim / 2
                        const float c0 = cos_s[2 * i], s0 = sin_s[2 * i], c1 = cos_s[2 * i + 1], s1 = sin_s[2 * i + 1];
                        const float ax = va.x * c0 - vb.x * s0, bx = vb.x * c0 + va.x * s0;
                        const float ay = va.y * c1 - vb.y * s1, by = vb.y * c1 + va.y * s1;
                        va = make_float2(ax, ay);
                        vb = make_float2(bx, by);
                    }
                    const P pa = Pair<T>::narrow(va.x, va.y), pb = Pair<T>::narrow(vb.x, vb.y);
                    x[i] = pa;
                    x[i + half_pairs] = pb;
                    if (dst) {
                        dst[i] = pa;
                        dst[i + half_pairs] = pb;
                    }
                }
            }
        }
    }
}

// The same work for bf16 heads of 64, 128 or 256: LANES = head_dim / 16 lanes share a head, each with eight adjacent
// values of both halves (16-byte loads and stores), so that a warp handles 32 / LANES heads at once.  With one pair
// of values per lane and instruction the kernel above is bound by its instruction count when there are thousands of
// tokens (16.9 M warp instructions for 2,048 tokens of 48 heads); this form needs about a sixth per value.
template <int LANES>
__global__ void __launch_bounds__(FUSED_WARPS * 32)
qk_norm_rope_kv_write_wide_kernel(bf16* __restrict__ qkv, const float* __restrict__ q_weight, const float* __restrict__ k_weight,
                                  const float* __restrict__ inv_freq, bf16* __restrict__ cache,
                                  const int* __restrict__ block_table, const int* __restrict__ request_of_token,
                                  const int* __restrict__ positions, int rows, int q_heads, int kv_heads, float eps,
                                  int page_size, int table_width, int num_pages, int write_cache,
                                  int* __restrict__ error_flag) {
    constexpr int HEAD_DIM = LANES * 16, HALF = HEAD_DIM / 2, HEADS_PER_WARP = 32 / LANES;
    pdl_launch_dependents();
    // positions, the request of each token and the block tables are constant during a step: the angles and the
    // page are worked out before the kernel before this one (the q, k, v product) has finished
    __shared__ __align__(16) float cos_s[HALF], sin_s[HALF];
    const int heads_total = q_heads + 2 * kv_heads;
    const int row = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int pos = positions[row];
    if (inv_freq) {
        for (int i = threadIdx.x; i < HALF; i += blockDim.x) sincosf((float)pos * inv_freq[i], &sin_s[i], &cos_s[i]);
        __syncthreads();
    }
    int page = -1;
    if (write_cache) {
        const int logical = pos / page_size;
        page = logical < table_width ? block_table[(long)request_of_token[row] * table_width + logical] : -1;
        if (page < 0 || page >= num_pages) {
            if (threadIdx.x == 0) atomicExch(error_flag, 2);
            page = -1;
        }
    }
    const int slot_in_page = pos % page_size;
    pdl_wait();
    const int sub = lane % LANES;  // this lane's eight values of each half start at 8 * sub
    const int stride = gridDim.y * FUSED_WARPS * HEADS_PER_WARP;  // heads that the token's warps take per round
    const bool any_norm = q_weight != nullptr || k_weight != nullptr;
    for (int base = (blockIdx.y * FUSED_WARPS + warp) * HEADS_PER_WARP; base < heads_total; base += stride) {
        // whole warps stay in the loop for the shuffles; lanes past the last head carry zeros and store nothing
        const int head = base + lane / LANES;
        const bool live = head < heads_total;
        const bool is_q = head < q_heads;
        const bool is_k = !is_q && head < q_heads + kv_heads;
        uint4* x = reinterpret_cast<uint4*>(qkv + (size_t)row * heads_total * HEAD_DIM + (size_t)(live ? head : 0) * HEAD_DIM);
        uint4 raw_lo = make_uint4(0u, 0u, 0u, 0u), raw_hi = raw_lo;
        if (live) {
            raw_lo = x[sub];
            raw_hi = x[sub + LANES];
        }
        uint4* dst = nullptr;
        if (live && !is_q && write_cache && page >= 0) {
            const int kv_head = is_k ? head - q_heads : head - q_heads - kv_heads;
            dst = reinterpret_cast<uint4*>(cache + kv_row_offset(page, is_k ? 0 : 1, kv_head, slot_in_page, kv_heads, page_size, HEAD_DIM));
        }
        const bool transform = live && (is_q || is_k);
        float lo[8], hi[8];
        {
            const __nv_bfloat162* pl = reinterpret_cast<const __nv_bfloat162*>(&raw_lo);
            const __nv_bfloat162* ph = reinterpret_cast<const __nv_bfloat162*>(&raw_hi);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 a = __bfloat1622float2(pl[j]), b = __bfloat1622float2(ph[j]);
                lo[2 * j] = a.x, lo[2 * j + 1] = a.y, hi[2 * j] = b.x, hi[2 * j + 1] = b.y;
            }
        }
        const float* weight = is_q ? q_weight : k_weight;
        if (any_norm) {  // the same for every lane of the warp
            float acc = 0.0f;
#pragma unroll
            for (int j = 0; j < 8; ++j) acc = fmaf(lo[j], lo[j], fmaf(hi[j], hi[j], acc));
#pragma unroll
            for (int d = 1; d < LANES; d <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, d);
            if (transform && weight) {
                const float variance = acc / (float)HEAD_DIM + eps;
                const float scale = variance == 0.0f ? 0.0f : 1.0f / sqrtf(variance);
                const float4* wl = reinterpret_cast<const float4*>(weight + 8 * sub);
                const float4* wh = reinterpret_cast<const float4*>(weight + HALF + 8 * sub);
                const float4 w0 = wl[0], w1 = wl[1], w2 = wh[0], w3 = wh[1];
                const float wlo[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
                const float whi[8] = {w2.x, w2.y, w2.z, w2.w, w3.x, w3.y, w3.z, w3.w};
#pragma unroll
                for (int j = 0; j < 8; ++j) lo[j] = lo[j] * scale * wlo[j], hi[j] = hi[j] * scale * whi[j];
            }
        }
        if (transform && inv_freq) {
            const float4* cs = reinterpret_cast<const float4*>(cos_s + 8 * sub);
            const float4* sn = reinterpret_cast<const float4*>(sin_s + 8 * sub);
            const float4 c0 = cs[0], c1 = cs[1], s0 = sn[0], s1 = sn[1];
            const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
            const float sv[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float a = lo[j], b = hi[j];
                lo[j] = a * c[j] - b * sv[j];
                hi[j] = b * c[j] + a * sv[j];
            }
        }
        if (!live) continue;
        uint4 out_lo = raw_lo, out_hi = raw_hi;
        if (transform) {
            __nv_bfloat162* pl = reinterpret_cast<__nv_bfloat162*>(&out_lo);
            __nv_bfloat162* ph = reinterpret_cast<__nv_bfloat162*>(&out_hi);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                pl[j] = __floats2bfloat162_rn(lo[2 * j], lo[2 * j + 1]);
                ph[j] = __floats2bfloat162_rn(hi[2 * j], hi[2 * j + 1]);
            }
            x[sub] = out_lo;
            x[sub + LANES] = out_hi;
        }
        if (dst) {
            dst[sub] = out_lo;
            dst[sub + LANES] = out_hi;
        }
    }
}

template <typename T>
static int qk_norm_rope_kv_write_launch(void* qkv, const float* q_weight, const float* k_weight, const float* inv_freq,
                                        void* cache, const int* block_table, const int* request_of_token,
                                        const int* positions, int rows, int q_heads, int kv_heads, int head_dim,
                                        int rotary_dim, float eps, int page_size, int table_width, int num_pages,
                                        int write_cache, int* error_flag, cudaStream_t stream) {
    if (head_dim > 64 * FUSED_MAX_PAIRS || (head_dim & 1)) return KIRAI_ERR_BAD_SIZE;
    if (inv_freq && rotary_dim != head_dim) return KIRAI_ERR_UNSUPPORTED;  // partial rotation goes through rope_kernel
    if (rows <= 0 || q_heads + 2 * kv_heads <= 0) return 0;
    if (rows > 65535 * 1024) return KIRAI_ERR_BAD_SIZE;
    const int heads_total = q_heads + 2 * kv_heads;
    const int head_blocks = rows >= 1024 ? 1 : (heads_total + FUSED_WARPS - 1) / FUSED_WARPS;
    const bool pairs_aligned = head_dim % 4 == 0 && ((uintptr_t)qkv & 7) == 0 && ((uintptr_t)cache & 7) == 0 &&
                               ((uintptr_t)q_weight & 7) == 0 && ((uintptr_t)k_weight & 7) == 0;
    // bf16 heads of 64, 128 or 256 on 16-byte boundaries: the wide kernel
    if (sizeof(T) == 2 && (head_dim == 64 || head_dim == 128 || head_dim == 256) && ((uintptr_t)qkv & 15) == 0 &&
        ((uintptr_t)cache & 15) == 0 && ((uintptr_t)q_weight & 15) == 0 && ((uintptr_t)k_weight & 15) == 0) {
        const int per_warp = 32 / (head_dim / 16);
        const int wide_blocks = rows >= 1024 ? 1 : (heads_total + FUSED_WARPS * per_warp - 1) / (FUSED_WARPS * per_warp);
#define KIRAI_FUSED_WIDE(LANES)                                                                                         \
    return launch_pdl(qk_norm_rope_kv_write_wide_kernel<LANES>, dim3(rows, wide_blocks), dim3(FUSED_WARPS * 32), 0, stream, \
                      1u, (bf16*)qkv, q_weight, k_weight, inv_freq, (bf16*)cache, block_table, request_of_token, positions, \
                      rows, q_heads, kv_heads, eps, page_size, table_width, num_pages, write_cache, error_flag)
        if (head_dim == 64) KIRAI_FUSED_WIDE(4);
        if (head_dim == 128) KIRAI_FUSED_WIDE(8);
        KIRAI_FUSED_WIDE(16);
#undef KIRAI_FUSED_WIDE
    }
#define KIRAI_FUSED_VEC(SLOTS)                                                                                          \
    return launch_pdl(qk_norm_rope_kv_write_vec_kernel<T, SLOTS>, dim3(rows, head_blocks), dim3(FUSED_WARPS * 32), 0, stream, \
                      1u, (T*)qkv, q_weight, k_weight, inv_freq, (T*)cache, block_table, request_of_token, positions, rows, \
                      q_heads, kv_heads, head_dim, eps, page_size, table_width, num_pages, write_cache, error_flag)
    if (pairs_aligned && head_dim <= 128) KIRAI_FUSED_VEC(1);
    if (pairs_aligned && head_dim <= 256) KIRAI_FUSED_VEC(2);
    if (pairs_aligned) KIRAI_FUSED_VEC(4);
#undef KIRAI_FUSED_VEC
    return launch_pdl(qk_norm_rope_kv_write_kernel<T>, dim3(rows, head_blocks), dim3(FUSED_WARPS * 32), 0, stream, 1u, (T*)qkv, q_weight,
                      k_weight, inv_freq, (T*)cache, block_table, request_of_token, positions, rows, q_heads, kv_heads,
                      head_dim, rotary_dim, eps, page_size, table_width, num_pages, write_cache, error_flag);
}
KIRAI_EXPORT int kirai_qk_norm_rope_kv_write_f32(void* qkv, const float* q_weight, const float* k_weight,
                                                 const float* inv_freq, void* cache, const int* block_table,
                                                 const int* request_of_token, const int* positions, int rows,
                                                 int q_heads, int kv_heads, int head_dim, int rotary_dim, float eps,
                                                 int page_size, int table_width, int num_pages, int write_cache,
                                                 int* error_flag, cudaStream_t stream) {
    return qk_norm_rope_kv_write_launch<float>(qkv, q_weight, k_weight, inv_freq, cache, block_table, request_of_token,
                                               positions, rows, q_heads, kv_heads, head_dim, rotary_dim, eps, page_size,
                                               table_width, num_pages, write_cache, error_flag, stream);
}
KIRAI_EXPORT int kirai_qk_norm_rope_kv_write_bf16(void* qkv, const float* q_weight, const float* k_weight,
                                                  const float* inv_freq, void* cache, const int* block_table,
                                                  const int* request_of_token, const int* positions, int rows,
                                                  int q_heads, int kv_heads, int head_dim, int rotary_dim, float eps,
                                                  int page_size, int table_width, int num_pages, int write_cache,
                                                  int* error_flag, cudaStream_t stream) {
    return qk_norm_rope_kv_write_launch<bf16>(qkv, q_weight, k_weight, inv_freq, cache, block_table, request_of_token,
                                              positions, rows, q_heads, kv_heads, head_dim, rotary_dim, eps, page_size,
                                              table_width, num_pages, write_cache, error_flag, stream);
}

// ------------------------------------------------------------------------ SwiGLU
// gate_up is [rows, 2 * inter]: the gate half, then the up half.  out = silu(gate) * up.
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gate_up, T* __restrict__ out, long rows, int inter) {
    pdl_launch_dependents();
    pdl_wait();
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= rows * inter) return;
    const long row = idx / inter;
    const int i = (int)(idx % inter);
    const float g = to_f32<T>(gate_up[row * 2 * inter + i]);
    const float u = to_f32<T>(gate_up[row * 2 * inter + inter + i]);
    out[idx] = from_f32<T>(g / (1.0f + expf(-g)) * u);
}
template <typename T>
static int swiglu_launch(const void* gate_up, void* out, int rows, int inter, cudaStream_t stream) {
    const long total = (long)rows * inter;
    if (total <= 0) return 0;
    const int threads = 256;
    const int pdl_status = launch_pdl(swiglu_kernel<T>, dim3((unsigned)((total + threads - 1) / threads)), dim3(threads), 0, stream, 1u, (const T*)gate_up, (T*)out,
                                                                                        rows, inter);
    return pdl_status;
}
KIRAI_EXPORT int kirai_swiglu_f32(const void* gate_up, void* out, int rows, int inter, cudaStream_t stream) {
    return swiglu_launch<float>(gate_up, out, rows, inter, stream);
}
KIRAI_EXPORT int kirai_swiglu_bf16(const void* gate_up, void* out, int rows, int inter, cudaStream_t stream) {
    return swiglu_launch<bf16>(gate_up, out, rows, inter, stream);
}

// ------------------------------------------------------- residual accumulate
// resid (32-bit) += delta, for arrangements whose sub-layer outputs are not
// followed by a norm that could fold the add in.
template <typename T>
__global__ void add_residual_kernel(float* __restrict__ resid, const T* __restrict__ delta, long count) {
    pdl_launch_dependents();
    pdl_wait();
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx < count) resid[idx] += to_f32<T>(delta[idx]);
}
template <typename T>
static int add_residual_launch(float* resid, const void* delta, long count, cudaStream_t stream) {
    if (count <= 0) return 0;
    const int pdl_status = launch_pdl(add_residual_kernel<T>, dim3((unsigned)((count + 255) / 256)), dim3(256), 0, stream, 1u, resid, (const T*)delta, count);
    return pdl_status;
}
KIRAI_EXPORT int kirai_add_residual_f32(float* resid, const void* delta, long count, cudaStream_t stream) {
    return add_residual_launch<float>(resid, delta, count, stream);
}
KIRAI_EXPORT int kirai_add_residual_bf16(float* resid, const void* delta, long count, cudaStream_t stream) {
    return add_residual_launch<bf16>(resid, delta, count, stream);
}

// ------------------------------------------------------------- decode advance
// After a captured decode step: the sampled tokens become the next step's input
// and every request moves one position on, so the same graph can be replayed
// without the host in between.
__global__ void decode_advance_kernel(int* __restrict__ token_ids, const int* __restrict__ sampled,
                                      int* __restrict__ positions, int* __restrict__ context_len, int count) {
    pdl_launch_dependents();
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= count) return;
    token_ids[i] = sampled[i];
    positions[i] += 1;
    context_len[i] += 1;
}
KIRAI_EXPORT int kirai_decode_advance(int* token_ids, const int* sampled, int* positions, int* context_len, int count,
                                      cudaStream_t stream) {
    if (count <= 0) return 0;
    const int pdl_status = launch_pdl(decode_advance_kernel, dim3((count + 127) / 128), dim3(128), 0, stream, 1u, token_ids, sampled, positions, context_len, count);
    return pdl_status;
}
