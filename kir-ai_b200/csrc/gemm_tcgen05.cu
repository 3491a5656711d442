// bf16 matrix product on the fifth-generation tensor cores:
// C[M, N] = A[M, K] * W[N, K]^T, 32-bit accumulation in tensor memory.
//
// One CTA computes one 128 x BN tile of the "X x Y" product, where X is the
// operand that fills the 128 rows of the MMA and Y the one that fills its N
// columns.  For many tokens X = A (activations) and Y = W; for few tokens
// (decode) the operands are swapped, X = W and Y = A, so that the weight rows
// fill the MMA and the token count, padded to 16, becomes N.  Both operands are
// K-major, so both are loaded by TMA as [rows, 64] boxes with the 128-byte
// swizzle and fed to tcgen05.mma through shared-memory descriptors.
//
// Warp roles: warp 0 issues TMA loads into a ring of STAGES buffers, one thread
// of warp 1 issues the MMAs and owns the tensor-memory allocation, warps 2-5
// read the accumulator back (tcgen05.ld) and store the tile.  With split-K each
// CTA of a tile covers a range of K and stores 32-bit partial sums that a
// second kernel adds in a fixed order.  Every barrier wait is bounded; a wait
// that runs out sets the device error flag and the CTA winds down.
#include "sm100.cuh"
#include "tensor_map.cuh"

using namespace sm100;

#define GEMM_BM 128
#define GEMM_BK 64
#define GEMM_THREADS 192

template <int BN>
struct GemmSmem {
    static constexpr int x_bytes = GEMM_BM * GEMM_BK * 2;
    static constexpr int y_bytes = BN * GEMM_BK * 2;
    static constexpr int stage_bytes = x_bytes + y_bytes;
    static constexpr int max_bytes = 200 * 1024;
    static constexpr int stages = (max_bytes / stage_bytes) > 10 ? 10 : (max_bytes / stage_bytes);
    static constexpr int barrier_bytes = 256;
    static constexpr int total = stages * stage_bytes + barrier_bytes + 1024;  // + slack for the 1024-byte alignment
};

template <int BN>
__host__ __device__ constexpr int tmem_columns() { return BN <= 32 ? 32 : (BN <= 64 ? 64 : (BN <= 128 ? 128 : 256)); }

// SWAP false: X = A (rows m), Y = W (rows n), C[m, n].  SWAP true: X = W, Y = A.
// PARTIAL: store 32-bit sums to partial[split][M][N] instead of C.
template <int BN, bool SWAP, typename OutT, bool PARTIAL>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_y,
                    OutT* __restrict__ C, float* __restrict__ partial, int M, int N, int K, long ldc,
                    int k_blocks_per_split, int* __restrict__ error_flag) {
    using Smem = GemmSmem<BN>;
    constexpr int STAGES = Smem::stages;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = (uint64_t*)(smem + STAGES * Smem::stage_bytes);
    uint64_t* full_bar = bars;                 // [STAGES] TMA -> MMA
    uint64_t* empty_bar = bars + STAGES;       // [STAGES] MMA -> TMA
    uint64_t* done_bar = bars + 2 * STAGES;    // accumulator complete
    uint32_t* tmem_slot = (uint32_t*)(bars + 2 * STAGES + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int x0 = blockIdx.x * GEMM_BM;  // first row of X in this tile
    const int y0 = blockIdx.y * BN;       // first row of Y
    const int total_k_blocks = (K + GEMM_BK - 1) / GEMM_BK;
    const int kb_begin = blockIdx.z * k_blocks_per_split;
    const int kb_end = min(total_k_blocks, kb_begin + k_blocks_per_split);
    const int num_kb = kb_end - kb_begin;

    if (threadIdx.x == 0) {
        tma_prefetch_descriptor(&map_x);
        tma_prefetch_descriptor(&map_y);
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_addr(&full_bar[s]), 1);
            mbar_init(smem_addr(&empty_bar[s]), 1);
        }
        mbar_init(smem_addr(done_bar), 1);
        mbar_fence_init();
    }
    if (warp == 1) {
        tmem_alloc(smem_addr(tmem_slot), tmem_columns<BN>());
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    bool ok = true;

    if (warp == 0) {
        if (elect_one()) {
            for (int i = 0; i < num_kb; ++i) {
                const int s = i % STAGES;
                const uint32_t phase = (uint32_t)(i / STAGES) & 1u;
                if (!mbar_wait(smem_addr(&empty_bar[s]), phase ^ 1u)) { ok = false; break; }
                const uint32_t full = smem_addr(&full_bar[s]);
                mbar_expect_tx(full, Smem::stage_bytes);
                const uint32_t dst = smem_addr(smem + s * Smem::stage_bytes);
                const int k = (kb_begin + i) * GEMM_BK;
                tma_load_2d(dst, &map_x, full, k, x0);
                tma_load_2d(dst + Smem::x_bytes, &map_y, full, k, y0);
            }
        }
    } else if (warp == 1) {
        if (elect_one()) {
            constexpr uint32_t idesc = instr_desc_bf16(GEMM_BM, BN);
            for (int i = 0; i < num_kb; ++i) {
                const int s = i % STAGES;
                const uint32_t phase = (uint32_t)(i / STAGES) & 1u;
                if (!mbar_wait(smem_addr(&full_bar[s]), phase)) { ok = false; break; }
                tc_fence_after();
                const uint32_t x_addr = smem_addr(smem + s * Smem::stage_bytes);
                const uint64_t desc_x = smem_desc_k_major_sw128(x_addr);
                const uint64_t desc_y = smem_desc_k_major_sw128(x_addr + Smem::x_bytes);
#pragma unroll
                for (int k = 0; k < GEMM_BK / 16; ++k) {
                    // 16 bf16 = 32 bytes further along K inside the swizzle atom: +2 in the 16-byte address field
                    mma_bf16_ss(tmem_base, desc_x + (uint64_t)(2 * k), desc_y + (uint64_t)(2 * k), idesc,
                                (i > 0 || k > 0) ? 1u : 0u);
                }
                mma_commit(smem_addr(&empty_bar[s]));  // frees the stage once these MMAs have read it
            }
            mma_commit(smem_addr(done_bar));
        }
    } else {
        // Epilogue: warp w reads tensor-memory lanes 32 (w % 4) .. +31, one lane per thread.
        const int lane_group = warp & 3;
        const int x_row = x0 + lane_group * 32 + lane;  // row of X that this thread holds
        const int x_rows = SWAP ? N : M;
        const int y_rows = SWAP ? M : N;
        if (num_kb > 0) ok = mbar_wait(smem_addr(done_bar), 0);
        tc_fence_after();
        if (ok) {
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 16) {
                if (y0 + c0 >= y_rows) break;  // uniform across the warp
                uint32_t r[16];
                if (num_kb > 0) {
                    tmem_load_32x16(tmem_base + ((uint32_t)(lane_group * 32) << 16) + (uint32_t)c0, r);
                    tmem_load_wait();
                } else {
#pragma unroll
                    for (int j = 0; j < 16; ++j) r[j] = 0u;
                }
                if (x_row >= x_rows) continue;
                if (PARTIAL) {
                    float* base = partial + (size_t)blockIdx.z * M * N;
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int y = y0 + c0 + j;
                        if (y < y_rows) {
                            if (SWAP) base[(size_t)y * N + x_row] = __uint_as_float(r[j]);
                            else base[(size_t)x_row * N + y] = __uint_as_float(r[j]);
                        }
                    }
                } else if (SWAP) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int y = y0 + c0 + j;
                        if (y < y_rows) C[(size_t)y * ldc + x_row] = from_f32<OutT>(__uint_as_float(r[j]));
                    }
                } else {
                    OutT* dst = C + (size_t)x_row * ldc + y0 + c0;
                    const bool full = (y0 + c0 + 16 <= y_rows) && (((uintptr_t)dst & 15) == 0);
                    if (full && sizeof(OutT) == 2) {
                        uint32_t packed[8];
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            __nv_bfloat162 pair = __floats2bfloat162_rn(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
                            packed[j] = *reinterpret_cast<uint32_t*>(&pair);
                        }
                        uint4* out = reinterpret_cast<uint4*>(dst);
                        out[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                        out[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
                    } else if (full && sizeof(OutT) == 4) {
                        uint4* out = reinterpret_cast<uint4*>(dst);
#pragma unroll
                        for (int j = 0; j < 4; ++j) out[j] = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (y0 + c0 + j < y_rows) dst[j] = from_f32<OutT>(__uint_as_float(r[j]));
                    }
                }
            }
        }
    }
    if (!ok) atomicExch(error_flag, 4);
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, tmem_columns<BN>());
    }
}

// Adds the split-K partial sums in split order and converts.
template <typename OutT>
__global__ void splitk_reduce_kernel(const float* __restrict__ partial, OutT* __restrict__ C, int splits, int M, int N,
                                     long ldc) {
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long)M * N) return;
    float acc = 0.0f;
    for (int s = 0; s < splits; ++s) acc += partial[(size_t)s * M * N + idx];
    C[(size_t)(idx / N) * ldc + (idx % N)] = from_f32<OutT>(acc);
}

template <int BN, bool SWAP, typename OutT>
static int launch_config(const void* A, const void* W, void* C, float* workspace, size_t workspace_bytes, int M, int N,
                         int K, long lda, long ldc, int splits, int* error_flag, cudaStream_t stream) {
    using Smem = GemmSmem<BN>;
    CUtensorMap map_a, map_w;
    const void* x_ptr = SWAP ? W : A;
    const void* y_ptr = SWAP ? A : W;
    const uint64_t x_rows = SWAP ? N : M, y_rows = SWAP ? M : N;
    const uint64_t x_stride = SWAP ? K : lda, y_stride = SWAP ? lda : K;
    if (!tmap::bf16_2d_sw128(&map_a, x_ptr, x_rows, K, x_stride, GEMM_BM, GEMM_BK)) return KIRAI_ERR_BAD_ALIGN;
    if (!tmap::bf16_2d_sw128(&map_w, y_ptr, y_rows, K, y_stride, BN, GEMM_BK)) return KIRAI_ERR_BAD_ALIGN;
    const int total_k_blocks = (K + GEMM_BK - 1) / GEMM_BK;
    if (splits < 1) splits = 1;
    if (splits > total_k_blocks) splits = total_k_blocks;
    const int per_split = (total_k_blocks + splits - 1) / splits;
    splits = (total_k_blocks + per_split - 1) / per_split;
    dim3 grid((unsigned)((x_rows + GEMM_BM - 1) / GEMM_BM), (unsigned)((y_rows + BN - 1) / BN), (unsigned)splits);
    if (grid.y > 65535 || grid.z > 65535) return KIRAI_ERR_BAD_SIZE;
    cudaError_t err;
    if (splits == 1) {
        auto kernel = gemm_tcgen05_kernel<BN, SWAP, OutT, false>;
        err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem::total);
        if (err != cudaSuccess) return (int)err;
        kernel<<<grid, GEMM_THREADS, Smem::total, stream>>>(map_a, map_w, (OutT*)C, nullptr, M, N, K, ldc, per_split,
                                                           error_flag);
        return launch_status();
    }
    if (!workspace || workspace_bytes < (size_t)splits * M * N * sizeof(float)) return KIRAI_ERR_BAD_SIZE;
    auto kernel = gemm_tcgen05_kernel<BN, SWAP, OutT, true>;
    err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem::total);
    if (err != cudaSuccess) return (int)err;
    kernel<<<grid, GEMM_THREADS, Smem::total, stream>>>(map_a, map_w, (OutT*)C, workspace, M, N, K, ldc, per_split,
                                                       error_flag);
    int status = launch_status();
    if (status) return status;
    const long count = (long)M * N;
    splitk_reduce_kernel<OutT><<<(unsigned)((count + 255) / 256), 256, 0, stream>>>(workspace, (OutT*)C, splits, M, N, ldc);
    return launch_status();
}

// Split count for the swapped (few tokens) case, which is bound by the weight
// stream: enough CTAs to fill the 148 SMs in whole waves, each split at least 8
// k-blocks long, and no more partial-sum traffic than a fraction of the weights.
static int choose_splits(int M, int N, int K) {
    const int tiles = (N + GEMM_BM - 1) / GEMM_BM;
    const int k_blocks = (K + GEMM_BK - 1) / GEMM_BK;
    const int sms = 148;
    int best = 1;
    double best_score = 0.0;
    for (int s = 1; s <= 16 && s * 8 <= k_blocks; ++s) {
        const int ctas = tiles * s;
        const int waves = (ctas + sms - 1) / sms;
        double score = (double)ctas / ((double)waves * sms);
        // partial sums are written and read once: 8 bytes per output per split, against 2 K bytes of weights per row
        const double extra = s > 1 ? (8.0 * s * M) / (2.0 * K) : 0.0;
        score /= (1.0 + extra);
        if (score > best_score + 1e-9) {
            best_score = score;
            best = s;
        }
    }
    return best;
}

template <typename OutT>
static int gemm_dispatch(const void* A, const void* W, void* C, float* workspace, size_t workspace_bytes, int M, int N,
                         int K, long lda, long ldc, int splits, int* error_flag, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0) return KIRAI_ERR_BAD_SIZE;
    if (K % 8 != 0 || lda % 8 != 0) return KIRAI_ERR_BAD_ALIGN;  // TMA needs 16-byte row strides
    if (splits <= 0) splits = M <= 64 ? choose_splits(M, N, K) : 1;
#define KIRAI_GEMM_CASE(BN, SWAP) \
    return launch_config<BN, SWAP, OutT>(A, W, C, workspace, workspace_bytes, M, N, K, lda, ldc, splits, error_flag, stream)
    if (M <= 16) KIRAI_GEMM_CASE(16, true);
    if (M <= 32) KIRAI_GEMM_CASE(32, true);
    if (M <= 64) KIRAI_GEMM_CASE(64, true);
    if (N <= 128) KIRAI_GEMM_CASE(128, false);
    KIRAI_GEMM_CASE(256, false);
#undef KIRAI_GEMM_CASE
}

// Split count that kirai_gemm_bf16 picks for splits <= 0 (callers size the workspace with it).
KIRAI_EXPORT int kirai_gemm_bf16_auto_splits(int M, int N, int K) { return M <= 64 ? choose_splits(M, N, K) : 1; }

// workspace: 32-bit scratch for split-K partial sums, at least splits * M * N floats when splits > 1.
// splits <= 0 picks the count itself.
KIRAI_EXPORT int kirai_gemm_bf16(const void* A, const void* W, void* C, float* workspace, size_t workspace_bytes, int M,
                                 int N, int K, long lda, long ldc, int splits, int* error_flag, cudaStream_t stream) {
    return gemm_dispatch<bf16>(A, W, C, workspace, workspace_bytes, M, N, K, lda, ldc, splits, error_flag, stream);
}
KIRAI_EXPORT int kirai_gemm_bf16_out_f32(const void* A, const void* W, void* C, float* workspace,
                                         size_t workspace_bytes, int M, int N, int K, long lda, long ldc, int splits,
                                         int* error_flag, cudaStream_t stream) {
    return gemm_dispatch<float>(A, W, C, workspace, workspace_bytes, M, N, K, lda, ldc, splits, error_flag, stream);
}
