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
// read the accumulator back (tcgen05.ld) and store the tile.  With split-K the
// CTAs of a thread-block cluster cover ranges of K of one tile and the partial
// tiles are added through distributed shared memory, in rank order.  Epilogue
// variants: SwiGLU over interleaved gate and up rows; the residual add with the
// next RMSNorm's unscaled rows and sums of squares; a per-row 1/rms scale on the
// result (see Epilogue).  Every barrier wait is bounded; a wait that runs out sets
// the device error flag and the CTA winds down.
//
// The kernel is launched with programmatic stream serialization and starts
// fetching W before the kernel before it in the stream has finished; it waits
// for that kernel only before it reads A or writes C.  W must therefore not be
// written by the kernel that directly precedes a product in the same stream
// (weights are constants of a loaded model).
//
// W comes either row-major [N, K], read through a tiled tensor map, or "tiled": cut at load time into boxes of
// 128 rows x 64 columns, each stored as the 16 KB image that the 128-byte swizzle leaves in shared memory, box
// (row tile, k block) at index row_tile * ceil(K / 64) + k_block, zero-padded at the edges.  A tiled box is one
// contiguous bulk copy; streaming whole boxes reads HBM about a sixth faster than gathering 128 rows of 128 bytes.
#include <cstdlib>
#include <map>
#include <mutex>
#include <tuple>

#include "sm100.cuh"
#include "tensor_map.cuh"

using namespace sm100;

#define GEMM_BM 128
#define GEMM_BK 64
#define GEMM_THREADS 192
#define GEMM_BOX_BYTES (GEMM_BM * GEMM_BK * 2)  // one box of tiled weights

// Shared memory of one CTA: the ring of stages, the barriers, then (only with split-K) one slot
// per CTA of the cluster for the partial tiles.  The swapped, weight-streaming case (BN <= 64)
// keeps the ring small enough for two CTAs per SM, so that every SM streams weights even when
// there are fewer tiles than two waves (but see DEEP below); the many-token case takes as many stages as fit.
// DEEP (weight-streaming case, BN <= 32): a launch with no more CTAs than SMs gains nothing from a second CTA per
// SM; its CTAs take a longer ring instead, because 4 stages of 16 KB in each of 128 CTAs are 8 MB in flight, fewer
// than the memory system needs to run at its rate (about 1.5 us of latency x 6.4 TB/s).  Ten stages for up to 16
// tokens (the 96 CTAs of the 8B shape's q, k, v product then stream at the memory's rate: 7 stages 9.5 us, 10 stages 8.5).
// Tried on top of this and taken out: the partial tiles of a cluster row by row, sent with 16-byte stores (no faster:
// what the first CTA waits for at the end of a split product is the slowest of its cluster, not the stores).
// STREAM (the swapped, weight-streaming kernel) with BN = 128 (65 to 128 tokens): a partial tile is 64 KB, so slots
// for the other CTAs' partial results do not fit beside a ring.  They lie IN the receiving CTA's ring instead, which is
// free once its products are done: the cluster meets once before anything is sent (LATE), every CTA keeps the chunks it
// owns in tensor memory (see `scatter` in the kernel), and the staged stores go through the rest of the ring 64 tokens
// at a time.  One CTA per SM with six stages and up to three splits where the launch fits the SMs, else three stages,
// two CTAs per SM and no split.  Tiles of 64 tokens take the same way where the launch fits the SMs (eight stages,
// up to four splits), and slots beside a ring of four otherwise.
template <int BN, bool DEEP = false, bool STREAM = (BN <= 64)>
struct GemmSmem {
    static constexpr bool streaming = STREAM;
    static constexpr bool late_slots = STREAM && (BN > 64 || (BN == 64 && DEEP));  // (tiles of 256 tokens: one CTA per SM and four stages, DEEP or not)
    static constexpr int x_bytes = GEMM_BM * GEMM_BK * 2;
    static constexpr int y_bytes = BN * GEMM_BK * 2;
    static constexpr int stage_bytes = x_bytes + y_bytes;
    static constexpr int max_splits = !STREAM ? 1 : (BN <= 64 ? 4 : (DEEP || BN > 128 ? 3 : 1));  // BN <= 64: up to 128 KB of slots beside the ring
    static constexpr int slot_bytes = BN * GEMM_BM * 4;  // one 32-bit partial tile
    static constexpr int stages = !STREAM ? (200 * 1024 / stage_bytes)
                                          : (BN > 128 ? 4 : (BN > 64 ? (DEEP ? 6 : 3) : (DEEP ? (BN <= 16 ? 10 : (BN <= 32 ? 7 : 8)) : 4)));
    static constexpr int barrier_bytes = 2048;  // barriers [0, 256), row scales [256, 256 + 4 BN) (BN <= 256)
    static constexpr int stage_tokens = BN < 64 ? BN : 64;  // tokens that the staged stores take through shared memory at a time
    static_assert(!streaming || (2 * stages + 1) * 8 + 4 <= 256, "the streaming kernel's barriers must end before the row scales");
    static_assert(!DEEP || BN <= 32 || late_slots, "a long ring beside slots is for the smallest tiles");
    // LATE: what a CTA receives (from each other CTA the 16-token chunks that it owns, 8 KB each) and the staged tokens
    // lie in its ring; the most is received with two splits (half the tile from one sender) or with max_splits
    static constexpr int chunks = BN / 16;
    static constexpr int most_received = (((chunks + 1) / 2) > (max_splits - 1) * ((chunks + max_splits - 1) / max_splits)
                                              ? (chunks + 1) / 2 : (max_splits - 1) * ((chunks + max_splits - 1) / max_splits)) * 16 * GEMM_BM * 4;
    static_assert(!late_slots || max_splits == 1 || most_received + stage_tokens * 132 * 4 <= stages * stage_bytes,
                  "the other CTAs' partial chunks and the staged tokens lie in the ring");
    static constexpr int ctas_per_sm = streaming && !DEEP && BN <= 128 ? 2 : 1;
    static constexpr int total(int splits) {  // + slack to align the base to 1024 bytes
        return stages * stage_bytes + barrier_bytes + (splits > 1 && !late_slots ? splits * slot_bytes : 0) + 1024;
    }
};

template <int BN>
__host__ __device__ constexpr int tmem_columns() { return BN <= 32 ? 32 : (BN <= 64 ? 64 : (BN <= 128 ? 128 : 256)); }

// What the epilogue does beyond storing the product.
//  * row_sumsq != nullptr: the rows of A were left unscaled by an RMSNorm whose sums of squares came in parts,
//    row_sumsq[part][M]; output row m is multiplied by 1 / sqrt(sum_p row_sumsq[p][m] / row_count + row_eps)
//    (0 when that variance is 0), which is what the product of the normed rows would have been.
//  * EPI 2 (residual and next norm): residual[m][n] += product; C[m][n] = bf16(residual * norm_weight[n]) is the
//    unscaled input of the next product, and sumsq_out[tile][m] receives this tile's share of sum_n residual^2.
struct Epilogue {
    const float* row_sumsq;
    int row_parts;
    float row_count, row_eps;
    float* residual;
    const float* norm_weight;
    float* sumsq_out;
    unsigned long long* stamps;  // null, or [CTAs][8] clock stamps (ns) of the streaming kernel, for measurements
};

// Clock stamps of one CTA of the streaming kernel, written only when a buffer is given: 0 the CTA starts, 1 the kernel
// before has finished (activations may be read), 2 the first stage is in shared memory, 3 the last product is done,
// 4 the partial tiles of the cluster are together, 5 the tile is stored.
__device__ __forceinline__ void gemm_stamp(const Epilogue& ep, int which) {
    if (ep.stamps) {
        unsigned long long now;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
        const size_t cta = ((size_t)blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;
        ep.stamps[cta * 8 + which] = now;
    }
}

__device__ __forceinline__ float row_scale_of(const Epilogue& ep, int m, int M) {
    float total = 0.0f;
    for (int p = 0; p < ep.row_parts; ++p) total += ep.row_sumsq[(size_t)p * M + m];
    const float variance = total / ep.row_count + ep.row_eps;
    return variance == 0.0f ? 0.0f : 1.0f / sqrtf(variance);
}
// The stream's values of column n for tokens y0 + c0 .. + 15 (0 where the tile hangs over), loads only.
// Sixteen of a row's values in the stream, when the chunk lies inside the matrix and on 16-byte boundaries
// (of the stream and of the norm's weights alike); otherwise the epilogue reads them one by one.
struct ResidualChunk {
    float4 r[4];
    bool vector;
};
__device__ __forceinline__ void load_residual_chunk(const Epilogue& ep, int row, int col, int M, int N, ResidualChunk& chunk) {
    chunk.vector = false;
    if (row >= M || col + 16 > N) return;
    const float* res = ep.residual + (size_t)row * N + col;
    if ((((uintptr_t)res | (uintptr_t)(ep.norm_weight + col)) & 15) != 0) return;
    chunk.vector = true;
#pragma unroll
    for (int q4 = 0; q4 < 4; ++q4) chunk.r[q4] = reinterpret_cast<const float4*>(res)[q4];
}
template <int BN>
__device__ __forceinline__ void load_residual_column(const Epilogue& ep, int n, int y0, int c0, int M, int N, float* res) {
#pragma unroll
    for (int j = 0; j < 16; ++j) {
        const int y = y0 + c0 + j;
        res[j] = (n < N && y < M) ? ep.residual[(size_t)y * N + n] : 0.0f;
    }
}
__device__ __forceinline__ void named_barrier_128() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// The address, in the cluster's shared window, that `local` has in CTA `rank`; and a store to it.
__device__ __forceinline__ uint32_t cluster_address(uint32_t local, uint32_t rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(rank));
    return remote;
}
__device__ __forceinline__ void st_cluster_f32(uint32_t address, float value) {
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(address), "f"(value) : "memory");
}

// silu(gate) * up with the fast exponential and the fast division (relative error about 2^-21, far below
// the bf16 rounding of the result); the epilogue runs beside the next tile's MMAs and must be short.  (The correctly
// rounded reciprocal, a sequence with a branch for special cases, made sixteen of these take 1.9 us a thread.)
__device__ __forceinline__ float silu_mul(float gate, float up) {
    return __fdividef(gate * up, 1.0f + __expf(-gate));
}

// SWAP false: X = A (rows m), Y = W (rows n), C[m, n].  SWAP true: X = W, Y = A.
// Split-K: the CTAs of a cluster (1, 1, splits) cover one tile; each stores its 32-bit partial
// tile into its slot in the shared memory of the cluster's first CTA (distributed shared memory),
// which adds the slots in rank order and stores the result: no partial sum goes to global memory.
// EPI 0 stores C.  EPI 1 expects W's rows interleaved in eights (8 gate rows, the 8 matching up
// rows, ...) and stores silu(gate) * up, [M, N / 2].
template <int BN, bool SWAP, typename OutT, int EPI, bool DEEP>
__global__ void __launch_bounds__(GEMM_THREADS, GemmSmem<BN, DEEP, true>::ctas_per_sm)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_y,
                    const uint8_t* __restrict__ w_tiled, OutT* __restrict__ C, int M, int N, int K, long ldc,
                    int k_blocks_per_split, int splits, Epilogue ep, int* __restrict__ error_flag) {
    using Smem = GemmSmem<BN, DEEP, true>;
    constexpr int STAGES = Smem::stages;
    constexpr bool LATE = Smem::late_slots;  // what other CTAs send lies in the receiver's ring (see GemmSmem)
    // Tiles of 32 tokens and more, split along K: every CTA of the cluster sums and stores a share of the tile's
    // 16-token chunks (chunk c belongs to CTA c % splits) instead of the first CTA all of it.  A CTA sends the chunks
    // it does not own to their owners and keeps its own in tensor memory; an owner adds the partial chunks in rank
    // order, which is the order in which the first CTA added whole tiles, so the sums are the same bits.  (With the
    // first CTA doing everything, a product of 64 tokens spent 3.7 us sending, 3.6 us adding and 4 us storing after
    // its last MMA; the o projection of the 8B shape took 18 us at 64 tokens and 8 us at 16.)
    const bool scatter = SWAP && BN >= 32 && splits > 1;
    constexpr int CHUNKS = BN / 16;
    const int owned_chunks = scatter ? (CHUNKS + splits - 1) / splits : CHUNKS;  // the most that one CTA owns
    const int first_c0 = scatter ? 16 * (int)blockIdx.z : 0;  // this CTA's first chunk of tokens (none if beyond the tile)
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = (uint64_t*)(smem + STAGES * Smem::stage_bytes);
    float* scale_s = reinterpret_cast<float*>(smem + STAGES * Smem::stage_bytes + 256);   // [BN] row scales of this tile's tokens
    // what other CTAs of the cluster send: behind the barriers, or (LATE) from the ring's start.  Tiles of 16 tokens:
    // [splits][BN][128] in the first CTA; wider tiles: [senders][owned chunks][16][128] in every CTA (see `scatter`)
    float* slots = LATE ? reinterpret_cast<float*>(smem)
                        : reinterpret_cast<float*>(smem + STAGES * Smem::stage_bytes + Smem::barrier_bytes);
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
    const int num_kb = max(0, kb_end - kb_begin);
    const uint32_t rank = blockIdx.z;  // the cluster is (1, 1, splits) and the grid's z extent is splits
    pdl_launch_dependents();  // the next kernel may set itself up while this one streams
    if (threadIdx.x == 0) gemm_stamp(ep, 0);

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
    float res[16];  // EPI 2: the stream's values under this thread's 16 outputs
    float norm_w = 0.0f;
    // Staged stores (SWAP): a thread holds one output column of 16 tokens, so storing from that layout takes 16 to 32
    // narrow store instructions a thread, which measured 0.4 to 2.6 us at the end of a launch (longest when the next
    // kernel's CTAs already stream beside it).  Where rows are 16-byte aligned the values go through shared memory
    // (the idle ring; 132 floats to a token) and every thread stores 16 adjacent columns of one token in 16-byte pieces.
    const bool c_aligned = ((uintptr_t)C & 15) == 0 && (ldc * (long)sizeof(OutT)) % 16 == 0;
    const bool staged = SWAP && c_aligned &&
                        (EPI == 2 ? (N % 8 == 0 && (((uintptr_t)ep.residual | (uintptr_t)ep.norm_weight) & 15) == 0)
                                  : (EPI == 1 ? N % 16 == 0 : N % 8 == 0));
    float4 res4[4], norm4[4];  // EPI 2, staged: the stream's values and the norm's weights under this thread's 16 columns of token y0 + tile_row / 8
    bool ok = true;
    const int lane_group = warp & 3;           // epilogue warps: tensor-memory lanes 32 (warp % 4) ..
    const int tile_row = lane_group * 32 + lane;

    if (warp == 0) {
        if (elect_one()) {
            // The weights do not depend on the kernel before this one: with SWAP the X operand (weights)
            // of the first ring of stages is fetched at once, and only the activations wait for it.
            const int x_first = SWAP ? 0 : 1, y_first = SWAP ? 1 : 0;  // which operand is the weights
            // tiled weights (SWAP only): this tile's boxes lie one after the other
            const uint8_t* boxes = w_tiled ? w_tiled + ((size_t)blockIdx.x * total_k_blocks + kb_begin) * GEMM_BOX_BYTES : nullptr;
            auto load_x = [&](uint32_t dst, uint32_t full, int i) {
                if (SWAP && boxes) bulk_load_1d(dst, boxes + (size_t)i * GEMM_BOX_BYTES, GEMM_BOX_BYTES, full);
                else tma_load_2d(dst, &map_x, full, (kb_begin + i) * GEMM_BK, x0);
            };
            const int head = num_kb < STAGES ? num_kb : STAGES;
            for (int i = 0; i < head; ++i) {
                const uint32_t full = smem_addr(&full_bar[i]);
                mbar_expect_tx(full, Smem::stage_bytes);
                const uint32_t dst = smem_addr(smem + i * Smem::stage_bytes);
                const int k = (kb_begin + i) * GEMM_BK;
                if (x_first == 0) load_x(dst, full, i);
                if (y_first == 0) tma_load_2d(dst + Smem::x_bytes, &map_y, full, k, y0);
            }
            pdl_wait();  // what the kernel before wrote (the activations) is complete and visible
            gemm_stamp(ep, 1);
            for (int i = 0; i < head; ++i) {
                const uint32_t full = smem_addr(&full_bar[i]);
                const uint32_t dst = smem_addr(smem + i * Smem::stage_bytes);
                const int k = (kb_begin + i) * GEMM_BK;
                if (x_first == 1) load_x(dst, full, i);
                if (y_first == 1) tma_load_2d(dst + Smem::x_bytes, &map_y, full, k, y0);
            }
            for (int i = head; i < num_kb; ++i) {
                const int s = i % STAGES;
                const uint32_t phase = (uint32_t)(i / STAGES) & 1u;
                if (!mbar_wait(smem_addr(&empty_bar[s]), phase ^ 1u)) { ok = false; break; }
                const uint32_t full = smem_addr(&full_bar[s]);
                mbar_expect_tx(full, Smem::stage_bytes);
                const uint32_t dst = smem_addr(smem + s * Smem::stage_bytes);
                const int k = (kb_begin + i) * GEMM_BK;
                load_x(dst, full, i);
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
                if (i == 0) gemm_stamp(ep, 2);
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
        pdl_wait();  // the output buffer may still be read by the kernel before this one
        // what the epilogue reads from global memory is fetched while the products run
        if ((rank == 0 || scatter) && SWAP) {
            if (ep.row_sumsq) {
                // the scales of this tile's tokens, computed once by the first BN threads
                for (int t = tile_row; t < BN; t += GEMM_BM) scale_s[t] = (y0 + t < M) ? row_scale_of(ep, y0 + t, M) : 0.0f;
                named_barrier_128();
            }
            if (EPI == 2 && staged) {
                const int token = y0 + first_c0 + (tile_row >> 3), col = x0 + 16 * (tile_row & 7);
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const bool inside = col + 4 * q + 4 <= N;
                    res4[q] = (inside && token < M) ? *reinterpret_cast<const float4*>(ep.residual + (size_t)token * N + col + 4 * q)
                                                    : make_float4(0.f, 0.f, 0.f, 0.f);
                    norm4[q] = inside ? *reinterpret_cast<const float4*>(ep.norm_weight + col + 4 * q) : make_float4(0.f, 0.f, 0.f, 0.f);
                }
            } else if (EPI == 2) {
                load_residual_column<BN>(ep, x0 + tile_row, y0, first_c0, M, N, res);
                norm_w = x0 + tile_row < N ? ep.norm_weight[x0 + tile_row] : 0.0f;
            }
        }
        // (polling without sleeping here and in the load and MMA threads' waits measured no faster: 3.72 against 3.70 ms
        // a decode step of 8 requests, 3.05 both ways at one)
        if (num_kb > 0) ok = mbar_wait(smem_addr(done_bar), 0);
        tc_fence_after();
        if (tile_row == 0) gemm_stamp(ep, 3);
    }
    // LATE: the receivers' rings take what is sent, so nothing is sent before every CTA of the cluster has seen its
    // last product finish (all threads arrive here, the epilogue warps after their wait for the accumulator)
    if (splits > 1 && LATE) cluster_sync_all();
    if (warp >= 2 && scatter) {
        // every chunk of 16 tokens that another CTA owns goes to that CTA: its slot [sender][chunk / splits], the senders
        // in rank order without the owner itself, 16 x 128 floats column-major (lanes side by side)
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 16) {
            const uint32_t owner = (uint32_t)(c0 >> 4) % (uint32_t)splits;
            if (owner == rank) continue;
            const uint32_t sender = rank < owner ? rank : rank - 1u;
            const uint32_t slot = cluster_address(
                smem_addr(slots) + ((sender * (uint32_t)owned_chunks + (uint32_t)(c0 >> 4) / (uint32_t)splits) * (16u * GEMM_BM)) * 4u, owner);
            uint32_t r[16];
            if (num_kb > 0 && ok) {
                tmem_load_32x16(tmem_base + ((uint32_t)(lane_group * 32) << 16) + (uint32_t)c0, r);
                tmem_load_wait();
            } else {
#pragma unroll
                for (int j = 0; j < 16; ++j) r[j] = 0u;
            }
#pragma unroll
            for (int j = 0; j < 16; ++j) st_cluster_f32(slot + (uint32_t)((j * GEMM_BM + tile_row) * 4), __uint_as_float(r[j]));
        }
    } else if (warp >= 2 && splits > 1) {
        // (tiles of 16 tokens) store this CTA's partial tile into its slot in the first CTA (column-major: lanes side by side)
        const uint32_t slot = cluster_address(smem_addr(slots) + rank * (uint32_t)Smem::slot_bytes, 0);
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 16) {
            uint32_t r[16];
            if (num_kb > 0 && ok) {
                tmem_load_32x16(tmem_base + ((uint32_t)(lane_group * 32) << 16) + (uint32_t)c0, r);
                tmem_load_wait();
            } else {
#pragma unroll
                for (int j = 0; j < 16; ++j) r[j] = 0u;
            }
#pragma unroll
            for (int j = 0; j < 16; ++j)
                st_cluster_f32(slot + (uint32_t)(((c0 + j) * GEMM_BM + tile_row) * 4), __uint_as_float(r[j]));
        }
    }
    if (splits > 1) cluster_sync_all();  // every partial tile (or chunk) has arrived where it is added
    if (threadIdx.x == 64) gemm_stamp(ep, 4);

    if (warp >= 2 && (rank == 0 || scatter)) {
        const int x_row = x0 + tile_row;  // row of X that this thread holds
        const int x_rows = SWAP ? N : M;
        const int y_rows = SWAP ? M : N;
        const float my_scale = (!SWAP && ep.row_sumsq && x_row < M) ? row_scale_of(ep, x_row, M) : 1.0f;
        // The staged stores take Smem::stage_tokens tokens at a time through shared memory: all of a tile of up to 64
        // tokens through the idle ring; of 128 tokens two halves; LATE: through what the received chunks leave of it.
        constexpr int HALF = Smem::stage_tokens;
        float* const stage = reinterpret_cast<float*>(smem) + (LATE ? (size_t)(splits - 1) * owned_chunks * (16 * GEMM_BM) : 0);
#pragma unroll 1
        for (int h0 = 0; h0 < BN; h0 += HALF) {
        if (y0 + h0 >= y_rows) break;  // uniform across the CTA
#pragma unroll 1
        for (int c0 = h0; c0 < h0 + HALF; c0 += 16) {
            if (y0 + c0 >= y_rows) break;  // uniform across the warp
            if (scatter && (uint32_t)(c0 >> 4) % (uint32_t)splits != rank) continue;  // another CTA's chunk
            if (EPI == 2 && SWAP && c0 != first_c0) load_residual_column<BN>(ep, x_row, y0, c0, M, N, res);
            float v[16];
            if (scatter) {
                // the partial chunks in rank order: the other CTAs' from the slots, this CTA's own from tensor memory
                uint32_t r[16];
                if (num_kb > 0 && ok) {
                    tmem_load_32x16(tmem_base + ((uint32_t)(lane_group * 32) << 16) + (uint32_t)c0, r);
                    tmem_load_wait();
                } else {
#pragma unroll
                    for (int j = 0; j < 16; ++j) r[j] = 0u;
                }
                const int local = (c0 >> 4) / splits;
                for (int q = 0; q < splits; ++q) {
                    if ((uint32_t)q == rank) {
#pragma unroll
                        for (int j = 0; j < 16; ++j) v[j] = q == 0 ? __uint_as_float(r[j]) : v[j] + __uint_as_float(r[j]);
                    } else {
                        const float* slot = slots + ((size_t)((uint32_t)q < rank ? q : q - 1) * owned_chunks + local) * (16 * GEMM_BM);
#pragma unroll
                        for (int j = 0; j < 16; ++j) v[j] = q == 0 ? slot[j * GEMM_BM + tile_row] : v[j] + slot[j * GEMM_BM + tile_row];
                    }
                }
            } else if (splits > 1) {
#pragma unroll
                for (int j = 0; j < 16; ++j) v[j] = slots[(c0 + j) * GEMM_BM + tile_row];
                for (int other = 1; other < splits; ++other) {
                    const float* slot = slots + (size_t)other * (BN * GEMM_BM);
#pragma unroll
                    for (int j = 0; j < 16; ++j) v[j] += slot[(c0 + j) * GEMM_BM + tile_row];
                }
            } else {
                uint32_t r[16];
                if (num_kb > 0 && ok) {
                    tmem_load_32x16(tmem_base + ((uint32_t)(lane_group * 32) << 16) + (uint32_t)c0, r);
                    tmem_load_wait();
                } else {
#pragma unroll
                    for (int j = 0; j < 16; ++j) r[j] = 0u;
                }
#pragma unroll
                for (int j = 0; j < 16; ++j) v[j] = __uint_as_float(r[j]);
            }
            if (ep.row_sumsq) {
#pragma unroll
                for (int j = 0; j < 16; ++j) v[j] *= SWAP ? scale_s[c0 + j] : my_scale;
            }
            if (tile_row == 0) gemm_stamp(ep, 6);
            if (SWAP && staged) {
                // (every product has read the ring: it is free)
                if (EPI == 1) {
                    // this lane holds weight row x_row: rows 16k..16k+7 are gate rows, 16k+8..16k+15 their up rows
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const float out = silu_mul(v[j], __shfl_xor_sync(0xffffffffu, v[j], 8));
                        if ((lane & 8) == 0) stage[(c0 - h0 + j) * 132 + (tile_row >> 4) * 8 + (tile_row & 7)] = out;
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 16; ++j) stage[(c0 - h0 + j) * 132 + tile_row] = v[j];
                }
                continue;
            }
            if (EPI == 2 && SWAP) {
                // this lane holds output column x_row of tokens y0 + c0 .. + 15.  The squares of the sums go to shared
                // memory (the ring is idle: every product has read it), token by token, 132 floats to a token; they
                // are added up after the loop.  (Sixteen warp reductions here, one after the other, took 2 us.)
                float* sq_s = stage;  // (behind the partial tiles where those lie in the ring)
                const bool row_ok = x_row < x_rows;
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const int y = y0 + c0 + j;
                    const bool live = row_ok && y < y_rows;
                    const float r = res[j] + v[j];
                    if (live) {
                        ep.residual[(size_t)y * N + x_row] = r;
                        C[(size_t)y * ldc + x_row] = from_f32<OutT>(r * norm_w);
                    }
                    sq_s[(c0 + j) * 132 + tile_row] = live ? r * r : 0.0f;
                }
                continue;
            }
            if (EPI == 1 && SWAP) {
                // this lane holds weight row x_row: rows 16k..16k+7 are gate rows, 16k+8..16k+15 their up rows
                float out[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) out[j] = silu_mul(v[j], __shfl_xor_sync(0xffffffffu, v[j], 8));
                if ((lane & 8) == 0 && x_row < x_rows) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int y = y0 + c0 + j;
                        if (y < y_rows) C[(size_t)y * ldc + (x_row >> 4) * 8 + (x_row & 7)] = from_f32<OutT>(out[j]);
                    }
                }
                continue;
            }
            if (x_row >= x_rows) continue;
            if (EPI == 1) {
                // columns y0 + c0 .. + 15 are 8 gate rows then their 8 up rows: 8 outputs at (y0 + c0) / 2
                OutT* dst = C + (size_t)x_row * ldc + ((y0 + c0) >> 1);
                if (y0 + c0 + 16 <= y_rows && sizeof(OutT) == 2 && (((uintptr_t)dst & 15) == 0)) {
                    uint32_t packed[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        __nv_bfloat162 pair = __floats2bfloat162_rn(silu_mul(v[2 * j], v[2 * j + 8]), silu_mul(v[2 * j + 1], v[2 * j + 9]));
                        packed[j] = *reinterpret_cast<uint32_t*>(&pair);
                    }
                    *reinterpret_cast<uint4*>(dst) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                } else {
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        if (y0 + c0 + j + 8 < y_rows) dst[j] = from_f32<OutT>(silu_mul(v[j], v[j + 8]));
                }
            } else if (SWAP) {
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const int y = y0 + c0 + j;
                    if (y < y_rows) C[(size_t)y * ldc + x_row] = from_f32<OutT>(v[j]);
                }
            } else {
                OutT* dst = C + (size_t)x_row * ldc + y0 + c0;
                const bool full = (y0 + c0 + 16 <= y_rows) && (((uintptr_t)dst & 15) == 0);
                if (full && sizeof(OutT) == 2) {
                    uint32_t packed[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        __nv_bfloat162 pair = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
                        packed[j] = *reinterpret_cast<uint32_t*>(&pair);
                    }
                    uint4* out = reinterpret_cast<uint4*>(dst);
                    out[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                    out[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
                } else if (full && sizeof(OutT) == 4) {
                    float4* out = reinterpret_cast<float4*>(dst);
#pragma unroll
                    for (int j = 0; j < 4; ++j) out[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                } else {
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        if (y0 + c0 + j < y_rows) dst[j] = from_f32<OutT>(v[j]);
                }
            }
        }
        if (tile_row == 0) gemm_stamp(ep, 7);
        if (SWAP && staged) {
            named_barrier_128();
            const int part = tile_row & 7;
#pragma unroll 1
            for (int base = h0; base < h0 + HALF; base += 16) {
                if (y0 + base >= y_rows) break;  // uniform
                if (scatter && (uint32_t)(base >> 4) % (uint32_t)splits != rank) continue;  // another CTA's chunk
                const int local = base + (tile_row >> 3), token = y0 + local;
                if (EPI == 1) {
                    // 64 outputs a token: eight to a thread
                    const int col = (x0 >> 1) + 8 * part;
                    if (token < y_rows && col + 8 <= (N >> 1)) {
                        const float4 a = *reinterpret_cast<const float4*>(stage + (local - h0) * 132 + 8 * part);
                        const float4 b = *reinterpret_cast<const float4*>(stage + (local - h0) * 132 + 8 * part + 4);
                        __nv_bfloat162 p0 = __floats2bfloat162_rn(a.x, a.y), p1 = __floats2bfloat162_rn(a.z, a.w);
                        __nv_bfloat162 p2 = __floats2bfloat162_rn(b.x, b.y), p3 = __floats2bfloat162_rn(b.z, b.w);
                        *reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(C) + (size_t)token * ldc + col) =
                            make_uint4(*reinterpret_cast<uint32_t*>(&p0), *reinterpret_cast<uint32_t*>(&p1),
                                       *reinterpret_cast<uint32_t*>(&p2), *reinterpret_cast<uint32_t*>(&p3));
                    }
                    continue;
                }
                const int col = x0 + 16 * part;
                float4 value[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) value[q] = *reinterpret_cast<const float4*>(stage + (local - h0) * 132 + 16 * part + 4 * q);
                float sq = 0.0f;
                if (EPI == 2) {
                    if (base != first_c0) {
#pragma unroll
                        for (int q = 0; q < 4; ++q)
                            res4[q] = (col + 4 * q + 4 <= N && token < M)
                                          ? *reinterpret_cast<const float4*>(ep.residual + (size_t)token * N + col + 4 * q)
                                          : make_float4(0.f, 0.f, 0.f, 0.f);
                    }
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        float4 sum = res4[q];
                        sum.x += value[q].x, sum.y += value[q].y, sum.z += value[q].z, sum.w += value[q].w;
                        if (token < M && col + 4 * q + 4 <= N) {
                            *reinterpret_cast<float4*>(ep.residual + (size_t)token * N + col + 4 * q) = sum;
                            sq += (sum.x * sum.x + sum.y * sum.y) + (sum.z * sum.z + sum.w * sum.w);
                        }
                        value[q] = make_float4(sum.x * norm4[q].x, sum.y * norm4[q].y, sum.z * norm4[q].z, sum.w * norm4[q].w);
                    }
                }
                if (token < y_rows) {
                    if (sizeof(OutT) == 2) {
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            if (col + 8 * h + 8 <= N) {
                                const float4 a = value[2 * h], b = value[2 * h + 1];
                                __nv_bfloat162 p0 = __floats2bfloat162_rn(a.x, a.y), p1 = __floats2bfloat162_rn(a.z, a.w);
                                __nv_bfloat162 p2 = __floats2bfloat162_rn(b.x, b.y), p3 = __floats2bfloat162_rn(b.z, b.w);
                                *reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(C) + (size_t)token * ldc + col + 8 * h) =
                                    make_uint4(*reinterpret_cast<uint32_t*>(&p0), *reinterpret_cast<uint32_t*>(&p1),
                                               *reinterpret_cast<uint32_t*>(&p2), *reinterpret_cast<uint32_t*>(&p3));
                            }
                        }
                    } else {
#pragma unroll
                        for (int q = 0; q < 4; ++q)
                            if (col + 4 * q + 4 <= N)
                                *reinterpret_cast<float4*>(reinterpret_cast<float*>(C) + (size_t)token * ldc + col + 4 * q) = value[q];
                    }
                }
                if (EPI == 2) {
                    // this tile's share of the token's sum of squares: its eight threads, in a fixed order
                    sq += __shfl_xor_sync(0xffffffffu, sq, 1);
                    sq += __shfl_xor_sync(0xffffffffu, sq, 2);
                    sq += __shfl_xor_sync(0xffffffffu, sq, 4);
                    if (part == 0 && token < M) ep.sumsq_out[(size_t)blockIdx.x * M + token] = sq;
                }
            }
            if (h0 + HALF < BN) named_barrier_128();  // the next half is staged where this one was read
        }
        }  // halves
        if (EPI == 2 && SWAP && !staged) {
            // this tile's share of each token's sum of squares: eight lanes add a token's 128 squares, sixteen each
            // (rotated so that the 32 lanes of a warp read 32 banks), in a fixed order.  (Tiles of up to 64 tokens only:
            // the launch gives wider tiles to this kernel only where the staged stores apply.)
            named_barrier_128();
            const float* sq_s = stage;
            const int part = tile_row & 7;
#pragma unroll 1
            for (int base = 0; base < BN; base += 16) {
                if (scatter && (uint32_t)(base >> 4) % (uint32_t)splits != rank) continue;  // another CTA's chunk
                const int j = base + (tile_row >> 3);
                float sum = 0.0f;
#pragma unroll
                for (int i = 0; i < 16; ++i) sum += sq_s[j * 132 + part * 16 + ((i + (part >> 1)) & 15)];
                sum += __shfl_xor_sync(0xffffffffu, sum, 1);
                sum += __shfl_xor_sync(0xffffffffu, sum, 2);
                sum += __shfl_xor_sync(0xffffffffu, sum, 4);
                if (part == 0 && y0 + j < M) ep.sumsq_out[(size_t)blockIdx.x * M + y0 + j] = sum;
            }
        }
    }
    if (!ok) atomicExch(error_flag, 4);
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0) gemm_stamp(ep, 5);
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, tmem_columns<BN>());
    }
}

// ---------------------------------------------------------------- many tokens: persistent kernel
// One CTA per SM walks tiles t = blockIdx.x, + gridDim.x, ... (token tile fastest, so CTAs that
// run side by side share a weight tile in L2).  Tensor memory holds two accumulators of BN
// columns: while the epilogue warps read one back, convert and store it, the MMA thread already
// fills the other with the next tile, and the TMA warp runs ahead across tile borders.
// Tried and taken out: the last wave shared out evenly (its tiles' k-blocks cut into one range per SM, partial tiles
// through a workspace, summed in the order of the ranges by the CTA that counts last).  Even with the sums left out
// the 8B shapes at 2,048 tokens gained 0 to 4 % (q, k, v 99 to 95 us, o 72 to 71, gate/up 283 to 282, down 166 to
// 160): a wave that leaves SMs idle runs its tiles faster, the products being bound by the power cap and by L2, and
// the partial tiles' way through memory cost more than that (o 90 us with them).
// The residual-and-norm epilogue of one 128 x BN tile for one warp (32 rows), with coalesced global accesses.  A
// thread holds a row of the accumulator, so touching the 32-bit stream from that layout costs a cache-line
// wavefront per row and instruction, eight times the lines' worth; measured, the epilogue then took longer than
// the tile's products.  Here 32 columns at a time go through a per-warp staging buffer in shared memory (16-byte
// slots, slot c of row r at c ^ (r % 8)) and come back with eight lanes per row, so that an instruction covers four
// rows of 128 contiguous bytes.  Needs N % 4 == 0 and 16-byte aligned stream, norm weights and output.
__device__ __forceinline__ void epilogue_residual_norm_coalesced(const Epilogue& ep, __nv_bfloat16* __restrict__ C, long ldc,
                                                                 uint32_t tmem_acc, float4* stage, int row0, int y0,
                                                                 int columns, int M, int N, int n_tile, int lane) {
    const int sub_row = lane >> 3, slot = lane & 7;  // in the coalesced layout: row 4 i + sub_row, columns 4 slot .. + 3
    float row_sq[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
    // the stream's values of a chunk, in the coalesced layout; requested one chunk ahead of their use
    auto load_chunk = [&](int c0, float4 (&res)[8]) {
        const int gc = y0 + c0 + slot * 4;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int gr = row0 + 4 * i + sub_row;
            res[i] = (c0 < columns && gr < M && gc + 4 <= N) ? *reinterpret_cast<const float4*>(ep.residual + (size_t)gr * N + gc)
                                                             : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    };
    float4 res[8], res_next[8];
    load_chunk(0, res);
#pragma unroll 1
    for (int c0 = 0; c0 < columns; c0 += 32) {
        if (y0 + c0 >= N) break;  // uniform across the warp
        const int gc = y0 + c0 + slot * 4;
        const bool col_ok = gc + 4 <= N;
        load_chunk(c0 + 32, res_next);
        const float4 w = col_ok ? *reinterpret_cast<const float4*>(ep.norm_weight + gc) : make_float4(0.f, 0.f, 0.f, 0.f);
        uint32_t r[32];
        tmem_load_32x32(tmem_acc + (uint32_t)c0, r);
        tmem_load_wait();
#pragma unroll
        for (int q = 0; q < 8; ++q)
            stage[lane * 8 + (q ^ (lane & 7))] = make_float4(__uint_as_float(r[4 * q]), __uint_as_float(r[4 * q + 1]),
                                                             __uint_as_float(r[4 * q + 2]), __uint_as_float(r[4 * q + 3]));
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int local_row = 4 * i + sub_row;
            const int gr = row0 + local_row;
            const float4 acc = stage[local_row * 8 + (slot ^ (local_row & 7))];
            float sq = 0.0f;
            if (gr < M && col_ok) {
                float4 sum = res[i];
                sum.x += acc.x, sum.y += acc.y, sum.z += acc.z, sum.w += acc.w;
                *reinterpret_cast<float4*>(ep.residual + (size_t)gr * N + gc) = sum;
                sq = (sum.x * sum.x + sum.y * sum.y) + (sum.z * sum.z + sum.w * sum.w);
                __nv_bfloat162 lo = __floats2bfloat162_rn(sum.x * w.x, sum.y * w.y), hi = __floats2bfloat162_rn(sum.z * w.z, sum.w * w.w);
                uint2 packed;
                packed.x = *reinterpret_cast<uint32_t*>(&lo);
                packed.y = *reinterpret_cast<uint32_t*>(&hi);
                *reinterpret_cast<uint2*>(C + (size_t)gr * ldc + gc) = packed;
            }
            sq += __shfl_xor_sync(0xffffffffu, sq, 1);
            sq += __shfl_xor_sync(0xffffffffu, sq, 2);
            sq += __shfl_xor_sync(0xffffffffu, sq, 4);
            row_sq[i] += sq;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) res[i] = res_next[i];
        __syncwarp();  // the staging buffer is rewritten by the next chunk
    }
    if (slot == 0) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int gr = row0 + 4 * i + sub_row;
            if (gr < M) ep.sumsq_out[(size_t)n_tile * M + gr] = row_sq[i];  // this column tile's share
        }
    }
}

template <int BN, typename OutT, int EPI>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_tcgen05_persistent_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_y,
                               const uint8_t* __restrict__ w_tiled, OutT* __restrict__ C, int M, int N, int K, long ldc,
                               Epilogue ep, int* __restrict__ error_flag) {
    using Smem = GemmSmem<BN>;
    constexpr int STAGES = Smem::stages;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = (uint64_t*)(smem + STAGES * Smem::stage_bytes);
    uint64_t* full_bar = bars;                    // [STAGES] TMA -> MMA
    uint64_t* empty_bar = bars + STAGES;          // [STAGES] MMA -> TMA
    uint64_t* acc_full = bars + 2 * STAGES;       // [2] MMA -> epilogue
    uint64_t* acc_empty = bars + 2 * STAGES + 2;  // [2] epilogue -> MMA
    uint32_t* tmem_slot = (uint32_t*)(bars + 2 * STAGES + 4);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m_tiles = (M + GEMM_BM - 1) / GEMM_BM, n_tiles = (N + BN - 1) / BN;
    const int total_tiles = m_tiles * n_tiles;
    const int num_kb = (K + GEMM_BK - 1) / GEMM_BK;
    pdl_launch_dependents();

    if (threadIdx.x == 0) {
        tma_prefetch_descriptor(&map_x);
        tma_prefetch_descriptor(&map_y);
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_addr(&full_bar[s]), 1);
            mbar_init(smem_addr(&empty_bar[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_addr(&acc_full[b]), 1);
            mbar_init(smem_addr(&acc_empty[b]), 4);  // one arrival per epilogue warp
        }
        mbar_fence_init();
    }
    if (warp == 1) {
        tmem_alloc(smem_addr(tmem_slot), 2 * tmem_columns<BN>());
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    bool ok = true;

    if (warp == 0) {
        if (elect_one()) {
            // Walks this CTA's (tile, k-block) sequence and the ring of stages with counters only: this thread's
            // issue rate bounds the kernel, and a division per k-block showed in the product's time.
            struct Cursor {
                int t, kb, stage, m_tile, n_tile;
                uint32_t round;  // how often the ring has wrapped
            };
            auto place = [&](Cursor& c) { c.m_tile = c.t % m_tiles, c.n_tile = c.t / m_tiles; };
            auto advance = [&](Cursor& c) {
                if (++c.kb == num_kb) { c.kb = 0, c.t += (int)gridDim.x; place(c); }
                if (++c.stage == STAGES) { c.stage = 0, ++c.round; }
            };
            const int row_tiles = (N + GEMM_BM - 1) / GEMM_BM;
            auto issue = [&](const Cursor& c, bool weights, bool activations) {
                const uint32_t full = smem_addr(&full_bar[c.stage]);
                const uint32_t dst = smem_addr(smem + c.stage * Smem::stage_bytes);
                if (weights && w_tiled) {
                    // BN / 128 boxes of 128 weight rows, stacked as the MMA reads them; a box past the last row
                    // tile is left out (its columns of the accumulator are never stored)
                    const int first = c.n_tile * (BN / GEMM_BM);
                    const int boxes = min(BN / GEMM_BM, row_tiles - first);
                    mbar_expect_tx(full, Smem::x_bytes + boxes * GEMM_BOX_BYTES);
                    const uint8_t* src = w_tiled + ((size_t)first * num_kb + c.kb) * GEMM_BOX_BYTES;
                    for (int b = 0; b < boxes; ++b)
                        bulk_load_1d(dst + Smem::x_bytes + b * GEMM_BOX_BYTES, src + (size_t)b * num_kb * GEMM_BOX_BYTES,
                                     GEMM_BOX_BYTES, full);
                } else if (weights) {
                    mbar_expect_tx(full, Smem::stage_bytes);
                    tma_load_2d(dst + Smem::x_bytes, &map_y, full, c.kb * GEMM_BK, c.n_tile * BN);
                }
                if (activations) tma_load_2d(dst, &map_x, full, c.kb * GEMM_BK, c.m_tile * GEMM_BM);
            };
            // The weights do not depend on the kernel before this one: the first ring of weight tiles is
            // fetched at once, and only the activation tiles wait for that kernel to finish.
            Cursor ahead{(int)blockIdx.x, 0, 0, 0, 0, 0u};
            place(ahead);
            Cursor behind = ahead;
            int head = 0;
            for (; head < STAGES && ahead.t < total_tiles; ++head) { issue(ahead, true, false); advance(ahead); }
            pdl_wait();
            for (int i = 0; i < head; ++i) { issue(behind, false, true); advance(behind); }
            while (ahead.t < total_tiles) {
                if (!mbar_wait(smem_addr(&empty_bar[ahead.stage]), (ahead.round - 1u) & 1u)) { ok = false; break; }
                issue(ahead, true, true);
                advance(ahead);
            }
        }
    } else if (warp == 1) {
        if (elect_one()) {
            constexpr uint32_t idesc = instr_desc_bf16(GEMM_BM, BN);
            int it = 0, local = 0;
            for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++local) {
                const int buf = local & 1;
                // the epilogue must have drained this accumulator (two tiles ago)
                if (local >= 2 && !mbar_wait(smem_addr(&acc_empty[buf]), (uint32_t)((local >> 1) - 1) & 1u)) { ok = false; break; }
                tc_fence_after();
                const uint32_t tmem_acc = tmem_base + (uint32_t)(buf * tmem_columns<BN>());
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (!mbar_wait(smem_addr(&full_bar[s]), (uint32_t)(it / STAGES) & 1u)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t x_addr = smem_addr(smem + s * Smem::stage_bytes);
                    const uint64_t desc_x = smem_desc_k_major_sw128(x_addr);
                    const uint64_t desc_y = smem_desc_k_major_sw128(x_addr + Smem::x_bytes);
#pragma unroll
                    for (int k = 0; k < GEMM_BK / 16; ++k)
                        mma_bf16_ss(tmem_acc, desc_x + (uint64_t)(2 * k), desc_y + (uint64_t)(2 * k), idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    mma_commit(smem_addr(&empty_bar[s]));
                }
                if (!ok) break;
                mma_commit(smem_addr(&acc_full[buf]));
            }
        }
    } else {
        const int lane_group = warp & 3;
        const int tile_row = lane_group * 32 + lane;
        pdl_wait();  // the output buffer may still be read by the kernel before this one
        // whether the residual-and-norm epilogue can take its coalesced form (whole 16-byte pieces everywhere)
        const bool coalesced = EPI == 2 && N % 4 == 0 && ldc % 4 == 0 &&
                               (((uintptr_t)ep.residual | (uintptr_t)ep.norm_weight | (uintptr_t)C) & 15) == 0;
        int local = 0;
        for (int t = blockIdx.x; t < total_tiles; t += gridDim.x, ++local) {
            const int buf = local & 1;
            const int n_tile = t / m_tiles;
            const int x0 = (t % m_tiles) * GEMM_BM, y0 = n_tile * BN;
            const int x_row = x0 + tile_row;
            // EPI 2: the stream's values are fetched two chunks of 16 columns ahead of their use, the first two
            // before this tile's products are done
            ResidualChunk cur, next, after;
            if (EPI == 2 && !coalesced) {
                load_residual_chunk(ep, x_row, y0, M, N, cur);
                load_residual_chunk(ep, x_row, y0 + 16, M, N, next);
            }
            if (EPI == 2 && coalesced) {
                // while this tile's products run: ask for its part of the stream to be brought into L2 (the weights
                // that stream through in between push it out); a line of 128 bytes per request, a row per lane
                const int gr = x0 + lane_group * 32 + lane;
                if (gr < M) {
                    const char* line = reinterpret_cast<const char*>(ep.residual + (size_t)gr * N + y0);
                    const int bytes = min(BN, N - y0) * 4;
                    for (int off = 0; off < bytes; off += 128) asm volatile("prefetch.global.L2 [%0];" ::"l"(line + off));
                }
            }
            if (!mbar_wait(smem_addr(&acc_full[buf]), (uint32_t)(local >> 1) & 1u)) { ok = false; break; }
            tc_fence_after();
            const uint32_t tmem_acc = tmem_base + (uint32_t)(buf * tmem_columns<BN>()) + ((uint32_t)(lane_group * 32) << 16);
            if (EPI == 2 && sizeof(OutT) == 2 && coalesced) {
                float4* stage = reinterpret_cast<float4*>(smem + STAGES * Smem::stage_bytes + Smem::barrier_bytes) + lane_group * 256;
                epilogue_residual_norm_coalesced(ep, reinterpret_cast<__nv_bfloat16*>(C), ldc, tmem_acc, stage, x0 + lane_group * 32,
                                                 y0, BN, M, N, n_tile, lane);
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_addr(&acc_empty[buf]));
                continue;
            }
            const float my_scale = (ep.row_sumsq && x_row < M) ? row_scale_of(ep, x_row, M) : 1.0f;
            float row_sq = 0.0f;
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 16) {
                if (y0 + c0 >= N) break;  // uniform across the warp
                float4 w4[4];
                if (EPI == 2) {
                    if (c0 > 0) { cur = next; next = after; }
                    load_residual_chunk(ep, x_row, c0 + 32 < BN ? y0 + c0 + 32 : N, M, N, after);
                    if (cur.vector) {
#pragma unroll
                        for (int q4 = 0; q4 < 4; ++q4) w4[q4] = reinterpret_cast<const float4*>(ep.norm_weight + y0 + c0)[q4];
                    }
                }
                const bool vector = EPI == 2 && cur.vector;
                uint32_t r[16];
                tmem_load_32x16(tmem_acc + (uint32_t)c0, r);
                tmem_load_wait();
                if (x_row >= M) continue;
                float v[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) v[j] = __uint_as_float(r[j]) * my_scale;
                if (EPI == 2) {
                    float* res = ep.residual + (size_t)x_row * N + y0 + c0;
                    OutT* dst = C + (size_t)x_row * ldc + y0 + c0;
                    if (vector && sizeof(OutT) == 2 && (((uintptr_t)dst & 15) == 0)) {
                        uint32_t packed[8];
#pragma unroll
                        for (int q4 = 0; q4 < 4; ++q4) {
                            float4 sum = cur.r[q4];
                            const float4 w = w4[q4];
                            sum.x += v[4 * q4]; sum.y += v[4 * q4 + 1]; sum.z += v[4 * q4 + 2]; sum.w += v[4 * q4 + 3];
                            reinterpret_cast<float4*>(res)[q4] = sum;
                            row_sq += (sum.x * sum.x + sum.y * sum.y) + (sum.z * sum.z + sum.w * sum.w);
                            __nv_bfloat162 lo = __floats2bfloat162_rn(sum.x * w.x, sum.y * w.y), hi = __floats2bfloat162_rn(sum.z * w.z, sum.w * w.w);
                            packed[2 * q4] = *reinterpret_cast<uint32_t*>(&lo);
                            packed[2 * q4 + 1] = *reinterpret_cast<uint32_t*>(&hi);
                        }
                        uint4* out = reinterpret_cast<uint4*>(dst);
                        out[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                        out[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            if (y0 + c0 + j < N) {
                                const float sum = res[j] + v[j];
                                res[j] = sum;
                                row_sq += sum * sum;
                                dst[j] = from_f32<OutT>(sum * ep.norm_weight[y0 + c0 + j]);
                            }
                        }
                    }
                } else if (EPI == 1) {
                    // columns y0 + c0 .. + 15 are 8 gate rows then their 8 up rows: 8 outputs at (y0 + c0) / 2
                    OutT* dst = C + (size_t)x_row * ldc + ((y0 + c0) >> 1);
                    if (y0 + c0 + 16 <= N && sizeof(OutT) == 2 && (((uintptr_t)dst & 15) == 0)) {
                        uint32_t packed[4];
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            __nv_bfloat162 pair = __floats2bfloat162_rn(silu_mul(v[2 * j], v[2 * j + 8]), silu_mul(v[2 * j + 1], v[2 * j + 9]));
                            packed[j] = *reinterpret_cast<uint32_t*>(&pair);
                        }
                        *reinterpret_cast<uint4*>(dst) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                    } else {
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            if (y0 + c0 + j + 8 < N) dst[j] = from_f32<OutT>(silu_mul(v[j], v[j + 8]));
                    }
                } else {
                    OutT* dst = C + (size_t)x_row * ldc + y0 + c0;
                    const bool full = (y0 + c0 + 16 <= N) && (((uintptr_t)dst & 15) == 0);
                    if (full && sizeof(OutT) == 2) {
                        uint32_t packed[8];
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            __nv_bfloat162 pair = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
                            packed[j] = *reinterpret_cast<uint32_t*>(&pair);
                        }
                        uint4* out = reinterpret_cast<uint4*>(dst);
                        out[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                        out[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
                    } else if (full && sizeof(OutT) == 4) {
                        float4* out = reinterpret_cast<float4*>(dst);
#pragma unroll
                        for (int j = 0; j < 4; ++j) out[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (y0 + c0 + j < N) dst[j] = from_f32<OutT>(v[j]);
                    }
                }
            }
            if (EPI == 2 && x_row < M) ep.sumsq_out[(size_t)n_tile * M + x_row] = row_sq;  // this column tile's share
            // this warp has read its lanes of the accumulator: hand it back to the MMA thread
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_addr(&acc_empty[buf]));
        }
    }
    if (!ok) atomicExch(error_flag, 4);
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 2 * tmem_columns<BN>());
    }
}

static int sm_count() {
    static const int count = [] {
        int device = 0, value = 0;
        if (cudaGetDevice(&device) != cudaSuccess) return 0;
        if (cudaDeviceGetAttribute(&value, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return 0;
        return value;
    }();
    return count;
}
template <int BN, typename OutT, int EPI>
static int launch_persistent(const void* A, const void* W, bool tiled, void* C, int M, int N, int K, long lda, long ldc,
                             const Epilogue& ep, int* error_flag, cudaStream_t stream) {
    using Smem = GemmSmem<BN>;
    CUtensorMap map_a, map_w;
    if (!tmap::bf16_2d_sw128(&map_a, A, M, K, lda, GEMM_BM, GEMM_BK)) return KIRAI_ERR_BAD_ALIGN;
    if (tiled) map_w = map_a;  // not read: the boxes are fetched by address
    else if (!tmap::bf16_2d_sw128(&map_w, W, N, K, K, BN, GEMM_BK)) return KIRAI_ERR_BAD_ALIGN;
    if (tiled && ((uintptr_t)W & 15)) return KIRAI_ERR_BAD_ALIGN;
    const long tiles = (long)((M + GEMM_BM - 1) / GEMM_BM) * ((N + BN - 1) / BN);
    const int sms = sm_count();
    if (sms <= 0) return KIRAI_ERR_UNSUPPORTED;  // the device did not say how many SMs it has
    const unsigned grid = (unsigned)(tiles < sms ? tiles : sms);
    auto kernel = gemm_tcgen05_persistent_kernel<BN, OutT, EPI>;
    const int smem_bytes = Smem::total(1) + (EPI == 2 ? 4 * 32 * 32 * 4 : 0);  // + the epilogue's staging buffers
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
    if (err != cudaSuccess) return (int)err;
    return launch_pdl(kernel, dim3(grid), dim3(GEMM_THREADS), (size_t)smem_bytes, stream, 1u, map_a, map_w,
                      tiled ? (const uint8_t*)W : (const uint8_t*)nullptr, (OutT*)C, M, N, K, ldc, ep, error_flag);
}

static bool deep_rings() {
    static const bool on = [] {
        const char* text = getenv("KIRAI_GEMM_DEEP");
        return !(text && text[0] == '0');
    }();
    return on;
}

// How many clusters of (1, 1, cluster_z) CTAs of `kernel` the device can hold at once, by its own account; asked once
// per kernel, shared-memory size and cluster size.  A failed query counts as "all fit".
template <typename Kernel>
static long max_resident_clusters(Kernel kernel, int smem_bytes, int cluster_z) {
    static std::mutex mutex;
    static std::map<std::tuple<const void*, int, int>, long> known;
    const auto key = std::make_tuple((const void*)kernel, smem_bytes, cluster_z);
    std::lock_guard<std::mutex> lock(mutex);
    auto found = known.find(key);
    if (found != known.end()) return found->second;
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(1, 1, (unsigned)cluster_z);
    config.blockDim = dim3(GEMM_THREADS);
    config.dynamicSmemBytes = (size_t)smem_bytes;
    cudaLaunchAttribute attribute;
    attribute.id = cudaLaunchAttributeClusterDimension;
    attribute.val.clusterDim.x = 1, attribute.val.clusterDim.y = 1, attribute.val.clusterDim.z = (unsigned)cluster_z;
    config.attrs = &attribute;
    config.numAttrs = 1;
    int clusters = 0;
    long answer = 1L << 40;
    if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &config) == cudaSuccess && clusters > 0) answer = clusters;
    else cudaGetLastError();  // a failed query leaves no error behind
    known.emplace(key, answer);
    return answer;
}

template <int BN, bool SWAP, typename OutT, int EPI>
static int launch_config(const void* A, const void* W, bool tiled, void* C, int M, int N, int K, long lda, long ldc,
                         int splits, const Epilogue& ep, int* error_flag, cudaStream_t stream) {
    using Smem = GemmSmem<BN, false, true>;
    CUtensorMap map_x, map_y;
    const void* x_ptr = SWAP ? W : A;
    const void* y_ptr = SWAP ? A : W;
    const uint64_t x_rows = SWAP ? N : M, y_rows = SWAP ? M : N;
    const uint64_t x_stride = SWAP ? K : lda, y_stride = SWAP ? lda : K;
    if (tiled && (!SWAP || ((uintptr_t)W & 15))) return KIRAI_ERR_BAD_ALIGN;
    if (!tmap::bf16_2d_sw128(&map_y, y_ptr, y_rows, K, y_stride, BN, GEMM_BK)) return KIRAI_ERR_BAD_ALIGN;
    if (tiled) map_x = map_y;  // not read: the boxes are fetched by address
    else if (!tmap::bf16_2d_sw128(&map_x, x_ptr, x_rows, K, x_stride, GEMM_BM, GEMM_BK)) return KIRAI_ERR_BAD_ALIGN;
    const int total_k_blocks = (K + GEMM_BK - 1) / GEMM_BK;
    if (splits < 1) splits = 1;
    int max_splits = Smem::max_splits;
    if constexpr (BN == 128) max_splits = GemmSmem<BN, true, true>::max_splits;  // (tiles of 128 tokens split only with the long ring)
    if (splits > max_splits) splits = max_splits;  // slots in the first CTA's shared memory
    if (splits > total_k_blocks) splits = total_k_blocks;
    const uint8_t* boxes = tiled ? (const uint8_t*)W : (const uint8_t*)nullptr;
    // The CTAs of a tile are a cluster, and a cluster's CTAs must find room in one GPC at the same time: 48 clusters of
    // 3 one-per-SM CTAs do not all fit a B200 (39 did; the other 9 started 7 us later, when the first had finished, and
    // the q, k, v product of the 8B shape took 15 us in place of 9).  So the split count goes down until the device
    // says that all clusters of the launch can be resident together.
    for (;; --splits) {
        const int per_split = (total_k_blocks + splits - 1) / splits;
        const int used = (total_k_blocks + per_split - 1) / per_split;
        dim3 grid((unsigned)((x_rows + GEMM_BM - 1) / GEMM_BM), (unsigned)((y_rows + BN - 1) / BN), (unsigned)used);
        if (grid.y > 65535) return KIRAI_ERR_BAD_SIZE;
        const long clusters = (long)grid.x * grid.y;
        if constexpr (BN <= 128) {  // (tiles of 256 tokens have one configuration: four stages, one CTA per SM)
            // no more CTAs than SMs: one CTA per SM with the long ring (KIRAI_GEMM_DEEP=0 keeps the short one, to compare)
            if (clusters * used <= sm_count() && deep_rings()) {
                using Deep = GemmSmem<BN, true, true>;
                auto kernel = gemm_tcgen05_kernel<BN, SWAP, OutT, EPI, true>;
                cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Deep::total(Deep::max_splits));
                if (err != cudaSuccess) return (int)err;
                if (used > 1 && splits > 1 && clusters > max_resident_clusters(kernel, Deep::total(used), used)) continue;
                return launch_pdl(kernel, grid, dim3(GEMM_THREADS), (size_t)Deep::total(used), stream, (unsigned)used, map_x,
                                  map_y, boxes, (OutT*)C, M, N, K, ldc, per_split, used, ep, error_flag);
            }
        }
        if (used > Smem::max_splits) continue;  // (tiles of 128 tokens split only with the long ring)
        auto kernel = gemm_tcgen05_kernel<BN, SWAP, OutT, EPI, false>;
        cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem::total(Smem::max_splits));
        if (err != cudaSuccess) return (int)err;
        // launches of more CTAs than SMs run in waves anyway; only a launch meant to be one wave is fitted
        if (used > 1 && splits > 1 && clusters * used <= 2L * sm_count() &&
            clusters > max_resident_clusters(kernel, Smem::total(used), used))
            continue;
        return launch_pdl(kernel, grid, dim3(GEMM_THREADS), (size_t)Smem::total(used), stream, (unsigned)used, map_x, map_y,
                          boxes, (OutT*)C, M, N, K, ldc, per_split, used, ep, error_flag);
    }
}

// Split count for the swapped (few tokens) case, which is bound by the weight
// stream: enough CTAs that every SM streams (two of these CTAs fit an SM), each
// split at least 8 k-blocks long, and no more splits than the first CTA has slots.
static int choose_splits(int M, int N, int K) {
    const int x_tiles = (N + GEMM_BM - 1) / GEMM_BM;
    const int max_splits = 4;
    const int k_blocks = (K + GEMM_BK - 1) / GEMM_BK;
    // about one CTA per SM (a few SMs fewer, so that a launch fits one wave whatever the tile count is); with more
    // than 32 tokens a CTA with slots for 3 or 4 partial tiles fills an SM by itself and fewer, longer CTAs measured
    // faster: three quarters of the SMs
    const int sms = sm_count() > 0 ? sm_count() : 148;
    const int target = M <= 32 ? sms - 4 : 3 * sms / 4 + 1;
    int splits = (2 * target + x_tiles) / (2 * x_tiles);  // target / x_tiles, rounded
    if (splits > max_splits) splits = max_splits;
    while (splits > 1 && k_blocks / splits < 8) --splits;
    return splits < 1 ? 1 : splits;
}

// Whether the epilogue of the weight-streaming kernel can store through shared memory (its `staged` condition), which
// tiles of 128 tokens need.
static bool streams_wide_tiles(const void* C, long ldc, size_t element, int N, int epi, const Epilogue& ep) {
    if (((uintptr_t)C & 15) != 0 || (ldc * (long)element) % 16 != 0) return false;
    if (epi == 2) return N % 8 == 0 && (((uintptr_t)ep.residual | (uintptr_t)ep.norm_weight) & 15) == 0;
    return epi == 1 ? N % 16 == 0 : N % 8 == 0;
}

template <typename OutT, int EPI>
static int gemm_dispatch(const void* A, const void* W, bool tiled, void* C, int M, int N, int K, long lda, long ldc,
                         int splits, const Epilogue& ep, int* error_flag, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0) return KIRAI_ERR_BAD_SIZE;
    if (K % 8 != 0 || lda % 8 != 0) return KIRAI_ERR_BAD_ALIGN;  // TMA needs 16-byte row strides
    if (EPI == 1 && N % 16 != 0) return KIRAI_ERR_BAD_SIZE;      // whole groups of 8 gate + 8 up rows
    if (splits <= 0) splits = M <= 256 ? choose_splits(M, N, K) : 1;
#define KIRAI_GEMM_CASE(BN, SWAP) \
    return launch_config<BN, SWAP, OutT, EPI>(A, W, tiled, C, M, N, K, lda, ldc, splits, ep, error_flag, stream)
    if (M <= 16) KIRAI_GEMM_CASE(16, true);
    if (M <= 32) KIRAI_GEMM_CASE(32, true);
    if (M <= 64) KIRAI_GEMM_CASE(64, true);
    // 65 to 128 tokens: still bound by the weight stream, which the many-token kernel below leaves to 16 to 96 CTAs
    // (230 us for the four products of an 8B layer against 66 us at 64 tokens).  The weight-streaming kernel takes
    // them where its staged stores apply (they do for every 16-byte aligned output).
    if (M <= 128 && streams_wide_tiles(C, ldc, sizeof(OutT), N, EPI, ep)) KIRAI_GEMM_CASE(128, true);
    // 129 to 256 tokens: tiles of 256 tokens fill an SM each, so only launches of no more tiles than SMs (the 8B shape's
    // gate/up product, 192 tiles, ran as two waves: 99 us against 59 us in the many-token kernel; its down product, 32
    // tiles split three ways, 38 against 67)
    const bool one_wave = (N + GEMM_BM - 1) / GEMM_BM <= sm_count();
    if (M <= 256 && one_wave && streams_wide_tiles(C, ldc, sizeof(OutT), N, EPI, ep)) KIRAI_GEMM_CASE(256, true);
    if (M <= 256 && EPI == 2 && N % 8 == 0 && (M <= 128 || one_wave)) return KIRAI_ERR_BAD_ALIGN;  // see kirai_gemm_bf16_residual_parts
#undef KIRAI_GEMM_CASE
    if (N <= 128) return launch_persistent<128, OutT, EPI>(A, W, tiled, C, M, N, K, lda, ldc, ep, error_flag, stream);
    return launch_persistent<256, OutT, EPI>(A, W, tiled, C, M, N, K, lda, ldc, ep, error_flag, stream);
}

// Split count that the entry points pick for splits <= 0.
KIRAI_EXPORT int kirai_gemm_bf16_auto_splits(int M, int N, int K) { return M <= 256 ? choose_splits(M, N, K) : 1; }

// How many parts the residual-and-norm form writes into sumsq_out for a product of this shape.
KIRAI_EXPORT int kirai_gemm_bf16_residual_parts(int M, int N) {
    // (65 to 256 tokens go to the weight-streaming kernel where whole 16-byte pieces can be stored, above 128 tokens
    // only launches of no more tiles than SMs; form 3 with such a
    // shape and buffers that are not 16-byte aligned is refused rather than sent to the kernel with the other layout)
    if (M <= 64 || (M <= 128 && N % 8 == 0) || (M <= 256 && N % 8 == 0 && (N + GEMM_BM - 1) / GEMM_BM <= sm_count()))
        return (N + GEMM_BM - 1) / GEMM_BM;
    return N <= 128 ? 1 : (N + 255) / 256;
}

// Bytes of the tiled form of a [N, K] weight matrix.
KIRAI_EXPORT long kirai_gemm_bf16_tiled_bytes(int N, int K) {
    return (long)((N + GEMM_BM - 1) / GEMM_BM) * ((K + GEMM_BK - 1) / GEMM_BK) * GEMM_BOX_BYTES;
}

// Measurements: while a buffer is set, every launch of the streaming kernel writes its CTAs' clock stamps (see
// gemm_stamp) to the next 8 * 1,024 words of it.  Null (the default) switches the stamps off.
static unsigned long long* g_gemm_stamps = nullptr;
KIRAI_EXPORT void kirai_gemm_bf16_set_stamps(unsigned long long* buffer) { g_gemm_stamps = buffer; }

// The one entry point of the tensor-core product, A[M, K] (row stride lda) times W[N, K] transposed.
//   tiled:  W is in the tiled form described at the top of this file, else row-major.
//   form 0: C[M, N] bf16.  1: C[M, N] float.  2: C[M, N / 2] = silu(gate) * up, W's rows in groups of 8 gate rows
//           followed by their 8 up rows.  3: residual[M, N] (float, in place) += product, C[M, N] =
//           bf16(residual * norm_weight[n]) and sumsq_out[parts][M] = each column tile's share of sum_n residual^2.
//   row_sumsq (forms 0-2, may be null): the rows of A were left unscaled by an RMSNorm; row m of the product is
//           multiplied by 1 / sqrt(sum_p row_sumsq[p][m] / row_count + row_eps).
//   splits <= 0 picks the split-K count itself (at most 4).
KIRAI_EXPORT int kirai_gemm_bf16_general(const void* A, const void* W, int tiled, void* C, int M, int N, int K, long lda,
                                         long ldc, int splits, int form, const float* row_sumsq, int row_parts,
                                         float row_count, float row_eps, float* residual, const float* norm_weight,
                                         float* sumsq_out, int* error_flag, cudaStream_t stream) {
    Epilogue ep{row_sumsq, row_sumsq ? row_parts : 0, row_count, row_eps, nullptr, nullptr, nullptr, g_gemm_stamps};
    if (g_gemm_stamps) g_gemm_stamps += 8 * 1024;  // the next launch's stamps follow (up to 1,024 CTAs a launch)
    if (row_sumsq && row_parts <= 0) return KIRAI_ERR_BAD_SIZE;
    switch (form) {
        case 0: return gemm_dispatch<bf16, 0>(A, W, tiled != 0, C, M, N, K, lda, ldc, splits, ep, error_flag, stream);
        case 1: return gemm_dispatch<float, 0>(A, W, tiled != 0, C, M, N, K, lda, ldc, splits, ep, error_flag, stream);
        case 2: return gemm_dispatch<bf16, 1>(A, W, tiled != 0, C, M, N, K, lda, ldc, splits, ep, error_flag, stream);
        case 3:
            if (!residual || !norm_weight || !sumsq_out || row_sumsq) return KIRAI_ERR_BAD_SIZE;
            ep.residual = residual, ep.norm_weight = norm_weight, ep.sumsq_out = sumsq_out;
            return gemm_dispatch<bf16, 2>(A, W, tiled != 0, C, M, N, K, lda, (long)N, splits, ep, error_flag, stream);
    }
    return KIRAI_ERR_BAD_SIZE;
}
