// Several weight-streaming products of a decode step as ONE persistent kernel.
//
// A decode step of a few tokens is bound by the weight stream, and a layer's products follow each other
// (output projection, gate/up, down, the next layer's q/k/v).  Launched one by one, every product pays its own
// ramp: its CTAs become resident only when the kernel before leaves the SMs, the first copies need a round trip to
// memory, and at the end the stream stops while the last tiles are reduced and stored.  Measured on the 8B layer
// sizes that is 4 to 7 us for each of the three small products, a sixth of a layer's time.  Here the products are
// phases of one kernel whose CTAs stay resident, one per SM, and whose load thread never stops: while a phase's last
// tiles are reduced and the CTAs wait for each other, the ring of every SM already fills with the next phase's
// weights (weights depend on nothing), and only the small activation tiles wait for the phase before.
//
// Work split.  Weights come in the tiled form of gemm_tcgen05.cu (boxes of 128 rows x 64 columns, 16 KB each, box
// (row tile, k block) at index row_tile * k_blocks + k_block), so a phase is a row of `row_tiles * k_blocks` boxes
// and CTA c of G takes the boxes [total * c / G, total * (c + 1) / G): a contiguous stretch of memory, the same number
// of bytes for every SM whatever the shape is.  Operands are swapped as in the streaming kernel (weight rows fill the
// 128 rows of the MMA, the tokens are its N).  A CTA's stretch covers whole row tiles and at most two pieces of
// tiles (at its begin and at its end).  A piece is written as a 32-bit partial tile into one of the CTA's two slots of
// a workspace; the CTA that arrives last at a tile (a counter per split tile) adds the pieces in the order of the
// CTAs, so the sum does not depend on who came last, and runs the epilogue.
//
// Phases.  Phase p + 1 reads what phase p wrote (activations through TMA, the residual stream and the norms'
// sums of squares through plain loads), so it may start its products only when every tile of phase p is stored:
// a counter per phase, incremented after a fence by each finished tile, polled with acquire loads.  All waits are
// bounded; one that runs out sets the device error word and the CTA winds down.  Data written inside the kernel is
// read back past L1 (ld.global.cg, or TMA after a proxy fence).
//
// Where it stands.  Correct against the single launches and against 32-bit arithmetic (tests), but slower: on the 8B
// layer sizes at 8 tokens the four phases take 22.5, 43.3, 34.8 and 14.6 us by the kernel's own clock stamps (116 us)
// against 75 us for the four single launches inside a captured step, so the model's steps do not use it unless
// ops.chain_products is set.  The stamps say why.  (1) Equal stretches do not end together: an SM's share of the
// memory system is its ring (176 KB) over the latency it sees, 3 to 4.7 us under load, so SMs differ by a quarter
// either way and a phase ends with the slowest (gate/up: the first CTA has issued its last box after 20.5 us, the last
// after 31.7).  (2) From a phase's last product to its counter pass 5 to 9 us (partial tiles through L2, two fences, two
// atomics, the reads of up to six pieces), the ring holds 4 us of stream, and memory idles for the rest, four times a
// layer.  (3) Asking for boxes to be brought into L2 ahead of the ring (24 boxes an SM) to bridge that made the chain
// slower still (134 us): requests and copies then fetch twice.  What would be needed: work handed out in small grains
// as CTAs finish, and a second buffer beside shared memory (tensor memory holds 240 KB more).
//
// The kernel needs its CTAs resident together (they wait for each other): the grid is at most one CTA per SM, each
// CTA asks for more than half an SM's shared memory, and nothing that is launched later can take an SM before all
// of them have started (the dependent launch is released by the last CTA's start).  The last CTA to leave puts the
// counters back to zero for the next launch.
#include <cstdlib>

#include "sm100.cuh"
#include "tensor_map.cuh"

using namespace sm100;

#define CHAIN_MAX_PHASES 6
#define CHAIN_THREADS 192
#define CHAIN_BM 128
#define CHAIN_BK 64
#define CHAIN_BOX_BYTES (CHAIN_BM * CHAIN_BK * 2)
#define CHAIN_POLL_LIMIT (1u << 22)

struct ChainPhase {
    const uint8_t* boxes;     // tiled weights [row_tiles][k_blocks][16 KB]
    void* out;                // C
    const float* row_sumsq;   // forms 0-2: parts of the input rows' sums of squares (an RMSNorm left them unscaled), or null
    float* residual;          // form 3: the 32-bit stream [M, N], updated in place
    const float* norm_weight; // form 3: [N]
    float* sumsq_out;         // form 3: [row_tiles][M]
    long ldc;
    long total_boxes;
    int N, K, form;           // form 0: bf16 C[M, N]; 1: float C[M, N]; 2: C[M, N / 2] = silu(gate) * up; 3: residual and next norm
    int row_tiles, k_blocks, row_parts;
    float row_count, row_eps;
};

struct ChainArgs {
    ChainPhase phase[CHAIN_MAX_PHASES];
    int phases, M;
    float* partial;   // [grid][2][BN][128]
    int* counters;    // arrive[grid], then done[CHAIN_MAX_PHASES], then one exit counter
    int* error_flag;
    unsigned long long* stamps;  // null, or [grid][CHAIN_MAX_PHASES][4] clock stamps (ns) for measurements: see chain_stamp
};

// Clock stamps of one CTA and phase, written only when a buffer is given: 0 the phase before is complete (its
// activations may be read), 1 the load thread has issued this phase's last box, 2 the epilogue has the last piece
// of this phase out of tensor memory, 3 this CTA's last tile (or piece) of the phase is stored and counted.
__device__ __forceinline__ void chain_stamp(const ChainArgs& args, int cta, int phase, int which) {
    if (args.stamps) {
        unsigned long long now;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
        args.stamps[((size_t)cta * CHAIN_MAX_PHASES + phase) * 4 + which] = now;
    }
}

struct ChainMaps {
    CUtensorMap map[CHAIN_MAX_PHASES];  // the activations of each phase, [M, K] in boxes of [BN, 64]
};

template <int BN>
struct ChainSmem {
    static constexpr int stage_bytes = CHAIN_BOX_BYTES + BN * CHAIN_BK * 2;
    static constexpr int stages = (200 * 1024) / stage_bytes;
    static constexpr int barrier_bytes = 2048;  // barriers [0, 256), flags [256, 272), row scales [512, 768), partial sums of squares [1024, 2048)
    static_assert((2 * stages + 4) * 8 + 4 <= 256, "barriers must end before the flags");
    static_assert(4 * BN * 4 <= 1024, "four warps' sums of squares must fit");
    static constexpr int total = stages * stage_bytes + barrier_bytes + 1024;  // + slack to align the base to 1024 bytes
    static constexpr int tmem_columns = 2 * BN < 32 ? 32 : 2 * BN;
};

__device__ __forceinline__ int ld_acquire(const int* address) {
    int value;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(value) : "l"(address) : "memory");
    return value;
}
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }
__device__ __forceinline__ void epilogue_barrier() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// Waits until `*counter` has reached `target` (every tile of a phase is stored).  Bounded.
__device__ __forceinline__ bool wait_counter(const int* counter, int target) {
    for (uint32_t spin = 0; spin < CHAIN_POLL_LIMIT; ++spin) {
        if (ld_acquire(counter) >= target) return true;
        if (spin > 16) __nanosleep(spin > 1024 ? 200 : 40);
    }
    return false;
}

__device__ __forceinline__ long chain_range_begin(long total, int cta, int grid) { return total * cta / grid; }
// The CTA whose stretch holds box `box`.
__device__ __forceinline__ int chain_owner(long box, long total, int grid) { return (int)(((box + 1) * grid + total - 1) / total) - 1; }

__device__ __forceinline__ float chain_silu_mul(float gate, float up) { return __fdividef(gate * up, 1.0f + __expf(-gate)); }

template <int BN>
__global__ void __launch_bounds__(CHAIN_THREADS, 1)
gemm_chain_kernel(const __grid_constant__ ChainMaps maps, const __grid_constant__ ChainArgs args) {
    using Smem = ChainSmem<BN>;
    constexpr int STAGES = Smem::stages;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* tail = smem + STAGES * Smem::stage_bytes;
    uint64_t* bars = (uint64_t*)tail;
    uint64_t* full_bar = bars;                    // [STAGES] copies -> MMA
    uint64_t* empty_bar = bars + STAGES;          // [STAGES] MMA -> copies
    uint64_t* acc_full = bars + 2 * STAGES;       // [2] MMA -> epilogue
    uint64_t* acc_empty = bars + 2 * STAGES + 2;  // [2] epilogue -> MMA
    uint32_t* tmem_slot = (uint32_t*)(bars + 2 * STAGES + 4);
    int* flag_s = (int*)(tail + 256);
    float* scale_s = (float*)(tail + 512);   // [BN]
    float* sumsq_s = (float*)(tail + 1024);  // [4][BN]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int G = (int)gridDim.x, cta = (int)blockIdx.x;
    const int M = args.M, P = args.phases;
    int* arrive = args.counters;
    int* done = args.counters + G;
    int* exit_counter = args.counters + G + CHAIN_MAX_PHASES;
    pdl_launch_dependents();  // what follows in the stream may set itself up; it waits for this whole grid before it reads

    if (threadIdx.x == 0) {
        for (int p = 0; p < P; ++p) tma_prefetch_descriptor(&maps.map[p]);
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
        tmem_alloc(smem_addr(tmem_slot), Smem::tmem_columns);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    bool ok = true;

    if (warp == 0) {
        if (elect_one()) {
            uint32_t issued = 0;  // stages issued so far, over all phases
            auto slot_free = [&](uint32_t n) {  // the stage that issue number n takes has been read by the MMAs
                if (n < (uint32_t)STAGES) return true;
                return mbar_wait(smem_addr(&empty_bar[n % STAGES]), ((n / STAGES) & 1u) ^ 1u);
            };
            auto issue_weights = [&](uint32_t n, const ChainPhase& ph, long box) {
                const uint32_t full = smem_addr(&full_bar[n % STAGES]);
                mbar_expect_tx(full, Smem::stage_bytes);
                bulk_load_1d(smem_addr(smem + (n % STAGES) * Smem::stage_bytes), ph.boxes + (size_t)box * CHAIN_BOX_BYTES,
                             CHAIN_BOX_BYTES, full);
            };
            auto issue_activations = [&](uint32_t n, int p, const ChainPhase& ph, long box) {
                const uint32_t full = smem_addr(&full_bar[n % STAGES]);
                const int kb = (int)(box % ph.k_blocks);
                tma_load_2d(smem_addr(smem + (n % STAGES) * Smem::stage_bytes) + CHAIN_BOX_BYTES, &maps.map[p], full, kb * CHAIN_BK, 0);
            };
            long pre = 0;  // boxes of the coming phase whose weights are already on their way
            {
                const ChainPhase& first = args.phase[0];
                const long b0 = chain_range_begin(first.total_boxes, cta, G), b1 = chain_range_begin(first.total_boxes, cta + 1, G);
                pre = b1 - b0 < STAGES ? b1 - b0 : STAGES;
                for (long i = 0; i < pre; ++i) issue_weights(issued + (uint32_t)i, first, b0 + i);
            }
            for (int p = 0; p < P && ok; ++p) {
                const ChainPhase& ph = args.phase[p];
                const long b0 = chain_range_begin(ph.total_boxes, cta, G), b1 = chain_range_begin(ph.total_boxes, cta + 1, G);
                // the activations are what the kernel before wrote (first phase) or what the phase before stored
                if (p == 0) pdl_wait();
                else if (!wait_counter(done + (p - 1), args.phase[p - 1].row_tiles)) { ok = false; break; }
                fence_proxy_async_all();  // the copies below read, through the async proxy, what other CTAs stored
                chain_stamp(args, cta, p, 0);
                for (long i = 0; i < pre; ++i) issue_activations(issued + (uint32_t)i, p, ph, b0 + i);
                for (long i = pre; i < b1 - b0; ++i) {
                    if (!slot_free(issued + (uint32_t)i)) { ok = false; break; }
                    issue_weights(issued + (uint32_t)i, ph, b0 + i);
                    issue_activations(issued + (uint32_t)i, p, ph, b0 + i);
                }
                if (!ok) break;
                chain_stamp(args, cta, p, 1);
                issued += (uint32_t)(b1 - b0);
                pre = 0;
                if (p + 1 < P) {  // the next phase's weights depend on nothing: they follow at once
                    const ChainPhase& next = args.phase[p + 1];
                    const long n0 = chain_range_begin(next.total_boxes, cta, G), n1 = chain_range_begin(next.total_boxes, cta + 1, G);
                    const long ahead = n1 - n0 < STAGES ? n1 - n0 : STAGES;
                    for (; pre < ahead; ++pre) {
                        if (!slot_free(issued + (uint32_t)pre)) { ok = false; break; }
                        issue_weights(issued + (uint32_t)pre, next, n0 + pre);
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (elect_one()) {
            constexpr uint32_t idesc = instr_desc_bf16(CHAIN_BM, BN);
            uint32_t consumed = 0, segments = 0;
            for (int p = 0; p < P && ok; ++p) {
                const ChainPhase& ph = args.phase[p];
                long b = chain_range_begin(ph.total_boxes, cta, G);
                const long b1 = chain_range_begin(ph.total_boxes, cta + 1, G);
                while (b < b1 && ok) {
                    const long tile_end = (b / ph.k_blocks + 1) * ph.k_blocks;
                    const long end = tile_end < b1 ? tile_end : b1;
                    const uint32_t buf = segments & 1u;
                    // the epilogue must have read this accumulator (two pieces ago)
                    if (segments >= 2 && !mbar_wait(smem_addr(&acc_empty[buf]), ((segments >> 1) - 1u) & 1u)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t tmem_acc = tmem_base + buf * (uint32_t)BN;
                    for (long box = b; box < end; ++box, ++consumed) {
                        const uint32_t s = consumed % STAGES;
                        if (!mbar_wait(smem_addr(&full_bar[s]), (consumed / STAGES) & 1u)) { ok = false; break; }
                        tc_fence_after();
                        const uint32_t x_addr = smem_addr(smem + s * Smem::stage_bytes);
                        const uint64_t desc_x = smem_desc_k_major_sw128(x_addr);
                        const uint64_t desc_y = smem_desc_k_major_sw128(x_addr + CHAIN_BOX_BYTES);
#pragma unroll
                        for (int k = 0; k < CHAIN_BK / 16; ++k)
                            mma_bf16_ss(tmem_acc, desc_x + (uint64_t)(2 * k), desc_y + (uint64_t)(2 * k), idesc, (box > b || k > 0) ? 1u : 0u);
                        mma_commit(smem_addr(&empty_bar[s]));
                    }
                    if (!ok) break;
                    mma_commit(smem_addr(&acc_full[buf]));
                    ++segments;
                    b = end;
                }
            }
        }
    } else {
        const int lane_group = warp & 3;  // tensor-memory lanes 32 (warp % 4) ..
        const int tile_row = lane_group * 32 + lane;
        uint32_t segments = 0;
        pdl_wait();  // the outputs may still be read by the kernel before this one
        for (int p = 0; p < P && ok; ++p) {
            const ChainPhase& ph = args.phase[p];
            if (p > 0) {
                // what this phase's epilogues read (sums of squares, the stream) was stored by the phase before
                if (tile_row == 0) flag_s[1] = wait_counter(done + (p - 1), args.phase[p - 1].row_tiles) ? 1 : 0;
                epilogue_barrier();
                if (!flag_s[1]) { ok = false; break; }
            }
            if (ph.row_sumsq) {
                if (tile_row < BN) {
                    float scale = 0.0f;
                    if (tile_row < M) {
                        float total = 0.0f;
                        for (int part = 0; part < ph.row_parts; ++part) total += __ldcg(ph.row_sumsq + (size_t)part * M + tile_row);
                        const float variance = total / ph.row_count + ph.row_eps;
                        scale = variance == 0.0f ? 0.0f : 1.0f / sqrtf(variance);
                    }
                    scale_s[tile_row] = scale;
                }
            }
            epilogue_barrier();
            long b = chain_range_begin(ph.total_boxes, cta, G);
            const long b1 = chain_range_begin(ph.total_boxes, cta + 1, G);
            while (b < b1 && ok) {
                const int tile = (int)(b / ph.k_blocks);
                const long tile_begin = (long)tile * ph.k_blocks, tile_end = tile_begin + ph.k_blocks;
                const long end = tile_end < b1 ? tile_end : b1;
                const bool whole = b == tile_begin && end == tile_end;
                const uint32_t buf = segments & 1u;
                if (!mbar_wait(smem_addr(&acc_full[buf]), (segments >> 1) & 1u)) { ok = false; break; }
                tc_fence_after();
                float v[BN];
#pragma unroll
                for (int c0 = 0; c0 < BN; c0 += 16) {
                    uint32_t r[16];
                    tmem_load_32x16(tmem_base + ((uint32_t)(lane_group * 32) << 16) + buf * (uint32_t)BN + (uint32_t)c0, r);
                    tmem_load_wait();
#pragma unroll
                    for (int j = 0; j < 16; ++j) v[c0 + j] = __uint_as_float(r[j]);
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_addr(&acc_empty[buf]));  // the MMAs may fill this accumulator again
                ++segments;
                b = end;
                if (b == b1 && tile_row == 0) chain_stamp(args, cta, p, 2);
                if (!whole) {
                    // a piece of a tile: into this CTA's slot (the piece at the begin of its stretch, or the one at its
                    // end), then count; whoever counts last adds the pieces up in the order of the CTAs
                    const int first = chain_owner(tile_begin, ph.total_boxes, G), last = chain_owner(tile_end - 1, ph.total_boxes, G);
                    float* mine = args.partial + ((size_t)cta * 2 + (cta == first ? 1 : 0)) * (BN * CHAIN_BM);
#pragma unroll
                    for (int j = 0; j < BN; ++j) __stcg(mine + j * CHAIN_BM + tile_row, v[j]);
                    __threadfence();
                    epilogue_barrier();
                    if (tile_row == 0) {
                        const int before = atomicAdd(arrive + first, 1);
                        const int is_last = before == last - first;
                        if (is_last) arrive[first] = 0;  // for the next split tile that begins in that CTA (a later phase)
                        flag_s[0] = is_last;
                    }
                    epilogue_barrier();
                    if (!flag_s[0]) continue;
                    __threadfence();
#pragma unroll
                    for (int j = 0; j < BN; ++j) v[j] = 0.0f;
                    // the pieces are added in the order of the CTAs; PAR of them are requested at a time, so that a
                    // tile in six pieces costs two round trips to L2 and not six
                    constexpr int PAR = BN <= 16 ? 4 : 2;
                    for (int base = first; base <= last; base += PAR) {
#pragma unroll
                        for (int c0 = 0; c0 < BN; c0 += 16) {
                            float piece_values[PAR][16];
#pragma unroll
                            for (int u = 0; u < PAR; ++u) {
                                const int other = base + u;
                                const float* piece = args.partial + ((size_t)(other <= last ? other : last) * 2 + (other == first ? 1 : 0)) * (BN * CHAIN_BM);
#pragma unroll
                                for (int j = 0; j < 16; ++j) piece_values[u][j] = __ldcg(piece + (c0 + j) * CHAIN_BM + tile_row);
                            }
#pragma unroll
                            for (int u = 0; u < PAR; ++u) {
                                if (base + u <= last) {
#pragma unroll
                                    for (int j = 0; j < 16; ++j) v[c0 + j] += piece_values[u][j];
                                }
                            }
                        }
                    }
                }
                // ---- the tile's epilogue: this thread holds output column n of tokens 0 .. BN - 1
                const int n = tile * CHAIN_BM + tile_row;
                if (ph.row_sumsq) {
#pragma unroll
                    for (int j = 0; j < BN; ++j) v[j] *= scale_s[j];
                }
                if (ph.form == 3) {
                    const float norm_w = n < ph.N ? ph.norm_weight[n] : 0.0f;
                    __nv_bfloat16* C = reinterpret_cast<__nv_bfloat16*>(ph.out);
#pragma unroll
                    for (int j = 0; j < BN; ++j) {
                        float sq = 0.0f;
                        if (n < ph.N && j < M) {
                            float* res = ph.residual + (size_t)j * ph.N + n;
                            const float r = __ldcg(res) + v[j];
                            __stcg(res, r);
                            C[(size_t)j * ph.ldc + n] = __float2bfloat16_rn(r * norm_w);
                            sq = r * r;
                        }
                        sq = warp_sum(sq);
                        if (lane == 0) sumsq_s[lane_group * BN + j] = sq;
                    }
                    epilogue_barrier();
                    if (tile_row < BN && tile_row < M)
                        ph.sumsq_out[(size_t)tile * M + tile_row] =
                            (sumsq_s[tile_row] + sumsq_s[BN + tile_row]) + (sumsq_s[2 * BN + tile_row] + sumsq_s[3 * BN + tile_row]);
                } else if (ph.form == 2) {
                    // rows 16 k .. 16 k + 7 are gate rows, 16 k + 8 .. 16 k + 15 their up rows
                    __nv_bfloat16* C = reinterpret_cast<__nv_bfloat16*>(ph.out);
#pragma unroll
                    for (int j = 0; j < BN; ++j) {
                        const float partner = __shfl_xor_sync(0xffffffffu, v[j], 8);
                        if ((lane & 8) == 0 && n < ph.N && j < M)
                            C[(size_t)j * ph.ldc + (n >> 4) * 8 + (n & 7)] = __float2bfloat16_rn(chain_silu_mul(v[j], partner));
                    }
                } else if (n < ph.N) {
                    if (ph.form == 0) {
                        __nv_bfloat16* C = reinterpret_cast<__nv_bfloat16*>(ph.out);
#pragma unroll
                        for (int j = 0; j < BN; ++j)
                            if (j < M) C[(size_t)j * ph.ldc + n] = __float2bfloat16_rn(v[j]);
                    } else {
                        float* C = reinterpret_cast<float*>(ph.out);
#pragma unroll
                        for (int j = 0; j < BN; ++j)
                            if (j < M) C[(size_t)j * ph.ldc + n] = v[j];
                    }
                }
                // the tile is stored: count it (the fence orders this CTA's stores before the count)
                __threadfence();
                epilogue_barrier();
                if (tile_row == 0) atomicAdd(done + p, 1);
                if (tile_row == 0) chain_stamp(args, cta, p, 3);
            }
        }
    }
    if (!ok) atomicExch(args.error_flag, KIRAI_FLAG_WAIT_RAN_OUT);
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, Smem::tmem_columns);
    }
    if (threadIdx.x == 0) {
        // the last CTA to leave puts the counters back for the next launch (nobody polls them any more)
        __threadfence();
        if (atomicAdd(exit_counter, 1) == G - 1) {
            for (int p = 0; p < CHAIN_MAX_PHASES; ++p) done[p] = 0;
            *exit_counter = 0;
            __threadfence();
        }
    }
}

namespace {

int chain_sm_count() {
    static const int count = [] {
        int device = 0, value = 0;
        if (cudaGetDevice(&device) != cudaSuccess) return 0;
        if (cudaDeviceGetAttribute(&value, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return 0;
        return value;
    }();
    return count;
}

template <int BN>
int chain_launch(const ChainMaps& maps, ChainArgs& args, int grid, cudaStream_t stream) {
    using Smem = ChainSmem<BN>;
    auto kernel = gemm_chain_kernel<BN>;
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem::total);
    if (err != cudaSuccess) return (int)err;
    return launch_pdl(kernel, dim3((unsigned)grid), dim3(CHAIN_THREADS), (size_t)Smem::total, stream, 1u, maps, args);
}

}  // namespace

// Bytes of workspace that a chain needs at most (partial tiles of every CTA, and the counters), zeroed once by the
// caller; the kernel leaves the counters zero again.
KIRAI_EXPORT long kirai_gemm_chain_workspace_bytes() {
    const long grid = chain_sm_count() > 0 ? chain_sm_count() : 148;
    return grid * 2 * 64 * CHAIN_BM * 4 + (grid + CHAIN_MAX_PHASES + 1) * 4 + 256;
}
KIRAI_EXPORT int kirai_gemm_chain_max_phases() { return CHAIN_MAX_PHASES; }

// `phases` products A_p[M, K_p] (row stride lda_p) times W_p[N_p, K_p] transposed, W_p tiled, run one after the other
// (each may read what the ones before it wrote) by one persistent kernel.  Forms, row_sumsq, residual, norm_weight and
// sumsq_out as in kirai_gemm_bf16_general (form 3 writes ceil(N / 128) parts).  M <= 64.  Refuses (-4) what it does
// not take; the caller then launches the products one by one.  stamps: null, or room for grid * 6 * 4 clock stamps.
KIRAI_EXPORT int kirai_gemm_chain_bf16(int phases, int M, const void* const* A, const long* lda, const void* const* W,
                                       void* const* C, const long* ldc, const int* N, const int* K, const int* form,
                                       const float* const* row_sumsq, const int* row_parts, const float* row_count,
                                       const float* row_eps, float* const* residual, const float* const* norm_weight,
                                       float* const* sumsq_out, void* workspace, long workspace_bytes, int* error_flag,
                                       unsigned long long* stamps, cudaStream_t stream) {
    if (phases < 1 || phases > CHAIN_MAX_PHASES || M < 1 || M > 64) return KIRAI_ERR_UNSUPPORTED;
    if (!workspace || ((uintptr_t)workspace & 15) || workspace_bytes < kirai_gemm_chain_workspace_bytes()) return KIRAI_ERR_BAD_SIZE;
    const int BN = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
    ChainMaps maps;
    ChainArgs args = {};
    long fewest = -1;
    for (int p = 0; p < phases; ++p) {
        if (N[p] <= 0 || K[p] <= 0) return KIRAI_ERR_BAD_SIZE;
        if (K[p] % 8 != 0 || lda[p] % 8 != 0 || ((uintptr_t)W[p] & 15)) return KIRAI_ERR_BAD_ALIGN;
        if (form[p] < 0 || form[p] > 3) return KIRAI_ERR_BAD_SIZE;
        if (form[p] == 2 && N[p] % 16 != 0) return KIRAI_ERR_BAD_SIZE;
        if (form[p] == 3 && (!residual[p] || !norm_weight[p] || !sumsq_out[p] || row_sumsq[p])) return KIRAI_ERR_BAD_SIZE;
        if (row_sumsq[p] && row_parts[p] <= 0) return KIRAI_ERR_BAD_SIZE;
        if (!tmap::bf16_2d_sw128(&maps.map[p], A[p], (uint64_t)M, (uint64_t)K[p], (uint64_t)lda[p], (uint32_t)BN, CHAIN_BK))
            return KIRAI_ERR_BAD_ALIGN;
        ChainPhase& ph = args.phase[p];
        ph.boxes = (const uint8_t*)W[p];
        ph.out = C[p];
        ph.row_sumsq = row_sumsq[p];
        ph.residual = residual[p];
        ph.norm_weight = norm_weight[p];
        ph.sumsq_out = sumsq_out[p];
        ph.ldc = form[p] == 3 ? (long)N[p] : ldc[p];
        ph.N = N[p], ph.K = K[p], ph.form = form[p];
        ph.row_tiles = (N[p] + CHAIN_BM - 1) / CHAIN_BM;
        ph.k_blocks = (K[p] + CHAIN_BK - 1) / CHAIN_BK;
        ph.total_boxes = (long)ph.row_tiles * ph.k_blocks;
        ph.row_parts = row_sumsq[p] ? row_parts[p] : 0;
        ph.row_count = row_count[p], ph.row_eps = row_eps[p];
        if (fewest < 0 || ph.total_boxes < fewest) fewest = ph.total_boxes;
    }
    // every CTA takes at least one box of every phase, so that the CTAs that share a tile are a run without gaps
    const int sms = chain_sm_count() > 0 ? chain_sm_count() : 148;
    const int grid = (int)(fewest < sms ? fewest : sms);
    args.phases = phases, args.M = M;
    args.partial = (float*)workspace;
    args.counters = (int*)((uint8_t*)workspace + (size_t)sms * 2 * 64 * CHAIN_BM * 4);
    args.error_flag = error_flag;
    args.stamps = stamps;
    if (BN == 16) return chain_launch<16>(maps, args, grid, stream);
    if (BN == 32) return chain_launch<32>(maps, args, grid, stream);
    return chain_launch<64>(maps, args, grid, stream);
}
