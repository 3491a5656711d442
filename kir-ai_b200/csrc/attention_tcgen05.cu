// Prompt attention over the paged cache on the tcgen05 tensor cores.
//
// One CTA per (request, kv head, tile of 128 query rows); the rows enumerate (token, head of
// the group) pairs, so the group's heads share every key/value tile.  Per tile of 64 keys:
//
//   S = Q K^T      tcgen05.mma, both operands from shared memory (K-major, 128-byte swizzle),
//                  S [128 x 64] in tensor memory;
//   softmax        128 threads, one query row each: the row comes back with tcgen05.ld, is masked
//                  by position, exponentiated against a running maximum, and goes to tensor
//                  memory again as bf16 (tcgen05.st) to be the A operand of the second product;
//   O += P V       tcgen05.mma with A from tensor memory and B = the V tile as it lies in shared
//                  memory (head dims contiguous: an MN-major operand).
//
// The running maximum is lazy: the output accumulator is rescaled only when a row's maximum has
// grown by more than 2^8 since the scale in use, which is exact (the final division uses the same
// scale) and spares most read-modify-write passes over the accumulator.
// Warp roles: warp 0 fetches K tiles and warp 6 V tiles by TMA straight from the pages (two slots each), one
// thread of warp 1 issues the MMAs, warps 2-5 are the softmax rows.  S has two buffers in tensor memory
// (P lies over the buffer its S came from): the first product of tile t + 1 is issued before the second
// product of tile t, so it runs while the rows of tile t exponentiate.  A CTA is small enough for two per
// SM, which fill each other's gaps.  Every barrier wait is bounded.
// A load warp's requests cost it about 100 cycles each (clock stamps) and one warp for both rings set the pace of
// the kernel: hence a warp per ring, and a page's rows come whole, both 64-column panels in one request, through a 4-dimensional tensor map (columns, 8 rows, panels, groups of
// 8 rows) that leaves a tile as [group][panel][8 rows][128 bytes]; head sizes that are no multiple of 64 and
// pages under 8 tokens take one request per panel and at most 8 rows into the same layout.
// Same visibility rule as the other attention kernels: row at position pos sees keys
// lo <= j <= pos.  head_dim: a multiple of 8 up to 128; the group size must divide 128.
#include "sm100.cuh"
#include "tensor_map.cuh"

using namespace sm100;

namespace {

#define TA_ROWS 128
#define TA_BN 64
#define TA_STAGES 2   // slots of the K ring, and of the V ring
#define TA_THREADS 224
#define TA_TMEM_COLS 256  // S buffers (and, over each one's first half, its P) in columns 0..63 and 64..127, O in 128..255

template <int D>
struct TcAttnSmem {
    static constexpr int panels = D / 64;
    static constexpr int q_bytes = TA_ROWS * D * 2;
    static constexpr int tile_bytes = TA_BN * D * 2;
    static constexpr int ring_bytes = TA_STAGES * 2 * tile_bytes;  // K ring, then V ring
    static constexpr int barrier_bytes = 256;
    static_assert((4 * TA_STAGES + 5) * 8 + 4 <= barrier_bytes, "the barriers and the tensor-memory slot must fit their region");
    static constexpr int table_entries = 1024;
    static constexpr int total = q_bytes + ring_bytes + barrier_bytes + table_entries * 4 + 1024;
};

// [rows][64 bf16] panels with the TMA 128-byte swizzle: chunk c of row r at chunk c ^ (r & 7).
template <int ROWS>
__device__ __forceinline__ uint32_t panel_offset(int row, int chunk) {
    return (uint32_t)((chunk >> 3) * (ROWS * 128) + row * 128 + (((chunk & 7) ^ (row & 7)) << 4));
}

// Key and value tiles lie in shared memory as [group of 8 rows][64-column panel][8 rows][128 bytes] with the
// 128-byte swizzle (a row's two panels in one group, so that one TMA request can bring whole rows): row `row` of
// panel `panel` starts here.
template <int PANELS>
__device__ __forceinline__ uint32_t kv_row_offset(int row, int panel) {
    return (uint32_t)((row >> 3) * (PANELS * 1024) + panel * 1024 + (row & 7) * 128);
}

// K-major operand (rows of 128 bytes, 8-row groups a given stride apart): see sm100::smem_desc_k_major_sw128_groups.
// MN-major operand with the 128-byte swizzle: 64 contiguous MN elements per 128-byte row, one row
// per K index, 8-row groups `group_bytes` apart (stride offset), the next 64 MN elements `panel_bytes`
// further (leading offset).
__device__ __forceinline__ uint64_t smem_desc_mn_major_sw128(uint32_t addr, uint32_t panel_bytes, uint32_t group_bytes) {
    uint64_t desc = 0;
    desc |= (uint64_t)((addr & 0x3FFFF) >> 4);
    desc |= (uint64_t)((panel_bytes >> 4) & 0x3FFF) << 16;
    desc |= (uint64_t)((group_bytes >> 4) & 0x3FFF) << 32;
    desc |= (uint64_t)1 << 46;
    desc |= (uint64_t)2 << 61;
    return desc;
}
__host__ __device__ constexpr uint32_t instr_desc_bf16_b_mn(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void mma_bf16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}\n"
        ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tmem_store_32x32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
          "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
          "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_store_32x16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void tmem_store_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// Two positive finite floats as a bf16 pair, rounded to nearest (ties upward) with integer instructions: the
// conversion instruction shares the pipe of ex2, which the softmax rows keep busy.
__device__ __forceinline__ uint32_t pack2_weights(float lo, float hi) {
    return __byte_perm(__float_as_uint(lo) + 0x8000u, __float_as_uint(hi) + 0x8000u, 0x7632);
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

template <int D>
__global__ void __launch_bounds__(TA_THREADS, 2)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap kv_map, const bf16* __restrict__ q, bf16* __restrict__ out,
                            const int* __restrict__ block_table, const int* __restrict__ query_start,
                            const int* __restrict__ context_len, int q_heads, int kv_heads, int head_dim,
                            long q_row_stride, int page_size, int box_rows, int piece_rows, int table_width, int num_pages,
                            int window, float scale_log2, int* __restrict__ error_flag) {
    pdl_launch_dependents();
    pdl_wait();
    using Smem = TcAttnSmem<D>;
    constexpr int PANELS = Smem::panels;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    // CTAs are handed out in the order of their linear index, x fastest: the kv heads are x and the row tiles y, last
    // tile first, so that of one prompt the tiles that see the most keys start first on every head, and the launch does
    // not end with a head's heavy tiles that were handed out late
    const int tile = gridDim.y - 1 - blockIdx.y;
    const int kv_head = blockIdx.x, req = blockIdx.z;
    const int group = q_heads / kv_heads;
    const int q_begin = query_start[req];
    const int q_len = query_start[req + 1] - q_begin;
    const int rows_total = q_len * group;
    const int row0 = tile * TA_ROWS;
    if (row0 >= rows_total) return;
    const int ctx = context_len[req];
    const int start_pos = ctx - q_len;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    const uint32_t q_smem = smem_addr(smem);
    const uint32_t ring = q_smem + Smem::q_bytes;
    uint64_t* bars = (uint64_t*)(smem + Smem::q_bytes + Smem::ring_bytes);
    uint64_t* k_full = bars;                        // [TA_STAGES] TMA -> MMA
    uint64_t* k_empty = bars + TA_STAGES;           // [TA_STAGES] first product done with the K tile
    uint64_t* v_full = bars + 2 * TA_STAGES;        // [TA_STAGES]
    uint64_t* v_empty = bars + 3 * TA_STAGES;       // [TA_STAGES] second product done with the V tile
    uint64_t* s_ready = bars + 4 * TA_STAGES;       // [2] S of a tile is in its buffer (and every product issued before is done)
    uint64_t* p_ready = s_ready + 2;                // [2] P of a tile is in tensor memory (4 warps arrive)
    uint64_t* o_ready = s_ready + 4;                // the second product of a tile is done
    uint32_t* tmem_slot = (uint32_t*)(s_ready + 5);
    int* table_s = reinterpret_cast<int*>(smem + Smem::q_bytes + Smem::ring_bytes + Smem::barrier_bytes);

    const int last_row = min(rows_total, row0 + TA_ROWS) - 1;
    const int pos_first = start_pos + row0 / group;
    const int pos_last = start_pos + last_row / group;
    const int key_lo = window > 0 ? max(0, pos_first - window + 1) : 0;
    const int first_tile = key_lo / TA_BN, last_tile = pos_last / TA_BN;
    const int num_tiles = last_tile - first_tile + 1;

    if (tid == 0) {
        tma_prefetch_descriptor(&kv_map);
        for (int s = 0; s < TA_STAGES; ++s) {
            mbar_init(smem_addr(&k_full[s]), 1);
            mbar_init(smem_addr(&k_empty[s]), 1);
            mbar_init(smem_addr(&v_full[s]), 1);
            mbar_init(smem_addr(&v_empty[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_addr(&s_ready[b]), 1);
            mbar_init(smem_addr(&p_ready[b]), 4);
        }
        mbar_init(smem_addr(o_ready), 1);
        mbar_fence_init();
    }
    if (warp == 1) {
        tmem_alloc(smem_addr(tmem_slot), TA_TMEM_COLS);
        tmem_relinquish();
    }
    // Q tile: row r is token (row0 + r) / group, head kv_head * group + (row0 + r) % group
    {
        constexpr int CH = D / 8;
        const int chunks_used = head_dim / 8;
        for (int id = tid; id < TA_ROWS * CH; id += TA_THREADS) {
            const int r = id / CH, chunk = id % CH;
            const int row = row0 + r;
            uint4 value = make_uint4(0u, 0u, 0u, 0u);
            if (row < rows_total && chunk < chunks_used) {
                const int token = row / group, head = kv_head * group + row % group;
                value = *reinterpret_cast<const uint4*>(q + (size_t)(q_begin + token) * q_row_stride + (size_t)head * head_dim + chunk * 8);
            }
            *reinterpret_cast<uint4*>(smem + panel_offset<TA_ROWS>(r, chunk)) = value;
        }
        // the block table of the keys this CTA reads
        const int* table_g = block_table + (long)req * table_width;
        const int first_page = (first_tile * TA_BN) / page_size;
        const int last_page = min(table_width - 1, pos_last / page_size);
        if (last_page - first_page < Smem::table_entries)
            for (int i = first_page + tid; i <= last_page; i += TA_THREADS) table_s[i - first_page] = table_g[i];
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the MMAs read the Q tile through the async proxy
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_s = tmem_base /* + 64 for odd tiles; P over the first 32 columns */, tmem_o = tmem_base + 128;
    bool ok = true;

    if (warp == 0 || warp == 6) {
        // the two load warps: warp 0 feeds the K ring, warp 6 the V ring, each at its own pace (a request costs its
        // warp about 100 cycles, and one warp for both rings set the pace of the kernel)
        const int which = warp == 0 ? 0 : 1;
        const int* table = block_table + (long)req * table_width;
        {
            const int first_page = (first_tile * TA_BN) / page_size;
            const int last_page = min(table_width - 1, pos_last / page_size);
            if (last_page - first_page < Smem::table_entries) table = table_s - first_page;
        }
        const int boxes = TA_BN / box_rows;
        const uint32_t box_bytes = (uint32_t)box_rows * 128u * PANELS;
        // This warp's pace bounds the kernel (two fills per tile), so a tile's pages are looked up once, for its
        // keys and its values alike, and sizes that are powers of two are shifted, not divided.
        const int page_shift = __ffs(page_size) - 1, box_shift = __ffs(box_rows) - 1;
        constexpr int PER_LANE = (TA_BN + 31) / 32;  // boxes per lane when a box is one row
        struct TilePlan {
            int row[PER_LANE];  // first cache row (of K; V lies kv_heads * page_size further) of this lane's boxes, or -1
            int count;          // boxes with a page, over the warp
        };
        auto plan_tile = [&](int t) {
            TilePlan plan;
            unsigned present = 0;
#pragma unroll
            for (int k = 0; k < PER_LANE; ++k) {
                const int b = lane + 32 * k;
                plan.row[k] = -1;
                if (b < boxes) {
                    const int j = t * TA_BN + (b << box_shift);
                    const int logical = j >> page_shift;
                    const int page = (j <= pos_last && logical < table_width) ? table[logical] : -1;
                    if (page >= 0 && page < num_pages)
                        plan.row[k] = ((page * 2) * kv_heads + kv_head) * page_size + (j & (page_size - 1));
                }
                present += __popc(__ballot_sync(0xffffffffu, plan.row[k] >= 0));
            }
            plan.count = (int)present;
            return plan;
        };
        // fills one slot of the K ring (which == 0) or of the V ring (which == 1) with the planned tile
        auto fill = [&](const TilePlan& plan, int which, uint32_t bar, uint32_t dst) {
            if (plan.count < boxes) {
                // boxes without a page hold masked keys only; their rows are cleared all the same, because a
                // value row is multiplied by its zero weight and must be finite
#pragma unroll
                for (int k = 0; k < PER_LANE; ++k) {
                    for (int owner = 0; owner < 32 && 32 * k + owner < boxes; ++owner) {
                        if (__shfl_sync(0xffffffffu, plan.row[k], owner) >= 0) continue;
                        const int b = 32 * k + owner;
                        for (int h = 0; h < PANELS; ++h) {
                            for (int i = lane; i < box_rows * 8; i += 32)
                                asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(dst + kv_row_offset<PANELS>((b << box_shift) + (i >> 3), h) + (i & 7) * 16), "r"(0u) : "memory");
                        }
                    }
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
            }
            if (lane == 0) {
                if (plan.count) mbar_expect_tx(bar, box_bytes * (uint32_t)plan.count);
                else mbar_arrive(bar);
            }
            __syncwarp();
            const int value_rows = which * kv_heads * page_size;
#pragma unroll
            for (int k = 0; k < PER_LANE; ++k) {
                if (plan.row[k] >= 0) {
                    const int first = (lane + 32 * k) << box_shift;  // the box's first row in the tile
                    if (piece_rows == 0) {
                        // one request for the box's whole rows (a multiple of 8 of them, both panels)
                        tma_load_4d(dst + kv_row_offset<PANELS>(first, 0), &kv_map, bar, 0, 0, 0, (plan.row[k] + value_rows) >> 3);
                    } else {
                        // pieces of at most 8 rows of one panel
                        for (int sub = 0; sub < box_rows; sub += piece_rows)
#pragma unroll
                            for (int h = 0; h < PANELS; ++h)
                                tma_load_2d(dst + kv_row_offset<PANELS>(first + sub, h), &kv_map, bar, h * 64,
                                            plan.row[k] + value_rows + sub);
                    }
                }
            }
            __syncwarp();
        };
        uint64_t* full = which == 0 ? k_full : v_full;
        uint64_t* empty = which == 0 ? k_empty : v_empty;
        for (int it = 0; it < num_tiles; ++it) {
            const TilePlan plan = plan_tile(first_tile + it);
            const int slot = it % TA_STAGES;
            if (it >= TA_STAGES && !mbar_wait_hot(smem_addr(&empty[slot]), (uint32_t)(it / TA_STAGES - 1) & 1u)) { ok = false; break; }
            fill(plan, which, smem_addr(&full[slot]), ring + (which * TA_STAGES + slot) * Smem::tile_bytes);
        }
    } else if (warp == 1) {
        if (elect_one()) {
            constexpr uint32_t idesc_qk = instr_desc_bf16(TA_ROWS, TA_BN);      // S[128 x 128 keys]
            constexpr uint32_t idesc_pv = instr_desc_bf16_b_mn(TA_ROWS, D);     // O[128 x D], B = V as it lies (MN-major)
            // S(it) = Q K(it)^T into buffer it & 1
            auto first_product = [&](int it) {
                const int slot = it % TA_STAGES;
                if (!mbar_wait_hot(smem_addr(&k_full[slot]), (uint32_t)(it / TA_STAGES) & 1u)) { ok = false; return; }
                tc_fence_after();
                const uint32_t k_addr = ring + slot * Smem::tile_bytes;
                const uint32_t s_acc = tmem_s + (uint32_t)((it & 1) * TA_BN);
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    // 16 dims further: 32 bytes inside the swizzle atom, or the next 64-column panel
                    const uint32_t off_q = (uint32_t)((kk >> 2) * (TA_ROWS * 128) + (kk & 3) * 32);
                    const uint32_t off_k = (uint32_t)((kk >> 2) * 1024 + (kk & 3) * 32);
                    mma_bf16_ss(s_acc, smem_desc_k_major_sw128(q_smem + off_q),
                                smem_desc_k_major_sw128_groups(k_addr + off_k, PANELS * 1024), idesc_qk, kk > 0 ? 1u : 0u);
                }
                mma_commit(smem_addr(&k_empty[slot]));
                mma_commit(smem_addr(&s_ready[it & 1]));
            };
            first_product(0);
            for (int it = 0; it < num_tiles && ok; ++it) {
                // the next tile's scores are computed while this tile's rows exponentiate; the products run in
                // issue order, so this one finds its buffer free (the second product of tile it - 1 read it)
                if (it + 1 < num_tiles) first_product(it + 1);
                if (!ok) break;
                const int slot = it % TA_STAGES;
                if (!mbar_wait_hot(smem_addr(&v_full[slot]), (uint32_t)(it / TA_STAGES) & 1u)) { ok = false; break; }
                if (!mbar_wait_hot(smem_addr(&p_ready[it & 1]), (uint32_t)(it >> 1) & 1u)) { ok = false; break; }
                tc_fence_after();
                const uint32_t v_addr = ring + (TA_STAGES + slot) * Smem::tile_bytes;
                const uint32_t tmem_p = tmem_s + (uint32_t)((it & 1) * TA_BN);
#pragma unroll
                for (int kk = 0; kk < TA_BN / 16; ++kk) {
                    // 16 keys further: 8 columns of packed bf16 pairs in tensor memory, two 8-row groups of the V tile
                    mma_bf16_ts(tmem_o, tmem_p + (uint32_t)(kk * 8),
                                smem_desc_mn_major_sw128(v_addr + (uint32_t)(kk * 2 * PANELS * 1024), 1024, PANELS * 1024), idesc_pv,
                                (it > 0 || kk > 0) ? 1u : 0u);
                }
                mma_commit(smem_addr(&v_empty[slot]));
                mma_commit(smem_addr(o_ready));
            }
        }
    } else {
        // softmax rows (warps 2-5): this thread owns query row r (tensor-memory lane r)
        const int lane_group = warp & 3;
        const int r = lane_group * 32 + lane;
        const uint32_t lane_bits = (uint32_t)(lane_group * 32) << 16;
        const int row = row0 + r;
        const bool valid = row < rows_total;
        const int pos = valid ? start_pos + row / group : -1;
        const int lo = (valid && window > 0) ? max(0, pos - window + 1) : 0;
        float m_used = -INFINITY;  // the maximum that the accumulator and the sum are scaled by (log2 domain)
        float l = 0.0f;
        for (int it = 0; it < num_tiles; ++it) {
            const int j0 = (first_tile + it) * TA_BN;
            // S of this tile is complete in buffer it & 1
            if (!mbar_wait_hot(smem_addr(&s_ready[it & 1]), (uint32_t)(it >> 1) & 1u)) { ok = false; break; }
            tc_fence_after();
            const uint32_t s_buf = tmem_s + lane_bits + (uint32_t)((it & 1) * TA_BN);
            // the row's 64 scores, read once
            uint32_t s[TA_BN];
            {
                uint32_t half0[32], half1[32];
                tmem_load_32x32(s_buf, half0);
                tmem_load_32x32(s_buf + 32u, half1);
                tmem_load_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    s[i] = half0[i];
                    s[32 + i] = half1[i];
                }
            }
            // a tile whose keys every row of this warp sees needs no mask
            const bool interior = __all_sync(0xffffffffu, j0 >= lo && j0 + TA_BN - 1 <= pos);
            if (!interior) {
#pragma unroll
                for (int i = 0; i < TA_BN; ++i) {
                    const int j = j0 + i;
                    if (!(j >= lo && j <= pos)) s[i] = __float_as_uint(-INFINITY);
                }
            }
            // the row's maximum (four running maxima, so that the chain of dependent compares is short)
            float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int i = 0; i < TA_BN; ++i) mx[i & 3] = fmaxf(mx[i & 3], __uint_as_float(s[i]));
            const float m_tile = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * scale_log2;  // the scale is positive
            const float m_new = fmaxf(m_used, m_tile);
            const bool grow = m_new > m_used + 8.0f || (m_used == -INFINITY && m_new != -INFINITY);
            const float factor = grow ? exp2f(m_used - m_new) : 1.0f;  // exp2(-inf) = 0 for a row that saw nothing yet
            if (grow) {
                l *= factor;
                m_used = m_new;
            }
            // The second product of the tile before is not behind this tile's scores in issue order.  Its barrier is
            // waited for in every tile, here if the accumulator must be rescaled and at the end of the tile
            // otherwise (by then it has long completed): a parity wait cannot tell a phase from the one two before
            // or after it, so no phase may be skipped.
            bool seen_before = it == 0;
            if (__any_sync(0xffffffffu, grow && it > 0)) {
                // rescale this warp's rows of the accumulator (rows that do not need it multiply by 1), once the
                // second product of the tile before has added into it
                if (!mbar_wait_hot(smem_addr(o_ready), (uint32_t)(it - 1) & 1u)) { ok = false; break; }
                seen_before = true;
                tc_fence_after();
#pragma unroll 1
                for (int c = 0; c < D / 32; ++c) {
                    uint32_t o[32];
                    tmem_load_32x32(tmem_o + lane_bits + (uint32_t)(c * 32), o);
                    tmem_load_wait();
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * factor);
                    tmem_store_32x32(tmem_o + lane_bits + (uint32_t)(c * 32), o);
                }
            }
            const float m_sub = m_used == -INFINITY ? 0.0f : m_used;
            // the weights: exp2(s * scale - m), one fused multiply-add and one ex2.approx per key (-inf gives 0);
            // their 32 columns of bf16 pairs go over the first half of this tile's S buffer
            float sum[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (int c = 0; c < TA_BN / 32; ++c) {
                uint32_t p[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const float a = ex2_approx(fmaf(__uint_as_float(s[c * 32 + 2 * i]), scale_log2, -m_sub));
                    const float b = ex2_approx(fmaf(__uint_as_float(s[c * 32 + 2 * i + 1]), scale_log2, -m_sub));
                    sum[i & 3] += a + b;
                    p[i] = pack2_weights(a, b);
                }
                tmem_store_32x16(s_buf + (uint32_t)(c * 16), p);
            }
            l += (sum[0] + sum[1]) + (sum[2] + sum[3]);
            tmem_store_wait();
            if (!seen_before && !mbar_wait_hot(smem_addr(o_ready), (uint32_t)(it - 1) & 1u)) { ok = false; break; }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_addr(&p_ready[it & 1]));
        }
        if (ok) ok = mbar_wait_hot(smem_addr(o_ready), (uint32_t)(num_tiles - 1) & 1u);
        tc_fence_after();
        if (ok) {
            const float inv = l > 0.0f ? 1.0f / l : 0.0f;
            bf16* dst = nullptr;
            if (valid) {
                const int token = row / group, head = kv_head * group + row % group;
                dst = out + ((size_t)(q_begin + token) * q_heads + head) * head_dim;
            }
#pragma unroll 1
            for (int c = 0; c < D / 32; ++c) {
                uint32_t o[32];
                tmem_load_32x32(tmem_o + lane_bits + (uint32_t)(c * 32), o);
                tmem_load_wait();
                if (dst) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        const int col = c * 32 + i;
                        if (col + 8 <= head_dim) {
                            uint4 packed;
                            packed.x = pack2(__uint_as_float(o[i]) * inv, __uint_as_float(o[i + 1]) * inv);
                            packed.y = pack2(__uint_as_float(o[i + 2]) * inv, __uint_as_float(o[i + 3]) * inv);
                            packed.z = pack2(__uint_as_float(o[i + 4]) * inv, __uint_as_float(o[i + 5]) * inv);
                            packed.w = pack2(__uint_as_float(o[i + 6]) * inv, __uint_as_float(o[i + 7]) * inv);
                            *reinterpret_cast<uint4*>(dst + col) = packed;
                        }
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
        tmem_dealloc(tmem_base, TA_TMEM_COLS);
    }
}

template <int D>
int launch(const void* q, const void* cache, void* out, const int* block_table, const int* query_start,
           const int* context_len, int requests, int max_query_len, int q_heads, int kv_heads, int head_dim,
           long q_row_stride, int page_size, int table_width, int num_pages, int window, float scale, int* error_flag,
           cudaStream_t stream) {
    using Smem = TcAttnSmem<D>;
    const int group = q_heads / kv_heads;
    const int box_rows = page_size < TA_BN ? page_size : TA_BN;
    if (TA_BN % box_rows != 0 || page_size % box_rows != 0) return KIRAI_ERR_UNSUPPORTED;
    CUtensorMap kv_map;
    const uint64_t rows = (uint64_t)num_pages * 2 * kv_heads * page_size;
    // whole rows of a box in one request where the sizes allow it; else pieces of one panel and at most 8 rows
    int piece_rows = 0;
    if (head_dim % 64 != 0 || box_rows % 8 != 0 || !tmap::bf16_kv_boxes_sw128(&kv_map, cache, rows, head_dim, box_rows)) {
        piece_rows = box_rows < 8 ? box_rows : 8;
        if (!tmap::bf16_2d_sw128(&kv_map, cache, rows, head_dim, head_dim, piece_rows, 64)) return KIRAI_ERR_BAD_ALIGN;
    }
    auto kernel = attention_prefill_tc_kernel<D>;
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem::total);
    if (err != cudaSuccess) return (int)err;
    dim3 grid(kv_heads, (unsigned)(((long)max_query_len * group + TA_ROWS - 1) / TA_ROWS), requests);
    if (grid.y > 65535) return KIRAI_ERR_BAD_SIZE;
    return launch_pdl(kernel, grid, dim3(TA_THREADS), (size_t)Smem::total, stream, 1u, kv_map, (const bf16*)q, (bf16*)out,
                      block_table, query_start, context_len, q_heads, kv_heads, head_dim, q_row_stride, page_size, box_rows,
                      piece_rows, table_width, num_pages, window, scale * 1.4426950408889634f, error_flag);
}

}  // namespace

// Same arguments as kirai_attention_prefill_bf16.  Refuses (KIRAI_ERR_UNSUPPORTED) head sizes above
// 128, groups that do not divide 128, and page sizes that are no power of two.
KIRAI_EXPORT int kirai_attention_prefill_tc_bf16(const void* q, const void* cache, void* out, const int* block_table,
                                                 const int* query_start, const int* context_len, int requests,
                                                 int max_query_len, int q_heads, int kv_heads, int head_dim,
                                                 long q_row_stride, int page_size, int table_width, int num_pages,
                                                 int window, float scale, int* error_flag, cudaStream_t stream) {
    if (requests <= 0 || max_query_len <= 0) return 0;
    if (kv_heads <= 0 || q_heads % kv_heads != 0) return KIRAI_ERR_BAD_SIZE;
    const int group = q_heads / kv_heads;
    if (head_dim <= 0 || head_dim % 8 != 0) return KIRAI_ERR_BAD_SIZE;
    if (head_dim > 128 || TA_ROWS % group != 0) return KIRAI_ERR_UNSUPPORTED;
    if (q_row_stride % 8 != 0 || ((uintptr_t)q & 15)) return KIRAI_ERR_BAD_ALIGN;
    if (requests > 65535 || kv_heads > 65535) return KIRAI_ERR_BAD_SIZE;
    if (head_dim <= 64)
        return launch<64>(q, cache, out, block_table, query_start, context_len, requests, max_query_len, q_heads, kv_heads,
                          head_dim, q_row_stride, page_size, table_width, num_pages, window, scale, error_flag, stream);
    return launch<128>(q, cache, out, block_table, query_start, context_len, requests, max_query_len, q_heads, kv_heads,
                       head_dim, q_row_stride, page_size, table_width, num_pages, window, scale, error_flag, stream);
}
