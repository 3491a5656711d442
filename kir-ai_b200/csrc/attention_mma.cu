// bf16 causal grouped-query attention over the paged cache on the tensor cores
// (warp-level mma.m16n8k16, 32-bit accumulation, softmax in 32-bit registers).
//
// Two kernels share one warp-level routine that folds a tile of keys into a
// running (max, sum, output) state, flash-attention style:
//
//  * the prompt kernel: one CTA per (request, kv head, tile of 64 query rows),
//    where the query rows enumerate (token, head of the group) pairs, so that
//    the heads of a group share each key/value tile; 4 warps own 16 rows each
//    and a fifth keeps a ring of 3 key/value tiles full by TMA from the pages;
//  * the decode kernels, for batches in which every request brings one token: the group's heads are the (few)
//    query rows, each of a CTA's warps walks its own 16-key tiles through its own three-slot TMA ring, and the
//    warps' states are merged in shared memory.  The split kernel runs one CTA per (request, kv head, split of
//    the context) and a second kernel merges the splits; the balanced kernel cuts the key tiles of all
//    (request, kv head) pairs into one equal range per CTA and merges only the pairs that a range border cut.
//    Both read what a step cannot change (block tables, lengths, keys and values of earlier steps) before they
//    wait for the kernel before them.
//
// Keys are visible to a row at position pos when lo <= j <= pos, lo = max(0,
// pos - window + 1) with a window, else 0 (same rule as the plain kernel).
// Key tiles start at absolute multiples of the tile size, so which keys share
// a tile does not depend on how a prompt was cut.  head_dim: any multiple of 8
// up to 256 (the tile is padded with zeros to 64, 128 or 256 columns).
#include "sm100.cuh"
#include "tensor_map.cuh"

namespace {

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// A tile in shared memory holds ROWS rows of D bf16 as D / 64 panels of [ROWS][64] (128-byte rows);
// inside a panel the 16-byte chunk c of row r sits at chunk c ^ (r & 7).  This is the layout that a
// TMA box of 64 columns with the 128-byte swizzle produces (panels based at multiples of 1024 bytes),
// and it keeps the 8 rows of an ldmatrix on different banks.
template <int ROWS>
__device__ __forceinline__ uint32_t tile_offset(int row, int chunk) {
    return (uint32_t)((chunk >> 3) * (ROWS * 128) + row * 128 + (((chunk & 7) ^ (row & 7)) << 4));
}

// Running softmax state of the two rows (g and g + 8) that a thread of an m16 tile holds.
template <int D>
struct WarpState {
    float m[2], l[2];
    float o[D / 8][4];
    __device__ __forceinline__ void init() {
        m[0] = m[1] = -INFINITY;
        l[0] = l[1] = 0.0f;
#pragma unroll
        for (int n = 0; n < D / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.0f;
    }
};

// Folds BN keys (tile at k_smem / v_smem, first key j0) into the state of this warp's 16 query
// rows, whose A-operand tile is at q_smem rows [q_row0, q_row0 + 16).  Row r (0..15) sees key j
// when lo[r] <= j <= hi[r]; the thread holds rows g = lane / 4 (index 0) and g + 8 (index 1).
template <int D, int BN, int QROWS, bool Q_IN_REGS>
__device__ __forceinline__ void warp_attend(WarpState<D>& st, uint32_t q_smem, int q_row0, const uint32_t (*q_regs)[4], uint32_t k_smem,
                                            uint32_t v_smem, int j0, const int (&lo)[2], const int (&hi)[2],
                                            float scale_log2, int lane) {
    float s[BN / 8][4];
#pragma unroll
    for (int n = 0; n < BN / 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.0f;
    // S = Q K^T
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
        uint32_t a[4];
        if (Q_IN_REGS) {
            a[0] = q_regs[kk][0]; a[1] = q_regs[kk][1]; a[2] = q_regs[kk][2]; a[3] = q_regs[kk][3];
        } else {
            const int row = q_row0 + (lane & 15);
            const int chunk = kk * 2 + (lane >> 4);
            ldmatrix_x4(q_smem + tile_offset<QROWS>(row, chunk), a[0], a[1], a[2], a[3]);
        }
#pragma unroll
        for (int n2 = 0; n2 < BN / 16; ++n2) {
            // two n-tiles (16 keys) per ldmatrix.x4: matrices (keys 0-7, k lo), (keys 0-7, k hi), (keys 8-15, k lo), (keys 8-15, k hi)
            uint32_t b0, b1, b2, b3;
            const int row = n2 * 16 + (lane & 7) + ((lane >> 4) << 3);
            const int chunk = kk * 2 + ((lane >> 3) & 1);
            ldmatrix_x4(k_smem + tile_offset<BN>(row, chunk), b0, b1, b2, b3);
            mma_bf16_16816(s[2 * n2], a, b0, b1);
            mma_bf16_16816(s[2 * n2 + 1], a, b2, b3);
        }
    }
    // mask, running maximum
    const int col0 = j0 + 2 * (lane & 3);
    float m_new[2] = {st.m[0], st.m[1]};
#pragma unroll
    for (int n = 0; n < BN / 8; ++n) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int r = e >> 1;
            const int j = col0 + n * 8 + (e & 1);
            const bool visible = j >= lo[r] && j <= hi[r];
            s[n][e] = visible ? s[n][e] * scale_log2 : -INFINITY;
            m_new[r] = fmaxf(m_new[r], s[n][e]);
        }
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        m_new[r] = fmaxf(m_new[r], __shfl_xor_sync(0xffffffffu, m_new[r], 1));
        m_new[r] = fmaxf(m_new[r], __shfl_xor_sync(0xffffffffu, m_new[r], 2));
    }
    float corr[2], m_use[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        m_use[r] = m_new[r] == -INFINITY ? 0.0f : m_new[r];  // a row that has seen no key yet
        corr[r] = exp2f(st.m[r] - m_use[r]);                  // exp2(-inf) = 0 on first contact
        st.m[r] = m_new[r];
    }
    float row_sum[2] = {0.0f, 0.0f};
    uint32_t p[BN / 16][4];  // P as A-operand tiles of 16 keys
#pragma unroll
    for (int n = 0; n < BN / 8; ++n) {
        const float p0 = exp2f(s[n][0] - m_use[0]), p1 = exp2f(s[n][1] - m_use[0]);
        const float p2 = exp2f(s[n][2] - m_use[1]), p3 = exp2f(s[n][3] - m_use[1]);
        row_sum[0] += p0 + p1;
        row_sum[1] += p2 + p3;
        // accumulator layout of two neighbouring n-tiles is the A layout of one k16 tile
        p[n >> 1][(n & 1) * 2 + 0] = pack_bf16(p0, p1);
        p[n >> 1][(n & 1) * 2 + 1] = pack_bf16(p2, p3);
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) st.l[r] = st.l[r] * corr[r] + row_sum[r];
#pragma unroll
    for (int n = 0; n < D / 8; ++n) {
        st.o[n][0] *= corr[0];
        st.o[n][1] *= corr[0];
        st.o[n][2] *= corr[1];
        st.o[n][3] *= corr[1];
    }
    // O += P V
#pragma unroll
    for (int kk = 0; kk < BN / 16; ++kk) {
#pragma unroll
        for (int n2 = 0; n2 < D / 16; ++n2) {
            // V rows are keys (k), columns head dims (n): transposed 8x8 loads give the col-major B operand
            uint32_t b0, b1, b2, b3;
            const int row = kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
            const int chunk = n2 * 2 + (lane >> 4);
            ldmatrix_x4_trans(v_smem + tile_offset<BN>(row, chunk), b0, b1, b2, b3);
            mma_bf16_16816(st.o[2 * n2], p[kk], b0, b1);
            mma_bf16_16816(st.o[2 * n2 + 1], p[kk], b2, b3);
        }
    }
}

// Fills one ring slot (K tile at k_dst, V tile at v_dst, `BN` keys from key t * BN on) by TMA, one
// box (a page, or part of one) per lane in turn; called by a whole warp.  Boxes without a page
// (past the last key, or given back by the window) hold masked keys only.
template <int BN, int PANELS>
__device__ __forceinline__ void fill_kv_slot(const CUtensorMap* kv_map, uint32_t bar, uint32_t k_dst, uint32_t v_dst, int t,
                                             int last_key, const int* table, int table_width, int num_pages,
                                             int kv_heads, int kv_head, int page_size, int box_rows, int lane) {
    // The warp that calls this sets the pace of the kernel it feeds (once per tile), so the pages are looked up
    // in one pass, a lane per box, and a page size that is a power of two is shifted by, not divided by.
    constexpr int PER_LANE = (BN + 31) / 32;  // boxes per lane when a box is one row
    const int boxes = BN / box_rows;
    const uint32_t box_bytes = (uint32_t)box_rows * 128u * PANELS;  // of K, and as much of V
    const bool shift = (page_size & (page_size - 1)) == 0;
    const int page_shift = __ffs(page_size) - 1;
    int row_k[PER_LANE];  // first cache row of this lane's boxes (K; V lies kv_heads * page_size further), or -1
    int count = 0;
#pragma unroll
    for (int k = 0; k < PER_LANE; ++k) {
        const int b = lane + 32 * k;
        row_k[k] = -1;
        if (b < boxes) {
            const int j = t * BN + b * box_rows;
            const int logical = shift ? j >> page_shift : j / page_size;
            const int page = (j <= last_key && logical < table_width) ? table[logical] : -1;
            if (page >= 0 && page < num_pages) row_k[k] = ((page * 2) * kv_heads + kv_head) * page_size + (j - logical * page_size);
        }
        count += __popc(__ballot_sync(0xffffffffu, row_k[k] >= 0));
    }
    // Boxes without a page (past the last key, or given back by the window): the warp clears their value rows
    // together (their keys are masked by position whatever they hold, but a value row is multiplied by its zero
    // weight and must be finite).  This happens before the barrier is armed, so that whoever passes the barrier
    // (another warp, in the prompt kernel) sees the cleared rows.
    if (count < boxes) {
#pragma unroll
        for (int k = 0; k < PER_LANE; ++k) {
            for (int owner = 0; owner < 32 && 32 * k + owner < boxes; ++owner) {
                if (__shfl_sync(0xffffffffu, row_k[k], owner) >= 0) continue;
                const int b = 32 * k + owner;
                for (int h = 0; h < PANELS; ++h) {
                    const uint32_t off = (uint32_t)(h * (BN * 128) + b * box_rows * 128);
                    for (int i = lane; i < box_rows * 8; i += 32)
                        asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(v_dst + off + i * 16), "r"(0u) : "memory");
                }
            }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
    }
    if (lane == 0) {
        if (count) sm100::mbar_expect_tx(bar, 2u * box_bytes * (uint32_t)count);
        else sm100::mbar_arrive(bar);
    }
    __syncwarp();
    const int value_rows = kv_heads * page_size;
#pragma unroll
    for (int k = 0; k < PER_LANE; ++k) {
        if (row_k[k] >= 0) {
            const int b = lane + 32 * k;
#pragma unroll
            for (int h = 0; h < PANELS; ++h) {
                const uint32_t off = (uint32_t)(h * (BN * 128) + b * box_rows * 128);
                sm100::tma_load_2d(k_dst + off, kv_map, bar, h * 64, row_k[k]);
                sm100::tma_load_2d(v_dst + off, kv_map, bar, h * 64, row_k[k] + value_rows);
            }
        }
    }
    __syncwarp();
}

// ------------------------------------------------------------------ prompt kernel
#define PF_WARPS 4      // consumer warps, 16 query rows each; one more warp feeds the ring
#define PF_ROWS 64
#define PF_BN 64
#define PF_STAGES 3

template <int D>
struct PrefillSmem {
    static constexpr int q_bytes = PF_ROWS * D * 2;
    static constexpr int tile_bytes = PF_BN * D * 2;
    static constexpr int ring_bytes = PF_STAGES * 2 * tile_bytes;
    static constexpr int total = q_bytes + ring_bytes + (2 * PF_STAGES + 1) * 8;  // no slack: the base must be 1024-aligned
    static constexpr int ctas_per_sm = (2 * (total + 1024) <= 227 * 1024) ? 2 : 1;
};

template <int D>
__global__ void __launch_bounds__((PF_WARPS + 1) * 32, PrefillSmem<D>::ctas_per_sm)
attention_prefill_kernel(const __grid_constant__ CUtensorMap kv_map, const bf16* __restrict__ q, bf16* __restrict__ out,
                         const int* __restrict__ block_table, const int* __restrict__ query_start,
                         const int* __restrict__ context_len, int q_heads, int kv_heads, int head_dim,
                         long q_row_stride, int page_size, int box_rows, int table_width, int num_pages, int window,
                         float scale_log2, int* __restrict__ error_flag) {
    pdl_launch_dependents();
    pdl_wait();
    using Smem = PrefillSmem<D>;
    constexpr int PANELS = D / 64;
    extern __shared__ __align__(1024) uint8_t smem[];
    // CTAs are handed out in the order of their linear index, x fastest: the kv heads are x and the row tiles y, last
    // tile first, so that of one prompt the tiles that see the most keys start first on every head, and the launch does
    // not end with a head's heavy tiles that were handed out late
    const int tile = gridDim.y - 1 - blockIdx.y;
    const int kv_head = blockIdx.x, req = blockIdx.z;
    const int group = q_heads / kv_heads;
    const int q_begin = query_start[req];
    const int q_len = query_start[req + 1] - q_begin;
    const int rows_total = q_len * group;
    const int row0 = tile * PF_ROWS;
    if (row0 >= rows_total) return;
    const uint32_t q_smem = sm100::smem_addr(smem);
    if (q_smem & 1023u) {  // the swizzled tiles need a 1024-byte aligned base: refuse rather than compute nonsense
        if (threadIdx.x == 0) atomicExch(error_flag, 5);
        return;
    }
    const int ctx = context_len[req];
    const int start_pos = ctx - q_len;  // position of the request's first new token
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t ring = q_smem + Smem::q_bytes;
    uint64_t* full_bar = (uint64_t*)(smem + Smem::q_bytes + Smem::ring_bytes);
    uint64_t* empty_bar = full_bar + PF_STAGES;
    uint64_t* q_free = empty_bar + PF_STAGES;  // the consumers have the query tile in registers

    if (tid == 0) {
        sm100::tma_prefetch_descriptor(&kv_map);
        for (int s = 0; s < PF_STAGES; ++s) {
            sm100::mbar_init(sm100::smem_addr(&full_bar[s]), 1);
            sm100::mbar_init(sm100::smem_addr(&empty_bar[s]), PF_WARPS);
        }
        sm100::mbar_init(sm100::smem_addr(q_free), PF_WARPS);
        sm100::mbar_fence_init();
    }
    // Q tile: row r is token (row0 + r) / group, head kv_head * group + (row0 + r) % group
    {
        constexpr int CH = D / 8;
        const int chunks_used = head_dim / 8;
        for (int id = tid; id < PF_ROWS * CH; id += (PF_WARPS + 1) * 32) {
            const int r = id / CH, chunk = id % CH;
            const int row = row0 + r;
            uint4 value = make_uint4(0u, 0u, 0u, 0u);
            if (row < rows_total && chunk < chunks_used) {
                const int token = row / group, head = kv_head * group + row % group;
                value = *reinterpret_cast<const uint4*>(q + (size_t)(q_begin + token) * q_row_stride + (size_t)head * head_dim + chunk * 8);
            }
            *reinterpret_cast<uint4*>(smem + tile_offset<PF_ROWS>(r, chunk)) = value;
        }
    }
    __syncthreads();

    const int last_row = min(rows_total, row0 + PF_ROWS) - 1;
    const int pos_first = start_pos + row0 / group;
    const int pos_last = start_pos + last_row / group;
    const int key_lo = window > 0 ? max(0, pos_first - window + 1) : 0;
    const int first_tile = key_lo / PF_BN, last_tile = pos_last / PF_BN;
    const int num_tiles = last_tile - first_tile + 1;
    bool ok = true;

    if (warp == PF_WARPS) {
        // producer: keeps the ring full.  Once the consumers hold the query tile in registers its
        // shared memory is free, and the pages of this CTA's keys are copied there: a lookup in global
        // memory for every tile would put its latency in front of every TMA issue.
        const int* table = block_table + (long)req * table_width;
        if (D <= 128) {
            int* table_s = reinterpret_cast<int*>(smem);
            const int first_page = (first_tile * PF_BN) / page_size;
            const int last_page = min(table_width - 1, pos_last / page_size);
            if (last_page - first_page < Smem::q_bytes / 4 && sm100::mbar_wait(sm100::smem_addr(q_free), 0)) {
                for (int i = first_page + lane; i <= last_page; i += 32) table_s[i - first_page] = table[i];
                table = table_s - first_page;
                __syncwarp();
            }
        }
        for (int it = 0; it < num_tiles; ++it) {
            const int slot = it % PF_STAGES;
            if (it >= PF_STAGES && !sm100::mbar_wait(sm100::smem_addr(&empty_bar[slot]), (uint32_t)(it / PF_STAGES - 1) & 1u)) {
                ok = false;
                break;
            }
            const uint32_t k_dst = ring + slot * 2 * Smem::tile_bytes;
            fill_kv_slot<PF_BN, PANELS>(&kv_map, sm100::smem_addr(&full_bar[slot]), k_dst, k_dst + Smem::tile_bytes,
                                        first_tile + it, pos_last, table, table_width, num_pages, kv_heads, kv_head,
                                        page_size, box_rows, lane);
        }
        if (!ok && lane == 0) atomicExch(error_flag, 4);
        return;
    }

    // consumers: per-thread rows g and g + 8 of this warp's 16
    int lo[2], hi[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = row0 + warp * 16 + (lane >> 2) + r * 8;
        if (row < rows_total) {
            const int pos = start_pos + row / group;
            hi[r] = pos;
            lo[r] = window > 0 ? max(0, pos - window + 1) : 0;
        } else {
            hi[r] = -1;
            lo[r] = 0;  // sees nothing
        }
    }
    constexpr bool Q_IN_REGS = D <= 128;
    uint32_t q_regs[Q_IN_REGS ? D / 16 : 1][4];
    if (Q_IN_REGS) {
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
            ldmatrix_x4(q_smem + tile_offset<PF_ROWS>(warp * 16 + (lane & 15), kk * 2 + (lane >> 4)), q_regs[kk][0],
                        q_regs[kk][1], q_regs[kk][2], q_regs[kk][3]);
        __syncwarp();
        if (lane == 0) sm100::mbar_arrive(sm100::smem_addr(q_free));
    }
    WarpState<D> st;
    st.init();
    const int warp_first_row = row0 + warp * 16;
    const int warp_last_row = min(rows_total - 1, warp_first_row + 15);
    const int warp_pos_last = warp_first_row < rows_total ? start_pos + warp_last_row / group : -1;
    const int warp_key_lo = (window > 0 && warp_first_row < rows_total) ? max(0, start_pos + warp_first_row / group - window + 1) : 0;
    for (int it = 0; it < num_tiles; ++it) {
        const int slot = it % PF_STAGES;
        const int t = first_tile + it;
        if (!sm100::mbar_wait(sm100::smem_addr(&full_bar[slot]), (uint32_t)(it / PF_STAGES) & 1u)) {
            ok = false;
            break;
        }
        // a warp whose rows all lie before this tile, or whose windows all start after it, adds nothing
        const bool warp_active = warp_pos_last >= t * PF_BN && warp_key_lo < (t + 1) * PF_BN;
        if (warp_active) {
            const uint32_t k_s = ring + slot * 2 * Smem::tile_bytes;
            warp_attend<D, PF_BN, PF_ROWS, Q_IN_REGS>(st, q_smem, warp * 16, q_regs, k_s, k_s + Smem::tile_bytes, t * PF_BN, lo, hi,
                                                     scale_log2, lane);
        }
        __syncwarp();
        if (lane == 0) sm100::mbar_arrive(sm100::smem_addr(&empty_bar[slot]));
    }
    if (!ok && lane == 0) atomicExch(error_flag, 4);
    // normalise and store
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        float l = st.l[r];
        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
        const int row = row0 + warp * 16 + (lane >> 2) + r * 8;
        if (row >= rows_total) continue;
        const float inv = l > 0.0f ? 1.0f / l : 0.0f;
        const int token = row / group, head = kv_head * group + row % group;
        bf16* dst = out + ((size_t)(q_begin + token) * q_heads + head) * head_dim;
#pragma unroll
        for (int n = 0; n < D / 8; ++n) {
            const int col = n * 8 + 2 * (lane & 3);
            if (col < head_dim)
                *reinterpret_cast<uint32_t*>(dst + col) = pack_bf16(st.o[n][2 * r] * inv, st.o[n][2 * r + 1] * inv);
        }
    }
}

__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
    return d;
}

// The decode kernel's state when the keys, not the (few) query heads, fill the 16 rows of the
// MMA: scores are S^T[key, head] = K Q^T and the output is O^T[dim, head] = V^T P^T, with the
// heads (at most 8) as the 8 columns.  A thread holds heads 2t and 2t + 1 (t = lane % 4).
template <int D>
struct HeadState {
    float m[2], l[2];
    float o[D / 16][4];  // m-tile i: (dim 16 i + g, heads 2t, 2t+1), (dim 16 i + g + 8, heads 2t, 2t+1)
    __device__ __forceinline__ void init() {
        m[0] = m[1] = -INFINITY;
        l[0] = l[1] = 0.0f;
#pragma unroll
        for (int i = 0; i < D / 16; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
    }
};

// Folds BN keys (first key j0) into the state; every head sees key j when lo <= j <= hi.
// q_b[kk] are the B-operand fragments of Q^T for dims 16 kk .. 16 kk + 15.
template <int D, int BN>
__device__ __forceinline__ void warp_attend_heads(HeadState<D>& st, const uint32_t (*q_b)[2], uint32_t k_smem,
                                                  uint32_t v_smem, int j0, int lo, int hi, float scale_log2, int lane) {
    constexpr int MT = BN / 16;
    float s[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
        s[mt][0] = s[mt][1] = s[mt][2] = s[mt][3] = 0.0f;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
            uint32_t a[4];
            ldmatrix_x4(k_smem + tile_offset<BN>(mt * 16 + (lane & 15), kk * 2 + (lane >> 4)), a[0], a[1], a[2], a[3]);
            mma_bf16_16816(s[mt], a, q_b[kk][0], q_b[kk][1]);
        }
    }
    // mask by key position (rows g and g + 8 of each m-tile), running maximum per head
    const int g = lane >> 2;
    const bool interior = j0 >= lo && j0 + BN - 1 <= hi;
    float m_new[2] = {st.m[0], st.m[1]};
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int j = j0 + mt * 16 + g + (e >> 1) * 8;
            const bool visible = interior || (j >= lo && j <= hi);
            s[mt][e] = visible ? s[mt][e] * scale_log2 : -INFINITY;
            m_new[e & 1] = fmaxf(m_new[e & 1], s[mt][e]);
        }
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        m_new[h] = fmaxf(m_new[h], __shfl_xor_sync(0xffffffffu, m_new[h], 4));
        m_new[h] = fmaxf(m_new[h], __shfl_xor_sync(0xffffffffu, m_new[h], 8));
        m_new[h] = fmaxf(m_new[h], __shfl_xor_sync(0xffffffffu, m_new[h], 16));
    }
    float corr[2], m_use[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        m_use[h] = m_new[h] == -INFINITY ? 0.0f : m_new[h];
        corr[h] = exp2f(st.m[h] - m_use[h]);
        st.m[h] = m_new[h];
    }
    uint32_t p_b[MT][2];  // P^T as B-operand fragments, one k16 step per m-tile of keys
    float sum[2] = {0.0f, 0.0f};
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
        const float p0 = exp2f(s[mt][0] - m_use[0]), p1 = exp2f(s[mt][1] - m_use[1]);
        const float p2 = exp2f(s[mt][2] - m_use[0]), p3 = exp2f(s[mt][3] - m_use[1]);
        sum[0] += p0 + p2;
        sum[1] += p1 + p3;
        // (key g, heads 2t, 2t+1) -> (keys 2t, 2t+1, head g): the transposed 8 x 8 block is the B fragment
        p_b[mt][0] = movmatrix_trans(pack_bf16(p0, p1));
        p_b[mt][1] = movmatrix_trans(pack_bf16(p2, p3));
    }
    st.l[0] = st.l[0] * corr[0] + sum[0];
    st.l[1] = st.l[1] * corr[1] + sum[1];
    // the running maximum settles after a few tiles: skip the rescaling when nothing changed
    if (__any_sync(0xffffffffu, corr[0] != 1.0f || corr[1] != 1.0f)) {
#pragma unroll
        for (int i = 0; i < D / 16; ++i) {
            st.o[i][0] *= corr[0];
            st.o[i][1] *= corr[1];
            st.o[i][2] *= corr[0];
            st.o[i][3] *= corr[1];
        }
    }
    // O^T += V^T P^T: A = V^T (dims x keys) through transposed 8 x 8 loads of the [key][dim] tile
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
        for (int i = 0; i < D / 16; ++i) {
            uint32_t a[4];
            const int row = mt * 16 + (lane & 7) + ((lane >> 4) << 3);
            const int chunk = 2 * i + ((lane >> 3) & 1);
            ldmatrix_x4_trans(v_smem + tile_offset<BN>(row, chunk), a[0], a[1], a[2], a[3]);
            mma_bf16_16816(st.o[i], a, p_b[mt][0], p_b[mt][1]);
        }
    }
}

// ------------------------------------------------------------------ decode kernel
#define DC_STAGES 3
// Keys per warp tile: 16 (one page at the usual page size); eight warps, four for the widest heads so that the
// warps' rings fit shared memory.
template <int D>
struct DecodeTile {
    static constexpr int BN = 16;
    static constexpr int WARPS = D > 128 ? 4 : 8;
};

// Shared memory of the decode kernel: the query tile, per warp a ring of DC_STAGES (K tile, V tile)
// filled by TMA, one mbarrier per ring slot; after the key loop the ring is reused to merge the warps.
template <int D>
struct DecodeSmem {
    static constexpr int BN = DecodeTile<D>::BN;
    static constexpr int DC_WARPS = DecodeTile<D>::WARPS;
    static constexpr int q_bytes = 16 * D * 2;
    static constexpr int tile_bytes = BN * D * 2;
    static constexpr int ring_bytes = DC_WARPS * DC_STAGES * 2 * tile_bytes;
    static constexpr int merge_bytes = DC_WARPS * 16 * (D + 2) * 4;
    static constexpr int body = q_bytes + (ring_bytes > merge_bytes ? ring_bytes : merge_bytes);
    static constexpr int table_entries = 1024;  // block-table entries kept in shared memory (longer ranges read global memory)
    static constexpr int prefix_entries = 1025;  // balanced kernel: where each request's tiles start (up to 1,024 requests)
    static constexpr int rope_offset = body + DC_WARPS * DC_STAGES * 8 + table_entries * 4 + prefix_entries * 4 + 12;  // 16-byte aligned
    // fused q/k preparation: cos [D / 2], sin [D / 2] of the request's position, then the q and the k norm's weights [D] each
    static constexpr int rope_bytes = 3 * D * 4;
    static_assert(rope_offset % 16 == 0, "the cosines are read in 16-byte pieces");
    // a pair of CTAs that shares a (request, kv head): the second CTA's rows, written by it into the first CTA's
    // shared memory; outside the ring, which the first CTA may still be streaming through (heads up to 128 only:
    // wider heads leave no room)
    static constexpr int pair_offset = rope_offset + rope_bytes;
    static constexpr int pair_bytes = D <= 128 ? 16 * (D + 2) * 4 : 0;
    static constexpr int total = pair_offset + pair_bytes + 1024;  // + slack to align to 1024
};

// What a decode CTA needs to attend one range of key tiles of one (request, kv head).
struct DecodeArgs {
    const bf16* q;
    const int* block_table;
    int q_heads, kv_heads, head_dim;
    long q_row_stride;
    int page_size, box_rows, table_width, num_pages, window;
    float scale_log2;
    int* error_flag;
    // Fused preparation (fuse != 0; head_dim is then the template's D): q points to the rows that the q, k, v product
    // left, [requests, (q_heads + 2 kv_heads) * head_dim] with row stride q_row_stride, untouched.  Every CTA norms and
    // rotates its group's query rows on the way into shared memory; the warp that takes the request's last key tile
    // norms and rotates the new token's key, puts it and the value into that tile in shared memory and into their
    // page (cache) for the steps to come.  Null weights skip the norm, null inv_freq the rotation.
    int fuse;
    const float* q_weight;
    const float* k_weight;
    const float* inv_freq;
    float eps;
    bf16* cache;
    unsigned long long* stamps;  // null, or [CTAs][8] clock stamps (ns) of the decode kernel, for measurements
};

// Clock stamps of one CTA of the decode kernel (split form), written only when a buffer is given: 0 the CTA starts,
// 1 the kernel before has finished, 2 the queries are in shared memory, 3 the warps have attended their tiles,
// 4 the CTA's result is merged and stored.
__device__ __forceinline__ void decode_stamp(const DecodeArgs& args, int which) {
    if (args.stamps && threadIdx.x == 0) {
        unsigned long long now;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
        const size_t cta = ((size_t)blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;
        args.stamps[cta * 8 + which] = now;
    }
}

// Per-head RMSNorm and half-split rotation of the sixteen values that a lane holds of one head (eight adjacent values of
// each half; LANES = D / 16 lanes share a head), the arithmetic of qk_norm_rope_kv_write_wide_kernel in elementwise.cu:
// statistics, scale, weights and angles in 32-bit, one rounding to bf16 at the end.  Called by whole warps.
template <int D>
__device__ __forceinline__ void prepare_head(uint4& lo_raw, uint4& hi_raw, const float* __restrict__ weight,
                                             const float* rope_s, bool rotate, float eps, int sub) {
    constexpr int LANES = D / 16, HALF = D / 2;
    float lo[8], hi[8];
    {
        const __nv_bfloat162* pl = reinterpret_cast<const __nv_bfloat162*>(&lo_raw);
        const __nv_bfloat162* ph = reinterpret_cast<const __nv_bfloat162*>(&hi_raw);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 a = __bfloat1622float2(pl[j]), b = __bfloat1622float2(ph[j]);
            lo[2 * j] = a.x, lo[2 * j + 1] = a.y, hi[2 * j] = b.x, hi[2 * j + 1] = b.y;
        }
    }
    if (weight) {
        float acc = 0.0f;
#pragma unroll
        for (int j = 0; j < 8; ++j) acc = fmaf(lo[j], lo[j], fmaf(hi[j], hi[j], acc));
#pragma unroll
        for (int d = 1; d < LANES; d <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, d);
        const float variance = acc / (float)D + eps;
        const float scale = variance == 0.0f ? 0.0f : 1.0f / sqrtf(variance);
        const float4* wl = reinterpret_cast<const float4*>(weight + 8 * sub);
        const float4* wh = reinterpret_cast<const float4*>(weight + HALF + 8 * sub);
        const float4 w0 = wl[0], w1 = wl[1], w2 = wh[0], w3 = wh[1];
        const float wlo[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
        const float whi[8] = {w2.x, w2.y, w2.z, w2.w, w3.x, w3.y, w3.z, w3.w};
#pragma unroll
        for (int j = 0; j < 8; ++j) lo[j] = lo[j] * scale * wlo[j], hi[j] = hi[j] * scale * whi[j];
    }
    if (rotate) {
        const float4* cs = reinterpret_cast<const float4*>(rope_s + 8 * sub);
        const float4* sn = reinterpret_cast<const float4*>(rope_s + HALF + 8 * sub);
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
    __nv_bfloat162* pl = reinterpret_cast<__nv_bfloat162*>(&lo_raw);
    __nv_bfloat162* ph = reinterpret_cast<__nv_bfloat162*>(&hi_raw);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        pl[j] = __floats2bfloat162_rn(lo[2 * j], lo[2 * j + 1]);
        ph[j] = __floats2bfloat162_rn(hi[2 * j], hi[2 * j + 1]);
    }
}

__device__ __forceinline__ void st_shared_16(uint32_t address, const uint4& v) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(address), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// The new token's key (normed, rotated) and value into row `pos % BN` of the tile at k_s / v_s, which TMA has just
// filled from the pages, and into the token's page.  Called by the whole warp that is about to attend that tile.
template <int D, int BN>
__device__ __forceinline__ void append_new_token(const DecodeArgs& args, const float* rope_s, const float* k_weight, const int* table, int req,
                                                 int kv_head, int pos, uint32_t k_s, uint32_t v_s, int lane) {
    constexpr int LANES = D / 16;
    const int row = pos % BN;
    const bf16* x = args.q + (size_t)req * args.q_row_stride;
    const int logical = pos / args.page_size;
    int page = logical < args.table_width ? table[logical] : -1;
    if (page < 0 || page >= args.num_pages) {
        if (lane == 0) atomicExch(args.error_flag, KIRAI_FLAG_NO_PAGE_WRITE);
        page = -1;
    }
    const long slot_rows = (long)(pos % args.page_size);
    // cache layer [pages][2][kv_heads][page_size][D]
    bf16* k_dst = page < 0 ? nullptr : args.cache + ((((long)page * 2 + 0) * args.kv_heads + kv_head) * args.page_size + slot_rows) * D;
    bf16* v_dst = page < 0 ? nullptr : args.cache + ((((long)page * 2 + 1) * args.kv_heads + kv_head) * args.page_size + slot_rows) * D;
    const bool k_live = lane < LANES;
    const uint4* xk = reinterpret_cast<const uint4*>(x + (size_t)(args.q_heads + kv_head) * D);
    uint4 lo = make_uint4(0u, 0u, 0u, 0u), hi = lo;
    if (k_live) {
        lo = xk[lane];
        hi = xk[lane + LANES];
    }
    prepare_head<D>(lo, hi, k_weight, rope_s, args.inv_freq != nullptr, args.eps, lane % LANES);
    if (k_live) {
        st_shared_16(k_s + tile_offset<BN>(row, lane), lo);
        st_shared_16(k_s + tile_offset<BN>(row, lane + LANES), hi);
        if (k_dst) {
            reinterpret_cast<uint4*>(k_dst)[lane] = lo;
            reinterpret_cast<uint4*>(k_dst)[lane + LANES] = hi;
        }
    }
    const uint4* xv = reinterpret_cast<const uint4*>(x + (size_t)(args.q_heads + args.kv_heads + kv_head) * D);
    for (int chunk = lane; chunk < D / 8; chunk += 32) {
        const uint4 value = xv[chunk];
        st_shared_16(v_s + tile_offset<BN>(row, chunk), value);
        if (v_dst) reinterpret_cast<uint4*>(v_dst)[chunk] = value;
    }
    __syncwarp();
}

// The CTA's warps attend key tiles [t_begin, t_end) of (req, kv_head) for the query at position pos (the keys from
// key_lo on; last_tile holds pos) and merge their states.  The result for the group's heads goes, unnormalised with
// its maximum and sum, to dst_partial (row g at dst_partial + g * partial_stride: head_dim values, max, sum), or, if
// dst_partial is null, normalised to `out`.  k_base: how many tiles this warp has put through its ring before (the
// barriers' phases go on from there); the number for the next call is returned.  With `first` the call is the
// CTA's first work: the tiles that earlier steps filled are requested before griddepcontrol.wait, the rest after.
template <int D, bool HEADS>
__device__ __forceinline__ int decode_attend_range(const CUtensorMap& kv_map, const DecodeArgs& args, uint8_t* smem, int req,
                                                   int kv_head, int pos, int key_lo, int last_tile, int t_begin, int t_end,
                                                   int k_base, bool first, bf16* __restrict__ out,
                                                   float* __restrict__ dst_partial, long partial_stride) {
    using Smem = DecodeSmem<D>;
    constexpr int BN = Smem::BN;
    constexpr int DC_WARPS = Smem::DC_WARPS;
    constexpr int PANELS = D / 64;
    const int q_heads = args.q_heads, kv_heads = args.kv_heads, head_dim = args.head_dim;
    const int page_size = args.page_size, table_width = args.table_width;
    const float scale_log2 = args.scale_log2;
    const int group = q_heads / kv_heads;  // <= 16 rows
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t q_smem = sm100::smem_addr(smem);
    const uint32_t ring = q_smem + Smem::q_bytes + warp * DC_STAGES * 2 * Smem::tile_bytes;
    uint64_t* bars = (uint64_t*)(smem + Smem::body) + warp * DC_STAGES;
    float* merge = reinterpret_cast<float*>(smem + Smem::q_bytes);  // [warps][16][D + 2], over the ring

    // What the set-up reads from global memory (block table, rotation frequencies, norm weights) is constant during a
    // step and is asked for in one go, before anything waits for any of it: a CTA that starts late (its SM was busy
    // with the kernel before) has these round trips in front of its first key tile, one after the other if each
    // load waited for the one before.
    constexpr int THREADS = DC_WARPS * 32;
    constexpr int PER_THREAD = (D + THREADS - 1) / THREADS;
    float* rope_s = reinterpret_cast<float*>(smem + Smem::rope_offset);
    float* q_weight_s = args.q_weight ? rope_s + D : nullptr;
    float* k_weight_s = args.k_weight ? rope_s + 2 * D : nullptr;
    const bool rotate = args.fuse && args.inv_freq;
    float freq[PER_THREAD], wq[PER_THREAD], wk[PER_THREAD];
#pragma unroll
    for (int i = 0; i < PER_THREAD; ++i) {
        const int d = tid + i * THREADS;
        freq[i] = rotate && d < D / 2 ? args.inv_freq[d] : 0.0f;
        wq[i] = args.fuse && first && q_weight_s && d < D ? args.q_weight[d] : 0.0f;
        wk[i] = args.fuse && first && k_weight_s && d < D ? args.k_weight[d] : 0.0f;
    }
    // The pages of this request's keys: copied to shared memory once, because a lookup in global memory for every
    // tile would put its latency in front of every TMA issue.  A table that fits is copied whole, which needs no
    // context length; of a longer one this range's part.
    const int* table = args.block_table + (long)req * table_width;
    {
        int* table_s = reinterpret_cast<int*>(smem + Smem::body + DC_WARPS * DC_STAGES * 8);
        if (table_width <= Smem::table_entries) {
            for (int i = tid; i < table_width; i += THREADS) table_s[i] = table[i];
            table = table_s;
        } else {
            const int first_page = (t_begin * BN) / page_size;
            const int last_page = min(table_width - 1, (min(t_end, last_tile + 1) * BN - 1) / page_size);
            if (last_page - first_page < Smem::table_entries) {
                for (int i = first_page + tid; i <= last_page; i += THREADS) table_s[i - first_page] = table[i];
                table = table_s - first_page;
            }
        }
    }
    bool ok = true;
#pragma unroll
    for (int i = 0; i < PER_THREAD; ++i) {
        const int d = tid + i * THREADS;
        // the angles depend on the position only
        if (rotate && d < D / 2) sincosf((float)pos * freq[i], &rope_s[D / 2 + d], &rope_s[d]);
        if (args.fuse && first && d < D) {
            if (q_weight_s) q_weight_s[d] = wq[i];
            if (k_weight_s) k_weight_s[d] = wk[i];
        }
    }
    __syncthreads();  // the table is in place (and, for the query rows further down, angles and weights)
    // Fills ring slot `slot` with key tile `t`.
    auto issue = [&](int t, int slot) {
        const uint32_t k_dst = ring + slot * 2 * Smem::tile_bytes;
        fill_kv_slot<BN, PANELS>(&kv_map, sm100::smem_addr(&bars[slot]), k_dst, k_dst + Smem::tile_bytes, t, pos, table,
                                 table_width, args.num_pages, kv_heads, kv_head, page_size, args.box_rows, lane);
    };

    // this warp's tiles: t_begin + warp, + DC_WARPS, ...; the ring holds DC_STAGES of them: a slot is asked for the tile
    // DC_STAGES further on as soon as its tile has been attended
    const int my_first = t_begin + warp;
    const int my_count = my_first < t_end ? (t_end - my_first + DC_WARPS - 1) / DC_WARPS : 0;
    // Everything up to here read only what is constant during a step (context lengths, block tables).  Keys and
    // values of earlier steps are constant too: the first tiles of the ring are fetched before the kernel before
    // this one has finished, all but the request's last tile, which holds the token that this step appends.
    uint32_t early = 0u;
    if (first) {
        for (int k = 0; k < DC_STAGES && k < my_count; ++k) {
            if (my_first + k * DC_WARPS < last_tile) {
                issue(my_first + k * DC_WARPS, (k_base + k) % DC_STAGES);
                early |= 1u << k;
            }
        }
        pdl_wait();  // the queries, and the new token's key and value, are complete and visible
        decode_stamp(args, 1);
    }
    // the query rows (the group's heads), zero beyond the group and beyond head_dim
    if (args.fuse) {
        // raw rows of the q, k, v product: normed and rotated on the way in (head_dim == D here)
        constexpr int CH = D / 8, LANES = D / 16, HEADS_PER_WARP = 32 / LANES;
        for (int id = tid; id < (16 - group) * CH; id += DC_WARPS * 32)
            *reinterpret_cast<uint4*>(smem + tile_offset<16>(group + id / CH, id % CH)) = make_uint4(0u, 0u, 0u, 0u);
        for (int base = warp * HEADS_PER_WARP; base < group; base += DC_WARPS * HEADS_PER_WARP) {
            const int r = base + lane / LANES, sub = lane % LANES;
            const bool live = r < group;
            const uint4* x = reinterpret_cast<const uint4*>(args.q + (size_t)req * args.q_row_stride + (size_t)(kv_head * group + (live ? r : 0)) * D);
            uint4 lo = make_uint4(0u, 0u, 0u, 0u), hi = lo;
            if (live) {
                lo = x[sub];
                hi = x[sub + LANES];
            }
            prepare_head<D>(lo, hi, q_weight_s, rope_s, args.inv_freq != nullptr, args.eps, sub);
            if (live) {
                *reinterpret_cast<uint4*>(smem + tile_offset<16>(r, sub)) = lo;
                *reinterpret_cast<uint4*>(smem + tile_offset<16>(r, sub + LANES)) = hi;
            }
        }
    } else {
        constexpr int CH = D / 8;
        const int chunks_used = head_dim / 8;
        for (int id = tid; id < 16 * CH; id += DC_WARPS * 32) {
            const int r = id / CH, chunk = id % CH;
            uint4 value = make_uint4(0u, 0u, 0u, 0u);
            if (r < group && chunk < chunks_used)
                value = *reinterpret_cast<const uint4*>(args.q + (size_t)req * args.q_row_stride + (size_t)(kv_head * group + r) * head_dim + chunk * 8);
            *reinterpret_cast<uint4*>(smem + tile_offset<16>(r, chunk)) = value;
        }
    }
    __syncthreads();
    decode_stamp(args, 2);

    constexpr int MS = D + 2;
    if (HEADS) {
        // B-operand fragments of Q^T: (dims 16 kk + 2t, + 1 and + 8; head g), read once
        uint32_t q_b[D / 16][2];
        {
            const int g = lane >> 2, t = lane & 3;
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
                q_b[kk][0] = *reinterpret_cast<const uint32_t*>(smem + tile_offset<16>(g, 2 * kk) + 4 * t);
                q_b[kk][1] = *reinterpret_cast<const uint32_t*>(smem + tile_offset<16>(g, 2 * kk + 1) + 4 * t);
            }
        }
        HeadState<D> st;
        st.init();
        for (int k = 0; k < DC_STAGES && k < my_count; ++k)
            if (!((early >> k) & 1u)) issue(my_first + k * DC_WARPS, (k_base + k) % DC_STAGES);
        for (int k = 0; k < my_count; ++k) {
            const int slot = (k_base + k) % DC_STAGES;
            if (!sm100::mbar_wait(sm100::smem_addr(&bars[slot]), (uint32_t)((k_base + k) / DC_STAGES) & 1u)) {
                ok = false;
                break;
            }
            const uint32_t k_s = ring + slot * 2 * Smem::tile_bytes;
            if (args.fuse && my_first + k * DC_WARPS == last_tile)
                append_new_token<D, BN>(args, rope_s, k_weight_s, table, req, kv_head, pos, k_s, k_s + Smem::tile_bytes, lane);
            warp_attend_heads<D, BN>(st, q_b, k_s, k_s + Smem::tile_bytes, (my_first + k * DC_WARPS) * BN, key_lo, pos, scale_log2, lane);
            __syncwarp();
            if (k + DC_STAGES < my_count) issue(my_first + (k + DC_STAGES) * DC_WARPS, slot);
        }
        if (!ok && lane == 0) atomicExch(args.error_flag, 4);
        __syncthreads();  // every warp is done with its ring: it becomes the merge buffer
        decode_stamp(args, 3);
        const int g = lane >> 2, t = lane & 3;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            float l = st.l[h];
            l += __shfl_xor_sync(0xffffffffu, l, 4);
            l += __shfl_xor_sync(0xffffffffu, l, 8);
            l += __shfl_xor_sync(0xffffffffu, l, 16);
            float* dst = merge + ((size_t)warp * 16 + (2 * t + h)) * MS;
#pragma unroll
            for (int i = 0; i < D / 16; ++i) {
                dst[16 * i + g] = st.o[i][h];
                dst[16 * i + g + 8] = st.o[i][2 + h];
            }
            if (g == 0) {
                dst[D] = st.m[h];
                dst[D + 1] = l;
            }
        }
    } else {
    int lo[2], hi[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = (lane >> 2) + r * 8;
        hi[r] = row < group ? pos : -1;
        lo[r] = key_lo;
    }
    // query fragments stay in registers for the narrower heads
    constexpr bool Q_IN_REGS = D <= 128;
    uint32_t q_regs[Q_IN_REGS ? D / 16 : 1][4];
    if (Q_IN_REGS) {
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
            ldmatrix_x4(q_smem + tile_offset<16>(lane & 15, kk * 2 + (lane >> 4)), q_regs[kk][0], q_regs[kk][1], q_regs[kk][2], q_regs[kk][3]);
    }
    WarpState<D> st;
    st.init();
    for (int k = 0; k < DC_STAGES && k < my_count; ++k)
            if (!((early >> k) & 1u)) issue(my_first + k * DC_WARPS, (k_base + k) % DC_STAGES);
    for (int k = 0; k < my_count; ++k) {
        const int slot = (k_base + k) % DC_STAGES;
        if (!sm100::mbar_wait(sm100::smem_addr(&bars[slot]), (uint32_t)((k_base + k) / DC_STAGES) & 1u)) {
            ok = false;
            break;
        }
        const uint32_t k_s = ring + slot * 2 * Smem::tile_bytes;
        if (args.fuse && my_first + k * DC_WARPS == last_tile)
            append_new_token<D, BN>(args, rope_s, k_weight_s, table, req, kv_head, pos, k_s, k_s + Smem::tile_bytes, lane);
        warp_attend<D, BN, 16, Q_IN_REGS>(st, q_smem, 0, q_regs, k_s, k_s + Smem::tile_bytes, (my_first + k * DC_WARPS) * BN, lo, hi,
                                          scale_log2, lane);
        __syncwarp();
        if (k + DC_STAGES < my_count) issue(my_first + (k + DC_STAGES) * DC_WARPS, slot);
    }
    if (!ok && lane == 0) atomicExch(args.error_flag, 4);
    __syncthreads();  // every warp is done with its ring: it becomes the merge buffer
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        float l = st.l[r];
        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
        const int row = (lane >> 2) + r * 8;
        float* dst = merge + ((size_t)warp * 16 + row) * MS;
#pragma unroll
        for (int n = 0; n < D / 8; ++n) {
            const int col = n * 8 + 2 * (lane & 3);
            dst[col] = st.o[n][2 * r];
            dst[col + 1] = st.o[n][2 * r + 1];
        }
        if ((lane & 3) == 0) {
            dst[D] = st.m[r];
            dst[D + 1] = l;
        }
    }
    }
    __syncthreads();
    for (int id = tid; id < group * head_dim; id += DC_WARPS * 32) {
        const int row = id / head_dim, col = id % head_dim;
        float m_all = -INFINITY;
#pragma unroll
        for (int w = 0; w < DC_WARPS; ++w) m_all = fmaxf(m_all, merge[((size_t)w * 16 + row) * MS + D]);
        float acc = 0.0f, l_all = 0.0f;
#pragma unroll
        for (int w = 0; w < DC_WARPS; ++w) {
            const float* src = merge + ((size_t)w * 16 + row) * MS;
            const float weight = src[D] == -INFINITY ? 0.0f : exp2f(src[D] - m_all);
            acc += src[col] * weight;
            l_all += src[D + 1] * weight;
        }
        if (dst_partial == nullptr) {
            out[((size_t)req * q_heads + kv_head * group + row) * head_dim + col] = from_f32<bf16>(l_all > 0.0f ? acc / l_all : 0.0f);
        } else {
            float* dst = dst_partial + (size_t)row * partial_stride;
            dst[col] = acc;
            if (col == 0) {
                dst[head_dim] = m_all;
                dst[head_dim + 1] = l_all;
            }
        }
    }
    return k_base + my_count;
}

// One barrier per ring slot and warp; called by every thread before the first range.
template <int D>
__device__ __forceinline__ void decode_init_barriers(uint8_t* smem) {
    using Smem = DecodeSmem<D>;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint64_t* bars = (uint64_t*)(smem + Smem::body) + warp * DC_STAGES;
    if (lane == 0) {
        for (int s = 0; s < DC_STAGES; ++s) sm100::mbar_init(sm100::smem_addr(&bars[s]), 1);
        sm100::mbar_fence_init();
    }
    __syncthreads();
}

// partial: [requests, q_heads, splits, head_dim + 2] floats: unnormalised output, then max (log2 domain), then sum.
// kv_map: the cache layer as a 2-D bf16 matrix [num_pages * 2 * kv_heads * page_size, head_dim], boxes of
// [box_rows, 64] with the 128-byte swizzle; box_rows = min(page_size, BN) and divides BN.
// HEADS: the group has at most 8 heads and they are the MMA's columns (keys fill its rows);
// otherwise the group's (at most 16) heads are the rows, as in the prompt kernel.
// Grid (splits, kv_heads, requests): every request's keys are cut into the same number of ranges.
// The ranges' partial results go through `partial` and attention_merge_splits_kernel.  (Merging them inside this
// kernel was built twice and taken out again: as thread-block clusters through distributed shared memory, which must
// be placed inside one GPC and therefore started late beside the product before them, 3.07 against 3.00 ms a step at
// one request and 8 ranges, equal at 8 requests; and by the CTA of a pair that finishes last, behind a fence and a
// counter, 3.06 against 2.98 ms at 16 ranges.)
// PAIR: two to five ranges, whose CTAs are a thread-block cluster.  Every CTA but the first writes its rows straight
// into a slot of its own in the first CTA's shared memory (its last loop stores through a pointer mapped to the first
// CTA), the cluster meets once, and the first CTA adds its own rows and the slots', in rank order and with the
// arithmetic of attention_merge_splits_kernel, and stores the result: no buffer in global memory and no second kernel,
// whose way through a kernel boundary cost 4.5 us a layer at 8 requests.  The slots (group rows each) share
// DecodeSmem::pair_bytes, which the launch checks.
template <int D, bool HEADS, bool PAIR>
__global__ void __launch_bounds__(DecodeTile<D>::WARPS * 32)
attention_decode_kernel(const __grid_constant__ CUtensorMap kv_map, DecodeArgs args, bf16* __restrict__ out,
                        float* __restrict__ partial, const int* __restrict__ context_len, int num_splits) {
    pdl_launch_dependents();
    decode_stamp(args, 0);
    using Smem = DecodeSmem<D>;
    constexpr int BN = Smem::BN;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const int split = blockIdx.x, kv_head = blockIdx.y, req = blockIdx.z;
    const int group = args.q_heads / args.kv_heads;
    const int pos = context_len[req] - 1;
    const int key_lo = args.window > 0 ? max(0, pos - args.window + 1) : 0;
    const int first_tile = key_lo / BN, last_tile = pos / BN;
    const int tiles = last_tile - first_tile + 1;
    const int per_split = (tiles + num_splits - 1) / num_splits;
    const int t_begin = first_tile + split * per_split;
    const int t_end = min(last_tile + 1, t_begin + per_split);
    if (threadIdx.x == 0) sm100::tma_prefetch_descriptor(&kv_map);
    decode_init_barriers<D>(smem);
    if (PAIR) {
        const int stride = args.head_dim + 2;
        float* own = reinterpret_cast<float*>(smem + Smem::q_bytes + Smem::merge_bytes);  // this CTA's rows, behind its warps' merge buffer
        float* slots = reinterpret_cast<float*>(smem + Smem::pair_offset);  // in the first CTA: the other CTAs' rows, [rank - 1][group][stride]
        float* dst = own;
        if (split > 0) {
            // this CTA's slot in the first CTA's shared memory, as an address that ordinary stores take
            unsigned long long mapped;
            asm volatile("mapa.u64 %0, %1, %2;" : "=l"(mapped) : "l"((unsigned long long)(uintptr_t)(slots + (size_t)(split - 1) * group * stride)), "r"(0u));
            dst = reinterpret_cast<float*>((uintptr_t)mapped);
        }
        decode_attend_range<D, HEADS>(kv_map, args, smem, req, kv_head, pos, key_lo, last_tile, t_begin, t_end, 0, true, out,
                                      dst, (long)stride);
        // the rows are in place in the first CTA (release), which may read them after the meeting (acquire)
        asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
        if (split == 0) {
            const int head_dim = args.head_dim;
            for (int e = threadIdx.x; e < group * head_dim; e += blockDim.x) {
                const int row = e / head_dim, col = e % head_dim;
                float m_all = own[row * stride + head_dim];
                for (int r = 1; r < num_splits; ++r) m_all = fmaxf(m_all, slots[((size_t)(r - 1) * group + row) * stride + head_dim]);
                float acc = 0.0f, l_all = 0.0f;
                for (int r = 0; r < num_splits; ++r) {
                    const float* src = r == 0 ? own + row * stride : slots + ((size_t)(r - 1) * group + row) * stride;
                    const float weight = src[head_dim] == -INFINITY ? 0.0f : exp2f(src[head_dim] - m_all);
                    acc += src[col] * weight;
                    l_all += src[head_dim + 1] * weight;
                }
                out[((size_t)req * args.q_heads + kv_head * group + row) * head_dim + col] = from_f32<bf16>(l_all > 0.0f ? acc / l_all : 0.0f);
            }
        }
        decode_stamp(args, 4);
        return;
    }
    float* dst_partial = num_splits == 1 ? nullptr
        : partial + (((size_t)req * args.q_heads + kv_head * group) * num_splits + split) * (args.head_dim + 2);
    decode_attend_range<D, HEADS>(kv_map, args, smem, req, kv_head, pos, key_lo, last_tile, t_begin, t_end, 0, true, out,
                                  dst_partial, (long)num_splits * (args.head_dim + 2));
    decode_stamp(args, 4);
}

// How the balanced kernel and its merge cut the work: the key tiles of all (request, kv head) pairs form one
// sequence (requests in order, a request's kv heads one after the other), cut into equal ranges, one per CTA.
#define DECODE_MAX_REQUESTS 1024

// prefix[r] = tiles of one kv head of the requests before r, prefix[requests] = of all; computed by the whole block
// (every thread loads its requests' lengths at once; a serial walk would pay a memory round trip per request).
__device__ __forceinline__ void decode_tile_prefix(const int* __restrict__ context_len, int requests, int window,
                                                   int tile_keys, int* prefix) {
    for (int r = threadIdx.x; r < requests; r += blockDim.x) {
        const int pos = context_len[r] - 1;
        int tiles = 0;
        if (pos >= 0) {
            const int key_lo = window > 0 ? max(0, pos - window + 1) : 0;
            tiles = pos / tile_keys - key_lo / tile_keys + 1;
        }
        prefix[r + 1] = tiles;
    }
    if (threadIdx.x == 0) prefix[0] = 0;
    __syncthreads();
    if (threadIdx.x < 32) {  // one warp scans: 32 requests per round
        int carry = 0;
        for (int base = 0; base < requests; base += 32) {
            const int r = base + (int)threadIdx.x;
            int value = r < requests ? prefix[r + 1] : 0;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const int other = __shfl_up_sync(0xffffffffu, value, d);
                if ((int)threadIdx.x >= d) value += other;
            }
            if (r < requests) prefix[r + 1] = carry + value;
            carry += __shfl_sync(0xffffffffu, value, 31);
        }
    }
    __syncthreads();
}

// Grid (ctas): CTA c attends tiles [c * per_cta, (c + 1) * per_cta) of the sequence above, one pair after the
// other.  A pair that lies inside one CTA's range is finished there; a pair cut by a range border leaves a partial
// result in slot 0 (the piece starts where the CTA's range starts) or 1 of its CTA,
// partial[cta][slot][group row][head_dim + 2], which attention_merge_balanced_kernel adds up.  Whatever the batch
// and the context lengths are, every CTA reads the same number of keys.
template <int D, bool HEADS>
__global__ void __launch_bounds__(DecodeTile<D>::WARPS * 32)
attention_decode_balanced_kernel(const __grid_constant__ CUtensorMap kv_map, DecodeArgs args, bf16* __restrict__ out,
                                 float* __restrict__ partial, const int* __restrict__ context_len, int requests) {
    pdl_launch_dependents();
    using Smem = DecodeSmem<D>;
    constexpr int BN = Smem::BN;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    int* prefix = reinterpret_cast<int*>(smem + Smem::body + Smem::DC_WARPS * DC_STAGES * 8 + Smem::table_entries * 4);
    const int kv_heads = args.kv_heads, window = args.window;
    if (threadIdx.x == 0) sm100::tma_prefetch_descriptor(&kv_map);
    decode_tile_prefix(context_len, requests, window, BN, prefix);
    const long total = (long)kv_heads * prefix[requests];
    const long per_cta = (total + gridDim.x - 1) / gridDim.x;
    const long begin = (long)blockIdx.x * per_cta, end = min(total, begin + per_cta);
    decode_init_barriers<D>(smem);
    bool first = true;
    int k_base = 0;
    // the first request with tiles in this CTA's range: the last r with kv_heads * prefix[r] <= begin
    int req = 0;
    {
        int lo = 0, hi = requests;
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if ((long)kv_heads * prefix[mid] <= begin) lo = mid; else hi = mid - 1;
        }
        req = lo;
    }
    for (; req < requests && begin < end; ++req) {
        const long pair_begin = (long)kv_heads * prefix[req];
        if (pair_begin >= end) break;
        const int tiles = prefix[req + 1] - prefix[req];
        if (tiles == 0) continue;
        const int pos = context_len[req] - 1;
        const int key_lo = window > 0 ? max(0, pos - window + 1) : 0;
        const int first_tile = key_lo / BN, last_tile = pos / BN;
        const int head_first = begin > pair_begin ? (int)((begin - pair_begin) / tiles) : 0;
        for (int kv_head = head_first; kv_head < kv_heads; ++kv_head) {
            const long start = pair_begin + (long)kv_head * tiles;
            if (start >= end) break;
            const long from = max(start, begin), to = min(start + tiles, end);
            const bool whole = from == start && to == start + tiles;
            float* dst_partial = whole ? nullptr
                : partial + ((size_t)blockIdx.x * 2 + (from == begin ? 0 : 1)) * 16 * (args.head_dim + 2);
            if (!first) __syncthreads();  // the merge buffer of the range before lies over the ring
            k_base = decode_attend_range<D, HEADS>(kv_map, args, smem, req, kv_head, pos, key_lo, last_tile,
                                                   first_tile + (int)(from - start), first_tile + (int)(to - start),
                                                   k_base, first, out, dst_partial, (long)(args.head_dim + 2));
            first = false;
        }
    }
    if (first) pdl_wait();  // a CTA without work still orders itself after the kernel before it
}

// One block per (request, query head): adds up the pieces of a pair that more than one CTA of the balanced kernel
// attended, in CTA order; a pair finished inside one CTA is left as that CTA wrote it.
__global__ void __launch_bounds__(128)
attention_merge_balanced_kernel(const float* __restrict__ partial, bf16* __restrict__ out,
                                const int* __restrict__ context_len, int requests, int q_heads, int kv_heads,
                                int head_dim, int window, int tile_keys, int ctas) {
    pdl_launch_dependents();
    __shared__ int prefix[DECODE_MAX_REQUESTS + 1];
    __shared__ float warp_max[4];
    const int req = blockIdx.x / q_heads, head = blockIdx.x % q_heads;
    const int group = q_heads / kv_heads, kv_head = head / group, row = head % group;
    decode_tile_prefix(context_len, requests, window, tile_keys, prefix);
    const int my_tiles = prefix[req + 1] - prefix[req];
    const long total = (long)kv_heads * prefix[requests];
    const long start = (long)kv_heads * prefix[req] + (long)kv_head * my_tiles;
    pdl_wait();
    bf16* dst = out + ((size_t)req * q_heads + head) * head_dim;
    if (my_tiles == 0) {
        for (int col = threadIdx.x; col < head_dim; col += blockDim.x) dst[col] = from_f32<bf16>(0.0f);
        return;
    }
    const long per_cta = (total + ctas - 1) / ctas;
    const int c_first = (int)(start / per_cta), c_last = (int)((start + my_tiles - 1) / per_cta);
    if (c_first == c_last) return;  // finished by its CTA
    const int stride = head_dim + 2;
    // piece of CTA c: slot 0 unless the pair starts inside that CTA's range (only c_first can)
    const int first_slot = start == (long)c_first * per_cta ? 0 : 1;
    auto piece = [&](int c) { return partial + (((size_t)c * 2 + (c == c_first ? first_slot : 0)) * 16 + row) * stride; };
    float m_all = -INFINITY;
    for (int c = c_first + (int)threadIdx.x; c <= c_last; c += blockDim.x) m_all = fmaxf(m_all, piece(c)[head_dim]);
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) m_all = fmaxf(m_all, __shfl_xor_sync(0xffffffffu, m_all, d));
    if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = m_all;
    __syncthreads();
    m_all = fmaxf(fmaxf(warp_max[0], warp_max[1]), fmaxf(warp_max[2], warp_max[3]));
    for (int col = threadIdx.x; col < head_dim; col += blockDim.x) {
        float acc = 0.0f, l_all = 0.0f;
#pragma unroll 4
        for (int c = c_first; c <= c_last; ++c) {
            const float* src = piece(c);
            const float weight = src[head_dim] == -INFINITY ? 0.0f : exp2f(src[head_dim] - m_all);
            acc += src[col] * weight;
            l_all += src[head_dim + 1] * weight;
        }
        dst[col] = from_f32<bf16>(l_all > 0.0f ? acc / l_all : 0.0f);
    }
}

__global__ void attention_merge_splits_kernel(const float* __restrict__ partial, bf16* __restrict__ out, int head_dim,
                                              int num_splits) {
    pdl_launch_dependents();
    pdl_wait();
    // one block per (request, head); the splits are read eight at a time, so that their loads are in flight together
    const size_t rh = blockIdx.x;
    const int stride = head_dim + 2;
    const float* base = partial + rh * num_splits * stride;
    float m_all = -INFINITY;
    for (int s0 = 0; s0 < num_splits; s0 += 8) {
        float m[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) m[u] = s0 + u < num_splits ? base[(size_t)(s0 + u) * stride + head_dim] : -INFINITY;
#pragma unroll
        for (int u = 0; u < 8; ++u) m_all = fmaxf(m_all, m[u]);
    }
    for (int col = threadIdx.x; col < head_dim; col += blockDim.x) {
        float acc = 0.0f, l_all = 0.0f;
        for (int s0 = 0; s0 < num_splits; s0 += 8) {
            float m[8], l[8], value[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const bool live = s0 + u < num_splits;
                const float* src = base + (size_t)(live ? s0 + u : 0) * stride;
                m[u] = live ? src[head_dim] : -INFINITY;
                l[u] = live ? src[head_dim + 1] : 0.0f;
                value[u] = live ? src[col] : 0.0f;
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const float weight = m[u] == -INFINITY ? 0.0f : exp2f(m[u] - m_all);
                acc += value[u] * weight;
                l_all += l[u] * weight;
            }
        }
        out[rh * head_dim + col] = from_f32<bf16>(l_all > 0.0f ? acc / l_all : 0.0f);
    }
}

// Measurements: while a buffer is set, every launch of the split decode kernel writes its CTAs' clock stamps (see
// decode_stamp) to the next 8 * 1,024 words of it.  Null (the default) switches the stamps off.
unsigned long long* g_decode_stamps = nullptr;

// What the decode kernels need to prepare queries and the new token's key themselves (see DecodeArgs).
struct FuseQK {
    const float* q_weight;
    const float* k_weight;
    const float* inv_freq;
    float eps;
};

template <int D>
int prefill_launch(const void* q, const void* cache, void* out, const int* block_table, const int* query_start,
                   const int* context_len, int requests, int max_query_len, int q_heads, int kv_heads, int head_dim,
                   long q_row_stride, int page_size, int table_width, int num_pages, int window, float scale,
                   int* error_flag, cudaStream_t stream) {
    using Smem = PrefillSmem<D>;
    const int group = q_heads / kv_heads;
    const int box_rows = page_size < PF_BN ? page_size : PF_BN;
    if (PF_BN % box_rows != 0 || page_size % box_rows != 0) return KIRAI_ERR_UNSUPPORTED;  // page sizes: powers of two
    CUtensorMap kv_map;
    const uint64_t rows = (uint64_t)num_pages * 2 * kv_heads * page_size;
    if (!tmap::bf16_2d_sw128(&kv_map, cache, rows, head_dim, head_dim, box_rows, 64)) return KIRAI_ERR_BAD_ALIGN;
    auto kernel = attention_prefill_kernel<D>;
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem::total);
    if (err != cudaSuccess) return (int)err;
    dim3 grid(kv_heads, (unsigned)(((long)max_query_len * group + PF_ROWS - 1) / PF_ROWS), requests);
    if (grid.y > 65535) return KIRAI_ERR_BAD_SIZE;
    return launch_pdl(kernel, grid, dim3((PF_WARPS + 1) * 32), (size_t)Smem::total, stream, 1u, kv_map, (const bf16*)q,
                      (bf16*)out, block_table, query_start, context_len, q_heads, kv_heads, head_dim, q_row_stride,
                      page_size, box_rows, table_width, num_pages, window, scale * 1.4426950408889634f, error_flag);
}

template <int D>
int decode_launch(const void* q, const void* cache, void* out, float* partial, const int* block_table,
                  const int* context_len, int requests, int q_heads, int kv_heads, int head_dim, long q_row_stride,
                  int page_size, int table_width, int num_pages, int window, float scale, int num_splits,
                  int* error_flag, cudaStream_t stream, const FuseQK* fuse = nullptr) {
    using Smem = DecodeSmem<D>;
    const int box_rows = page_size < Smem::BN ? page_size : Smem::BN;
    if (Smem::BN % box_rows != 0 || page_size % box_rows != 0) return KIRAI_ERR_UNSUPPORTED;  // page sizes: powers of two
    CUtensorMap kv_map;
    const uint64_t rows = (uint64_t)num_pages * 2 * kv_heads * page_size;
    if (!tmap::bf16_2d_sw128(&kv_map, cache, rows, head_dim, head_dim, box_rows, 64)) return KIRAI_ERR_BAD_ALIGN;
    const bool heads = q_heads / kv_heads <= 8;
    // a few ranges and no buffer: they merge in the first CTA's shared memory, if their rows fit its slots
    const bool pair = num_splits >= 2 && num_splits <= 8 && partial == nullptr;
    if (pair && (size_t)(num_splits - 1) * (q_heads / kv_heads) * (head_dim + 2) * 4 > (size_t)Smem::pair_bytes) return KIRAI_ERR_UNSUPPORTED;
    auto kernel = pair ? (heads ? attention_decode_kernel<D, true, true> : attention_decode_kernel<D, false, true>)
                       : (heads ? attention_decode_kernel<D, true, false> : attention_decode_kernel<D, false, false>);
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem::total);
    if (err != cudaSuccess) return (int)err;
    if (fuse && head_dim != D) return KIRAI_ERR_UNSUPPORTED;  // the fused preparation works on whole heads of 64, 128 or 256
    DecodeArgs args{(const bf16*)q, block_table, q_heads, kv_heads, head_dim, q_row_stride, page_size, box_rows,
                    table_width, num_pages, window, scale * 1.4426950408889634f, error_flag};
    if (fuse) {
        args.fuse = 1, args.q_weight = fuse->q_weight, args.k_weight = fuse->k_weight, args.inv_freq = fuse->inv_freq;
        args.eps = fuse->eps, args.cache = (bf16*)const_cast<void*>(cache);
    }
    args.stamps = g_decode_stamps;
    if (g_decode_stamps) g_decode_stamps += 8 * 1024;  // the next launch's stamps follow
    dim3 grid(num_splits, kv_heads, requests);
    if (pair)
        return launch_pdl_clusters(kernel, grid, dim3(Smem::DC_WARPS * 32), (size_t)Smem::total, stream, dim3(num_splits, 1, 1),
                                   kv_map, args, (bf16*)out, partial, context_len, num_splits);
    int status = launch_pdl(kernel, grid, dim3(Smem::DC_WARPS * 32), (size_t)Smem::total, stream, 1u, kv_map, args,
                            (bf16*)out, partial, context_len, num_splits);
    if (status || num_splits == 1) return status;
    return launch_pdl(attention_merge_splits_kernel, dim3(requests * q_heads), dim3(128), 0, stream, 1u,
                      (const float*)partial, (bf16*)out, head_dim, num_splits);
}

template <int D>
int decode_balanced_launch(const void* q, const void* cache, void* out, float* partial, const int* block_table,
                           const int* context_len, int requests, int q_heads, int kv_heads, int head_dim,
                           long q_row_stride, int page_size, int table_width, int num_pages, int window, float scale,
                           int ctas, int* error_flag, cudaStream_t stream, const FuseQK* fuse = nullptr) {
    using Smem = DecodeSmem<D>;
    const int box_rows = page_size < Smem::BN ? page_size : Smem::BN;
    if (Smem::BN % box_rows != 0 || page_size % box_rows != 0) return KIRAI_ERR_UNSUPPORTED;  // page sizes: powers of two
    CUtensorMap kv_map;
    const uint64_t rows = (uint64_t)num_pages * 2 * kv_heads * page_size;
    if (!tmap::bf16_2d_sw128(&kv_map, cache, rows, head_dim, head_dim, box_rows, 64)) return KIRAI_ERR_BAD_ALIGN;
    auto kernel = (q_heads / kv_heads <= 8) ? attention_decode_balanced_kernel<D, true> : attention_decode_balanced_kernel<D, false>;
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem::total);
    if (err != cudaSuccess) return (int)err;
    if (fuse && head_dim != D) return KIRAI_ERR_UNSUPPORTED;  // the fused preparation works on whole heads of 64, 128 or 256
    DecodeArgs args{(const bf16*)q, block_table, q_heads, kv_heads, head_dim, q_row_stride, page_size, box_rows,
                    table_width, num_pages, window, scale * 1.4426950408889634f, error_flag};
    if (fuse) {
        args.fuse = 1, args.q_weight = fuse->q_weight, args.k_weight = fuse->k_weight, args.inv_freq = fuse->inv_freq;
        args.eps = fuse->eps, args.cache = (bf16*)const_cast<void*>(cache);
    }
    int status = launch_pdl(kernel, dim3(ctas), dim3(Smem::DC_WARPS * 32), (size_t)Smem::total, stream, 1u, kv_map, args,
                            (bf16*)out, partial, context_len, requests);
    if (status) return status;
    return launch_pdl(attention_merge_balanced_kernel, dim3(requests * q_heads), dim3(128), 0, stream, 1u,
                      (const float*)partial, (bf16*)out, context_len, requests, q_heads, kv_heads, head_dim, window,
                      (int)Smem::BN, ctas);
}

int check_common(int q_heads, int kv_heads, int head_dim, long q_row_stride, const void* q) {
    if (kv_heads <= 0 || q_heads % kv_heads != 0) return KIRAI_ERR_BAD_SIZE;
    if (head_dim <= 0 || head_dim > 256 || head_dim % 8 != 0) return KIRAI_ERR_BAD_SIZE;
    if (q_row_stride % 8 != 0 || ((uintptr_t)q & 15)) return KIRAI_ERR_BAD_ALIGN;  // 16-byte row chunks
    if (kv_heads > 65535) return KIRAI_ERR_BAD_SIZE;
    return 0;
}

}  // namespace

// Attention for the new tokens of a step: q [tokens, q_heads, head_dim] (row stride in elements),
// requests described by query_start [requests + 1] and context_len [requests] (tokens in the cache
// after this step, the new ones included).  out [tokens, q_heads * head_dim].
KIRAI_EXPORT int kirai_attention_prefill_bf16(const void* q, const void* cache, void* out, const int* block_table,
                                              const int* query_start, const int* context_len, int requests,
                                              int max_query_len, int q_heads, int kv_heads, int head_dim,
                                              long q_row_stride, int page_size, int table_width, int num_pages,
                                              int window, float scale, int* error_flag, cudaStream_t stream) {
    if (requests <= 0 || max_query_len <= 0) return 0;
    int bad = check_common(q_heads, kv_heads, head_dim, q_row_stride, q);
    if (bad) return bad;
    if (requests > 65535) return KIRAI_ERR_BAD_SIZE;
#define KIRAI_PF(D) \
    return prefill_launch<D>(q, cache, out, block_table, query_start, context_len, requests, max_query_len, q_heads, \
                             kv_heads, head_dim, q_row_stride, page_size, table_width, num_pages, window, scale, \
                             error_flag, stream)
    if (head_dim <= 64) KIRAI_PF(64);
    if (head_dim <= 128) KIRAI_PF(128);
    KIRAI_PF(256);
#undef KIRAI_PF
}

// How many clusters of `cluster` CTAs of the decode kernel the device can hold at once, 0 if it refuses the size.
// A CTA of this kernel fills an SM, so a cluster needs that many free SMs inside one GPC, and how many SMs the GPCs
// have differs from chip to chip (clusters of 3: 39 on one B200, 45 on another): whoever plans a launch whose ranges
// merge as clusters, and which should run as one wave, asks here.
template <int D>
int decode_resident_clusters(bool heads, int cluster) {
    using Smem = DecodeSmem<D>;
    auto kernel = heads ? attention_decode_kernel<D, true, true> : attention_decode_kernel<D, false, true>;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem::total) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(cluster, 1, 1), config.blockDim = dim3(Smem::DC_WARPS * 32), config.dynamicSmemBytes = (size_t)Smem::total;
    cudaLaunchAttribute attribute;
    attribute.id = cudaLaunchAttributeClusterDimension;
    attribute.val.clusterDim.x = (unsigned)cluster, attribute.val.clusterDim.y = 1, attribute.val.clusterDim.z = 1;
    config.attrs = &attribute, config.numAttrs = 1;
    int resident = 0;
    if (cudaOccupancyMaxActiveClusters(&resident, kernel, &config) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return resident;
}

KIRAI_EXPORT int kirai_attention_decode_resident_clusters(int head_dim, int group, int cluster) {
    if (cluster < 1 || cluster > 8 || group < 1 || group > 16 || head_dim < 1 || head_dim > 256) return 0;
    if (head_dim <= 64) return decode_resident_clusters<64>(group <= 8, cluster);
    if (head_dim <= 128) return decode_resident_clusters<128>(group <= 8, cluster);
    return decode_resident_clusters<256>(group <= 8, cluster);
}

// Attention for a batch in which every request brings exactly one token (token r belongs to request r).
// With num_splits > 1 and a buffer `partial` of requests * q_heads * num_splits * (head_dim + 2) floats, the ranges'
// results go through that buffer and a second kernel merges them.
KIRAI_EXPORT int kirai_attention_decode_bf16(const void* q, const void* cache, void* out, float* partial,
                                             const int* block_table, const int* context_len, int requests,
                                             int q_heads, int kv_heads, int head_dim, long q_row_stride, int page_size,
                                             int table_width, int num_pages, int window, float scale, int num_splits,
                                             int* error_flag, cudaStream_t stream) {
    if (requests <= 0) return 0;
    int bad = check_common(q_heads, kv_heads, head_dim, q_row_stride, q);
    if (bad) return bad;
    if (q_heads / kv_heads > 16) return KIRAI_ERR_UNSUPPORTED;  // the group's heads are the rows of one m16 tile
    if (num_splits < 1 || num_splits > 65535 || requests > 65535) return KIRAI_ERR_BAD_SIZE;
    if (num_splits > 8 && !partial) return KIRAI_ERR_BAD_SIZE;  // (up to 8 ranges may merge without a buffer, if their rows fit)
#define KIRAI_DC(D) \
    return decode_launch<D>(q, cache, out, partial, block_table, context_len, requests, q_heads, kv_heads, head_dim, \
                            q_row_stride, page_size, table_width, num_pages, window, scale, num_splits, error_flag, \
                            stream)
    if (head_dim <= 64) KIRAI_DC(64);
    if (head_dim <= 128) KIRAI_DC(128);
    KIRAI_DC(256);
#undef KIRAI_DC
}

// The same with the work cut evenly: `ctas` CTAs (one per SM is the intent) each attend the same number of key
// tiles, whatever the batch size and the context lengths are.  partial holds ctas * 2 * 16 * (head_dim + 2) floats.
KIRAI_EXPORT int kirai_attention_decode_balanced_bf16(const void* q, const void* cache, void* out, float* partial,
                                                      const int* block_table, const int* context_len, int requests,
                                                      int q_heads, int kv_heads, int head_dim, long q_row_stride,
                                                      int page_size, int table_width, int num_pages, int window,
                                                      float scale, int ctas, int* error_flag, cudaStream_t stream) {
    if (requests <= 0) return 0;
    int bad = check_common(q_heads, kv_heads, head_dim, q_row_stride, q);
    if (bad) return bad;
    if (q_heads / kv_heads > 16) return KIRAI_ERR_UNSUPPORTED;  // the group's heads are the rows of one m16 tile
    if (ctas < 1 || ctas > 65535 || !partial) return KIRAI_ERR_BAD_SIZE;
    if (requests > DECODE_MAX_REQUESTS) return KIRAI_ERR_UNSUPPORTED;  // the tile prefix lives in shared memory
#define KIRAI_DCB(D) \
    return decode_balanced_launch<D>(q, cache, out, partial, block_table, context_len, requests, q_heads, kv_heads, \
                                     head_dim, q_row_stride, page_size, table_width, num_pages, window, scale, ctas, \
                                     error_flag, stream)
    if (head_dim <= 64) KIRAI_DCB(64);
    if (head_dim <= 128) KIRAI_DCB(128);
    KIRAI_DCB(256);
#undef KIRAI_DCB
}

// The two decode entry points with the preparation of queries and keys inside: `qkv` holds the rows that the q, k, v
// product left, [requests, (q_heads + 2 kv_heads) * head_dim] (row stride in elements), and is not modified.  Per-head
// RMSNorm of q and k (weights [head_dim], may be null), half-split rotation at position context_len - 1 (inv_freq
// [head_dim / 2], may be null), the new token's key and value appended to their page of `cache`, then attention.
// head_dim must be 64, 128 or 256; everything else as in the entry points above.
KIRAI_EXPORT int kirai_attention_decode_qk_bf16(const void* qkv, void* cache, void* out, float* partial,
                                                const int* block_table, const int* context_len, int requests,
                                                int q_heads, int kv_heads, int head_dim, long qkv_row_stride,
                                                int page_size, int table_width, int num_pages, int window, float scale,
                                                int num_splits, const float* q_weight, const float* k_weight,
                                                const float* inv_freq, float eps, int* error_flag, cudaStream_t stream) {
    if (requests <= 0) return 0;
    int bad = check_common(q_heads, kv_heads, head_dim, qkv_row_stride, qkv);
    if (bad) return bad;
    if (q_heads / kv_heads > 16) return KIRAI_ERR_UNSUPPORTED;
    if (num_splits < 1 || num_splits > 65535 || requests > 65535) return KIRAI_ERR_BAD_SIZE;
    if (num_splits > 8 && !partial) return KIRAI_ERR_BAD_SIZE;
    if (((uintptr_t)q_weight | (uintptr_t)k_weight | (uintptr_t)inv_freq | (uintptr_t)cache) & 15) return KIRAI_ERR_BAD_ALIGN;
    const FuseQK fuse{q_weight, k_weight, inv_freq, eps};
#define KIRAI_DCQ(D) \
    return decode_launch<D>(qkv, cache, out, partial, block_table, context_len, requests, q_heads, kv_heads, head_dim, \
                            qkv_row_stride, page_size, table_width, num_pages, window, scale, num_splits, error_flag, \
                            stream, &fuse)
    if (head_dim == 64) KIRAI_DCQ(64);
    if (head_dim == 128) KIRAI_DCQ(128);
    if (head_dim == 256) KIRAI_DCQ(256);
#undef KIRAI_DCQ
    return KIRAI_ERR_UNSUPPORTED;
}

KIRAI_EXPORT int kirai_attention_decode_balanced_qk_bf16(const void* qkv, void* cache, void* out, float* partial,
                                                         const int* block_table, const int* context_len, int requests,
                                                         int q_heads, int kv_heads, int head_dim, long qkv_row_stride,
                                                         int page_size, int table_width, int num_pages, int window,
                                                         float scale, int ctas, const float* q_weight,
                                                         const float* k_weight, const float* inv_freq, float eps,
                                                         int* error_flag, cudaStream_t stream) {
    if (requests <= 0) return 0;
    int bad = check_common(q_heads, kv_heads, head_dim, qkv_row_stride, qkv);
    if (bad) return bad;
    if (q_heads / kv_heads > 16) return KIRAI_ERR_UNSUPPORTED;
    if (ctas < 1 || ctas > 65535 || !partial) return KIRAI_ERR_BAD_SIZE;
    if (requests > DECODE_MAX_REQUESTS) return KIRAI_ERR_UNSUPPORTED;
    if (((uintptr_t)q_weight | (uintptr_t)k_weight | (uintptr_t)inv_freq | (uintptr_t)cache) & 15) return KIRAI_ERR_BAD_ALIGN;
    const FuseQK fuse{q_weight, k_weight, inv_freq, eps};
#define KIRAI_DCBQ(D) \
    return decode_balanced_launch<D>(qkv, cache, out, partial, block_table, context_len, requests, q_heads, kv_heads, \
                                     head_dim, qkv_row_stride, page_size, table_width, num_pages, window, scale, ctas, \
                                     error_flag, stream, &fuse)
    if (head_dim == 64) KIRAI_DCBQ(64);
    if (head_dim == 128) KIRAI_DCBQ(128);
    if (head_dim == 256) KIRAI_DCBQ(256);
#undef KIRAI_DCBQ
    return KIRAI_ERR_UNSUPPORTED;
}

KIRAI_EXPORT void kirai_attention_decode_set_stamps(unsigned long long* buffer) { g_decode_stamps = buffer; }

// ----------------------------------------------------- decode without allocation
// The same decode kernels, with the splits' partial results in a file-scope device array
// instead of a buffer from the caller; see no_alloc.h for who needs this and for the rules.
#include "no_alloc.h"

#include <mutex>

// In host code this name is only a handle for cudaGetSymbolAddress, never a device pointer.
static __device__ __align__(256) float kirai_static_scratch[KIRAI_STATIC_SCRATCH_FLOATS];

namespace {
constexpr int kMaxDevices = 64;
float* static_scratch_address[kMaxDevices];  // per device, found on the first call there
std::mutex static_scratch_mutex;

// The device address of the array on the current device (looked up once per device).
int static_scratch_for_current_device(float** address) {
    int device = -1;
    cudaError_t err = cudaGetDevice(&device);
    if (err != cudaSuccess) return (int)err;
    if (device < 0 || device >= kMaxDevices) return KIRAI_ERR_STATIC_SCRATCH_SETUP;
    std::lock_guard<std::mutex> lock(static_scratch_mutex);
    if (static_scratch_address[device] == nullptr) {
        float* found = nullptr;
        err = cudaGetSymbolAddress((void**)&found, kirai_static_scratch);
        if (err != cudaSuccess) return (int)err;
        if (found == nullptr) return KIRAI_ERR_STATIC_SCRATCH_SETUP;
        static_scratch_address[device] = found;
    }
    *address = static_scratch_address[device];
    return 0;
}
}  // namespace

KIRAI_EXPORT unsigned kirai_static_scratch_capacity_floats(void) { return KIRAI_STATIC_SCRATCH_FLOATS; }

KIRAI_EXPORT int kirai_attention_decode_bf16_static_scratch(const void* q, const void* cache, void* out,
                                                            const int* block_table, const int* context_len,
                                                            int requests, int q_heads, int kv_heads, int head_dim,
                                                            long q_row_stride, int page_size, int table_width,
                                                            int num_pages, int window, float scale, int num_splits,
                                                            int* error_flag, cudaStream_t stream) {
    if (requests <= 0) return 0;
    if (num_splits < 1 || q_heads <= 0 || head_dim <= 0) return KIRAI_ERR_BAD_SIZE;
    float* scratch = nullptr;
    if (num_splits > 1) {
        const unsigned long long need =
            (unsigned long long)requests * (unsigned long long)q_heads * (unsigned long long)num_splits *
            (unsigned long long)(head_dim + 2);
        if (need > KIRAI_STATIC_SCRATCH_FLOATS) return KIRAI_ERR_STATIC_SCRATCH_TOO_SMALL;
        const int status = static_scratch_for_current_device(&scratch);
        if (status) return status;
    }
    return kirai_attention_decode_bf16(q, cache, out, scratch, block_table, context_len, requests, q_heads, kv_heads,
                                       head_dim, q_row_stride, page_size, table_width, num_pages, window, scale,
                                       num_splits, error_flag, stream);
}
