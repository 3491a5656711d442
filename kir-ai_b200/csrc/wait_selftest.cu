// A self-test of the bounded waits: what a kernel of this library does when a barrier that it waits for never
// completes.  Every pipeline here waits on mbarriers through mbar_wait (sm100.cuh), which gives up after a number of
// polls; the kernel then sets the device error word to KIRAI_FLAG_WAIT_RAN_OUT and winds down, so that the host
// reads an error instead of meeting a hung device.  This kernel shows exactly that path in the smallest form: one
// barrier in shared memory on which nothing ever arrives, one thread that waits for it with a limit given by the
// caller, no copy and no tensor-core work in flight.  It returns in microseconds and leaves the context usable.
// (The reference checks for cancellation between its steps on the host instead,
// crates/llm-backend/src/core/qwen/ops/decoder.rs:497-523.)
#include "sm100.cuh"

using namespace sm100;

__global__ void wait_runs_out_kernel(uint32_t limit, int arrive, int* __restrict__ error_flag, int* __restrict__ polls_done) {
    __shared__ uint64_t barrier;
    if (threadIdx.x == 0) {
        mbar_init(smem_addr(&barrier), 1);
        mbar_fence_init();
    }
    __syncthreads();
    if (threadIdx.x == 1 && arrive) mbar_arrive(smem_addr(&barrier));  // the control case: the wait is answered
    if (threadIdx.x == 0) {
        const bool ok = mbar_wait_limited(smem_addr(&barrier), 0u, limit);
        if (!ok) atomicExch(error_flag, KIRAI_FLAG_WAIT_RAN_OUT);
        if (polls_done) *polls_done = ok ? 0 : (int)limit;
    }
}

// limit: polls before the wait gives up (1 .. 2^20).  arrive != 0: another thread completes the barrier, and the wait
// succeeds.  polls_done (may be null) receives the limit when the wait ran out, else 0.
KIRAI_EXPORT int kirai_wait_selftest(unsigned limit, int arrive, int* error_flag, int* polls_done, cudaStream_t stream) {
    if (limit < 1 || limit > (1u << 20) || !error_flag) return KIRAI_ERR_BAD_SIZE;
    wait_runs_out_kernel<<<1, 32, 0, stream>>>(limit, arrive, error_flag, polls_done);
    return launch_status();
}

// ---------------------------------------------------------------------------------------------------------------
// A read-only stream at the rate of the memory system, for measurements: every CTA (one per SM, all of shared
// memory) copies a contiguous stretch of `bytes` into a ring of 16 KB slots with cp.async.bulk, as the
// weight-streaming products do, and drops the data.  What it reaches is the ceiling for a kernel that only reads; the
// copy figure that roofline fractions are usually taken against counts a read and a write.
__global__ void __launch_bounds__(32, 1) stream_read_kernel(const uint8_t* __restrict__ data, long boxes, int* __restrict__ error_flag) {
    constexpr int SLOTS = 12, BOX = 16384;
    extern __shared__ uint8_t stream_smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)stream_smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = (uint64_t*)(smem + SLOTS * BOX);
    if (threadIdx.x == 0) {
        for (int s = 0; s < SLOTS; ++s) mbar_init(smem_addr(&bars[s]), 1);
        mbar_fence_init();
    }
    __syncwarp();
    if (threadIdx.x != 0) return;
    const long begin = boxes * blockIdx.x / gridDim.x, end = boxes * (blockIdx.x + 1) / gridDim.x;
    bool ok = true;
    for (long i = begin; i < end + SLOTS && ok; ++i) {
        const long waited = i - SLOTS;  // the copy that took this slot before has to be in
        if (waited >= begin) ok = mbar_wait(smem_addr(&bars[waited % SLOTS]), (uint32_t)(((waited - begin) / SLOTS) & 1));
        if (i < end && ok) {
            const uint32_t bar = smem_addr(&bars[i % SLOTS]);
            mbar_expect_tx(bar, BOX);
            bulk_load_1d(smem_addr(smem + (i % SLOTS) * BOX), data + (size_t)i * BOX, BOX, bar);
        }
    }
    if (!ok) atomicExch(error_flag, KIRAI_FLAG_WAIT_RAN_OUT);
}

// Reads `bytes` (a multiple of 16 KB, 16-byte aligned) once with `ctas` CTAs.
KIRAI_EXPORT int kirai_stream_read(const void* data, long bytes, int ctas, int* error_flag, cudaStream_t stream) {
    if (bytes <= 0 || bytes % 16384 != 0 || ((uintptr_t)data & 15) || ctas < 1 || !error_flag) return KIRAI_ERR_BAD_SIZE;
    const int smem_bytes = 12 * 16384 + 12 * 8 + 1024;
    cudaError_t err = cudaFuncSetAttribute(stream_read_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
    if (err != cudaSuccess) return (int)err;
    stream_read_kernel<<<ctas, 32, smem_bytes, stream>>>((const uint8_t*)data, bytes / 16384, error_flag);
    return launch_status();
}
