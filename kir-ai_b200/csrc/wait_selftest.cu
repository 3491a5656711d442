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
