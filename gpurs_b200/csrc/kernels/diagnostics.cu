// A kernel that exercises the bounded-wait path on purpose: one block waits on an mbarrier that nothing will ever
// complete.  The wait gives up after ptx::WAIT_LIMIT_NS like every wait of the GEMM kernels, the block records the
// failure in the status word and returns normally, so the context stays usable.  Nothing faults, traps or spins
// for ever.  (The reference's waits are unbounded: crates/gpurs/src/gpu/tensor/hopper/intrinsics.rs:15-16.)
#include "gemm_tcgen05.cuh"

extern "C" __global__ void __launch_bounds__(32) gpurs_wait_probe(unsigned int *status) {
    __shared__ __align__(8) unsigned long long barrier;
    __shared__ uint32_t abort_word;
    volatile uint32_t *abort_flag = &abort_word;
    const uint32_t bar = ptx::smem_u32(&barrier);
    if (threadIdx.x == 0) {
        *abort_flag = 0;
        ptx::mbarrier_init(bar, 1);
        ptx::fence_mbarrier_init();
    }
    __syncwarp();
    if (threadIdx.x == 0) {
        // phase 0 never completes: nobody arrives
        if (!ptx::mbarrier_wait(bar, 0, abort_flag)) gemm::report_status(status, abort_flag, gemm::STATUS_PROBE_TIMEOUT, -1, -1);
    }
}
