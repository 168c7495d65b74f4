// Bounded-wait self test: one CTA holds TMEM columns and waits on an mbarrier that nothing ever
// arrives on.  The wait uses the same ptx::mbar_wait as the production kernels, with a budget of
// microseconds instead of seconds, so it gives up, the kernel frees its TMEM, writes
// DEV_ERR_WAIT_TIMEOUT into the context's status word and returns normally.  Nothing faults and
// nothing hangs: this is how the time-out path of the tensor-core kernels (abort flag -> drain ->
// dealloc -> status word -> ZANT_E_DEVICE_TIMEOUT on the host) is exercised on a healthy GPU.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>

#include "fused_cnn.cuh"
#include "ptx_sm100.cuh"

namespace zb {

__global__ void __launch_bounds__(64, 1) bounded_wait_selftest_kernel(long long budget_cycles, int* status) {
    __shared__ __align__(8) uint64_t bar;
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag_mem;
    volatile int* abort_flag = &abort_flag_mem;
    const int tid = threadIdx.x, warp = tid >> 5;
    if (tid == 0) { ptx::mbar_init(ptx::smem_u32(&bar), 1); *abort_flag = 0; ptx::mbar_fence_init(); }
    if (warp == 0) { ptx::tmem_alloc(ptx::smem_u32(&tmem_slot), 32); ptx::tmem_relinquish(); }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = tmem_slot;
    // warp 1 plays the role that waits for a producer that never comes
    if (warp == 1 && ptx::elect_one()) ptx::mbar_wait(ptx::smem_u32(&bar), 0, abort_flag, budget_cycles);
    __syncthreads();
    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 0) ptx::tmem_dealloc(tmem_base, 32);
    if (tid == 0 && *abort_flag) atomicExch(status, (int)DEV_ERR_WAIT_TIMEOUT);
}

}  // namespace zb
