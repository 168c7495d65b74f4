// Resident-tile tcgen05 kind::i8 throughput probe: every CTA keeps one A tile (128 x 64 B) and one
// W tile (256 x 64 B) in shared memory and issues `iters` x 2 MMAs (128 x 256 x 32) on them, with no
// global traffic inside the loop.  The time of the launch gives the attainable int8 tensor rate
// of the device (the denominator for "tensor-bound" roofline fractions).
#pragma once
#include <cuda_runtime.h>

#include <cstdint>

#include "fused_cnn.cuh"
#include "ptx_sm100.cuh"

namespace zb {

constexpr int PEAK_SMEM = 128 * 64 + 256 * 64 + 64;

__global__ void __launch_bounds__(128, 1) tc_peak_i8_kernel(int iters, int* status) {
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* sA = smem;                      // [4 chunks][128][16]
    uint8_t* sW = smem + 128 * 64;           // [4 chunks][256][16]
    uint64_t* bar = reinterpret_cast<uint64_t*>(smem + 128 * 64 + 256 * 64);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + 128 * 64 + 256 * 64 + 16);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + 128 * 64 + 256 * 64 + 20);
    const int tid = threadIdx.x, warp = tid >> 5;
    for (int i = tid; i < (128 * 64 + 256 * 64) / 4; i += 128) reinterpret_cast<uint32_t*>(smem)[i] = 0x01ff7f03u * (uint32_t)(i + 1);
    if (tid == 0) { ptx::mbar_init(ptx::smem_u32(bar), 1); *abort_flag = 0; ptx::mbar_fence_init(); }
    ptx::fence_proxy_async_smem();
    if (warp == 0) { ptx::tmem_alloc(ptx::smem_u32(tmem_slot), 512); ptx::tmem_relinquish(); }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    if (warp == 1 && ptx::elect_one()) {
        constexpr uint32_t idesc = ptx::idesc_i8(128, 256, true, true);
        const uint32_t sa = ptx::smem_u32(sA), sw = ptx::smem_u32(sW);
        const uint64_t da0 = ptx::smem_desc_kmajor(sa, 2048, 128), da1 = ptx::smem_desc_kmajor(sa + 4096, 2048, 128);
        const uint64_t db0 = ptx::smem_desc_kmajor(sw, 4096, 128), db1 = ptx::smem_desc_kmajor(sw + 8192, 4096, 128);
        for (int i = 0; i < iters; ++i) {
            const uint32_t d = tmem_base + (uint32_t)((i & 1) * 256);
            ptx::mma_i8(d, da0, db0, idesc, i > 1);
            ptx::mma_i8(d, da1, db1, idesc, true);
        }
        ptx::mma_commit(ptx::smem_u32(bar));
        ptx::mbar_wait(ptx::smem_u32(bar), 0, abort_flag);
    }
    __syncthreads();
    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 0) ptx::tmem_dealloc(tmem_base, 512);
    if (tid == 0 && *abort_flag) atomicExch(status, (int)DEV_ERR_WAIT_TIMEOUT);
}

}  // namespace zb
