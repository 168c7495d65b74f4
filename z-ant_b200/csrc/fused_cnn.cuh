// Fused kernels for quantized 3x3 convolution stages followed by ReLU and a 2x2/2 MaxPool.
//
// Internal activation layout "C16 planar": [image][C/16][H*W positions][16 channels] int8, i.e.
// every pixel of a 16-channel group is one 16-byte chunk and consecutive pixels are consecutive
// chunks.  With that layout the A operand of an implicit-GEMM convolution needs no im2col at all:
// for filter tap (kh,kw) the rows of A are the SAME chunks shifted by (kh*W + kw) positions, so the
// tcgen05 shared-memory descriptor (K-major, no swizzle: 8 rows = 8 consecutive 16-byte chunks)
// simply starts (kh*W + kw)*16 bytes further.  One bulk async copy brings an image into shared
// memory once; nine (taps) x C/32 MMAs read it in place.
//
// MaxPool is applied to the int32 accumulators BEFORE requantisation.  That is exact because the
// requantisation y = sat(rne(float(acc + bias) * M) + zp) is non-decreasing in acc whenever M > 0
// (checked on the host), so max and requantise commute.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>

#include "kernels_q8.cuh"
#include "ptx_sm100.cuh"

namespace zb {

enum DeviceError : int {
    DEV_OK = 0,
    DEV_ERR_WAIT_TIMEOUT = 1,   // a bounded mbarrier wait gave up
};

// =============================================================================================
// Stage 1: QuantizeLinear(uint8) + QLinearConv(1 -> 32, 3x3, stride 1, no pad) + ReLU + MaxPool 2x2/2
//          float [N,1,28,28]  ->  int8 C16-planar [N][2][13*13][16]
// Host-side description of the stage (the plan fills it from the graph; the kernel below takes its
// own argument block derived from it).
// =============================================================================================
struct Conv1Args {
    const float* x;
    int8_t* y;
    int n_images;
    float x_scale; int x_zp;            // QuantizeLinear of the input (uint8)
    uint32_t wpack[32][3][2];           // [m][kh][dx]: dx=0 -> bytes (w0,w1,w2,0); dx=1 -> (0,w0,w1,w2)
    float mult[32];                     // (x_scale * w_scale[m]) / y_scale
    int32_t bias[32];                   // bias[m] - x_zp * sum(w[m])   (no padding: all 9 taps always valid)
    float y_scale; int y_zp; int act;
};

// =============================================================================================
// Stage 1 kernel.  The contraction is only 9 deep and the input has one channel, so the 128-row
// tcgen05 shape has nothing to contract over; the 3x3 contraction runs on warp-level int8 MMAs (mma.sync m16n8k16, u8 x s8 -> s32):
//   rows    = 16 pooled pixels (two per thread-row group g and g+8),
//   K (16)  = the 4x4 input patch of a pooled pixel, byte (r,s) at k = 4r + s, so a thread's A
//             register is simply patch row r = lane%4 as one packed word,
//   columns = 8 output channels; the four members (dy,dx) of the 2x2 pool window are four
//             MMAs with the filter shifted inside the patch (zero where it falls outside).
// All four members of one pooled pixel and channel land in the same thread and register slot,
// so the pool is three max instructions without any data exchange.  Channels are permuted
// (group j, column n <-> channel 8*(n/2) + 2j + n%2) so that a thread ends up with eight
// consecutive channels of its two pixels and stores them as one 8-byte word each.
// =============================================================================================
struct Conv1MmaArgs {
    const float* x;
    int8_t* y;
    int n_images;
    float x_scale; int x_zp;
    const uint32_t* wfrag;   // [4 members][4 groups][32 lanes] B-fragment words
    const int32_t* biasfrag; // [4 groups][32 lanes][2]  (bias - x_zp * sum(w)) of the lane's two columns
    const float* multfrag;   // [4 groups][32 lanes][2]
    int* status;             // device status word: DEV_ERR_WAIT_TIMEOUT when a bounded wait gave up
};

__device__ __forceinline__ void mma_m16n8k16_u8s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0, const int (&c)[4]) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%8,%9,%10};"
                 : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
                 : "r"(a0), "r"(a1), "r"(b0), "r"(c[0]), "r"(c[1]), "r"(c[2]), "r"(c[3]));
}

constexpr int C1M_G = 3;               // images per CTA iteration: 507 pooled pixels = 32 units of 16
constexpr int C1M_THREADS = 256;
constexpr int C1M_UNITS = (C1M_G * 169 + 15) / 16;

constexpr int C1M_IMG_FLOATS = 28 * 28;
constexpr int C1M_GROUP_BYTES = C1M_G * C1M_IMG_FLOATS * 4;   // 9408: a multiple of 16, as the bulk copy wants

// The float images of a group arrive by one bulk async copy into a two-deep shared-memory ring: the copy
// of group i+1 is issued when the MMA phase of group i starts, so no thread waits on global loads.  The
// quantized bytes are double-buffered too, which leaves one __syncthreads per group.
// Four CTAs per SM (64 registers per thread): measured faster than three at 80 registers.
__global__ void __launch_bounds__(C1M_THREADS, 4) conv1_mma_relu_pool_kernel(const Conv1MmaArgs a) {
    __shared__ __align__(128) float stage[2][C1M_G * C1M_IMG_FLOATS];
    __shared__ uint32_t img2[2][C1M_G][28][8];   // quantized uint8 rows of 32 bytes (28 pixels + 4 pad)
    __shared__ __align__(8) uint64_t bars[2];
    __shared__ int abort_flag;
    // Per pooled pixel of an iteration (the same in every iteration): x = word of img that holds the patch's
    // first byte | odd column << 16 | image within the group << 17 | exists << 19; y = byte offset of the
    // pixel's first 16-channel chunk from the group's first image.  Keeps divisions out of the main loop.
    __shared__ uint2 pix_tab[C1M_UNITS * 16];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int stride = gridDim.x * C1M_G;
    const uint32_t bar0 = ptx::smem_u32(&bars[0]);
    if (tid == 0) {
        abort_flag = 0;
        ptx::mbar_init(bar0, 1); ptx::mbar_init(bar0 + 8, 1);
        ptx::mbar_fence_init();
        const int base = blockIdx.x * C1M_G;
        if (base < a.n_images) {
            const uint32_t bytes = (uint32_t)min(C1M_G, a.n_images - base) * (C1M_IMG_FLOATS * 4);
            ptx::mbar_arrive_expect_tx(bar0, bytes);
            ptx::bulk_g2s(ptx::smem_u32(&stage[0][0]), a.x + (size_t)base * C1M_IMG_FLOATS, bytes, bar0);
        }
    }
    for (int i = tid; i < C1M_UNITS * 16; i += C1M_THREADS) {
        const bool exists = i < C1M_G * 169;
        const int pc = exists ? i : 0;
        const int gi = pc / 169, pp = pc - gi * 169;
        const int py = pp / 13, px = pp - py * 13;
        pix_tab[i] = make_uint2((uint32_t)(gi * 224 + 2 * py * 8 + (px >> 1)) | ((uint32_t)(px & 1) << 16) | ((uint32_t)gi << 17) | ((uint32_t)exists << 19),
                                (uint32_t)(gi * 2 * 169 * 16 + pp * 16));
    }
    uint32_t wf[4][4]; int bias[4][2]; float mult[4][2];
#pragma unroll
    for (int m = 0; m < 4; ++m)
#pragma unroll
        for (int j = 0; j < 4; ++j) wf[m][j] = __ldg(a.wfrag + (m * 4 + j) * 32 + lane);
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int b = 0; b < 2; ++b) { bias[j][b] = __ldg(a.biasfrag + (j * 32 + lane) * 2 + b); mult[j][b] = __ldg(a.multfrag + (j * 32 + lane) * 2 + b); }
    __syncthreads();                               // barriers and the abort flag are set up

    const float q_lo = (float)(-a.x_zp), q_hi = (float)(255 - a.x_zp);
    int it = 0;
    for (int base = blockIdx.x * C1M_G; base < a.n_images; base += stride, ++it) {
        const int s = it & 1;
        // ---- the group's floats have landed (bounded wait; after a time-out the results are void and the
        //      status word says so)
        ptx::mbar_wait(bar0 + 8 * s, (uint32_t)(it >> 1) & 1u, &abort_flag);
        // ---- quantize C1M_G images: float4 in, four uint8 out
        uint32_t (*img)[28][8] = img2[s];
        const int n_here = min(C1M_G, a.n_images - base);
        for (int i = tid; i < C1M_G * 196; i += C1M_THREADS) {
            const int gi = i / 196, p4 = i - gi * 196;        // 196 float4 per image, 7 per row
            uint32_t word = 0;
            if (gi < n_here) {
                const float4 v = reinterpret_cast<const float4*>(stage[s])[i];
                // sat_u8(rne(clamp(t, -512, 511)) + zp) == rne(clamp(t, -zp, 255 - zp)) + zp: the bounds are integers
                // inside [-512, 511] and rounding is monotonic; a NaN becomes the lower bound either way.
                const int q0 = __float2int_rn(fminf(fmaxf(__fdiv_rn(v.x, a.x_scale), q_lo), q_hi)) + a.x_zp;
                const int q1 = __float2int_rn(fminf(fmaxf(__fdiv_rn(v.y, a.x_scale), q_lo), q_hi)) + a.x_zp;
                const int q2 = __float2int_rn(fminf(fmaxf(__fdiv_rn(v.z, a.x_scale), q_lo), q_hi)) + a.x_zp;
                const int q3 = __float2int_rn(fminf(fmaxf(__fdiv_rn(v.w, a.x_scale), q_lo), q_hi)) + a.x_zp;
                word = (uint32_t)q0 | ((uint32_t)q1 << 8) | ((uint32_t)q2 << 16) | ((uint32_t)q3 << 24);
            }
            const int r = p4 / 7, c4 = p4 - r * 7;
            img[gi][r][c4] = word;
        }
        __syncthreads();
        // ---- every thread is done with the other ring slot (it was read one group ago): refill it
        if (tid == 0 && base + stride < a.n_images) {
            const int nb = base + stride;
            const uint32_t bytes = (uint32_t)min(C1M_G, a.n_images - nb) * (C1M_IMG_FLOATS * 4);
            const uint32_t bar = bar0 + 8 * (s ^ 1);
            ptx::mbar_arrive_expect_tx(bar, bytes);
            ptx::bulk_g2s(ptx::smem_u32(&stage[s ^ 1][0]), a.x + (size_t)nb * C1M_IMG_FLOATS, bytes, bar);
        }
        // ---- 16 pooled pixels per warp iteration
        for (int u = warp; u < C1M_UNITS; u += C1M_THREADS / 32) {
            bool ok[2]; uint32_t afrag[2], out_off[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint2 e = pix_tab[u * 16 + g + 8 * h];
                ok[h] = (e.x >> 19) != 0 && base + (int)((e.x >> 17) & 3u) < a.n_images;
                out_off[h] = e.y;
                const uint32_t* row = &img[0][0][0] + (e.x & 0xffffu) + t * 8;       // patch row t of the pooled pixel
                afrag[h] = __byte_perm(row[0], row[1], (e.x & 0x10000u) ? 0x5432u : 0x3210u);
            }
            uint32_t outw[2][2];
#pragma unroll
            for (int jp = 0; jp < 2; ++jp) {          // two channel groups at a time -> one packed word per pixel
                int r[2][4];                          // [j in pair][row g: ch0, ch1 ; row g+8: ch0, ch1]
#pragma unroll
                for (int jj = 0; jj < 2; ++jj) {
                    const int j = jp * 2 + jj;
                    const int c[4] = {bias[j][0], bias[j][1], bias[j][0], bias[j][1]};
                    int d0[4], d1[4], d2[4], d3[4];
                    mma_m16n8k16_u8s8(d0, afrag[0], afrag[1], wf[0][j], c);
                    mma_m16n8k16_u8s8(d1, afrag[0], afrag[1], wf[1][j], c);
                    mma_m16n8k16_u8s8(d2, afrag[0], afrag[1], wf[2][j], c);
                    mma_m16n8k16_u8s8(d3, afrag[0], afrag[1], wf[3][j], c);
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        r[jj][k] = rq_round(__vimax_s32_relu(__vimax3_s32(d0[k], d1[k], d2[k]), d3[k]), mult[j][k & 1]);   // max of the window and ReLU: two instructions
                }
                outw[0][jp] = pack_sat_s8x4(r[0][0], r[0][1], r[1][0], r[1][1]);   // row g   : ch 8t+4jp .. +3
                outw[1][jp] = pack_sat_s8x4(r[0][2], r[0][3], r[1][2], r[1][3]);   // row g+8
            }
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                if (!ok[h]) continue;
                int8_t* yo = a.y + (size_t)base * (2 * 169 * 16) + out_off[h] + (t >> 1) * (169 * 16) + (t & 1) * 8;
                *reinterpret_cast<uint2*>(yo) = make_uint2(outw[h][0], outw[h][1]);
            }
        }
    }
    if (tid == 0 && abort_flag) atomicExch(a.status, (int)DEV_ERR_WAIT_TIMEOUT);
}

// =============================================================================================
// Stage 2: QLinearConv(32 -> COUT, 3x3, stride 1, no pad) + ReLU + MaxPool 2x2/2 on tcgen05.
//   input  int8 C16-planar [N][2][IH*IW][16]
//   output int8, either row-major [N][PH*PW*COUT] in (h,w,c) order, or blocked for a following
//          GEMM: [N/128][K/16][128 images][16]  (K = PH*PW*COUT)
// One image per tile: the 128 MMA rows are the positions p = oh*IW + ow (0..127) of the input
// grid, which cover every conv output that the 2x2 pool keeps.  Persistent CTAs, warp roles:
//   warp 0   bulk-copy producer (one elected lane), STAGES-deep ring of images
//   warp 1   TMEM owner + MMA issuer (one elected lane): 9 MMAs (K=32) per image into one of two
//            TMEM accumulators
//   warps 2-9  epilogue, two groups of four warps that alternate images (group g owns TMEM
//            accumulator g): TMEM -> registers, + bias, requantise to int8, shared staging (int8),
//            2x2 max and ReLU on packed bytes, 16-byte stores
// =============================================================================================
constexpr int TCCONV_MAX_COUT = 128;
struct TcConvPoolArgs {
    const int8_t* x;
    const int8_t* w;        // [9 taps + bias block][2 chunks][COUT][16] int8 (TcConvPoolCfg::W_BYTES)
    float mult[TCCONV_MAX_COUT];     // per output channel; read as constant-bank operands (no loads)
    int8_t* y;
    int n_images;
    float y_scale; int y_zp; int act;
    int out_blocked;        // 0 row-major, 1 GEMM-blocked
    int* status;
};

template <int IH, int IW, int COUT>
struct TcConvPoolCfg {
    static constexpr int P = IH * IW;
    static constexpr int PH = (IH - 2) / 2, PW = (IW - 2) / 2;
    static constexpr int IMG_BYTES = 2 * P * 16;
    static constexpr int STAGE_BYTES = (IMG_BYTES + 127) / 128 * 128;
    static constexpr int STAGES = 4;
    static constexpr int W_TAP_BYTES = 2 * COUT * 16;
    // A tenth block after the nine taps holds the bias as int8 factors: the MMA issuer multiplies it with a
    // constant block of (1, 127, 127, ...) rows, so the accumulators arrive with the bias already added and the
    // epilogue saves one integer add per value.  Row m of the block: k = 0 the remainder r, k = 1..31 factors
    // v with bias = r + 127 * sum(v)  (|bias| <= 127 + 31 * 127 * 127; the host checks).
    static constexpr int W_BYTES = 10 * W_TAP_BYTES;
    static constexpr int ONES_BYTES = 2 * 128 * 16;          // [2 chunks][128 rows][16]: K-major like an image
    // Staging of the requantised rows (int8).  COUT == 64: rows of 64 bytes, two per 128-byte line, the eight
    // 16-byte slots of a line permuted per row pair (stg_chunk) so that both the row-wise stores (8 consecutive
    // rows, one chunk index) and the pooling loads (two windows two rows apart, four chunks each) of a quarter
    // warp touch eight distinct slots.  Otherwise rows padded by 16 bytes (conflict-free stores only).
    static constexpr int STG_ROW = COUT == 64 ? 64 : COUT + 16;
    __host__ __device__ static constexpr int stg_chunk(int row, int c) {     // byte offset of 16-byte chunk c of a staged row
        if (COUT == 64) { const int k = row >> 1; return k * 128 + (((((row & 1) << 2) | c) ^ ((k & 3) | ((k & 1) << 2))) << 4); }
        return row * STG_ROW + c * 16;
    }
    static constexpr int STG_BYTES = 128 * STG_ROW;
    static constexpr int OFF_W = 0;
    static constexpr int OFF_A = OFF_W + W_BYTES;
    static constexpr int OFF_ONES = OFF_A + STAGES * STAGE_BYTES;
    static constexpr int OFF_STG = OFF_ONES + ONES_BYTES;          // two staging areas, one per epilogue group
    static constexpr int OFF_CONST = OFF_STG + 2 * STG_BYTES;      // float mult[COUT]; int bias[COUT]
    static constexpr int OFF_BAR = OFF_CONST + 2 * COUT * 4;
    static constexpr int SMEM_BYTES = OFF_BAR + 256;
    static constexpr int TMEM_COLS = 2 * COUT >= 32 ? 2 * COUT : 32;
    static constexpr int KOUT = PH * PW * COUT;
    static constexpr int QUADS = COUT / 16;                  // 16-channel groups: one 16-byte word of int8
    static constexpr int TASKS = PH * PW * QUADS;
    static constexpr int TASKS_PER_THREAD = (TASKS + 127) / 128;
    static constexpr int THREADS = 320;                      // producer, MMA, 2 x 4 epilogue warps
    // every position the pool keeps must be one of the 128 MMA rows, and every shifted read must
    // stay inside the image's planes
    static_assert((2 * PH - 1) * IW + (2 * PW - 1) < 128, "pooled window exceeds one 128-row tile");
    static_assert(127 + 2 * IW + 2 < 2 * P, "shifted A rows would leave the staged image");
    static_assert(COUT % 32 == 0 && COUT <= TCCONV_MAX_COUT, "COUT must be a multiple of 32 within the parameter block");
    static_assert((TMEM_COLS & (TMEM_COLS - 1)) == 0, "TMEM columns must be a power of two");
};

// Three CTAs per SM (63 registers per thread, 3 x 64 KB of shared memory, 3 x 128 TMEM columns): six epilogue
// groups per SM hide the waits of one another; measured 0.176 ms against 0.193 ms with two.
constexpr int TCCONV_CTAS_PER_SM = 3;
// Requires: int8 output with zero point 0, ReLU, positive finite multipliers (host-checked).
template <int IH, int IW, int COUT>
__global__ void __launch_bounds__(320, TCCONV_CTAS_PER_SM) tc_conv3x3_relu_pool_kernel(const __grid_constant__ TcConvPoolArgs a) {
    using Cfg = TcConvPoolCfg<IH, IW, COUT>;
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* sW = smem + Cfg::OFF_W;
    uint8_t* sA = smem + Cfg::OFF_A;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::OFF_BAR);
    // barrier slots: full[STAGES], empty[STAGES], tfull[2], tempty[2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + Cfg::OFF_BAR + 128);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + Cfg::OFF_BAR + 132);
    volatile int* epi_ok = reinterpret_cast<volatile int*>(smem + Cfg::OFF_BAR + 136);   // [2]
    const uint32_t bar0 = ptx::smem_u32(bars);
    auto full = [&](int s) { return bar0 + 8u * s; };
    auto empty = [&](int s) { return bar0 + 8u * (Cfg::STAGES + s); };
    auto tfull = [&](int b) { return bar0 + 8u * (2 * Cfg::STAGES + b); };
    auto tempty = [&](int b) { return bar0 + 8u * (2 * Cfg::STAGES + 2 + b); };

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    if (tid == 0) {
        for (int s = 0; s < Cfg::STAGES; ++s) { ptx::mbar_init(full(s), 1); ptx::mbar_init(empty(s), 1); }
        for (int b = 0; b < 2; ++b) { ptx::mbar_init(tfull(b), 1); ptx::mbar_init(tempty(b), 4); }
        *abort_flag = 0;
        epi_ok[0] = 1; epi_ok[1] = 1;
        ptx::mbar_fence_init();
    }
    for (int i = tid; i < Cfg::W_BYTES / 16; i += Cfg::THREADS)
        reinterpret_cast<uint4*>(sW)[i] = __ldg(reinterpret_cast<const uint4*>(a.w) + i);
    for (int i = tid; i < Cfg::ONES_BYTES / 16; i += Cfg::THREADS)     // the constant operand of the bias MMA
        reinterpret_cast<uint4*>(smem + Cfg::OFF_ONES)[i] = make_uint4(i < 128 ? 0x7f7f7f01u : 0x7f7f7f7fu, 0x7f7f7f7fu, 0x7f7f7f7fu, 0x7f7f7f7fu);
    ptx::fence_proxy_async_smem();
    if (warp == 1) {
        ptx::tmem_alloc(ptx::smem_u32(tmem_slot), Cfg::TMEM_COLS);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------------ producer
        if (ptx::elect_one()) {
            int it = 0;
            for (int img = blockIdx.x; img < a.n_images; img += gridDim.x, ++it) {
                const int s = it % Cfg::STAGES;
                const uint32_t ph = (uint32_t)(it / Cfg::STAGES) & 1u;
                if (!ptx::mbar_wait(empty(s), ph ^ 1u, abort_flag)) break;
                ptx::mbar_arrive_expect_tx(full(s), Cfg::IMG_BYTES);
                ptx::bulk_g2s(ptx::smem_u32(sA + s * Cfg::STAGE_BYTES), a.x + (size_t)img * Cfg::IMG_BYTES, Cfg::IMG_BYTES, full(s));
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (ptx::elect_one()) {
            constexpr uint32_t idesc = ptx::idesc_i8(128, COUT, true, true);
            const uint32_t w_addr = ptx::smem_u32(sW);
            int it = 0;
            for (int img = blockIdx.x; img < a.n_images; img += gridDim.x, ++it) {
                const int s = it % Cfg::STAGES;
                const uint32_t ph = (uint32_t)(it / Cfg::STAGES) & 1u;
                const int b = it & 1;
                const uint32_t bph = (uint32_t)(it >> 1) & 1u;
                if (!ptx::mbar_wait(tempty(b), bph ^ 1u, abort_flag)) break;
                if (!ptx::mbar_wait(full(s), ph, abort_flag)) break;
                ptx::tc_fence_after();
                const uint32_t a_addr = ptx::smem_u32(sA + s * Cfg::STAGE_BYTES);
                const uint32_t d_tmem = tmem_base + (uint32_t)(b * COUT);
#pragma unroll
                for (int tap = 0; tap < 9; ++tap) {
                    const int kh = tap / 3, kw = tap - kh * 3;
                    const uint64_t da = ptx::smem_desc_kmajor(a_addr + (uint32_t)((kh * IW + kw) * 16), Cfg::P * 16, 128);
                    const uint64_t db = ptx::smem_desc_kmajor(w_addr + (uint32_t)(tap * Cfg::W_TAP_BYTES), COUT * 16, 128);
                    ptx::mma_i8(d_tmem, da, db, idesc, tap > 0);
                }
                ptx::mma_i8(d_tmem, ptx::smem_desc_kmajor(ptx::smem_u32(smem + Cfg::OFF_ONES), 128 * 16, 128),
                            ptx::smem_desc_kmajor(w_addr + (uint32_t)(9 * Cfg::W_TAP_BYTES), COUT * 16, 128), idesc, true);   // + bias
                ptx::mma_commit(empty(s));    // the image's smem stage is free once these MMAs retire
                ptx::mma_commit(tfull(b));    // ... and the accumulator is complete
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue: two groups of 4 warps;
        // group g owns TMEM accumulator g and handles the images whose iteration index is g mod 2.
        const int g = (warp - 2) >> 2;
        const int quarter = warp & 3;               // TMEM lane quarter this warp may access
        const int row = quarter * 32 + lane;        // MMA row = input-grid position
        const int e = ((warp - 2) & 3) * 32 + lane; // 0..127 within the group
        uint8_t* sStg = smem + Cfg::OFF_STG + g * Cfg::STG_BYTES;
        // this thread's pooled outputs (16 channels each): staging offset of the window's top-left
        // row and output offset
        int stg_off[Cfg::TASKS_PER_THREAD][4]; int out_off[Cfg::TASKS_PER_THREAD];   // the four members of the pool window
#pragma unroll
        for (int k = 0; k < Cfg::TASKS_PER_THREAD; ++k) {
            const int t = e + 128 * k;
            const int q = t / Cfg::QUADS, cg = t - q * Cfg::QUADS;
            const int py = q / Cfg::PW, px = q - py * Cfg::PW;
            const int p0 = 2 * py * IW + 2 * px;
            stg_off[k][0] = (t < Cfg::TASKS) ? Cfg::stg_chunk(p0, cg) : -1;
            stg_off[k][1] = Cfg::stg_chunk(p0 + 1, cg);
            stg_off[k][2] = Cfg::stg_chunk(p0 + IW, cg);
            stg_off[k][3] = Cfg::stg_chunk(p0 + IW + 1, cg);
            out_off[k] = a.out_blocked ? (q * Cfg::QUADS + cg) * 2048 : q * COUT + cg * 16;
        }
        const uint32_t bar_id = 1u + (uint32_t)g;
        int it = g;
        for (int img = blockIdx.x + g * (int)gridDim.x; img < a.n_images; img += 2 * (int)gridDim.x, it += 2) {
            const uint32_t bph = (uint32_t)(it >> 1) & 1u;
            if (e == 0) epi_ok[g] = ptx::mbar_wait(tfull(g), bph, abort_flag) ? 1 : 0;
            ptx::named_barrier_sync(bar_id, 128);   // also: the group finished reading the staging of its previous image
            if (!epi_ok[g]) break;
            ptx::tc_fence_after();
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(g * COUT);
            // requantise this row (max-pool and ReLU commute with it and are applied to the int8 values)
#pragma unroll
            for (int h = 0; h < COUT / 32; ++h) {
                uint32_t v[32];
                ptx::tmem_ld32(taddr + (uint32_t)(h * 32), v);
                ptx::tmem_wait_ld();
                uint32_t pk[8];
#pragma unroll
                for (int j4 = 0; j4 < 8; ++j4) {
                    const int c = h * 32 + j4 * 4;     // compile-time after unrolling: constant-bank operands
                    pk[j4] = pack_sat_s8x4(rq_round((int)v[j4 * 4 + 0], a.mult[c + 0]),
                                           rq_round((int)v[j4 * 4 + 1], a.mult[c + 1]),
                                           rq_round((int)v[j4 * 4 + 2], a.mult[c + 2]),
                                           rq_round((int)v[j4 * 4 + 3], a.mult[c + 3]));
                }
                *reinterpret_cast<uint4*>(sStg + Cfg::stg_chunk(row, 2 * h)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                *reinterpret_cast<uint4*>(sStg + Cfg::stg_chunk(row, 2 * h + 1)) = make_uint4(pk[4], pk[5], pk[6], pk[7]);
            }
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(tempty(g));   // accumulator g may be overwritten
            ptx::named_barrier_sync(bar_id, 128);
            int8_t* ybase = a.out_blocked ? a.y + (size_t)(img >> 7) * (Cfg::KOUT / 16) * 2048 + (size_t)(img & 127) * 16
                                          : a.y + (size_t)img * Cfg::KOUT;
#pragma unroll
            for (int k = 0; k < Cfg::TASKS_PER_THREAD; ++k) {
                if (stg_off[k][0] < 0) continue;
                const uint4 r0 = *reinterpret_cast<const uint4*>(sStg + stg_off[k][0]);
                const uint4 r1 = *reinterpret_cast<const uint4*>(sStg + stg_off[k][1]);
                const uint4 r2 = *reinterpret_cast<const uint4*>(sStg + stg_off[k][2]);
                const uint4 r3 = *reinterpret_cast<const uint4*>(sStg + stg_off[k][3]);
                uint4 o;
                o.x = relu_s8x4(__vmaxs4(__vmaxs4(r0.x, r1.x), __vmaxs4(r2.x, r3.x)));
                o.y = relu_s8x4(__vmaxs4(__vmaxs4(r0.y, r1.y), __vmaxs4(r2.y, r3.y)));
                o.z = relu_s8x4(__vmaxs4(__vmaxs4(r0.z, r1.z), __vmaxs4(r2.z, r3.z)));
                o.w = relu_s8x4(__vmaxs4(__vmaxs4(r0.w, r1.w), __vmaxs4(r2.w, r3.w)));
                *reinterpret_cast<uint4*>(ybase + out_off[k]) = o;
            }
        }
    }

    // ---------------------------------------------------------------------- teardown
    if (*abort_flag) {
        // give copies and MMAs that are still in flight time to land before the CTA's memory goes away
        for (int i = 0; i < 200; ++i) __nanosleep(1000);
    }
    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 1) ptx::tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
    if (tid == 0 && *abort_flag) atomicExch(a.status, (int)DEV_ERR_WAIT_TIMEOUT);
}

}  // namespace zb
