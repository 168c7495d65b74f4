// Fused kernels for quantized 3x3 convolution stages followed by ReLU and a 2x2/2 MaxPool.
//
// Internal activation layout between the two stages, "parity planes": every pixel of a 16-channel group is one
// 16-byte chunk, and the chunks of the pixels with the same (row parity, column parity) form one plane in
// row-major order of (row/2, column/2), images one after the other.  With that layout the A operand of an
// implicit-GEMM convolution FOLLOWED BY a 2x2/2 pool needs no im2col at all: for member (dy,dx) of a pool
// window and filter tap (kh,kw) the rows of A (one per pool window) are consecutive chunks of one plane,
// shifted by a constant, so the tcgen05 shared-memory descriptor (K-major, no swizzle: 8 rows = 8
// consecutive 16-byte chunks) simply starts a few rows further.
//
// MaxPool is applied to the int32 accumulators BEFORE requantisation.  That is exact because the
// requantisation y = sat(rne(float(acc + bias) * M) + zp) is non-decreasing in acc whenever M > 0
// (checked on the host), so max and requantise commute; the bias is the same for the four members of a
// window, so it is added after the max.
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
//          float [N,1,28,28]  ->  int8 parity planes (Conv1MmaArgs::plane_bytes)
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
    // Output layout: parity planes for tc_conv3x3_pool_parity_kernel, [2 chunks][4 parities][N*36 rows (+ padding)][16],
    // `plane_bytes` apart: pooled pixel (y, x), y and x below 12, lies in plane (y&1)*2 + (x&1) at row
    // n*36 + (y>>1)*6 + (x>>1); row and column 12 are neither computed nor stored (the next stage's pool never
    // reads them).
    long long plane_bytes;
};

__device__ __forceinline__ void mma_m16n8k16_u8s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0, const int (&c)[4]) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%8,%9,%10};"
                 : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
                 : "r"(a0), "r"(a1), "r"(b0), "r"(c[0]), "r"(c[1]), "r"(c[2]), "r"(c[3]));
}

// Images per CTA iteration: 4 x 144 pooled pixels = 36 units of 16.
constexpr int C1M_G = 4;
constexpr int C1M_THREADS = 256;
constexpr int C1M_UNITS = (C1M_G * 144 + 15) / 16;

constexpr int C1M_IMG_FLOATS = 28 * 28;
constexpr int C1M_GROUP_BYTES = C1M_G * C1M_IMG_FLOATS * 4;   // 9408: a multiple of 16, as the bulk copy wants

// The float images of a group arrive by one bulk async copy into a two-deep shared-memory ring: the copy
// of group i+1 is issued when the MMA phase of group i starts, so no thread waits on global loads.  The
// quantized bytes are double-buffered too, which leaves one __syncthreads per group.
// Three CTAs per SM (80 registers per thread; a fourth would need 64 registers and spills).
__global__ void __launch_bounds__(C1M_THREADS, 3) conv1_mma_relu_pool_kernel(const Conv1MmaArgs a) {
    __shared__ __align__(128) float stage[2][C1M_G * C1M_IMG_FLOATS];
    __shared__ uint32_t img2[2][C1M_G][28][8];   // quantized uint8 rows of 32 bytes (28 pixels + 4 pad)
    __shared__ __align__(8) uint64_t bars[2];
    __shared__ int abort_flag;
    // Per pooled pixel of an iteration (the same in every iteration): x = word of img that holds the patch's
    // first byte | odd column << 16 | image within the group << 17 (3 bits) | exists << 20; y = byte offset of the
    // pixel's first 16-channel chunk from the group's first image (and, with parity planes, from plane 0).  Keeps divisions out of the main loop.
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
    // Parity planes: only the 12 x 12 pooled pixels that the next stage reads are computed, enumerated plane by
    // plane (a unit's 16 pixels are 16 consecutive rows of one plane: contiguous stores).
    constexpr int n_pix = C1M_G * 144, n_units = (n_pix + 15) / 16;
    for (int i = tid; i < C1M_UNITS * 16; i += C1M_THREADS) {
        const bool exists = i < n_pix;
        const int pc = exists ? i : 0;
        const int gi = pc / 144, rem = pc - gi * 144;
        const int plane = rem / 36, rloc = rem - plane * 36;
        const int py = 2 * (rloc / 6) + (plane >> 1), px = 2 * (rloc % 6) + (plane & 1);
        const uint32_t off = (uint32_t)(plane * a.plane_bytes) + (uint32_t)((gi * 36 + rloc) * 16);
        pix_tab[i] = make_uint2((uint32_t)(gi * 224 + 2 * py * 8 + (px >> 1)) | ((uint32_t)(px & 1) << 16) | ((uint32_t)gi << 17) | ((uint32_t)exists << 20), off);
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
    // this thread's 8 channels: chunk t >> 1 (four parity planes further), half t & 1
    int8_t* const y_thread = a.y + (size_t)(t >> 1) * 4 * (size_t)a.plane_bytes + (t & 1) * 8;
    constexpr size_t img_bytes = 36 * 16;
    int it = 0;
    for (int base = blockIdx.x * C1M_G; base < a.n_images; base += stride, ++it) {
        const int s = it & 1;
        // ---- the group's floats have landed (bounded wait; after a time-out the results are void and the
        //      status word says so)
        ptx::mbar_wait(bar0 + 8 * s, (uint32_t)(it >> 1) & 1u, &abort_flag);
        // ---- quantize C1M_G images: float4 in, four uint8 out
        uint32_t (*img)[28][8] = img2[s];
        const int n_here = min(C1M_G, a.n_images - base);
        // pooled rows and columns 0..11 read input rows 0..25 only (26 rows of 7 float4)
        constexpr int f4_per_img = 182;
        for (int i = tid; i < C1M_G * f4_per_img; i += C1M_THREADS) {
            const int gi = i / f4_per_img, p4 = i - gi * f4_per_img;        // 7 float4 per row
            uint32_t word = 0;
            if (gi < n_here && a.x_zp == 0) {
                // zero point 0: sat_u8(rne(clamp(t, -512, 511))) is the float -> int32 conversion (rne, a NaN gives 0) followed
                // by the pack instruction's own saturation to [0, 255]; no clamps, no adds (the ALU pipe bounds this kernel)
                const float4 v = reinterpret_cast<const float4*>(stage[s])[gi * 196 + p4];
                const int q0 = __float2int_rn(__fdiv_rn(v.x, a.x_scale)), q1 = __float2int_rn(__fdiv_rn(v.y, a.x_scale));
                const int q2 = __float2int_rn(__fdiv_rn(v.z, a.x_scale)), q3 = __float2int_rn(__fdiv_rn(v.w, a.x_scale));
                uint32_t hi;
                asm("cvt.pack.sat.u8.s32.b32 %0, %1, %2, 0;" : "=r"(hi) : "r"(q3), "r"(q2));
                asm("cvt.pack.sat.u8.s32.b32 %0, %1, %2, %3;" : "=r"(word) : "r"(q1), "r"(q0), "r"(hi));
            } else if (gi < n_here) {
                const float4 v = reinterpret_cast<const float4*>(stage[s])[gi * 196 + p4];
                // sat_u8(rne(clamp(t, -512, 511)) + zp) == rne(clamp(t, -zp, 255 - zp)) + zp: the bounds are integers
                // inside [-512, 511] and rounding is monotonic; a NaN becomes the lower bound either way.
                // (the proof-by-residual form of quantize_fast costs this kernel more issue slots than the division it saves)
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
        for (int u = warp; u < n_units; u += C1M_THREADS / 32) {
            bool ok[2]; uint32_t afrag[2], out_off[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint2 e = pix_tab[u * 16 + g + 8 * h];
                ok[h] = (e.x >> 20) != 0 && base + (int)((e.x >> 17) & 7u) < a.n_images;
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
                int8_t* yo = y_thread + (size_t)base * img_bytes + out_off[h];
                *reinterpret_cast<uint2*>(yo) = make_uint2(outw[h][0], outw[h][1]);
            }
        }
    }
    if (tid == 0 && abort_flag) atomicExch(a.status, (int)DEV_ERR_WAIT_TIMEOUT);
}

// =============================================================================================
// Stage 2, pool windows on the MMA rows: QLinearConv(32 -> 64, 3x3, no pad) + ReLU + MaxPool 2x2/2 from the
// parity-plane layout that stage 1 writes (Conv1MmaArgs::plane_bytes).
//
// MMA row r of tile t is pool window R = t*128 + r of the whole batch: image R / 36, window (py, px) =
// ((R % 36) / 6, (R % 36) % 6) (py, px < 5 exist).  The four members (dy, dx) of a window are four
// accumulators (TMEM columns m*64 ..): member (dy, dx), tap (kh, kw) reads input pixel
// (2py + dy + kh, 2px + dx + kw), which lies in parity plane ((dy+kh)&1, (dx+kw)&1) at row
// R + ((dy+kh)>>1)*6 + ((dx+kw)>>1) -- the same 128 consecutive rows of that plane, shifted.  So a tile is
// eight bulk copies (2 chunks x 4 planes, 136 rows of 16 bytes each) and 24 MMAs (12 of 128x128x32 that serve two
// members at once, 12 of 128x64x32), and a thread
// of the epilogue holds all four members of its window: max, bias, ReLU and requantisation happen in
// registers on a quarter of the values, with no staging; a window's 64 channels leave as four 16-byte stores
// into the GEMM-blocked layout [N/128][1600/16][128 images][16].
//   warp 0 producer, warp 1 MMA issuer (TMEM: two sets of 4 x 64 columns, so the epilogue of a tile overlaps the
//   MMAs of the next), warps 2-17 epilogue.
// =============================================================================================
// Optional per-role cycle counters of the kernel below (debug builds with -DZB_TC_CONV_TIMERS only).
#ifdef ZB_TC_CONV_TIMERS
__device__ unsigned long long g_c2_timers[256 * 8];
#define ZB_C2T_DECL() long long c2t_[8] = {0, 0, 0, 0, 0, 0, 0, 0}; long long c2t0_ = clock64()
#define ZB_C2T(slot) do { const long long n_ = clock64(); c2t_[slot] += n_ - c2t0_; c2t0_ = n_; } while (0)
#define ZB_C2T_DUMP(lo, hi) do { for (int i_ = (lo); i_ < (hi); ++i_) g_c2_timers[blockIdx.x * 8 + i_] = (unsigned long long)c2t_[i_]; } while (0)
#else
#define ZB_C2T_DECL() do {} while (0)
#define ZB_C2T(slot) do {} while (0)
#define ZB_C2T_DUMP(lo, hi) do {} while (0)
#endif

struct TcConvParityArgs {
    const int8_t* x; long long plane_bytes;
    const int8_t* w;                 // [9 taps][2 chunks][64][16] int8, then the paired blocks (TcConvParityCfg::W_ALL_BYTES)
    float mult[64]; int32_t bias[64];   // per filter; bias includes -x_zp * sum(w); constant-bank operands
    int8_t* y;
    int n_images, n_tiles;           // n_tiles = ceil(n_images * 36 / 128)
    int* status;
};

struct TcConvParityCfg {
    static constexpr int ROWS = 136;                         // 128 + the largest shift (7), rounded up to 8
    static constexpr int PLANE_BYTES = ROWS * 16;
    static constexpr int STAGE_BYTES = 8 * PLANE_BYTES;
    static constexpr int STAGES = 6;                         // 104 KB of stages: also keeps a second CTA (which would wait for TMEM) off the SM
    static constexpr int W_TAP_BYTES = 2 * 64 * 16;
    static constexpr int W_BYTES = 9 * W_TAP_BYTES;
    // paired blocks after the nine taps: [kh][j][2 chunks][128 rows][16]; j = 0: rows 0-63 tap (kh,1), rows 64-127 tap
    // (kh,0); j = 1: rows 0-63 tap (kh,2), rows 64-127 tap (kh,1)   (member dx = 0 first, then dx = 1)
    static constexpr int W_PAIR_BYTES = 2 * 128 * 16;
    static constexpr int W_ALL_BYTES = W_BYTES + 6 * W_PAIR_BYTES;
    static constexpr int OFF_W = 0;
    static constexpr int OFF_A = OFF_W + W_ALL_BYTES;
    static constexpr int OFF_BAR = OFF_A + STAGES * STAGE_BYTES;
    static constexpr int SMEM_BYTES = OFF_BAR + 256;
    static constexpr int TMEM_COLS = 512;                    // 2 sets x 4 members x 64 filters
    static constexpr int THREADS = 576;                      // producer, MMA issuer, 16 epilogue warps
    // rows of a plane that a batch needs: every tile copies ROWS rows from its first row
    static long long plane_rows(long long n_tiles) { return n_tiles * 128 + (ROWS - 128); }
};

__global__ void __launch_bounds__(576, 1) tc_conv3x3_pool_parity_kernel(const __grid_constant__ TcConvParityArgs a) {
    using Cfg = TcConvParityCfg;
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* sW = smem + Cfg::OFF_W;
    uint8_t* sA = smem + Cfg::OFF_A;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::OFF_BAR);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + Cfg::OFF_BAR + 128);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + Cfg::OFF_BAR + 132);
    const uint32_t bar0 = ptx::smem_u32(bars);
    auto full = [&](int s) { return bar0 + 8u * s; };
    auto empty = [&](int s) { return bar0 + 8u * (Cfg::STAGES + s); };
    auto tfull = [&](int b) { return bar0 + 8u * (2 * Cfg::STAGES + b); };
    auto tempty = [&](int b) { return bar0 + 8u * (2 * Cfg::STAGES + 2 + b); };
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    if (tid == 0) {
        for (int s = 0; s < Cfg::STAGES; ++s) { ptx::mbar_init(full(s), 1); ptx::mbar_init(empty(s), 1); }
        for (int b = 0; b < 2; ++b) { ptx::mbar_init(tfull(b), 1); ptx::mbar_init(tempty(b), 16); }
        *abort_flag = 0;
        ptx::mbar_fence_init();
    }
    for (int i = tid; i < Cfg::W_ALL_BYTES / 16; i += Cfg::THREADS)
        reinterpret_cast<uint4*>(sW)[i] = __ldg(reinterpret_cast<const uint4*>(a.w) + i);
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
            ZB_C2T_DECL();
            for (int t = blockIdx.x; t < a.n_tiles; t += gridDim.x, ++it) {
                const int s = it % Cfg::STAGES;
                const uint32_t ph = (uint32_t)(it / Cfg::STAGES) & 1u;
                if (!ptx::mbar_wait(empty(s), ph ^ 1u, abort_flag)) break;
                ZB_C2T(3);
                ptx::mbar_arrive_expect_tx(full(s), Cfg::STAGE_BYTES);
                const int8_t* src = a.x + (size_t)t * (128 * 16);
                const uint32_t dst = ptx::smem_u32(sA + s * Cfg::STAGE_BYTES);
#pragma unroll
                for (int pl = 0; pl < 8; ++pl)
                    ptx::bulk_g2s(dst + (uint32_t)(pl * Cfg::PLANE_BYTES), src + (size_t)pl * (size_t)a.plane_bytes, Cfg::PLANE_BYTES, full(s));
                ZB_C2T(7);
            }
            ZB_C2T_DUMP(3, 4);
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (ptx::elect_one()) {
            constexpr uint32_t idesc64 = ptx::idesc_i8(128, 64, true, true), idesc128 = ptx::idesc_i8(128, 128, true, true);
            const uint32_t w_addr = ptx::smem_u32(sW);
            int it = 0;
            ZB_C2T_DECL();
            for (int t = blockIdx.x; t < a.n_tiles; t += gridDim.x, ++it) {
                const int s = it % Cfg::STAGES;
                const uint32_t ph = (uint32_t)(it / Cfg::STAGES) & 1u;
                const int b = it & 1;
                const uint32_t bph = (uint32_t)(it >> 1) & 1u;
                if (!ptx::mbar_wait(tempty(b), bph ^ 1u, abort_flag)) break;
                ZB_C2T(0);
                if (!ptx::mbar_wait(full(s), ph, abort_flag)) break;
                ZB_C2T(1);
                ptx::tc_fence_after();
                const uint32_t a_addr = ptx::smem_u32(sA + s * Cfg::STAGE_BYTES);
                // Input pixel (2py + ry, 2px + rx), ry = dy + kh, rx = dx + kw, 0..3 each: one shifted view of one plane.
                // The view (ry, rx = 1 or 2) serves both members dx = 0 (kw = rx) and dx = 1 (kw = rx - 1) of a row dy:
                // one MMA of 128 filters-times-members over the paired weight block instead of two of 64 (an N = 64
                // MMA is bound by its 6 KB of shared-memory operands, not by its 32 cycles of math).
#pragma unroll
                for (int kh = 0; kh < 3; ++kh) {
#pragma unroll
                    for (int dy = 0; dy < 2; ++dy) {
                        const int ry = dy + kh;
                        auto view = [&](int rx) {
                            const int plane = (ry & 1) * 2 + (rx & 1), shift = (ry >> 1) * 6 + (rx >> 1);
                            return ptx::smem_desc_kmajor(a_addr + (uint32_t)(plane * Cfg::PLANE_BYTES + shift * 16), 4 * Cfg::PLANE_BYTES, 128);
                        };
                        auto w64 = [&](int kw) { return ptx::smem_desc_kmajor(w_addr + (uint32_t)((kh * 3 + kw) * Cfg::W_TAP_BYTES), 64 * 16, 128); };
                        auto w128 = [&](int j) { return ptx::smem_desc_kmajor(w_addr + (uint32_t)(Cfg::W_BYTES + (kh * 2 + j) * Cfg::W_PAIR_BYTES), 128 * 16, 128); };
                        const uint32_t d = tmem_base + (uint32_t)(b * 256 + dy * 128);     // members (dy, 0) and (dy, 1): 2 x 64 columns
                        ptx::mma_i8(d, view(1), w128(0), idesc128, kh > 0);               // the first MMA of a set initialises both members
                        ptx::mma_i8(d, view(2), w128(1), idesc128, true);
                        ptx::mma_i8(d, view(0), w64(0), idesc64, true);
                        ptx::mma_i8(d + 64u, view(3), w64(2), idesc64, true);
                    }
                }
                ptx::mma_commit(empty(s));
                ptx::mma_commit(tfull(b));
                ZB_C2T(2);
            }
            ZB_C2T_DUMP(0, 3);
        }
    } else {
        // ------------------------------------------------------------------ epilogue: 16 warps, four per TMEM lane
        // quarter; each takes 16 of the 64 filters of its quarter's 32 windows, in every tile (a single warp per
        // quarter and tile would be latency-bound and slower than the MMAs of the next tile).
        const int quarter = warp & 3;               // TMEM lane quarter this warp may access
        const int cg = (warp - 2) >> 2;             // 16-filter group of this warp
        const int row = quarter * 32 + lane;        // MMA row = pool window within the tile
        float mult[16]; int bias[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) { mult[j] = a.mult[cg * 16 + j]; bias[j] = a.bias[cg * 16 + j]; }
        int it = 0;
        ZB_C2T_DECL();
        for (int t = blockIdx.x; t < a.n_tiles; t += gridDim.x, ++it) {
            const int b = it & 1;
            const uint32_t bph = (uint32_t)(it >> 1) & 1u;
            int ok = 1;
            if (lane == 0) ok = ptx::mbar_wait(tfull(b), bph, abort_flag) ? 1 : 0;
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) break;
            ZB_C2T(4);
            ptx::tc_fence_after();
            const int R = t * 128 + row;
            const int n = R / 36, q = R - 36 * n;
            const int py = q / 6, px = q - py * 6;
            const bool live = n < a.n_images && py < 5 && px < 5;
            int8_t* yw = a.y + (size_t)(n >> 7) * (1600 / 16) * 2048 + (size_t)(n & 127) * 16 + (size_t)((py * 5 + px) * 4 + cg) * 2048;
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(b * 256 + cg * 16);
            uint32_t v[4][16];
#pragma unroll
            for (int m = 0; m < 4; ++m) ptx::tmem_ld16(taddr + (uint32_t)(m * 64), v[m]);
            ptx::tmem_wait_ld();
            ZB_C2T(5);
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(tempty(b));   // this warp has its values: the set may be overwritten once all 16 arrived
            uint32_t pk[4];
#pragma unroll
            for (int j4 = 0; j4 < 4; ++j4) {
                int r[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int c = j4 * 4 + j;
                    const int mx = max(__vimax3_s32((int)v[0][c], (int)v[1][c], (int)v[2][c]), (int)v[3][c]);
                    r[j] = rq_round(mx + bias[c], mult[c]);
                }
                pk[j4] = relu_s8x4(pack_sat_s8x4(r[0], r[1], r[2], r[3]));
            }
            if (live) *reinterpret_cast<uint4*>(yw) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
            ZB_C2T(6);
        }
        if (warp == 2 && lane == 0) ZB_C2T_DUMP(4, 7);
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
