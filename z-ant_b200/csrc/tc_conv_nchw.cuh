// Implicit-GEMM QLinearConv on tcgen05 that reads and writes the reference's NCHW layout directly
// (group 1, stride 1, any kernel size / dilation / padding, weight zero points 0).
//
// A tile is RB row blocks of BH output rows x BW output columns of one image (a row block is what one
// 128-row MMA covers); its input patch (PH x PW pixels, halo included, shared by the row blocks so that
// the halo rows are fetched and transposed once per tile, not once per block) is brought in CB*16
// channels at a time:
//   1. the loader warp issues one tiled TMA load per stage: a box of CB*16 channels x the input bytes
//      that hold the patch rows (one run per channel when the tile spans the image width, else one
//      per row) into a staging buffer.  A box starts at the 16-byte boundary below its first wanted
//      byte, so the data sits `shift` bytes into its slot; the host admits only shapes for which
//      `shift` is the same for every channel of a stage (H*W % 16 == 0, and W % 16 == 0 when rows
//      are separate runs);
//   2. eight warps transpose staging -> "patch" [16-channel group][patch pixel][16 channels], one
//      16-byte chunk per pixel, pixels in row-major order of the patch (4x4 byte transposes with
//      prmt); pixels outside the image are replaced by the input zero point on the way.
// In that form filter tap (kh,kw) of the implicit GEMM is the same shared memory shifted by
// (kh*dh*PW + kw*dw) chunks, which a K-major no-swizzle shared-memory descriptor expresses
// directly: MMA row r of row block b stands for patch pixel b*BH*PW + r, i.e. output
// (b*BH + r / PW, r % PW) of the tile; rows with r % PW >= BW or r / PW >= BH are computed and
// dropped.  Each row block accumulates in its own TMEM columns.  No im2col matrix exists anywhere.
// 1x1 convolutions skip steps 1-2: a box of 128 pixels x CB*16 channels, loaded with the 128-byte swizzle,
// is already a valid MMA operand (MN-major: the pixel index is the contiguous one), so the loader
// signals the MMA issuer directly and the transposing warps stay idle.
// Weights are pre-blocked [filter tile][channel stage][tap][CB][NT][16]; they stay resident in
// shared memory when there is a single filter tile, else one bulk copy per stage streams them.
// The epilogue requantises into a shared-memory image of the tile's NCHW bytes and copies it out
// as one contiguous run per filter.
//
// Warp roles (576 threads, one persistent CTA per SM):
//   warp 0       loader (bulk copies)          warp 1        TMEM owner + MMA issuer
//   warps 2-9    transpose (1x1: epilogue)     warps 10-17   epilogue
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <type_traits>
#include <vector>

#include "context.cuh"
#include "geometry.hpp"
#include "kernels_q8.cuh"
#include "ptx_sm100.cuh"

namespace zb {

struct TcConvArgs {
    const uint8_t* x; uint8_t* y; const int8_t* w; const float* mult; const int32_t* bias;
    int N, C, H, W, M, OH, OW;        // M = filters; for 1x1 convolutions the host passes H = 1, W = H*W
    int KH, KW, dh, dw, pt, pl;
    int BH, BW, PH, PW, PR;           // row block, patch, allocated patch pixels per 16-channel group
    int RB, BHT;                      // row blocks per tile (1, 2 or 4); output rows per tile = RB * BH
    int hseg, wseg, c_stages, n_tiles;
    int CB;                           // 16-channel groups per stage (2, 4 or 8)
    int direct;                       // 1x1 convolution: the MMA operand is the input itself (MN-major, 128-byte swizzle), no transposes.
                                      // 1: a TMA box lands in that form; 2: image planes are not multiples of 16 bytes (no tensor map
                                      // exists), warps 2-9 copy the rows with 4-byte loads into the same swizzled form
    int full_width;                   // 1: a tile spans the image width and a channel's patch rows are one run; 0: one run per row
    int RP;                           // staging bytes between two patch rows of a channel (W, or the run pitch when rows are separate runs)
    int CP;                           // staging bytes per channel
    int KN;                           // staging words per patch row that the transpose visits (upper bound over tiles)
    int log2V;
    int w_resident;                   // all weights of the (single) filter tile stay in shared memory at off_wres
    int off_wres;
    int stages, stage_bytes, off_patch, off_stg, off_out;   // a stage = weights | patch | staging; off_out: output staging
    int V;                            // bytes per global store of the epilogue's copy-out (1, 2, 4, 8 or 16)
    uint32_t pad_word;                // the input zero point in all four bytes
    float y_scale; int y_zp; int act; int out_u8;
    int six;                          // lean epilogue: sat8(rne(6 / y_scale)), used by ReLU6
    int small_products;               // lean epilogue: every |accumulator * multiplier| is below 2^22 (host-checked bound)
    int m_pad;                        // filters rounded up to the tile width
    const uint8_t* lut;               // optional 256-entry table applied to the output codes (see Requant)
    int pool;                         // NCHW kernel: 1 = a 2x2 / stride-2 MaxPool follows; y is the POOLED tensor [N, M, OH/2, OW/2]
    int POH, POW;                     // pooled output dimensions (floor)
    int* status;
};

constexpr int kTcConvMaxStages = 6;
constexpr int kTcConvMaxFilters = 1024;
constexpr int kTcConvThreads = 576;                             // 2 + 8 producer + 8 epilogue warps
constexpr int kTcConvOutPitch = 128;                            // bytes per filter in the output staging buffer
constexpr int kTcConvTail = 2 * kTcConvMaxFilters * 4 + 512 + 256;   // constants + barriers + the activation table after the stages

// out[p] = bytes (a[p], b[p], c[p], d[p]) for p = 0..3
__device__ __forceinline__ void transpose_4x4_bytes(uint32_t a, uint32_t b, uint32_t c, uint32_t d, uint32_t out[4]) {
    const uint32_t t0 = __byte_perm(a, b, 0x5140), t1 = __byte_perm(c, d, 0x5140);
    const uint32_t t2 = __byte_perm(a, b, 0x7362), t3 = __byte_perm(c, d, 0x7362);
    out[0] = __byte_perm(t0, t1, 0x5410); out[1] = __byte_perm(t0, t1, 0x7632);
    out[2] = __byte_perm(t2, t3, 0x5410); out[3] = __byte_perm(t2, t3, 0x7632);
}

// Optional per-role cycle counters (debug builds with -DZB_TC_CONV_TIMERS only).
#ifdef ZB_TC_CONV_TIMERS
__device__ unsigned long long g_tc_conv_timers[256 * 32];
#define ZB_T0() long long zb_t_ = clock64()
#define ZB_TACC(slot) do { const long long n_ = clock64(); zb_acc_[slot] += n_ - zb_t_; zb_t_ = n_; } while (0)
#define ZB_TDECL() long long zb_acc_[8] = {0, 0, 0, 0, 0, 0, 0, 0}
#define ZB_TSUB0() long long zb_q_ = clock64()
#define ZB_TSUB(slot) do { const long long n_ = clock64(); zb_acc_[slot] += n_ - zb_q_; zb_q_ = n_; } while (0)
#define ZB_TDUMP(base) do { for (int i_ = 0; i_ < 8; ++i_) g_tc_conv_timers[blockIdx.x * 32 + (base) + i_] = (unsigned long long)zb_acc_[i_]; } while (0)
#else
#define ZB_T0() do {} while (0)
#define ZB_TACC(slot) do {} while (0)
#define ZB_TDECL() do {} while (0)
#define ZB_TSUB0() do {} while (0)
#define ZB_TSUB(slot) do {} while (0)
#define ZB_TDUMP(base) do {} while (0)
#endif

// Requantisation of the lean epilogue: rq_round (the float-to-int conversion saturates at the int32 range and
// the saturating pack that follows clamps to int8, which equals the reference's clamp for zero point 0).  Both
// CLAMP instantiations are the same code.
template <bool CLAMP>
__device__ __forceinline__ int tc_conv_round(int acc, float m) { return rq_round(acc, m); }

// Where a tile sits: image, first output row / column, filter tile, and the loader's view of its
// input patch: first input row / column, the patch rows and image columns that exist, and where
// the data of a run lands in its staging slot.
struct TcConvTile {
    int img, h0, w0, nt;
    int h_in0, w_in0;
    int hh_lo, hh_hi;        // patch rows [hh_lo, hh_hi) lie inside the image
    int iw_lo, iw_hi;        // image columns [iw_lo, iw_hi) are loaded
    int shift;               // bytes between the 16-byte boundary a run is copied from and its first wanted byte
    int S0;                  // staging byte (within a row of a run) that holds patch column 0
};

// Mixed-radix counter over (image, row segment, column segment, filter tile) that advances by the
// grid size without dividing: the per-tile paths of every role stay free of integer division.
struct TcConvCursor {
    int nt, ws, hs, img;
    int d_nt, d_ws, d_hs, d_img;
};

__device__ __forceinline__ void tc_conv_cursor_init(const TcConvArgs& a, int t0, int step, TcConvCursor& c) {
    c.nt = t0 % a.n_tiles; t0 /= a.n_tiles; c.ws = t0 % a.wseg; t0 /= a.wseg; c.hs = t0 % a.hseg; c.img = t0 / a.hseg;
    c.d_nt = step % a.n_tiles; step /= a.n_tiles; c.d_ws = step % a.wseg; step /= a.wseg; c.d_hs = step % a.hseg; c.d_img = step / a.hseg;
}

__device__ __forceinline__ void tc_conv_cursor_next(const TcConvArgs& a, TcConvCursor& c) {
    c.nt += c.d_nt; int carry = c.nt >= a.n_tiles ? 1 : 0; c.nt -= carry ? a.n_tiles : 0;
    c.ws += c.d_ws + carry; carry = c.ws >= a.wseg ? 1 : 0; c.ws -= carry ? a.wseg : 0;
    c.hs += c.d_hs + carry; carry = c.hs >= a.hseg ? 1 : 0; c.hs -= carry ? a.hseg : 0;
    c.img += c.d_img + carry;
}

__device__ __forceinline__ TcConvTile tc_conv_tile(const TcConvArgs& a, const TcConvCursor& c) {
    TcConvTile r;
    r.nt = c.nt; r.img = c.img; r.h0 = c.hs * a.BHT; r.w0 = c.ws * a.BW;
    r.h_in0 = r.h0 - a.pt; r.w_in0 = r.w0 - a.pl;
    r.hh_lo = max(0, -r.h_in0); r.hh_hi = min(a.PH, a.H - r.h_in0);
    if (a.full_width) {
        r.iw_lo = 0; r.iw_hi = a.W;
        r.shift = ((r.h_in0 + r.hh_lo) * a.W) & 15;      // H*W % 16 == 0: the same for every channel
    } else {
        r.iw_lo = max(r.w_in0, 0); r.iw_hi = min(r.w_in0 + a.PW, a.W);
        r.shift = r.iw_lo & 15;                          // W % 16 == 0: the same for every row and channel
    }
    r.S0 = r.shift + r.w_in0 - r.iw_lo;
    return r;
}

// LEAN: int8 output with zero point 0 and finite multipliers (requantisation by rni + saturating pack).
template <int NT, bool XU8, bool LEAN>
__global__ void __launch_bounds__(kTcConvThreads, 1) tc_conv_nchw_kernel(const __grid_constant__ TcConvArgs a, const __grid_constant__ CUtensorMap x_map) {
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* sStages = smem;
    uint8_t* sOut = smem + a.off_out;
    uint8_t* tail = sOut + 2 * NT * kTcConvOutPitch;
    float* sMult = reinterpret_cast<float*>(tail);
    int* sBias = reinterpret_cast<int*>(tail + kTcConvMaxFilters * 4);
    uint64_t* bars = reinterpret_cast<uint64_t*>(tail + 2 * kTcConvMaxFilters * 4);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tail + 2 * kTcConvMaxFilters * 4 + 400);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tail + 2 * kTcConvMaxFilters * 4 + 404);
    volatile int* epi_ok = reinterpret_cast<volatile int*>(tail + 2 * kTcConvMaxFilters * 4 + 408);
    uint8_t* sLut = tail + 2 * kTcConvMaxFilters * 4 + 512;
    const uint32_t bar0 = ptx::smem_u32(bars);
    const int S = a.stages;
    auto full = [&](int s) { return bar0 + 8u * s; };
    auto empty = [&](int s) { return bar0 + 8u * (kTcConvMaxStages + s); };
    auto tfull = [&](int b) { return bar0 + 8u * (2 * kTcConvMaxStages + b); };
    auto tempty = [&](int b) { return bar0 + 8u * (2 * kTcConvMaxStages + 2 + b); };
    const uint32_t wfull = bar0 + 8u * (2 * kTcConvMaxStages + 4);
    auto ld_full = [&](int s) { return bar0 + 8u * (2 * kTcConvMaxStages + 5 + s); };    // staging slot filled (bytes)
    auto ld_empty = [&](int s) { return bar0 + 8u * (3 * kTcConvMaxStages + 5 + s); };   // staging slot read by all 8 transpose warps

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int tiles = a.N * a.hseg * a.wseg * a.n_tiles;
    const int taps = a.KH * a.KW;
    const uint32_t w_tap_bytes = (uint32_t)a.CB * NT * 16u;
    const uint32_t w_stage_bytes = (uint32_t)taps * w_tap_bytes;

    if (tid == 0) {
        for (int s = 0; s < S; ++s) { ptx::mbar_init(full(s), (a.direct == 1 || a.w_resident) ? 1 : 2); ptx::mbar_init(empty(s), 1); }
        for (int b = 0; b < 2; ++b) { ptx::mbar_init(tfull(b), 1); ptx::mbar_init(tempty(b), 8); }
        for (int s = 0; s < S; ++s) { ptx::mbar_init(ld_full(s), 1); ptx::mbar_init(ld_empty(s), 8); }
        ptx::mbar_init(wfull, 1);
        *abort_flag = 0;
        epi_ok[0] = 1; epi_ok[1] = 1;
        ptx::mbar_fence_init();
    }
    for (int i = tid; i < a.m_pad; i += kTcConvThreads) { sMult[i] = __ldg(a.mult + i); sBias[i] = __ldg(a.bias + i); }
    if (a.lut && tid < 256) sLut[tid] = __ldg(a.lut + tid);
    if (warp == 1) {
        ptx::tmem_alloc(ptx::smem_u32(tmem_slot), 2 * a.RB * NT);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------------ loader: bulk copies of activations (and weights)
        if (a.w_resident && lane == 0) {
            // every tile uses the same weights: load them once
            ptx::mbar_arrive_expect_tx(wfull, (uint32_t)a.c_stages * w_stage_bytes);
            for (int cs = 0; cs < a.c_stages; ++cs)
                ptx::bulk_g2s(ptx::smem_u32(smem + a.off_wres) + (uint32_t)cs * w_stage_bytes, a.w + (size_t)cs * w_stage_bytes, w_stage_bytes, wfull);
        }
        // One tiled TMA load per stage: the box holds CB*16 channels x the bytes of the patch rows.  With
        // full-width tiles the image plane is addressed as one row of H*W bytes (4-byte elements) and the
        // box starts at the 16-byte boundary below the first wanted byte; otherwise the map is (W, H, C, N)
        // and rows above or below the image arrive as zero fill.
        const int CH = a.CB * 16;
        const uint32_t box_bytes = (uint32_t)(CH * a.CP);
        TcConvCursor cur;
        tc_conv_cursor_init(a, (int)blockIdx.x, (int)gridDim.x, cur);
        int s = 0; uint32_t ph = 0;
        bool alive = true;
        for (int t = blockIdx.x; t < tiles && alive; t += gridDim.x) {
            const TcConvTile T = tc_conv_tile(a, cur);
            tc_conv_cursor_next(a, cur);
            for (int cs = 0; cs < a.c_stages; ++cs) {
                if (a.direct == 2) {
                    // 1x1 without a tensor map: warps 2-9 copy the activations; only streamed weights are loaded here
                    if (!a.w_resident) {
                        if (!ptx::mbar_wait(empty(s), ph ^ 1u, abort_flag)) { alive = false; break; }
                        if (lane == 0) {
                            ptx::mbar_arrive_expect_tx(full(s), w_stage_bytes);
                            ptx::bulk_g2s(ptx::smem_u32(sStages + (size_t)s * a.stage_bytes), a.w + ((size_t)T.nt * a.c_stages + cs) * w_stage_bytes, w_stage_bytes, full(s));
                        }
                        __syncwarp();
                    }
                    if (++s == S) { s = 0; ph ^= 1u; }
                    continue;
                }
                if (a.direct) {
                    // 1x1: the box of 128 pixels x CB*16 channels lands where the MMA reads it
                    if (!ptx::mbar_wait(empty(s), ph ^ 1u, abort_flag)) { alive = false; break; }
                    if (lane == 0) {
                        const uint32_t stage0 = ptx::smem_u32(sStages + (size_t)s * a.stage_bytes);
                        ptx::mbar_arrive_expect_tx(full(s), box_bytes + (a.w_resident ? 0u : w_stage_bytes));
                        ptx::tma_load_3d(stage0 + (uint32_t)a.off_patch, &x_map, T.w0 >> 2, cs * CH, T.img, full(s));
                        if (!a.w_resident) ptx::bulk_g2s(stage0, a.w + ((size_t)T.nt * a.c_stages + cs) * w_stage_bytes, w_stage_bytes, full(s));
                    }
                    __syncwarp();
                    if (++s == S) { s = 0; ph ^= 1u; }
                    continue;
                }
                // the slot's previous contents have been transposed (and, for streamed weights, multiplied)
                bool ok = ptx::mbar_wait(ld_empty(s), ph ^ 1u, abort_flag);
                if (ok && !a.w_resident) ok = ptx::mbar_wait(empty(s), ph ^ 1u, abort_flag);
                if (!ok) { alive = false; break; }
                if (lane == 0) {
                    const uint32_t stage0 = ptx::smem_u32(sStages + (size_t)s * a.stage_bytes);
                    ptx::mbar_arrive_expect_tx(ld_full(s), box_bytes);
                    if (a.full_width) ptx::tma_load_3d(stage0 + (uint32_t)a.off_stg, &x_map, (((T.h_in0 + T.hh_lo) * a.W) - T.shift) >> 2, cs * CH, T.img, ld_full(s));
                    else ptx::tma_load_4d(stage0 + (uint32_t)a.off_stg, &x_map, (T.iw_lo - T.shift) >> 2, T.h_in0, cs * CH, T.img, ld_full(s));
                    if (!a.w_resident) {
                        ptx::mbar_arrive_expect_tx(full(s), w_stage_bytes);
                        ptx::bulk_g2s(stage0, a.w + ((size_t)T.nt * a.c_stages + cs) * w_stage_bytes, w_stage_bytes, full(s));
                    }
                }
                __syncwarp();
                if (++s == S) { s = 0; ph ^= 1u; }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (ptx::elect_one()) {
            constexpr uint32_t idesc = ptx::idesc_i8(128, NT, !XU8, true);
            const uint32_t a_lbo = (uint32_t)a.PR * 16u;
            const int ksteps = a.CB / 2;
            // descriptors advance by adding 16-byte units to their address field (shared memory is < 256 KiB, no carry)
            const uint32_t a_kstep = (2u * a_lbo) >> 4, b_kstep = (2u * NT * 16u) >> 4;
            const uint32_t a_col = (uint32_t)a.dw, a_rowstep = (uint32_t)(a.dh * a.PW), a_blkstep = (uint32_t)(a.BH * a.PW);
            const uint32_t b_tap = w_tap_bytes >> 4;
            int s = 0; uint32_t ph = 0;
            int tile_it = 0;
            ZB_TDECL(); ZB_T0();
            if (a.w_resident && !ptx::mbar_wait(wfull, 0, abort_flag)) goto mma_done;
            for (int t = blockIdx.x; t < tiles; t += gridDim.x, ++tile_it) {
                const int b = tile_it & 1;
                const uint32_t bph = (uint32_t)(tile_it >> 1) & 1u;
                if (!ptx::mbar_wait(tempty(b), bph ^ 1u, abort_flag)) goto mma_done;
                ZB_TACC(0);
                const uint32_t d_tmem = tmem_base + (uint32_t)(b * a.RB * NT);
                for (int cs = 0; cs < a.c_stages; ++cs) {
                    if (!ptx::mbar_wait(full(s), ph, abort_flag)) goto mma_done;
                    ZB_TACC(1);
                    ptx::tc_fence_after();
                    const uint32_t stage0 = ptx::smem_u32(sStages + (size_t)s * a.stage_bytes);
                    const uint32_t sw = a.w_resident ? ptx::smem_u32(smem + a.off_wres) + (uint32_t)cs * w_stage_bytes : stage0;
                    const uint64_t db0 = ptx::smem_desc_kmajor(sw, NT * 16, 128);
                    uint32_t acc = cs != 0 ? 1u : 0u;
                    if (a.direct) {
                        // A = [channel][128 pixels] rows of 128 bytes: MN-major; a K step of 32 channels is 4096 bytes
                        const uint64_t da0 = ptx::smem_desc_mnmajor_sw128(stage0 + (uint32_t)a.off_patch, (uint32_t)(a.CB * 16 * 128), 1024);
                        for (int kk = 0; kk < ksteps; ++kk) {
                            ptx::mma_i8(d_tmem, da0 + (uint64_t)kk * 256u, db0 + (uint64_t)(kk * b_kstep), idesc | ptx::kIdescAMnMajor, (acc | (uint32_t)kk) != 0);
                        }
                        ptx::mma_commit(empty(s));
                        if (++s == S) { s = 0; ph ^= 1u; }
                        ZB_TACC(2);
                        continue;
                    }
                    // Every row block multiplies its own window of the shared patch into its own accumulator.
                    // The blocks' MMAs alternate: consecutive instructions are then independent of one another
                    // (an MMA that accumulates onto the previous one's result waits for it).
                    // Only the start-address field of the descriptors changes inside the loops: 32-bit adds on the low halves.
                    const uint64_t da0 = ptx::smem_desc_kmajor(stage0 + (uint32_t)a.off_patch, a_lbo, 128);
                    const uint32_t a_hi = (uint32_t)(da0 >> 32), b_hi = (uint32_t)(db0 >> 32);
                    uint32_t a_row = (uint32_t)da0, b_lo = (uint32_t)db0;
                    for (int kh = 0; kh < a.KH; ++kh, a_row += a_rowstep) {
                        uint32_t a_tap = a_row;
                        for (int kw = 0; kw < a.KW; ++kw, a_tap += a_col, b_lo += b_tap) {
                            uint32_t a_k = a_tap, b_k = b_lo;
                            for (int kk = 0; kk < ksteps; ++kk, a_k += a_kstep, b_k += b_kstep) {
                                ptx::mma_i8_halves(d_tmem, a_k, a_hi, b_k, b_hi, idesc, acc);
                                if (a.RB > 1) ptx::mma_i8_halves(d_tmem + NT, a_k + a_blkstep, a_hi, b_k, b_hi, idesc, acc);
                                if (a.RB > 2) {
                                    ptx::mma_i8_halves(d_tmem + 2 * NT, a_k + 2 * a_blkstep, a_hi, b_k, b_hi, idesc, acc);
                                    ptx::mma_i8_halves(d_tmem + 3 * NT, a_k + 3 * a_blkstep, a_hi, b_k, b_hi, idesc, acc);
                                }
                                acc = 1u;
                            }
                        }
                    }
                    ptx::mma_commit(empty(s));
                    if (++s == S) { s = 0; ph ^= 1u; }
                    ZB_TACC(2);
                }
                ptx::mma_commit(tfull(b));
            }
            ZB_TDUMP(0);
        mma_done:;
        }
    } else if (warp < 10 && a.direct == 2) {
        // ------------------------------------------------------------------ 1x1 without a tensor map: copy 128 pixels x CB*16
        // channels per stage into the form a swizzled TMA box would have: one 128-byte row per channel, 16-byte
        // chunk k of row r stored at chunk position k ^ (r % 8).  Pixels past the image and channels past C are zero.
        const int p = tid - 64, lw = warp - 2;
        const int CH = a.CB * 16;
        const uint32_t lane_off = (uint32_t)((lane & 3) * 4);
        TcConvCursor lcur;
        tc_conv_cursor_init(a, (int)blockIdx.x, (int)gridDim.x, lcur);
        int s = 0; uint32_t ph = 0;
        bool alive = true;
        for (int t = blockIdx.x; t < tiles && alive; t += gridDim.x) {
            const TcConvTile T = tc_conv_tile(a, lcur);
            tc_conv_cursor_next(a, lcur);
            const bool px_ok = T.w0 + lane * 4 < a.W;          // W % 4 == 0: a word is inside the image or outside
            for (int cs = 0; cs < a.c_stages; ++cs) {
                if (p == 0) ptx::mbar_wait(empty(s), ph ^ 1u, abort_flag);      // the MMAs that read this slot are done
                ptx::named_barrier_sync(2, 256);
                if (*abort_flag) { alive = false; break; }
                uint8_t* dst = sStages + (size_t)s * a.stage_bytes + a.off_patch;
                const uint8_t* src = a.x + ((size_t)T.img * a.C + (size_t)cs * CH) * a.W + T.w0 + lane * 4;
#pragma unroll 4
                for (int rr = lw; rr < CH; rr += 8) {
                    uint32_t v = 0;
                    if (px_ok && cs * CH + rr < a.C) v = __ldg(reinterpret_cast<const uint32_t*>(src + (size_t)rr * a.W));
                    *reinterpret_cast<uint32_t*>(dst + rr * 128 + ((((uint32_t)lane >> 2) ^ ((uint32_t)rr & 7u)) << 4) + lane_off) = v;
                }
                ptx::fence_proxy_async_smem();
                ptx::named_barrier_sync(2, 256);
                if (p == 0) ptx::mbar_arrive(full(s));
                if (++s == S) { s = 0; ph ^= 1u; }
            }
        }
    } else if (warp < 10 && !a.direct) {
        // ------------------------------------------------------------------ transpose: staging -> patch (256 threads)
        const int p = tid - 64;
        const int my_tiles = (tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
        const int total_it = my_tiles * a.c_stages;

        // transpose items: 16 channels x 4 pixels each, decoded once; consecutive threads take consecutive
        // words of a patch row (conflict-free loads).  The 16-byte stores of a quarter warp would all fall
        // into two bank groups; each lane therefore rotates its four pixels by (lane / 2) % 4 before the
        // transposes and stores them in the rotated order, which spreads the stores over all banks.
        int t_stg[4], t_pat[4], t_hh[4], t_kk[4];
        {
            const int row_items = a.PH * a.KN, items = a.CB * row_items;
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const int i = p + 256 * r;
                const int blk = i / row_items, rem = i - blk * row_items;
                const int hh = rem / a.KN, kk = rem - hh * a.KN;
                const bool ok = i < items;
                t_hh[r] = ok ? hh : 0; t_kk[r] = ok ? kk : 0x7fff;
                t_stg[r] = ok ? blk * 16 * a.CP + hh * a.RP + kk * 4 : 0;
                t_pat[r] = ok ? (blk * a.PR + hh * a.PW + kk * 4) * 16 : 0;
            }
        }
        const int rot = (lane >> 1) & 3;
        const uint32_t rot_sel = rot == 0 ? 0x3210u : (rot == 1 ? 0x0321u : (rot == 2 ? 0x1032u : 0x2103u));
        int c_cs = 0, s = 0;
        uint32_t ph = 0;
        TcConvCursor ccur;
        tc_conv_cursor_init(a, (int)blockIdx.x, (int)gridDim.x, ccur);
        TcConvTile CT = tc_conv_tile(a, ccur);
        ZB_TDECL(); ZB_T0();
        for (int ci = 0; ci < total_it; ++ci) {
            // one thread polls (a time-out raises the abort flag); the others park at the barrier
            if (p == 0) {
                if (ptx::mbar_wait(ld_full(s), ph, abort_flag))                     // this stage's box has landed
                    ptx::mbar_wait(empty(s), ph ^ 1u, abort_flag);                  // the patch slot is free
            }
            ZB_TACC(2);
            ptx::named_barrier_sync(2, 256);
            if (*abort_flag) break;
            ZB_TACC(3);

            const int k_lo = CT.S0 >> 2;                                             // S0 may be negative: floor
            const int kn = ((CT.S0 + a.PW - 1) >> 2) - k_lo + 1;
            // full-width tiles: the run starts with patch row hh_lo; otherwise the box holds every patch row
            const uint8_t* stg = sStages + (size_t)s * a.stage_bytes + a.off_stg + k_lo * 4 - (a.full_width ? CT.hh_lo * a.RP : 0);
            uint8_t* patch = sStages + (size_t)s * a.stage_bytes + a.off_patch + (k_lo * 4 - CT.S0) * 16;
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                if (t_kk[r] < kn) {
                    const uint8_t* sp = stg + t_stg[r];
                    uint32_t wv[16];
#pragma unroll
                    for (int j = 0; j < 16; ++j) wv[j] = *reinterpret_cast<const uint32_t*>(sp + j * a.CP);
                    const int ww0 = (k_lo + t_kk[r]) * 4 - CT.S0;   // patch column of byte 0
                    const int iw0 = CT.w_in0 + ww0;
                    const bool row_ok = t_hh[r] >= CT.hh_lo && t_hh[r] < CT.hh_hi;
                    if (!row_ok || iw0 < 0 || iw0 + 3 >= a.W) {
                        // pixels outside the image hold the input zero point
                        uint32_t mask = 0;
#pragma unroll
                        for (int px = 0; px < 4; ++px) mask |= ((unsigned)(iw0 + px) < (unsigned)a.W) ? (0xffu << (8 * px)) : 0u;
                        if (!row_ok) mask = 0;
#pragma unroll
                        for (int j = 0; j < 16; ++j) wv[j] = (wv[j] & mask) | (a.pad_word & ~mask);
                    }
#pragma unroll
                    for (int j = 0; j < 16; ++j) wv[j] = __byte_perm(wv[j], wv[j], rot_sel);
                    uint32_t o[4][4];    // o[group of 4 channels][i] = pixel (i + rot) % 4
#pragma unroll
                    for (int q = 0; q < 4; ++q) transpose_4x4_bytes(wv[4 * q], wv[4 * q + 1], wv[4 * q + 2], wv[4 * q + 3], o[q]);
                    uint8_t* dst = patch + t_pat[r];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int px = (i + rot) & 3;
                        const int ww = ww0 + px;
                        if (ww >= 0 && ww < a.PW) *reinterpret_cast<uint4*>(dst + px * 16) = make_uint4(o[0][i], o[1][i], o[2][i], o[3][i]);
                    }
                }
            }
            ZB_TACC(4);
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(ld_empty(s));                           // this warp is done reading the staging slot
            ptx::fence_proxy_async_smem();
            ptx::named_barrier_sync(2, 256);
            if (p == 0) ptx::mbar_arrive(full(s));
            ZB_TACC(5);
            if (++s == S) { s = 0; ph ^= 1u; }
            if (++c_cs == a.c_stages) {
                c_cs = 0;
                tc_conv_cursor_next(a, ccur);
                CT = tc_conv_tile(a, ccur);
            }
        }
        if (p == 0) ZB_TDUMP(8);
    } else {
        // ------------------------------------------------------------------ epilogue: a group of 8 warps per tile (warps
        // 10..17); each TMEM lane quarter is served by two warps that split the tile's filters.  In 1x1 convolutions
        // with a TMA-fed operand warps 2..9 have nothing else to do and form a second group: the groups take
        // alternate tiles (group g owns accumulator g and staging buffer g), so that one group's waits
        // (accumulator ready, TMEM loads, barriers, stores) overlap the other's arithmetic.
        constexpr int n_epi = 8;
        const int n_grp = a.direct == 1 ? 2 : 1;
        const int grp = warp >= 10 ? 0 : 1;
        const int ew = warp >= 10 ? warp - 10 : warp - 2;     // 0..7 within the group
        const int quarter = warp & 3;
        const int part = ew >> 2;
        const int row = quarter * 32 + lane;
        const int e = ew * 32 + lane;
        const uint32_t epi_bar = grp == 0 ? 1u : 3u;           // named barrier of the group (2 belongs to warps 2..9 in their other roles)
        volatile int* grp_ok = epi_ok + grp;
        const Requant rq{a.y_scale, a.y_zp, a.act, a.lut};
        const int oh_l = row / a.PW, ow_l = row - oh_l * a.PW;
        const bool row_live = oh_l < a.BH && ow_l < a.BW;        // this MMA row is an output of the tile
        const int pix_off = oh_l * a.BW + ow_l;
        const size_t ohw = (size_t)a.OH * a.OW;
        const uint32_t hi4 = a.act == ZANT_QACT_RELU6 ? 0x01010101u * (uint32_t)(a.six & 255) : 0x7f7f7f7fu;   // upper bound of the lean activation
        // copy-out work split, fixed for the launch: a warp pass covers co_cpp filters x co_lpc lanes
        // (a power of two that holds the vectors of a full tile's run)
        int co_shift = 0;
        {
            const int l_full = a.wseg == 1 ? a.BH * a.OW : a.BW;
            const int slots_full = (l_full >> a.log2V) + ((l_full & (a.V - 1)) ? 1 : 0);
            while ((1 << co_shift) < slots_full && co_shift < 5) ++co_shift;
        }
        const int co_lpc = 1 << co_shift, co_cpp = 32 >> co_shift;
        const int co_c0 = ew * co_cpp + (lane >> co_shift), co_v0 = lane & (co_lpc - 1);
        const size_t co_dst_step = (size_t)(n_epi * co_cpp) * ohw;
        int tile_it = grp;
        int blk_it = grp;                                      // one group: row blocks done, parity selects the staging buffer; two groups: buffer = group
        const int t_step = n_grp * (int)gridDim.x;
        TcConvCursor ecur;
        tc_conv_cursor_init(a, (int)blockIdx.x + grp * (int)gridDim.x, t_step, ecur);
        ZB_TDECL(); ZB_T0();
        for (int t = (int)blockIdx.x + grp * (int)gridDim.x; t < tiles; t += t_step, tile_it += n_grp) {
            const TcConvTile T = tc_conv_tile(a, ecur);
            tc_conv_cursor_next(a, ecur);
            const int b = tile_it & 1;
            const uint32_t bph = (uint32_t)(tile_it >> 1) & 1u;
            ZB_TACC(0);
            if (e == 0) *grp_ok = ptx::mbar_wait(tfull(b), bph, abort_flag) ? 1 : 0;
            ptx::named_barrier_sync(epi_bar, n_epi * 32);       // also: the group's previous copy-out has left the staging buffer
            if (!*grp_ok) break;
            ZB_TACC(1);
            ptx::tc_fence_after();
            // the tile's real filters, in chunks of 16, split evenly between the two warps of a lane quarter
            const int n_chunks = (min(NT, a.M - T.nt * NT) + 15) >> 4;
            const int h_lo = part ? (n_chunks + 1) >> 1 : 0, h_hi = part ? n_chunks : (n_chunks + 1) >> 1;
            // row blocks of the tile, one after the other; those below the image's last row do not exist
            const int n_blk = min(a.RB, (a.OH - T.h0 + a.BH - 1) / a.BH);
            for (int rb = 0; rb < n_blk; ++rb, blk_it += (n_grp == 1 ? 1 : 0)) {
            const int hb = T.h0 + rb * a.BH;
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)((b * a.RB + rb) * NT);
            uint8_t* ob = sOut + (size_t)(blk_it & 1) * NT * kTcConvOutPitch;
            uint8_t* orow = ob + pix_off;
#pragma unroll 1
            for (int h = h_lo; h < h_hi; ++h) {
                const int col0 = T.nt * NT + h * 16;                 // filters past M in the last chunk are padding: staged, never copied out
                uint32_t v[16];
                ZB_TSUB0();
                ptx::tmem_ld16(taddr + (uint32_t)(h * 16), v);
                ptx::tmem_wait_ld();
                ZB_TSUB(5);
                uint8_t* oc = orow + (size_t)h * 16 * kTcConvOutPitch;
                // All loads and arithmetic of the chunk come before its first store: the byte stores may alias anything
                // in the compiler's eyes, and loads placed after them would wait for them, one group of four at a time.
                uint32_t pk[4];
                if constexpr (LEAN) {
                    float4 m4[4]; int4 b4[4];
#pragma unroll
                    for (int j4 = 0; j4 < 4; ++j4) {
                        m4[j4] = *reinterpret_cast<const float4*>(sMult + col0 + j4 * 4);
                        b4[j4] = *reinterpret_cast<const int4*>(sBias + col0 + j4 * 4);
                    }
                    auto lean_chunk = [&](auto clamp) {
                        constexpr bool CL = decltype(clamp)::value;
#pragma unroll
                        for (int j4 = 0; j4 < 4; ++j4) {
                            const int q0 = tc_conv_round<CL>((int)v[j4 * 4 + 0] + b4[j4].x, m4[j4].x);
                            const int q1 = tc_conv_round<CL>((int)v[j4 * 4 + 1] + b4[j4].y, m4[j4].y);
                            const int q2 = tc_conv_round<CL>((int)v[j4 * 4 + 2] + b4[j4].z, m4[j4].z);
                            const int q3 = tc_conv_round<CL>((int)v[j4 * 4 + 3] + b4[j4].w, m4[j4].w);
                            uint32_t w4 = pack_act_s8x4(q0, q1, q2, q3, a.act != ZANT_QACT_NONE, hi4);
                            if (a.lut) w4 = lut4_smem(sLut, w4);
                            pk[j4] = w4;
                        }
                    };
                    if (a.small_products) lean_chunk(std::false_type{});
                    else lean_chunk(std::true_type{});
                } else {
                    float mv[16]; int bv[16];
#pragma unroll
                    for (int j = 0; j < 16; ++j) { mv[j] = sMult[col0 + j]; bv[j] = sBias[col0 + j]; }
#pragma unroll
                    for (int j4 = 0; j4 < 4; ++j4) {
                        uint32_t w4 = 0;
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const int acc = (int)v[j4 * 4 + j] + bv[j4 * 4 + j];
                            const int q = a.out_u8 ? requant_one<true>(acc, mv[j4 * 4 + j], rq) : requant_one<false>(acc, mv[j4 * 4 + j], rq);
                            w4 |= (uint32_t)(q & 255) << (8 * j);
                        }
                        pk[j4] = w4;
                    }
                }
                if (row_live) {
#pragma unroll
                    for (int j4 = 0; j4 < 4; ++j4) {
                        oc[(j4 * 4 + 0) * kTcConvOutPitch] = (uint8_t)pk[j4];
                        oc[(j4 * 4 + 1) * kTcConvOutPitch] = (uint8_t)(pk[j4] >> 8);
                        oc[(j4 * 4 + 2) * kTcConvOutPitch] = (uint8_t)(pk[j4] >> 16);
                        oc[(j4 * 4 + 3) * kTcConvOutPitch] = (uint8_t)(pk[j4] >> 24);
                    }
                }
                ZB_TSUB(6);
            }
            if (rb == n_blk - 1) {
                ptx::tc_fence_before();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(tempty(b));      // the tile's accumulators are free again
            }
            ZB_TACC(2);
            // The block's bytes are staged.  The staging buffer written two blocks later is this one: every
            // thread has left this block's copy-out before it reaches the next block's barrier.
            ptx::named_barrier_sync(epi_bar, n_epi * 32);
            ZB_TACC(3);

            const int ncv = min(NT, a.M - T.nt * NT);
            if (a.pool) {
                // A 2x2 / stride-2 MaxPool follows: the pooled bytes are written instead of the block's own.  The window's
                // two rows are two rows of this block (BH even), or this block and the previous one (BH == 1: blocks are
                // single output rows, an even block only stages).  Tiles and row blocks start at even rows and columns, so
                // windows never straddle a tile.  The maximum is taken on the finished codes, which is what the separate
                // MaxPool operator does on the int8 tensor.
                const bool pair = a.BH == 1;
                if (!pair || (rb & 1)) {
                    const uint8_t* ob_top = pair ? sOut + (size_t)((blk_it ^ 1) & 1) * NT * kTcConvOutPitch : ob;
                    const int rows = pair ? 2 : min(a.BH, a.OH - hb);
                    const int cols = a.wseg == 1 ? a.OW : min(a.BW, a.OW - T.w0);
                    const int pr_n = rows >> 1, pc_n = cols >> 1, half = (pc_n + 1) >> 1;
                    const int per_c = pr_n * half;
                    const int prow0 = (pair ? hb - 1 : hb) >> 1;
                    for (int c = ew; c < ncv; c += n_epi) {
                        uint8_t* dst_c = a.y + (((size_t)T.img * a.M + (size_t)(T.nt * NT + c)) * a.POH + prow0) * a.POW + (T.w0 >> 1);
                        for (int j = lane; j < per_c; j += 32) {
                            const int pr = j / half, k = j - pr * half;
                            const uint8_t* p0 = (pair ? ob_top : ob + (size_t)(2 * pr) * a.BW) + c * kTcConvOutPitch + 4 * k;
                            const uint8_t* p1 = pair ? ob + c * kTcConvOutPitch + 4 * k : p0 + a.BW;
                            const uint32_t w0 = (uint32_t)*reinterpret_cast<const uint16_t*>(p0) | ((uint32_t)*reinterpret_cast<const uint16_t*>(p0 + 2) << 16);
                            const uint32_t w1 = (uint32_t)*reinterpret_cast<const uint16_t*>(p1) | ((uint32_t)*reinterpret_cast<const uint16_t*>(p1 + 2) << 16);
                            uint32_t m = a.out_u8 ? __vmaxu4(w0, w1) : __vmaxs4(w0, w1);
                            m = a.out_u8 ? __vmaxu4(m, m >> 8) : __vmaxs4(m, m >> 8);     // bytes 0 and 2: the two windows' maxima
                            uint8_t* d = dst_c + (size_t)pr * a.POW + 2 * k;
                            if (2 * k + 1 < pc_n) {
                                if ((reinterpret_cast<uintptr_t>(d) & 1u) == 0) *reinterpret_cast<uint16_t*>(d) = (uint16_t)__byte_perm(m, 0u, 0x4420u);
                                else { d[0] = (uint8_t)m; d[1] = (uint8_t)(m >> 16); }
                            } else {
                                d[0] = (uint8_t)m;
                            }
                        }
                    }
                    if (pair) ptx::named_barrier_sync(epi_bar, n_epi * 32);   // both buffers are read: the next block's staging waits
                }
                ZB_TACC(4);
                continue;
            }
            // copy-out: per filter one contiguous run of the NCHW output
            const int L = a.wseg == 1 ? min(a.BH, a.OH - hb) * a.OW : min(a.BW, a.OW - T.w0);
            const int nvec = L >> a.log2V, tail_bytes = L - (nvec << a.log2V);
            const int slots = nvec + (tail_bytes ? 1 : 0);
            uint8_t* dst = a.y + ((size_t)T.img * a.M + (size_t)(T.nt * NT + co_c0)) * ohw + (size_t)hb * a.OW + T.w0;
            const uint8_t* src = ob + co_c0 * kTcConvOutPitch;
            for (int c = co_c0; c < ncv; c += n_epi * co_cpp, dst += co_dst_step, src += n_epi * co_cpp * kTcConvOutPitch) {
                for (int vv = co_v0; vv < slots; vv += co_lpc) {
                    const int o = vv << a.log2V;
                    if (vv < nvec) {
                        if (a.V == 16) *reinterpret_cast<uint4*>(dst + o) = *reinterpret_cast<const uint4*>(src + o);
                        else if (a.V == 8) *reinterpret_cast<uint2*>(dst + o) = *reinterpret_cast<const uint2*>(src + o);
                        else if (a.V == 4) *reinterpret_cast<uint32_t*>(dst + o) = *reinterpret_cast<const uint32_t*>(src + o);
                        else if (a.V == 2) *reinterpret_cast<uint16_t*>(dst + o) = *reinterpret_cast<const uint16_t*>(src + o);
                        else dst[o] = src[o];
                    } else {
                        for (int i = 0; i < tail_bytes; ++i) dst[o + i] = src[o + i];
                    }
                }
            }
            ZB_TACC(4);
            }
        }
        if (e == 32) ZB_TDUMP(16);
    }

    if (*abort_flag) {
        for (int i = 0; i < 200; ++i) __nanosleep(1000);
    }
    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 1) ptx::tmem_dealloc(tmem_base, 2 * a.RB * NT);
    if (tid == 0 && *abort_flag) atomicExch(a.status, (int)DEV_ERR_WAIT_TIMEOUT);
}

// =============================================================================================
// Host side: tiling, weight blocking and launch.
// =============================================================================================
struct TcConvPlan {
    TcConvArgs a{};            // geometry and tiling; pointers are filled in at launch
    int NT = 0;
    size_t smem_bytes = 0;
    size_t w_bytes = 0;        // blocked weights
    double row_efficiency = 0; // useful MMA rows / issued MMA rows
};

inline int tc_gcd(int a, int b) { while (b) { const int t = a % b; a = b; b = t; } return a; }

// Chooses tiling for `g`.  Returns false when the kernel does not apply (the caller then uses the
// im2col path or the generic kernel).
// `pool`: the epilogue also applies a 2x2 / stride-2 MaxPool (no padding, floor) and writes only the pooled tensor; tiles and
// row blocks then start at even rows and columns (BH even, or single-row blocks in pairs).
inline bool tc_conv_plan(const ConvGeom& g, bool w_zp_all_zero, TcConvPlan& p, bool pool = false) {
    if (g.G != 1 || !w_zp_all_zero || g.sh != 1 || g.sw != 1) return false;
    if (pool && (g.OH < 2 || g.OW < 2)) return false;
    if (g.M > kTcConvMaxFilters || g.N <= 0 || g.OH <= 0 || g.OW <= 0) return false;
    TcConvArgs& a = p.a;
    a = TcConvArgs{};
    const bool pointwise = g.KH == 1 && g.KW == 1 && g.pt == 0 && g.pl == 0 && g.pb == 0 && g.pr == 0;
    a.N = g.N; a.C = g.C; a.M = g.M; a.KH = g.KH; a.KW = g.KW; a.dh = g.dh; a.dw = g.dw;
    if (pointwise) {           // pixels of an image are one long row
        a.H = 1; a.W = g.H * g.W; a.OH = 1; a.OW = g.OH * g.OW; a.pt = a.pl = 0;
    } else {
        a.H = g.H; a.W = g.W; a.OH = g.OH; a.OW = g.OW; a.pt = g.pt; a.pl = g.pl;
    }
    if (a.W % 4 != 0) return false;
    const int halo_w = (a.KW - 1) * a.dw, halo_h = (a.KH - 1) * a.dh;
    if (halo_w > 32 || halo_h > 32) return false;
    if (!pointwise && (g.pl > halo_w || g.pr > halo_w || g.pt > halo_h || g.pb > halo_h)) return false;   // every tile overlaps the image
    if (pool && pointwise) return false;      // the pooled epilogue belongs to the patch form of the kernel
    a.BW = std::min(a.OW, 128 - halo_w);
    if (pool && a.BW < a.OW && (a.BW & 1)) a.BW -= 1;          // column segments start at even columns
    a.PW = a.BW + halo_w;
    a.BH = std::max(1, std::min(a.OH, 128 / a.PW));
    if (pool && a.BH > 1 && (a.BH & 1)) a.BH -= 1;            // row blocks hold whole window rows
    a.pool = pool ? 1 : 0; a.POH = g.OH / 2; a.POW = g.OW / 2;
    a.wseg = (a.OW + a.BW - 1) / a.BW;
    a.full_width = a.wseg == 1 ? 1 : 0;
    a.direct = pointwise ? 1 : 0;
    // the TMA boxes start at 16-byte boundaries; every channel of a stage must see the same offset
    if (((long long)a.H * a.W) % 16 != 0) {
        if (!pointwise) return false;
        a.direct = 2;          // no tensor map over planes of such a size (W % 4 == 0 holds): the rows are copied with plain loads
    }
    if (!a.direct && !a.full_width && a.W % 16 != 0) return false;
    p.NT = g.M <= 64 ? 64 : 128;
    if (pointwise && g.M > 128) p.NT = 256;
    a.m_pad = (g.M + p.NT - 1) / p.NT * p.NT;
    a.n_tiles = a.m_pad / p.NT;
    const int taps = a.KH * a.KW;
    const int out_bytes = 2 * p.NT * kTcConvOutPitch;
    const int budget = 232448 - kTcConvTail - out_bytes - 1024;
    const int blocks_in_image = (a.OH + a.BH - 1) / a.BH;
    const TcConvArgs base = a;
    // Row blocks per tile: the more blocks share a patch, the fewer halo rows are fetched and transposed
    // (a 3x3 filter on a 56-wide image: 4 input rows per 2 output rows with one block, 10 per 8 with four).
    // The accumulators of a tile take RB * NT TMEM columns, twice (double buffering), out of 512.  A count
    // that wastes more than an eighth of the last tile's blocks, or that does not fit, gives way to a smaller one.
    bool placed = false;
    for (int rb = (a.direct || halo_h == 0) ? 1 : 4; rb >= 1 && !placed; rb /= 2) {
        if (2 * rb * p.NT > 512 || (rb > 1 && rb > blocks_in_image)) continue;
        if (pool && base.BH == 1 && (rb & 1)) continue;        // single-row blocks pool in pairs
        a = base;
        a.RB = rb; a.BHT = rb * a.BH;
        a.PH = a.BHT + halo_h;
        a.hseg = (a.OH + a.BHT - 1) / a.BHT;
        if (rb > 1 && (long long)a.hseg * rb * 7 > (long long)blocks_in_image * 8) continue;
        // patch pixels a 16-channel group holds: the last block's 128 MMA rows plus the filter's reach;
        // 1 mod 8, so that the channel groups of a pixel fall into different banks
        a.PR = ((rb - 1) * a.BH * a.PW + 128 + halo_h * a.PW + halo_w + 7) / 8 * 8 + 1;
        if (a.direct) {
            a.RP = 128; a.CP = 128; a.KN = 1;               // the box row is the operand row: 128 pixels of one channel
        } else if (a.full_width) {
            a.RP = a.W;
            a.CP = (a.PH * a.W + 15 + 15) / 16 * 16;        // box row: the run plus its alignment slack
            if (a.CP > 1024) continue;                      // box rows hold at most 256 four-byte elements
            const int s0 = ((-a.pl) % 4 + 4) % 4;
            a.KN = ((s0 + a.PW - 1) >> 2) + 1;
        } else {
            a.RP = (a.PW + 15 + 15) / 16 * 16;
            a.CP = a.PH * a.RP;
            if (a.PH > 256) continue;
            a.KN = 1;
            for (int ws = 0; ws < a.wseg; ++ws) {   // most staging words any tile's patch row spans
                const int w_in0 = ws * a.BW - a.pl, lo = std::max(w_in0, 0);
                const int s0 = (lo & 15) + w_in0 - lo;
                a.KN = std::max(a.KN, ((s0 + a.PW - 1) >> 2) - (s0 >> 2) + 1);
            }
        }
        // Shared-memory plan.  Preference: 64 channels per stage over 32 (fewer hand-offs per byte), weights
        // resident over streamed (possible when there is one filter tile: no re-fetch per tile), at least 3 stages.
        for (int min_stages = 3; min_stages >= 2 && !placed; --min_stages)
            for (int cb = (a.C > 64 ? 8 : (a.C > 32 ? 4 : 2)); cb >= 2 && !placed; cb /= 2)
                for (int resident = 1; resident >= 0 && !placed; --resident) {
                    if (!a.direct && cb * a.PH * a.KN > 1024) continue;   // the transposers' per-thread work lists hold 4 entries
                    const int c_stages = (a.C + cb * 16 - 1) / (cb * 16);
                    const int w_stage = taps * cb * p.NT * 16;
                    const long long w_all = (long long)c_stages * w_stage;
                    if (resident && (a.n_tiles != 1 || w_all > 112 * 1024)) continue;
                    const int off_patch = resident ? 0 : w_stage;
                    int off_stg, stage_bytes;
                    if (a.direct) {       // operand tile = TMA destination: 1024-byte aligned, no staging
                        off_stg = off_patch;
                        stage_bytes = (off_patch + cb * 16 * 128 + 1023) / 1024 * 1024;
                    } else {
                        off_stg = (off_patch + cb * a.PR * 16 + 127) / 128 * 128;   // TMA destination
                        stage_bytes = (off_stg + cb * 16 * a.CP + 128 + 127) / 128 * 128;   // + 128: the transposes may read a few bytes past the last channel
                    }
                    const int stages = std::min<long long>(kTcConvMaxStages, (budget - (resident ? w_all : 0)) / stage_bytes);
                    if (stages < min_stages) continue;
                    a.CB = cb; a.c_stages = c_stages; a.w_resident = resident; a.off_patch = off_patch; a.off_stg = off_stg;
                    a.stage_bytes = stage_bytes; a.stages = stages;
                    a.off_wres = stages * stage_bytes;
                    a.off_out = a.off_wres + (resident ? (int)w_all : 0);
                    placed = true;
                }
    }
    if (!placed) return false;
    p.smem_bytes = (size_t)a.off_out + out_bytes + kTcConvTail;
    p.w_bytes = (size_t)a.n_tiles * a.c_stages * taps * a.CB * p.NT * 16;
    // one contiguous output run per filter and tile; V = widest store that every run start and length allows
    const int ohw_gcd = tc_gcd(16, (int)(((long long)a.OH * a.OW) % 16 == 0 ? 16 : ((long long)a.OH * a.OW) % 16));
    a.V = a.wseg == 1 ? tc_gcd(ohw_gcd, tc_gcd(16, (a.BH * a.OW) % 16 == 0 ? 16 : (a.BH * a.OW) % 16))
                      : tc_gcd(ohw_gcd, tc_gcd(tc_gcd(16, a.OW % 16 == 0 ? 16 : a.OW % 16), tc_gcd(16, a.BW % 16 == 0 ? 16 : a.BW % 16)));
    for (a.log2V = 0; (1 << a.log2V) < a.V; ++a.log2V) {}
    p.row_efficiency = (double)a.OH * a.OW / ((double)a.hseg * a.RB * a.wseg * 128.0);
    const long long tiles = (long long)a.N * a.hseg * a.wseg * a.n_tiles;
    if (tiles > 0x7fffffffLL || p.row_efficiency < 0.5) return false;
    return true;
}

// Blocks `w` ([M][C][KH][KW] int8) as [filter tile][channel stage][tap][CB][NT][16] and pads the
// per-filter constants; the input zero point is folded into the bias (halo pixels hold x_zp).
inline void tc_conv_prepare(const TcConvPlan& p, const int8_t* w, const float* mult, const int32_t* bias, int x_zp,
                            std::vector<int8_t>& w_blk, std::vector<float>& mult_pad, std::vector<int32_t>& bias_pad) {
    const TcConvArgs& a = p.a;
    const int taps = a.KH * a.KW, NT = p.NT, CH = a.CB * 16;
    w_blk.assign(p.w_bytes, 0);
    mult_pad.assign(a.m_pad, 1.0f);
    bias_pad.assign(a.m_pad, 0);
    for (int m = 0; m < a.M; ++m) {
        const int nt = m / NT, mm = m % NT;
        long long sum = 0;
        for (int c = 0; c < a.C; ++c) {
            const int cs = c / CH, blk = (c % CH) / 16, j = c % 16;
            for (int tap = 0; tap < taps; ++tap) {
                const int8_t v = w[((size_t)m * a.C + c) * taps + tap];
                w_blk[((((size_t)nt * a.c_stages + cs) * taps + tap) * a.CB + blk) * NT * 16 + (size_t)mm * 16 + j] = v;
                sum += v;
            }
        }
        mult_pad[m] = mult[m];
        bias_pad[m] = (int32_t)((bias ? bias[m] : 0) - (long long)x_zp * sum);
    }
}

template <int NT, bool XU8, bool LEAN>
inline int32_t tc_conv_launch_t(zant_ctx* ctx, const TcConvPlan& p, const TcConvArgs& a, const CUtensorMap& x_map, int grid) {
    ZB_SMEM_ATTR(ctx, (tc_conv_nchw_kernel<NT, XU8, LEAN>), 232448);
    tc_conv_nchw_kernel<NT, XU8, LEAN><<<grid, kTcConvThreads, p.smem_bytes, ctx->stream>>>(a, x_map);
    return check_launch(ctx, "tc_conv_nchw_kernel");
}

template <int NT>
inline int32_t tc_conv_launch_nt(zant_ctx* ctx, const TcConvPlan& p, const TcConvArgs& a, const CUtensorMap& m, int grid, bool x_u8, bool lean) {
    if (x_u8) return lean ? tc_conv_launch_t<NT, true, true>(ctx, p, a, m, grid) : tc_conv_launch_t<NT, true, false>(ctx, p, a, m, grid);
    return lean ? tc_conv_launch_t<NT, false, true>(ctx, p, a, m, grid) : tc_conv_launch_t<NT, false, false>(ctx, p, a, m, grid);
}

// Tensor map over the NCHW input in 4-byte elements: (H*W/4, C, N) for full-width tiles (an image plane
// is one row), (W/4, H, C, N) otherwise; box = the bytes of a stage.  Out-of-range elements read as zero.
inline int32_t tc_conv_encode_map(const TcConvArgs& a, const void* x, CUtensorMap* map) {
    const cuuint64_t W = (cuuint64_t)a.W, H = (cuuint64_t)a.H, C = (cuuint64_t)a.C, N = (cuuint64_t)a.N;
    cuuint64_t dims[4], strides[3];
    cuuint32_t box[4], estr[4] = {1, 1, 1, 1};
    cuuint32_t rank;
    CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_NONE;
    if (a.direct) {
        rank = 3;
        dims[0] = H * W / 4; dims[1] = C; dims[2] = N;
        strides[0] = H * W; strides[1] = C * H * W;
        box[0] = 32; box[1] = (cuuint32_t)(a.CB * 16); box[2] = 1;     // 128 pixels x the stage's channels
        swizzle = CU_TENSOR_MAP_SWIZZLE_128B;
    } else if (a.full_width) {
        rank = 3;
        dims[0] = H * W / 4; dims[1] = C; dims[2] = N;
        strides[0] = H * W; strides[1] = C * H * W;
        box[0] = (cuuint32_t)(a.CP / 4); box[1] = (cuuint32_t)(a.CB * 16); box[2] = 1;
    } else {
        rank = 4;
        dims[0] = W / 4; dims[1] = H; dims[2] = C; dims[3] = N;
        strides[0] = W; strides[1] = H * W; strides[2] = C * H * W;
        box[0] = (cuuint32_t)(a.RP / 4); box[1] = (cuuint32_t)a.PH; box[2] = (cuuint32_t)(a.CB * 16); box[3] = 1;
    }
    // The driver entry point is looked up at run time, so that the library itself does not link against
    // libcuda (it must load on machines without a driver, where only its symbols are inspected).
    using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static EncodeFn encode = nullptr;
    if (!encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
        const cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
        if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !fn) {
            cudaGetLastError();
            return fail(ZANT_E_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
        }
        encode = reinterpret_cast<EncodeFn>(fn);
    }
    const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, rank, const_cast<void*>(x), dims, strides, box, estr,
                                              CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(ZANT_E_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
    return ZANT_OK;
}

// x must be 16-byte aligned (cp.async granules); a y that is not falls back to byte stores.
inline bool tc_conv_ptr_ok(const void* x) { return (reinterpret_cast<uintptr_t>(x) & 15u) == 0; }

// `max_product`: upper bound of |accumulator * multiplier| over all filters (tc_conv_max_product), infinity if
// some multiplier is not finite.
inline int32_t tc_conv_run(zant_ctx* ctx, const TcConvPlan& p, const void* x, bool x_u8, int x_zp, const int8_t* w_blk_dev,
                           const float* mult_dev, const int32_t* bias_dev, void* y, bool y_u8, const Requant& rq, double max_product) {
    const bool mult_finite = std::isfinite(max_product);
    TcConvArgs a = p.a;
    a.x = (const uint8_t*)x; a.y = (uint8_t*)y; a.w = w_blk_dev; a.mult = mult_dev; a.bias = bias_dev;
    a.pad_word = 0x01010101u * (uint32_t)(x_zp & 255);
    a.y_scale = rq.y_scale; a.y_zp = rq.y_zp; a.act = rq.act; a.out_u8 = y_u8 ? 1 : 0; a.lut = rq.lut;
    if (!tc_conv_ptr_ok(y)) { a.V = 1; a.log2V = 0; }
    const bool lean = !y_u8 && rq.y_zp == 0 && mult_finite;
    a.small_products = max_product < 4194304.0 ? 1 : 0;
    if (lean) {
        float v = 6.0f / rq.y_scale;
        v = std::fmin(std::fmax(v, -512.0f), 511.0f);
        a.six = std::min(std::max((int)std::nearbyintf(v), -128), 127);
    }
    a.status = ctx->status_word;
    const long long tiles = (long long)a.N * a.hseg * a.wseg * a.n_tiles;
    const int grid = (int)std::min<long long>(tiles, ctx->sm_count);
    alignas(64) CUtensorMap x_map{};
    if (a.direct != 2) ZB_TRY(tc_conv_encode_map(a, x, &x_map));
    if (p.NT == 64) return tc_conv_launch_nt<64>(ctx, p, a, x_map, grid, x_u8, lean);
    if (p.NT == 128) return tc_conv_launch_nt<128>(ctx, p, a, x_map, grid, x_u8, lean);
    return tc_conv_launch_nt<256>(ctx, p, a, x_map, grid, x_u8, lean);
}

// Bound of |accumulator * multiplier|: an accumulator is at most 255 * 128 * K in magnitude plus the bias.
inline double tc_conv_max_product(const std::vector<float>& mult, const std::vector<int32_t>& bias_folded, long long K) {
    double worst = 0.0;
    for (size_t m = 0; m < mult.size(); ++m) {
        if (!std::isfinite(mult[m])) return INFINITY;
        const double acc = 255.0 * 128.0 * (double)K + std::fabs((double)(m < bias_folded.size() ? bias_folded[m] : 0));
        worst = std::max(worst, acc * std::fabs((double)mult[m]));
    }
    return worst;
}

}  // namespace zb
