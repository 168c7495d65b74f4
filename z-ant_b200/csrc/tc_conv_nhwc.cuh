// Implicit-GEMM QLinearConv on tcgen05 for channels-last tensors: x [N][H][W][C], y [N][OH][OW][M]
// (group 1, stride 1, any kernel size / dilation, weight zero points 0, C % 64 == 0, M % 16 == 0;
// with padding the input zero point must be 0, because the halo arrives as TMA zero fill).
//
// Channels-last is the layout the tensor core wants: a pixel's channels are contiguous, so ONE tiled
// TMA load per stage (box = KC channels x PW x PH pixels, 64- or 128-byte swizzle) leaves the input
// patch in shared memory as a valid K-major MMA operand, pixel (hh, ww) of the patch in row
// hh*PW + ww.  Filter tap (kh, kw) is the same memory, (kh*dh*PW + kw*dw) rows further on; MMA row
// r of row block b stands for patch pixel b*BH*PW + r, rows in the halo columns are computed and
// dropped.  Nothing is transposed or staged: the epilogue requantises a pixel's filters in
// registers and stores them as 16-byte words of the channels-last output.
//
// Warp roles (576 threads, one persistent CTA per SM):
//   warp 0  loader (TMA boxes, weights)      warp 1  TMEM owner + MMA issuer      warps 2-17  epilogue
// Tiling (row blocks, tile walk, shared-memory stages) is that of tc_conv_nchw.cuh, whose argument
// block and cursor this kernel reuses.
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
#include "tc_conv_nchw.cuh"

namespace zb {

// K-major operand whose rows are `row_bytes` (64 or 128) wide and were written with the matching
// swizzle (by TMA, or by the host for the weights): 8-row groups lie 8 * row_bytes apart.  The swizzle
// is a function of the shared-memory address itself, for the TMA write and for the MMA read alike
// (measured: with the base-offset field left 0, views that start any whole number of rows into the
// patch, and K steps of 32 bytes into a row, read the right bytes; with the field set to the row phase
// they do not).  So the start address may be any row of a buffer whose base is 1024-byte aligned.
__device__ __forceinline__ uint64_t smem_desc_kmajor_swizzled(uint32_t addr, uint32_t row_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((addr >> 4) & 0x3FFFu);
    d |= (uint64_t)1 << 16;                                    // leading-dimension offset: unused for swizzled K-major operands
    d |= (uint64_t)(((8u * row_bytes) >> 4) & 0x3FFFu) << 32;
    d |= (uint64_t)1 << 46;                                    // descriptor version for sm_100
    d |= (uint64_t)(row_bytes == 128 ? 2u : 4u) << 61;         // layout type: 128-byte / 64-byte swizzle
    return d;
}

// Uses TcConvArgs with: CB = channels per stage / 16 (4 or 8), PR = patch rows allocated per stage,
// off_patch = patch offset inside a stage (after streamed weights).
template <int NT, bool XU8, bool LEAN>
__global__ void __launch_bounds__(kTcConvThreads, 1) tc_conv_nhwc_kernel(const __grid_constant__ TcConvArgs a, const __grid_constant__ CUtensorMap x_map) {
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* sStages = smem;
    uint8_t* tail = smem + a.off_out;
    float* sMult = reinterpret_cast<float*>(tail);
    int* sBias = reinterpret_cast<int*>(tail + kTcConvMaxFilters * 4);
    uint64_t* bars = reinterpret_cast<uint64_t*>(tail + 2 * kTcConvMaxFilters * 4);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tail + 2 * kTcConvMaxFilters * 4 + 400);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tail + 2 * kTcConvMaxFilters * 4 + 404);
    uint8_t* sLut = tail + 2 * kTcConvMaxFilters * 4 + 512;          // copy of the optional activation table
    const uint32_t bar0 = ptx::smem_u32(bars);
    const int S = a.stages;
    auto full = [&](int s) { return bar0 + 8u * s; };
    auto empty = [&](int s) { return bar0 + 8u * (kTcConvMaxStages + s); };
    auto tfull = [&](int b) { return bar0 + 8u * (2 * kTcConvMaxStages + b); };
    auto tempty = [&](int b) { return bar0 + 8u * (2 * kTcConvMaxStages + 2 + b); };
    const uint32_t wfull = bar0 + 8u * (2 * kTcConvMaxStages + 4);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int tiles = a.N * a.hseg * a.wseg * a.n_tiles;
    const int taps = a.KH * a.KW;
    const int KC = a.CB * 16;                                   // channels (= bytes per operand row) per stage
    const uint32_t w_tap_bytes = (uint32_t)(NT * KC);
    const uint32_t w_stage_bytes = (uint32_t)taps * w_tap_bytes;
    constexpr int kEpiWarps = 16;

    if (tid == 0) {
        for (int s = 0; s < S; ++s) { ptx::mbar_init(full(s), 1); ptx::mbar_init(empty(s), 1); }
        for (int b = 0; b < 2; ++b) { ptx::mbar_init(tfull(b), 1); ptx::mbar_init(tempty(b), kEpiWarps); }
        ptx::mbar_init(wfull, 1);
        *abort_flag = 0;
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
        // ------------------------------------------------------------------ loader
        if (a.w_resident && lane == 0) {
            ptx::mbar_arrive_expect_tx(wfull, (uint32_t)a.c_stages * w_stage_bytes);
            for (int cs = 0; cs < a.c_stages; ++cs)
                ptx::bulk_g2s(ptx::smem_u32(smem + a.off_wres) + (uint32_t)cs * w_stage_bytes, a.w + (size_t)cs * w_stage_bytes, w_stage_bytes, wfull);
        }
        const uint32_t box_bytes = (uint32_t)(KC * a.PW * a.PH);
        TcConvCursor cur;
        tc_conv_cursor_init(a, (int)blockIdx.x, (int)gridDim.x, cur);
        int s = 0; uint32_t ph = 0;
        bool alive = true;
        for (int t = blockIdx.x; t < tiles && alive; t += gridDim.x) {
            const TcConvTile T = tc_conv_tile(a, cur);
            tc_conv_cursor_next(a, cur);
            for (int cs = 0; cs < a.c_stages; ++cs) {
                if (!ptx::mbar_wait(empty(s), ph ^ 1u, abort_flag)) { alive = false; break; }
                if (lane == 0) {
                    const uint32_t stage0 = ptx::smem_u32(sStages + (size_t)s * a.stage_bytes);
                    ptx::mbar_arrive_expect_tx(full(s), box_bytes + (a.w_resident ? 0u : w_stage_bytes));
                    // pixels outside the image (negative or too large coordinates) arrive as zeros
                    ptx::tma_load_4d(stage0 + (uint32_t)a.off_patch, &x_map, cs * KC, T.w_in0, T.h_in0, T.img, full(s));
                    if (!a.w_resident) ptx::bulk_g2s(stage0, a.w + ((size_t)T.nt * a.c_stages + cs) * w_stage_bytes, w_stage_bytes, full(s));
                }
                __syncwarp();
                if (++s == S) { s = 0; ph ^= 1u; }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (ptx::elect_one()) {
            constexpr uint32_t idesc = ptx::idesc_i8(128, NT, !XU8, true);
            const int ksteps = KC / 32;
            const uint32_t row_bytes = (uint32_t)KC;
            const uint32_t row_units = row_bytes >> 4;                          // descriptor address units per patch row
            const uint32_t a_col = (uint32_t)a.dw * row_units, a_rowstep = (uint32_t)(a.dh * a.PW) * row_units;
            const uint32_t a_blkstep = (uint32_t)(a.BH * a.PW) * row_units, b_tap = w_tap_bytes >> 4;
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
                    uint32_t acc = cs != 0 ? 1u : 0u;
                    // Only the start-address field (16-byte units) of the descriptors changes inside the loops: 32-bit adds
                    // on the low halves.  The row blocks' MMAs alternate, so that consecutive instructions are independent.
                    const uint64_t da0 = smem_desc_kmajor_swizzled(stage0 + (uint32_t)a.off_patch, row_bytes);
                    const uint64_t db0 = smem_desc_kmajor_swizzled(sw, row_bytes);
                    const uint32_t a_hi = (uint32_t)(da0 >> 32), b_hi = (uint32_t)(db0 >> 32);
                    uint32_t a_row = (uint32_t)da0, b_lo = (uint32_t)db0;
                    for (int kh = 0; kh < a.KH; ++kh, a_row += a_rowstep) {
                        uint32_t a_tap = a_row;
                        for (int kw = 0; kw < a.KW; ++kw, a_tap += a_col, b_lo += b_tap) {
                            uint32_t a_k = a_tap, b_k = b_lo;
                            for (int kk = 0; kk < ksteps; ++kk, a_k += 2u, b_k += 2u) {        // a K step is 32 bytes
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
    } else {
        // ------------------------------------------------------------------ epilogue: 16 warps, four per TMEM lane quarter,
        // each with a quarter of the tile's filters.  A thread is one pixel of the row block.
        const int ew = warp - 2;
        const int quarter = warp & 3;
        const int part = ew >> 2;
        constexpr int cols = NT / 4;
        const int row = quarter * 32 + lane;
        const Requant rq{a.y_scale, a.y_zp, a.act, a.lut};
        const int oh_l = row / a.PW, ow_l = row - oh_l * a.PW;
        const bool row_live = oh_l < a.BH && ow_l < a.BW;
        const uint32_t hi4 = a.act == ZANT_QACT_RELU6 ? 0x01010101u * (uint32_t)(a.six & 255) : 0x7f7f7f7fu;   // upper bound of the lean activation
        const int tcol0 = part * cols;
        // With one 64-filter tile a warp serves the same 16 filters in every tile: their constants stay in registers
        // (as broadcast shared-memory loads they would take about a third of the shared-memory pipe's time, which the
        // tensor core's operand fetches need).
        constexpr bool kRegConsts = NT == 64 && LEAN;
        float rm[kRegConsts ? 16 : 1]; int rbias[kRegConsts ? 16 : 1];
        if constexpr (kRegConsts) {
#pragma unroll
            for (int j = 0; j < 16; ++j) { rm[j] = sMult[tcol0 + j]; rbias[j] = sBias[tcol0 + j]; }
        }
        int tile_it = 0;
        TcConvCursor ecur;
        tc_conv_cursor_init(a, (int)blockIdx.x, (int)gridDim.x, ecur);
        ZB_TDECL(); ZB_T0();
        for (int t = blockIdx.x; t < tiles; t += gridDim.x, ++tile_it) {
            const TcConvTile T = tc_conv_tile(a, ecur);
            tc_conv_cursor_next(a, ecur);
            const int b = tile_it & 1;
            const uint32_t bph = (uint32_t)(tile_it >> 1) & 1u;
            ZB_TACC(0);
            const bool arrived = ptx::mbar_wait(tfull(b), bph, abort_flag);
            if (!__all_sync(0xffffffffu, arrived)) break;                // a time-out ends the whole warp together
            ZB_TACC(1);
            ptx::tc_fence_after();
            const int n_blk = min(a.RB, (a.OH - T.h0 + a.BH - 1) / a.BH);
            const int ow = T.w0 + ow_l;
            for (int rb = 0; rb < n_blk; ++rb) {
                const int oh = T.h0 + rb * a.BH + oh_l;
                const bool live = row_live && oh < a.OH && ow < a.OW;
                const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)((b * a.RB + rb) * NT + tcol0);
                uint8_t* yrow = a.y + (((size_t)T.img * a.OH + oh) * a.OW + ow) * a.M + (size_t)T.nt * NT + tcol0;
#pragma unroll 1
                for (int h = 0; h < cols / 16; ++h) {
                    const int col0 = T.nt * NT + tcol0 + h * 16;
                    if (col0 >= a.M) break;                          // filter padding
                    uint32_t v[16];
                    ptx::tmem_ld16(taddr + (uint32_t)(h * 16), v);
                    ptx::tmem_wait_ld();
                    uint32_t wd[4];
                    if constexpr (LEAN) {
                        auto lean_chunk = [&](auto clamp) {
                            constexpr bool CL = decltype(clamp)::value;
#pragma unroll
                            for (int j4 = 0; j4 < 4; ++j4) {
                                float4 m4; int4 b4;
                                if constexpr (kRegConsts) {
                                    m4 = make_float4(rm[j4 * 4], rm[j4 * 4 + 1], rm[j4 * 4 + 2], rm[j4 * 4 + 3]);
                                    b4 = make_int4(rbias[j4 * 4], rbias[j4 * 4 + 1], rbias[j4 * 4 + 2], rbias[j4 * 4 + 3]);
                                } else {
                                    m4 = *reinterpret_cast<const float4*>(sMult + col0 + j4 * 4);
                                    b4 = *reinterpret_cast<const int4*>(sBias + col0 + j4 * 4);
                                }
                                uint32_t pk = pack_act_s8x4(tc_conv_round<CL>((int)v[j4 * 4 + 0] + b4.x, m4.x), tc_conv_round<CL>((int)v[j4 * 4 + 1] + b4.y, m4.y),
                                                            tc_conv_round<CL>((int)v[j4 * 4 + 2] + b4.z, m4.z), tc_conv_round<CL>((int)v[j4 * 4 + 3] + b4.w, m4.w),
                                                            a.act != ZANT_QACT_NONE, hi4);
                                if (a.lut) pk = lut4_smem(sLut, pk);
                                wd[j4] = pk;
                            }
                        };
                        if (a.small_products) lean_chunk(std::false_type{});
                        else lean_chunk(std::true_type{});
                    } else {
#pragma unroll
                        for (int j4 = 0; j4 < 4; ++j4) {
                            uint32_t pk = 0;
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                const int c = col0 + j4 * 4 + j;
                                const int acc = (int)v[j4 * 4 + j] + sBias[c];
                                const int q = a.out_u8 ? requant_one<true>(acc, sMult[c], rq) : requant_one<false>(acc, sMult[c], rq);
                                pk |= (uint32_t)(q & 255) << (8 * j);
                            }
                            wd[j4] = pk;
                        }
                    }
                    if (live) *reinterpret_cast<uint4*>(yrow + h * 16) = make_uint4(wd[0], wd[1], wd[2], wd[3]);
                }
            }
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(tempty(b));          // this warp has read its part of the tile's accumulators
            ZB_TACC(2);
        }
        if (warp == 2 && lane == 0) ZB_TDUMP(16);
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
// Host side
// =============================================================================================
// `g` describes the convolution with H, W, C, M as usual; only the memory order of x and y differs.
inline bool tc_conv_nhwc_plan(const ConvGeom& g, bool w_zp_all_zero, int x_zp, TcConvPlan& p) {
    if (g.G != 1 || !w_zp_all_zero || g.sh != 1 || g.sw != 1) return false;
    if (g.M > kTcConvMaxFilters || g.M % 16 != 0 || g.C % 64 != 0 || g.N <= 0 || g.OH <= 0 || g.OW <= 0) return false;
    const bool padded = g.pt || g.pl || g.pb || g.pr;
    if (padded && x_zp != 0) return false;                       // the halo is zero fill
    TcConvArgs& a = p.a;
    a = TcConvArgs{};
    a.N = g.N; a.C = g.C; a.M = g.M; a.KH = g.KH; a.KW = g.KW; a.dh = g.dh; a.dw = g.dw;
    a.H = g.H; a.W = g.W; a.OH = g.OH; a.OW = g.OW; a.pt = g.pt; a.pl = g.pl;
    const int halo_w = (a.KW - 1) * a.dw, halo_h = (a.KH - 1) * a.dh;
    if (halo_w > 32 || halo_h > 32) return false;
    a.BW = std::min(a.OW, 128 - halo_w);
    a.PW = a.BW + halo_w;
    a.BH = std::max(1, std::min(a.OH, 128 / a.PW));
    a.wseg = (a.OW + a.BW - 1) / a.BW;
    a.full_width = 0;
    p.NT = g.M <= 64 ? 64 : (g.M <= 128 ? 128 : 256);
    a.m_pad = (g.M + p.NT - 1) / p.NT * p.NT;
    a.n_tiles = a.m_pad / p.NT;
    const int taps = a.KH * a.KW;
    const int budget = 232448 - kTcConvTail - 2048;
    const int blocks_in_image = (a.OH + a.BH - 1) / a.BH;
    const TcConvArgs base = a;
    bool placed = false;
    int w_stage = 0;
    // 128 channels per stage when C allows and the stage's weights leave room for two stages, else 64
    for (int KC = g.C % 128 == 0 ? 128 : 64; KC >= 64 && !placed; KC -= 64)
    for (int rb = 4; rb >= 1 && !placed; rb /= 2) {
        w_stage = taps * p.NT * KC;
        const long long w_all = (long long)(g.C / KC) * w_stage;
        if (2 * rb * p.NT > 512 || (rb > 1 && rb > blocks_in_image)) continue;
        a = base;
        a.CB = KC / 16; a.c_stages = g.C / KC;
        a.RB = rb; a.BHT = rb * a.BH;
        a.PH = a.BHT + halo_h;
        if (a.PH > 256) continue;
        a.hseg = (a.OH + a.BHT - 1) / a.BHT;
        if (rb > 1 && (long long)a.hseg * rb * 7 > (long long)blocks_in_image * 8) continue;
        a.PR = std::max(a.PH * a.PW, (rb - 1) * a.BH * a.PW + 128 + halo_h * a.PW + halo_w);
        const int patch_bytes = (a.PR * KC + 1023) / 1024 * 1024;
        for (int resident = 1; resident >= 0 && !placed; --resident) {
            if (resident && (a.n_tiles != 1 || w_all > 112 * 1024)) continue;
            const int off_patch = resident ? 0 : w_stage;         // a multiple of 1024: NT * KC is
            const int stage_bytes = off_patch + patch_bytes;
            const int stages = (int)std::min<long long>(kTcConvMaxStages, (budget - (resident ? w_all : 0)) / stage_bytes);
            if (stages < 2) continue;
            a.w_resident = resident; a.off_patch = off_patch; a.stage_bytes = stage_bytes; a.stages = stages;
            a.off_wres = stages * stage_bytes;
            a.off_out = a.off_wres + (resident ? (int)w_all : 0);   // here: the constants and barriers
            placed = true;
        }
    }
    if (!placed) return false;
    p.smem_bytes = (size_t)a.off_out + kTcConvTail;
    p.w_bytes = (size_t)a.n_tiles * a.c_stages * w_stage;
    p.row_efficiency = (double)a.OH * a.OW / ((double)a.hseg * a.RB * a.wseg * 128.0);
    const long long tiles = (long long)a.N * a.hseg * a.wseg * a.n_tiles;
    return tiles <= 0x7fffffffLL && p.row_efficiency >= 0.5;
}

// Blocks `w` ([M][C][KH][KW] int8) as [filter tile][channel stage][tap][NT rows of KC bytes], every row
// swizzled the way the tensor core reads it (16-byte chunk c of row j at chunk position c ^ (j % 8) for
// 128-byte rows, c ^ ((j / 2) % 4) for 64-byte rows), and pads the per-filter constants.
inline void tc_conv_nhwc_prepare(const TcConvPlan& p, const int8_t* w, const float* mult, const int32_t* bias, int x_zp,
                                 std::vector<int8_t>& w_blk, std::vector<float>& mult_pad, std::vector<int32_t>& bias_pad) {
    const TcConvArgs& a = p.a;
    const int taps = a.KH * a.KW, NT = p.NT, KC = a.CB * 16;
    w_blk.assign(p.w_bytes, 0);
    mult_pad.assign(a.m_pad, 1.0f);
    bias_pad.assign(a.m_pad, 0);
    for (int m = 0; m < a.M; ++m) {
        const int nt = m / NT, j = m % NT;
        const int x = KC == 128 ? (j & 7) : ((j >> 1) & 3);
        long long sum = 0;
        for (int c = 0; c < a.C; ++c) {
            const int cs = c / KC, cc = c % KC;
            const int pos = (((cc >> 4) ^ x) << 4) | (cc & 15);
            for (int tap = 0; tap < taps; ++tap) {
                const int8_t v = w[((size_t)m * a.C + c) * taps + tap];
                w_blk[((((size_t)nt * a.c_stages + cs) * taps + tap) * NT + j) * KC + pos] = v;
                sum += v;
            }
        }
        mult_pad[m] = mult[m];
        bias_pad[m] = (int32_t)((bias ? bias[m] : 0) - (long long)x_zp * sum);
    }
}

// Tensor map over x as (C, W, H, N) bytes; box = the stage's channels x the patch.
inline int32_t tc_conv_nhwc_encode_map(const TcConvArgs& a, const void* x, CUtensorMap* map) {
    const cuuint64_t W = (cuuint64_t)a.W, H = (cuuint64_t)a.H, C = (cuuint64_t)a.C, N = (cuuint64_t)a.N;
    const int KC = a.CB * 16;
    cuuint64_t dims[4] = {C, W, H, N}, strides[3] = {C, W * C, H * W * C};
    cuuint32_t box[4] = {(cuuint32_t)KC, (cuuint32_t)a.PW, (cuuint32_t)a.PH, 1}, estr[4] = {1, 1, 1, 1};
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
    const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void*>(x), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                              KC == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(ZANT_E_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
    return ZANT_OK;
}

template <int NT>
inline int32_t tc_conv_nhwc_launch_nt(zant_ctx* ctx, const TcConvPlan& p, const TcConvArgs& a, const CUtensorMap& m, int grid, bool x_u8, bool lean) {
    auto go = [&](auto kernel) -> int32_t {
        ZB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448));
        kernel<<<grid, kTcConvThreads, p.smem_bytes, ctx->stream>>>(a, m);
        return check_launch(ctx, "tc_conv_nhwc_kernel");
    };
    if (x_u8) return lean ? go(tc_conv_nhwc_kernel<NT, true, true>) : go(tc_conv_nhwc_kernel<NT, true, false>);
    return lean ? go(tc_conv_nhwc_kernel<NT, false, true>) : go(tc_conv_nhwc_kernel<NT, false, false>);
}

// x and y are device pointers, 16-byte aligned.
inline int32_t tc_conv_nhwc_run(zant_ctx* ctx, const TcConvPlan& p, const void* x, bool x_u8, const int8_t* w_blk_dev, const float* mult_dev,
                                const int32_t* bias_dev, void* y, bool y_u8, const Requant& rq, double max_product) {
    TcConvArgs a = p.a;
    a.x = (const uint8_t*)x; a.y = (uint8_t*)y; a.w = w_blk_dev; a.mult = mult_dev; a.bias = bias_dev;
    a.y_scale = rq.y_scale; a.y_zp = rq.y_zp; a.act = rq.act; a.out_u8 = y_u8 ? 1 : 0; a.lut = rq.lut;
    const bool lean = !y_u8 && rq.y_zp == 0 && std::isfinite(max_product);
    a.small_products = max_product < 4194304.0 ? 1 : 0;
    if (lean) {
        float v = 6.0f / rq.y_scale;
        v = std::fmin(std::fmax(v, -512.0f), 511.0f);
        a.six = std::min(std::max((int)std::nearbyintf(v), -128), 127);
    }
    a.status = ctx->status_word;
    const long long tiles = (long long)a.N * a.hseg * a.wseg * a.n_tiles;
    const int grid = (int)std::min<long long>(tiles, ctx->sm_count);
    alignas(64) CUtensorMap x_map;
    ZB_TRY(tc_conv_nhwc_encode_map(a, x, &x_map));
    if (p.NT == 64) return tc_conv_nhwc_launch_nt<64>(ctx, p, a, x_map, grid, x_u8, lean);
    if (p.NT == 128) return tc_conv_nhwc_launch_nt<128>(ctx, p, a, x_map, grid, x_u8, lean);
    return tc_conv_nhwc_launch_nt<256>(ctx, p, a, x_map, grid, x_u8, lean);
}

}  // namespace zb
