// Implicit-GEMM QLinearConv on tcgen05 that reads and writes the reference's NCHW layout directly
// (group 1, stride 1, any kernel size / dilation / padding, weight zero points 0).
//
// A tile is BH output rows x BW output columns of one image; its input patch (PH x PW pixels, halo
// included) is brought in 32 channels at a time:
//   1. producer warps copy the patch rows of the 32 channel planes with cp.async into a staging
//      buffer (rows stay rows: [channel][patch row][bytes], every input column at the same byte
//      offset in every row);
//   2. the same warps transpose staging -> "patch" [16-channel group][patch pixel][16 channels],
//      one 16-byte chunk per pixel, pixels in row-major order of the patch (4x4 byte transposes
//      with prmt); pixels outside the image hold the input zero point.
// In that form filter tap (kh,kw) of the implicit GEMM is the same shared memory shifted by
// (kh*dh*PW + kw*dw) chunks, which a K-major no-swizzle shared-memory descriptor expresses
// directly: MMA row r stands for patch pixel r, i.e. output (r / PW, r % PW) of the tile; rows
// with r % PW >= BW or r / PW >= BH are computed and dropped.  No im2col matrix exists anywhere.
// Weights arrive pre-blocked [filter tile][channel stage][tap][2][NT][16] by one bulk copy per stage.
//
// Warp roles (448 threads, one persistent CTA per SM):
//   warp 0      weight bulk copies          warp 1      TMEM owner + MMA issuer (taps MMAs per stage)
//   warps 2-5   cp.async + transpose        warps 6-13  epilogue: TMEM -> requantise -> NCHW bytes
#pragma once
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdint>
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
    int BH, BW, PH, PW, PR;           // tile, patch, allocated patch pixels per 16-channel group
    int hseg, wseg, c_stages, n_tiles;
    int G, SP;                        // cp.async granule (4, 8 or 16 bytes); staging row pitch
    int stages, stage_bytes, off_patch, off_stg;   // a stage = weights | patch | staging
    uint32_t pad_word;                // the input zero point in all four bytes
    float y_scale; int y_zp; int act; int out_u8;
    int m_pad;                        // filters rounded up to the tile width
    int* status;
};

constexpr int kTcConvMaxStages = 6;
constexpr int kTcConvMaxFilters = 1024;
constexpr int kTcConvThreads = 448;
constexpr int kTcConvTail = 2 * kTcConvMaxFilters * 4 + 512;   // constants + barriers after the stages

__device__ __forceinline__ void cp_async_4(uint32_t dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_8(uint32_t dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// out[p] = bytes (a[p], b[p], c[p], d[p]) for p = 0..3
__device__ __forceinline__ void transpose_4x4_bytes(uint32_t a, uint32_t b, uint32_t c, uint32_t d, uint32_t out[4]) {
    const uint32_t t0 = __byte_perm(a, b, 0x5140), t1 = __byte_perm(c, d, 0x5140);
    const uint32_t t2 = __byte_perm(a, b, 0x7362), t3 = __byte_perm(c, d, 0x7362);
    out[0] = __byte_perm(t0, t1, 0x5410); out[1] = __byte_perm(t0, t1, 0x7632);
    out[2] = __byte_perm(t2, t3, 0x5410); out[3] = __byte_perm(t2, t3, 0x7632);
}

struct TcConvTile { int img, h0, w0, nt; };

__device__ __forceinline__ TcConvTile tc_conv_decode(const TcConvArgs& a, int t) {
    TcConvTile r;
    r.nt = t % a.n_tiles;
    int sp = t / a.n_tiles;
    const int ws = sp % a.wseg; sp /= a.wseg;
    const int hs = sp % a.hseg;
    r.img = sp / a.hseg; r.h0 = hs * a.BH; r.w0 = ws * a.BW;
    return r;
}

template <int NT, bool XU8>
__global__ void __launch_bounds__(kTcConvThreads, 1) tc_conv_nchw_kernel(const __grid_constant__ TcConvArgs a) {
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* sStages = smem;
    uint8_t* tail = smem + (size_t)a.stages * a.stage_bytes;
    float* sMult = reinterpret_cast<float*>(tail);
    int* sBias = reinterpret_cast<int*>(tail + kTcConvMaxFilters * 4);
    uint64_t* bars = reinterpret_cast<uint64_t*>(tail + 2 * kTcConvMaxFilters * 4);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tail + 2 * kTcConvMaxFilters * 4 + 400);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tail + 2 * kTcConvMaxFilters * 4 + 404);
    volatile int* epi_ok = reinterpret_cast<volatile int*>(tail + 2 * kTcConvMaxFilters * 4 + 408);
    const uint32_t bar0 = ptx::smem_u32(bars);
    const int S = a.stages;
    auto full = [&](int s) { return bar0 + 8u * s; };
    auto empty = [&](int s) { return bar0 + 8u * (kTcConvMaxStages + s); };
    auto tfull = [&](int b) { return bar0 + 8u * (2 * kTcConvMaxStages + b); };
    auto tempty = [&](int b) { return bar0 + 8u * (2 * kTcConvMaxStages + 2 + b); };

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int tiles = a.N * a.hseg * a.wseg * a.n_tiles;
    const int taps = a.KH * a.KW;
    const uint32_t w_stage_bytes = (uint32_t)taps * 2u * NT * 16u;

    if (tid == 0) {
        for (int s = 0; s < S; ++s) { ptx::mbar_init(full(s), 2); ptx::mbar_init(empty(s), 1); }
        for (int b = 0; b < 2; ++b) { ptx::mbar_init(tfull(b), 1); ptx::mbar_init(tempty(b), 8); }
        *abort_flag = 0;
        *epi_ok = 1;
        ptx::mbar_fence_init();
    }
    for (int i = tid; i < a.m_pad; i += kTcConvThreads) { sMult[i] = __ldg(a.mult + i); sBias[i] = __ldg(a.bias + i); }
    if (warp == 1) {
        ptx::tmem_alloc(ptx::smem_u32(tmem_slot), 2 * NT);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------------ weights: one bulk copy per stage
        if (ptx::elect_one()) {
            int it = 0;
            for (int t = blockIdx.x; t < tiles; t += gridDim.x) {
                const int nt = t % a.n_tiles;
                const int8_t* gw = a.w + (size_t)nt * a.c_stages * w_stage_bytes;
                for (int cs = 0; cs < a.c_stages; ++cs, ++it) {
                    const int s = it % S;
                    const uint32_t ph = (uint32_t)(it / S) & 1u;
                    if (!ptx::mbar_wait(empty(s), ph ^ 1u, abort_flag)) goto weights_done;
                    ptx::mbar_arrive_expect_tx(full(s), w_stage_bytes);
                    ptx::bulk_g2s(ptx::smem_u32(sStages + (size_t)s * a.stage_bytes), gw + (size_t)cs * w_stage_bytes, w_stage_bytes, full(s));
                }
            }
        weights_done:;
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (ptx::elect_one()) {
            constexpr uint32_t idesc = ptx::idesc_i8(128, NT, !XU8, true);
            const uint32_t a_lbo = (uint32_t)a.PR * 16u;
            int it = 0, tile_it = 0;
            for (int t = blockIdx.x; t < tiles; t += gridDim.x, ++tile_it) {
                const int b = tile_it & 1;
                const uint32_t bph = (uint32_t)(tile_it >> 1) & 1u;
                if (!ptx::mbar_wait(tempty(b), bph ^ 1u, abort_flag)) goto mma_done;
                const uint32_t d_tmem = tmem_base + (uint32_t)(b * NT);
                for (int cs = 0; cs < a.c_stages; ++cs, ++it) {
                    const int s = it % S;
                    const uint32_t ph = (uint32_t)(it / S) & 1u;
                    if (!ptx::mbar_wait(full(s), ph, abort_flag)) goto mma_done;
                    ptx::tc_fence_after();
                    const uint32_t sw = ptx::smem_u32(sStages + (size_t)s * a.stage_bytes);
                    const uint32_t sp = sw + (uint32_t)a.off_patch;
                    int tap = 0;
                    for (int kh = 0; kh < a.KH; ++kh)
                        for (int kw = 0; kw < a.KW; ++kw, ++tap) {
                            const uint32_t off = (uint32_t)(kh * a.dh * a.PW + kw * a.dw) * 16u;
                            const uint64_t da = ptx::smem_desc_kmajor(sp + off, a_lbo, 128);
                            const uint64_t db = ptx::smem_desc_kmajor(sw + (uint32_t)tap * (2u * NT * 16u), NT * 16, 128);
                            ptx::mma_i8(d_tmem, da, db, idesc, (cs | tap) != 0);
                        }
                    ptx::mma_commit(empty(s));
                }
                ptx::mma_commit(tfull(b));
            }
        mma_done:;
        }
    } else if (warp < 6) {
        // ------------------------------------------------------------------ activation producers (128 threads)
        const int p = tid - 64;
        const int GP = (a.SP - 32) / a.G;                       // granules per staging row (data region)
        const int runs = 32 * a.PH;
        const int slots = runs * GP;
        const int my_tiles = (tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
        const int total_it = my_tiles * a.c_stages;
        const size_t plane = (size_t)a.H * a.W;

        auto issue_loads = [&](int it) {
            if (it < total_it) {
                const int tl = it / a.c_stages, cs = it - tl * a.c_stages;
                const TcConvTile T = tc_conv_decode(a, (int)blockIdx.x + tl * (int)gridDim.x);
                const int s = it % S;
                const uint32_t stg = ptx::smem_u32(sStages + (size_t)s * a.stage_bytes + a.off_stg);
                const int w_in0 = T.w0 - a.pl, h_in0 = T.h0 - a.pt;
                const int iw_lo = max(w_in0, 0), iw_hi = min(w_in0 + a.PW, a.W);
                const int seg_base = iw_lo & ~(a.G - 1);
                const int n_gran = iw_hi > iw_lo ? (iw_hi - seg_base + a.G - 1) / a.G : 0;
                const uint8_t* ximg = a.x + ((size_t)T.img * a.C + (size_t)cs * 32) * plane + seg_base;
                for (int sl = p; sl < slots; sl += 128) {
                    const int run = sl / GP, gi = sl - run * GP;
                    const int cc = run / a.PH, hh = run - cc * a.PH;
                    const int ih = h_in0 + hh;
                    if (gi < n_gran && cs * 32 + cc < a.C && ih >= 0 && ih < a.H) {
                        const uint8_t* src = ximg + (size_t)cc * plane + (size_t)ih * a.W + (size_t)gi * a.G;
                        const uint32_t dst = stg + (uint32_t)(run * a.SP + 16 + gi * a.G);
                        if (a.G == 16) cp_async_16(dst, src);
                        else if (a.G == 8) cp_async_8(dst, src);
                        else cp_async_4(dst, src);
                    }
                }
                // halo columns that no copy covers hold the input zero point
                const int left = iw_lo - w_in0, right = w_in0 + a.PW - iw_hi;     // pixels outside the image on either side
                if (left + right > 0) {
                    const int per_run = left + right;
                    uint8_t* stg_g = sStages + (size_t)s * a.stage_bytes + a.off_stg;
                    for (int i = p; i < runs * per_run; i += 128) {
                        const int run = i / per_run, j = i - run * per_run;
                        const int col = j < left ? (16 + (iw_lo - seg_base) - left + j) : (16 + (iw_hi - seg_base) + (j - left));
                        stg_g[run * a.SP + col] = (uint8_t)a.pad_word;
                    }
                }
            }
            cp_async_commit();
        };

        for (int d = 0; d < S - 1; ++d) issue_loads(d);
        for (int it = 0; it < total_it; ++it) {
            issue_loads(it + S - 1);
            // all but the S-1 newest groups of this thread are complete
            switch (S - 1) {
                case 1: cp_async_wait<1>(); break;
                case 2: cp_async_wait<2>(); break;
                case 3: cp_async_wait<3>(); break;
                case 4: cp_async_wait<4>(); break;
                default: cp_async_wait<5>(); break;
            }
            const int s = it % S;
            const uint32_t ph = (uint32_t)(it / S) & 1u;
            const bool ok = ptx::mbar_wait(empty(s), ph ^ 1u, abort_flag);
            ptx::named_barrier_sync(2, 128);                    // every thread's copies of this stage have landed
            if (!ok || *abort_flag) break;

            const int tl = it / a.c_stages, cs = it - tl * a.c_stages;
            const TcConvTile T = tc_conv_decode(a, (int)blockIdx.x + tl * (int)gridDim.x);
            const int w_in0 = T.w0 - a.pl, h_in0 = T.h0 - a.pt;
            const int iw_lo = max(w_in0, 0);
            const int seg_base = iw_lo & ~(a.G - 1);
            const int S0 = w_in0 - seg_base + 16;               // staging column of patch column 0
            const int k_lo = S0 >> 2, k_hi = (S0 + a.PW - 1) >> 2;
            const int kn = k_hi - k_lo + 1;
            const uint8_t* stg = sStages + (size_t)s * a.stage_bytes + a.off_stg;
            uint8_t* patch = sStages + (size_t)s * a.stage_bytes + a.off_patch;
            const int items = 2 * a.PH * kn;
            for (int i = p; i < items; i += 128) {
                const int k = k_lo + i % kn;
                const int rest = i / kn;
                const int hh = rest % a.PH, blk = rest / a.PH;
                const int ih = h_in0 + hh;
                const bool row_ok = ih >= 0 && ih < a.H;
                const int c_base = cs * 32 + blk * 16;
                uint32_t wv[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const uint32_t v = *reinterpret_cast<const uint32_t*>(stg + (size_t)((blk * 16 + j) * a.PH + hh) * a.SP + k * 4);
                    wv[j] = (row_ok && c_base + j < a.C) ? v : a.pad_word;
                }
                uint32_t o[4][4];    // o[group of 4 channels][pixel]
#pragma unroll
                for (int q = 0; q < 4; ++q) transpose_4x4_bytes(wv[4 * q], wv[4 * q + 1], wv[4 * q + 2], wv[4 * q + 3], o[q]);
                uint8_t* dst_row = patch + (size_t)blk * a.PR * 16 + (size_t)hh * a.PW * 16;
#pragma unroll
                for (int px = 0; px < 4; ++px) {
                    const int ww = k * 4 + px - S0;
                    if (ww >= 0 && ww < a.PW) *reinterpret_cast<uint4*>(dst_row + (size_t)ww * 16) = make_uint4(o[0][px], o[1][px], o[2][px], o[3][px]);
                }
            }
            ptx::fence_proxy_async_smem();
            ptx::named_barrier_sync(2, 128);
            if (p == 0) ptx::mbar_arrive(full(s));
        }
        cp_async_wait<0>();
    } else {
        // ------------------------------------------------------------------ epilogue: warps 6..13
        const int quarter = warp & 3;
        const int half = (warp - 6) >> 2;
        const int row = quarter * 32 + lane;
        const int e = (warp - 6) * 32 + lane;
        const Requant rq{a.y_scale, a.y_zp, a.act};
        const int oh_l = row / a.PW, ow_l = row - oh_l * a.PW;
        const size_t ohw = (size_t)a.OH * a.OW;
        int tile_it = 0;
        for (int t = blockIdx.x; t < tiles; t += gridDim.x, ++tile_it) {
            const TcConvTile T = tc_conv_decode(a, t);
            const int b = tile_it & 1;
            const uint32_t bph = (uint32_t)(tile_it >> 1) & 1u;
            if (e == 0) *epi_ok = ptx::mbar_wait(tfull(b), bph, abort_flag) ? 1 : 0;
            ptx::named_barrier_sync(1, 256);
            if (!*epi_ok) break;
            ptx::tc_fence_after();
            const int tcol0 = half * (NT / 2);
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(b * NT + tcol0);
            const int oh = T.h0 + oh_l, ow = T.w0 + ow_l;
            const bool row_ok = oh_l < a.BH && ow_l < a.BW && oh < a.OH && ow < a.OW;
            uint8_t* ybase = a.y + (size_t)T.img * a.M * ohw + (size_t)oh * a.OW + ow;
#pragma unroll 1
            for (int h = 0; h < NT / 64; ++h) {
                uint32_t v[32];
                ptx::tmem_ld32(taddr + (uint32_t)(h * 32), v);
                ptx::tmem_wait_ld();
                const int col0 = T.nt * NT + tcol0 + h * 32;
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    const int col = col0 + j;
                    const int acc = (int)v[j] + sBias[col];
                    const int q = a.out_u8 ? requant_one<true>(acc, sMult[col], rq) : requant_one<false>(acc, sMult[col], rq);
                    if (row_ok && col < a.M) ybase[(size_t)col * ohw] = (uint8_t)q;
                }
            }
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(tempty(b));
        }
    }

    if (*abort_flag) {
        for (int i = 0; i < 200; ++i) __nanosleep(1000);
    }
    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 1) ptx::tmem_dealloc(tmem_base, 2 * NT);
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

// Chooses tiling for `g`.  Returns false when the kernel does not apply (the caller then uses the
// im2col path or the generic kernel).
inline bool tc_conv_plan(const ConvGeom& g, bool w_zp_all_zero, TcConvPlan& p) {
    if (g.G != 1 || !w_zp_all_zero || g.sh != 1 || g.sw != 1) return false;
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
    if (a.W % 4 != 0 || a.pl > 16) return false;
    a.G = a.W % 16 == 0 ? 16 : (a.W % 8 == 0 ? 8 : 4);
    const int halo_w = (a.KW - 1) * a.dw, halo_h = (a.KH - 1) * a.dh;
    if (halo_w > 32 || halo_h > 32) return false;
    if (!pointwise && (g.pl > halo_w || g.pr > halo_w || g.pt > halo_h || g.pb > halo_h)) return false;   // every tile overlaps the image
    a.BW = std::min(a.OW, 128 - halo_w);
    a.PW = a.BW + halo_w;
    a.BH = std::max(1, std::min(a.OH, 128 / a.PW));
    a.PH = a.BH + halo_h;
    a.PR = (128 + halo_h * a.PW + halo_w + 7) / 8 * 8;
    a.wseg = (a.OW + a.BW - 1) / a.BW;
    a.hseg = (a.OH + a.BH - 1) / a.BH;
    a.c_stages = (a.C + 31) / 32;
    p.NT = g.M <= 64 ? 64 : 128;
    if (pointwise && g.M > 128) p.NT = 256;
    a.m_pad = (g.M + p.NT - 1) / p.NT * p.NT;
    a.n_tiles = a.m_pad / p.NT;
    a.SP = 32 + (a.PW + 15 + 15) / 16 * 16;
    const int taps = a.KH * a.KW;
    const int w_stage = taps * 2 * p.NT * 16;
    a.off_patch = w_stage;
    a.off_stg = a.off_patch + 2 * a.PR * 16;
    a.stage_bytes = (a.off_stg + 32 * a.PH * a.SP + 127) / 128 * 128;
    const int budget = 232448 - kTcConvTail - 1024;
    a.stages = std::min(kTcConvMaxStages, budget / a.stage_bytes);
    if (a.stages < 2) return false;
    p.smem_bytes = (size_t)a.stages * a.stage_bytes + kTcConvTail;
    p.w_bytes = (size_t)a.n_tiles * a.c_stages * w_stage;
    const double useful = (double)a.OH * a.OW;
    const double issued = (double)a.hseg * a.wseg * 128.0;
    p.row_efficiency = useful / issued;
    const long long tiles = (long long)a.N * a.hseg * a.wseg * a.n_tiles;
    if (tiles > 0x7fffffffLL || p.row_efficiency < 0.5) return false;
    return true;
}

// Blocks `w` ([M][C][KH][KW] int8) as [filter tile][channel stage][tap][2][NT][16] and pads the
// per-filter constants; the input zero point is folded into the bias (halo pixels hold x_zp).
inline void tc_conv_prepare(const TcConvPlan& p, const int8_t* w, const float* mult, const int32_t* bias, int x_zp,
                            std::vector<int8_t>& w_blk, std::vector<float>& mult_pad, std::vector<int32_t>& bias_pad) {
    const TcConvArgs& a = p.a;
    const int taps = a.KH * a.KW, NT = p.NT;
    w_blk.assign(p.w_bytes, 0);
    mult_pad.assign(a.m_pad, 1.0f);
    bias_pad.assign(a.m_pad, 0);
    for (int m = 0; m < a.M; ++m) {
        const int nt = m / NT, mm = m % NT;
        long long sum = 0;
        for (int c = 0; c < a.C; ++c) {
            const int cs = c / 32, blk = (c % 32) / 16, j = c % 16;
            for (int tap = 0; tap < taps; ++tap) {
                const int8_t v = w[((size_t)m * a.C + c) * taps + tap];
                w_blk[((((size_t)nt * a.c_stages + cs) * taps + tap) * 2 + blk) * NT * 16 + (size_t)mm * 16 + j] = v;
                sum += v;
            }
        }
        mult_pad[m] = mult[m];
        bias_pad[m] = (int32_t)((bias ? bias[m] : 0) - (long long)x_zp * sum);
    }
}

template <int NT, bool XU8>
inline int32_t tc_conv_launch_t(zant_ctx* ctx, const TcConvPlan& p, const TcConvArgs& a, int grid) {
    static bool attr_set = false;
    if (!attr_set) {
        ZB_CUDA(cudaFuncSetAttribute(tc_conv_nchw_kernel<NT, XU8>, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448));
        attr_set = true;
    }
    tc_conv_nchw_kernel<NT, XU8><<<grid, kTcConvThreads, p.smem_bytes, ctx->stream>>>(a);
    return check_launch(ctx, "tc_conv_nchw_kernel");
}

// x must be 16-byte aligned (checked by the caller through tc_conv_ptr_ok).
inline bool tc_conv_ptr_ok(const void* x) { return (reinterpret_cast<uintptr_t>(x) & 15u) == 0; }

inline int32_t tc_conv_run(zant_ctx* ctx, const TcConvPlan& p, const void* x, bool x_u8, int x_zp, const int8_t* w_blk_dev,
                           const float* mult_dev, const int32_t* bias_dev, void* y, bool y_u8, const Requant& rq) {
    TcConvArgs a = p.a;
    a.x = (const uint8_t*)x; a.y = (uint8_t*)y; a.w = w_blk_dev; a.mult = mult_dev; a.bias = bias_dev;
    a.pad_word = 0x01010101u * (uint32_t)(x_zp & 255);
    a.y_scale = rq.y_scale; a.y_zp = rq.y_zp; a.act = rq.act; a.out_u8 = y_u8 ? 1 : 0;
    a.status = ctx->status_word;
    const long long tiles = (long long)a.N * a.hseg * a.wseg * a.n_tiles;
    const int grid = (int)std::min<long long>(tiles, ctx->sm_count);
    if (p.NT == 64) return x_u8 ? tc_conv_launch_t<64, true>(ctx, p, a, grid) : tc_conv_launch_t<64, false>(ctx, p, a, grid);
    if (p.NT == 128) return x_u8 ? tc_conv_launch_t<128, true>(ctx, p, a, grid) : tc_conv_launch_t<128, false>(ctx, p, a, grid);
    return x_u8 ? tc_conv_launch_t<256, true>(ctx, p, a, grid) : tc_conv_launch_t<256, false>(ctx, p, a, grid);
}

}  // namespace zb
