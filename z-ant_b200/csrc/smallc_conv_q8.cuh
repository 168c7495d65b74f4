// QLinearConv 3x3 for inputs with at most four channels (network stems: RGB -> 16..64 filters),
// stride 1 or 2, pads 0 or 1, NCHW in and out.
//
// The contraction is at most 36 deep, far too shallow for the 128-row tcgen05 shape (a K step of 32
// bytes would be mostly padding, and the NCHW -> channels-last transposition would cost more than the
// math).  It runs on warp-level int8 MMAs instead, with the roles of the operands swapped so that the
// result already has the layout of the output:
//   mma.sync m16n8k16 (s8 x u8|s8 -> s32):  rows    = 16 filters            (A: weights, registers, loaded once)
//                                           columns = 8 output pixels       (B: input patches)
//                                           K (16)  = 4 groups of 4 bytes; group q = (channel, kh) holds the
//                                                     bytes x[c][ih][iw0 .. iw0+3]: taps kw = 0..2 and one
//                                                     byte whose weight is zero.
// A B register of lane (g, t) is therefore ONE (unaligned) 4-byte window of an input row: two aligned
// shared-memory words and a byte permute.  The columns of the NTL MMAs of a unit are assigned to
// pixels so that a thread ends up with 2*NTL consecutive pixels of its two filters (g and g+8 of
// every 16-filter tile): after requantisation they are packed and stored as one 4- or 8-byte word
// per filter, no staging, and the per-filter constants are per-thread scalars.
//
// A CTA stages the input rows of a band of output rows in shared memory (pixels outside the image
// hold the input zero point, which the host folded into the bias), then its warps take units of
// 8*NTL pixels of one output row.
#pragma once
#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <vector>

#include "context.cuh"
#include "geometry.hpp"
#include "kernels_q8.cuh"
#include "tc_conv_nchw.cuh"

namespace zb {

constexpr int kSmallcThreads = 256;
constexpr int kSmallcMaxKs = 3;       // K steps of 16: up to 12 (channel, kh) groups

struct SmallcArgs {
    const uint8_t* x; uint8_t* y;
    const uint32_t* wfrag;            // [M/16][KS][2][32 lanes] A-fragment words
    const float* mult; const int32_t* bias;    // per filter; bias includes -x_zp * sum(w)
    int N, C, H, W, M, OH, OW;
    int s, pt, pl;
    int R, RIN, P;                    // output rows per band, staged input rows per channel, staged row pitch (bytes)
    int bands, upr;                   // bands per image, units per output row
    int KS;
    uint32_t pad_word;
    float y_scale; int y_zp; int act; int out_u8;
    const uint8_t* lut;       // optional table applied to the output codes (see Requant)
    int six; int small_products;
    int vec_ok;                       // output words of a thread are aligned (base and OW)
};

template <bool XU8>
__device__ __forceinline__ void mma_m16n8k16_s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    if (XU8)
        asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.s8.u8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
                     : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3]) : "r"(a0), "r"(a1), "r"(b0));
    else
        asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
                     : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3]) : "r"(a0), "r"(a1), "r"(b0));
}

// MT: 16-filter tiles (1..4); NTL: MMAs per unit along the pixels (2: 16 pixels, 4: 32 pixels); KSC: K steps issued per
// pixel block (1 for one input channel, 3 otherwise - a step whose groups do not exist multiplies zero weights), a
// compile-time count so that the unrolled MMA loops carry no tests.
template <int MT, int NTL, int KSC, bool XU8, bool LEAN>
__global__ void __launch_bounds__(kSmallcThreads) qconv3x3_smallc_kernel(const SmallcArgs a) {
    extern __shared__ __align__(16) uint8_t s_in[];      // [C][RIN][P]
    __shared__ uint8_t s_lut[256];                       // copy of the optional activation table
    if (a.lut) for (int i = threadIdx.x; i < 256; i += blockDim.x) s_lut[i] = __ldg(a.lut + i);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    constexpr int PXU = 8 * NTL;

    // weights (A fragments) and the constants of this thread's filters
    uint32_t wa[MT][kSmallcMaxKs][2];
    int bias[MT][2]; float mult[MT][2];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
        for (int ks = 0; ks < kSmallcMaxKs; ++ks)
#pragma unroll
            for (int h = 0; h < 2; ++h) wa[mt][ks][h] = ks < a.KS ? __ldg(a.wfrag + ((mt * a.KS + ks) * 2 + h) * 32 + lane) : 0u;
#pragma unroll
        for (int h = 0; h < 2; ++h) { bias[mt][h] = __ldg(a.bias + mt * 16 + g + 8 * h); mult[mt][h] = __ldg(a.mult + mt * 16 + g + 8 * h); }
    }
    // staged-row offset of this lane's K group in every K step (groups beyond 3*C have zero weights: any row will do)
    int qoff[kSmallcMaxKs];
#pragma unroll
    for (int ks = 0; ks < kSmallcMaxKs; ++ks) {
        const int q = 4 * ks + t, qq = q < 3 * a.C ? q : 0;
        qoff[ks] = ((qq / 3) * a.RIN + (qq % 3)) * a.P;
    }
    // pixel (within a unit) that this lane supplies to MMA nt: column g <-> pixel 2*NTL*(g/2) + 2*nt + g%2
    const int bpix0 = 2 * NTL * (g >> 1) + (g & 1);
    const Requant rq{a.y_scale, a.y_zp, a.act, a.lut};
    const uint32_t hi4 = a.act == ZANT_QACT_RELU6 ? 0x01010101u * (uint32_t)(a.six & 255) : 0x7f7f7f7fu;   // upper bound of the lean activation
    const bool relu = a.act != ZANT_QACT_NONE;
    const size_t ohw = (size_t)a.OH * a.OW;
    const int words_per_row = a.P >> 2;
    const int tiles = a.N * a.bands;

    for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
        const int n = tile / a.bands, band = tile - n * a.bands;
        const int oh0 = band * a.R;
        const int rows = min(a.R, a.OH - oh0);
        const int ih0 = oh0 * a.s - a.pt;
        // ---- stage the band's input rows: word k of a row holds image columns 4k-4 .. 4k-1
        for (int row = warp; row < a.C * a.RIN; row += kSmallcThreads / 32) {
            const int c = row / a.RIN, rr = row - c * a.RIN;
            const int ih = ih0 + rr;
            const bool row_ok = ih >= 0 && ih < a.H;
            const uint32_t* src = reinterpret_cast<const uint32_t*>(a.x + (((size_t)n * a.C + c) * a.H + (row_ok ? ih : 0)) * a.W);
            uint32_t* dst = reinterpret_cast<uint32_t*>(s_in + (size_t)row * a.P);
            for (int k = lane; k < words_per_row; k += 32)
                dst[k] = (row_ok && k >= 1 && k <= (a.W >> 2)) ? __ldg(src + k - 1) : a.pad_word;
        }
        __syncthreads();
        // ---- units of PXU pixels of one output row
        for (int u = warp; u < rows * a.upr; u += kSmallcThreads / 32) {
            const int r = u / a.upr, ow0 = (u - r * a.upr) * PXU;
            int acc[MT][NTL][4];
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int nt = 0; nt < NTL; ++nt) { acc[mt][nt][0] = acc[mt][nt][1] = bias[mt][0]; acc[mt][nt][2] = acc[mt][nt][3] = bias[mt][1]; }
            const int row_base = r * a.s * a.P + 4 - a.pl;
#pragma unroll
            for (int nt = 0; nt < NTL; ++nt) {
                const int ow = min(ow0 + bpix0 + 2 * nt, a.OW - 1);       // pixels past the row end are computed on valid data and dropped
                const int j0 = row_base + ow * a.s;
#pragma unroll
                for (int ks = 0; ks < KSC; ++ks) {
                    const int j = qoff[ks] + j0;
                    const uint32_t* wp = reinterpret_cast<const uint32_t*>(s_in + (j & ~3));
                    const uint32_t b0 = __byte_perm(wp[0], wp[1], 0x3210u + 0x1111u * (uint32_t)(j & 3));
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) mma_m16n8k16_s8<XU8>(acc[mt][nt], wa[mt][ks][0], wa[mt][ks][1], b0);
                }
            }
            // ---- requantise; this thread holds pixels ow0 + 2*NTL*t .. + 2*NTL-1 of filters 16*mt + g and + 8
            const int oh = oh0 + r;
            const int owt = ow0 + 2 * NTL * t;
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int f = mt * 16 + g + 8 * h;
                    uint32_t wd[NTL / 2];
#pragma unroll
                    for (int p = 0; p < NTL / 2; ++p) {
                        const int v0 = acc[mt][2 * p][2 * h], v1 = acc[mt][2 * p][2 * h + 1], v2 = acc[mt][2 * p + 1][2 * h], v3 = acc[mt][2 * p + 1][2 * h + 1];
                        if constexpr (LEAN) {
                            const int q0 = rq_round(v0, mult[mt][h]), q1 = rq_round(v1, mult[mt][h]), q2 = rq_round(v2, mult[mt][h]), q3 = rq_round(v3, mult[mt][h]);
                            wd[p] = relu ? __vminu4(pack_sat_u8x4(q0, q1, q2, q3), hi4) : pack_sat_s8x4(q0, q1, q2, q3);
                        } else {
                            const int q0 = a.out_u8 ? requant_one<true>(v0, mult[mt][h], rq) : requant_one<false>(v0, mult[mt][h], rq);
                            const int q1 = a.out_u8 ? requant_one<true>(v1, mult[mt][h], rq) : requant_one<false>(v1, mult[mt][h], rq);
                            const int q2 = a.out_u8 ? requant_one<true>(v2, mult[mt][h], rq) : requant_one<false>(v2, mult[mt][h], rq);
                            const int q3 = a.out_u8 ? requant_one<true>(v3, mult[mt][h], rq) : requant_one<false>(v3, mult[mt][h], rq);
                            wd[p] = (uint32_t)(q0 & 255) | ((uint32_t)(q1 & 255) << 8) | ((uint32_t)(q2 & 255) << 16) | ((uint32_t)(q3 & 255) << 24);
                        }
                    }
                    if (LEAN && a.lut) {
#pragma unroll
                        for (int p = 0; p < NTL / 2; ++p) wd[p] = lut4_smem(s_lut, wd[p]);
                    }
                    if (f < a.M && owt < a.OW) {
                        uint8_t* dst = a.y + ((size_t)n * a.M + f) * ohw + (size_t)oh * a.OW + owt;
                        if (a.vec_ok && owt + 2 * NTL <= a.OW) {
                            if constexpr (NTL == 4) *reinterpret_cast<uint2*>(dst) = make_uint2(wd[0], wd[1]);
                            else *reinterpret_cast<uint32_t*>(dst) = wd[0];
                        } else {
#pragma unroll
                            for (int i = 0; i < 2 * NTL; ++i)
                                if (owt + i < a.OW) dst[i] = (uint8_t)(wd[i >> 2] >> (8 * (i & 3)));
                        }
                    }
                }
            }
        }
        __syncthreads();
    }
}

// ---------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------
inline bool qconv_smallc_eligible(const ConvGeom& g, bool w_zp_all_zero) {
    if (g.G != 1 || !w_zp_all_zero || g.C > 4 || g.KH != 3 || g.KW != 3 || g.dh != 1 || g.dw != 1) return false;
    if (g.sh != g.sw || (g.sh != 1 && g.sh != 2)) return false;
    if (g.pt > 1 || g.pl > 1 || g.pb > 1 || g.pr > 1) return false;
    if (g.M % 16 != 0 || g.M > 64 || g.W % 4 != 0 || g.OH <= 0 || g.OW <= 0) return false;
    return (long long)g.N * g.OH * g.OW >= 4096;       // small outputs: the generic kernel is as good
}

inline bool qconv_smallc_ptr_ok(const void* x) { return (reinterpret_cast<uintptr_t>(x) & 3u) == 0; }

// A-fragment words of the weights ([M][C][3][3] int8): word (mt, ks, h, lane) = filter 16*mt + lane/4 + 8*h,
// K group q = 4*ks + lane%4 = (channel q/3, row q%3): bytes (w0, w1, w2, 0).  The input zero point is folded
// into the bias.
inline void qconv_smallc_prepare(const ConvGeom& g, const int8_t* w, const int32_t* bias, int x_zp, std::vector<uint32_t>& wfrag, std::vector<int32_t>& bias_f) {
    const int MT = g.M / 16, KS = (3 * g.C + 3) / 4;
    wfrag.assign((size_t)MT * KS * 2 * 32, 0u);
    bias_f.assign(g.M, 0);
    for (int mt = 0; mt < MT; ++mt)
        for (int ks = 0; ks < KS; ++ks)
            for (int h = 0; h < 2; ++h)
                for (int lane = 0; lane < 32; ++lane) {
                    const int f = 16 * mt + (lane >> 2) + 8 * h, q = 4 * ks + (lane & 3);
                    if (q >= 3 * g.C) continue;
                    const int8_t* wp = w + (((size_t)f * g.C + q / 3) * 3 + q % 3) * 3;
                    wfrag[((size_t)(mt * KS + ks) * 2 + h) * 32 + lane] = (uint32_t)(uint8_t)wp[0] | ((uint32_t)(uint8_t)wp[1] << 8) | ((uint32_t)(uint8_t)wp[2] << 16);
                }
    for (int m = 0; m < g.M; ++m) {
        long long sum = 0;
        for (int i = 0; i < g.C * 9; ++i) sum += w[(size_t)m * g.C * 9 + i];
        bias_f[m] = (int32_t)((bias ? bias[m] : 0) - (long long)x_zp * sum);
    }
}

template <int MT, int NTL>
inline int32_t smallc_launch(zant_ctx* ctx, const SmallcArgs& a, int grid, size_t smem, bool x_u8, bool lean) {
    auto go = [&](auto kernel) -> int32_t {
        if (smem > 48 * 1024) ZB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        kernel<<<grid, kSmallcThreads, smem, ctx->stream>>>(a);
        return check_launch(ctx, "qconv3x3_smallc_kernel");
    };
    if (a.KS == 1) {
        if (x_u8) return lean ? go(qconv3x3_smallc_kernel<MT, NTL, 1, true, true>) : go(qconv3x3_smallc_kernel<MT, NTL, 1, true, false>);
        return lean ? go(qconv3x3_smallc_kernel<MT, NTL, 1, false, true>) : go(qconv3x3_smallc_kernel<MT, NTL, 1, false, false>);
    }
    if (x_u8) return lean ? go(qconv3x3_smallc_kernel<MT, NTL, 3, true, true>) : go(qconv3x3_smallc_kernel<MT, NTL, 3, true, false>);
    return lean ? go(qconv3x3_smallc_kernel<MT, NTL, 3, false, true>) : go(qconv3x3_smallc_kernel<MT, NTL, 3, false, false>);
}

// `max_product`: bound of |accumulator * multiplier| (tc_conv_max_product), infinity if a multiplier is not finite.
inline int32_t run_qconv_smallc(zant_ctx* ctx, const ConvGeom& g, const void* x, bool x_u8, int x_zp, const uint32_t* wfrag_dev, const float* mult_dev,
                                const int32_t* bias_dev, void* y, bool y_u8, const Requant& rq, double max_product) {
    SmallcArgs a{};
    a.x = (const uint8_t*)x; a.y = (uint8_t*)y; a.wfrag = wfrag_dev; a.mult = mult_dev; a.bias = bias_dev;
    a.N = g.N; a.C = g.C; a.H = g.H; a.W = g.W; a.M = g.M; a.OH = g.OH; a.OW = g.OW;
    a.s = g.sh; a.pt = g.pt; a.pl = g.pl;
    a.KS = (3 * g.C + 3) / 4;
    a.P = (g.W + 12 + 15) / 16 * 16;
    // rows per band: the staged rows stay below 40 KiB, so that several CTAs share an SM
    a.R = std::min(g.OH, 8);
    while (a.R > 1 && (size_t)g.C * (a.R * a.s + 2) * a.P > 40 * 1024) --a.R;
    a.RIN = (a.R - 1) * a.s + 3;
    const size_t smem = (size_t)g.C * a.RIN * a.P;
    if (smem > 200 * 1024) return fail(ZANT_E_INVALID_INPUT, "QLinearConv(small-c): image rows of %d bytes do not fit in shared memory", g.W);
    a.bands = (g.OH + a.R - 1) / a.R;
    const int NTL = (g.OW % 32 == 0 || g.OW >= 256) ? 4 : 2;
    a.upr = (g.OW + 8 * NTL - 1) / (8 * NTL);
    a.pad_word = 0x01010101u * (uint32_t)(x_zp & 255);
    a.y_scale = rq.y_scale; a.y_zp = rq.y_zp; a.act = rq.act; a.out_u8 = y_u8 ? 1 : 0; a.lut = rq.lut;
    const bool lean = !y_u8 && rq.y_zp == 0 && std::isfinite(max_product);
    a.small_products = max_product < 4194304.0 ? 1 : 0;
    if (lean) {
        float v = 6.0f / rq.y_scale;
        v = std::fmin(std::fmax(v, -512.0f), 511.0f);
        a.six = std::min(std::max((int)std::nearbyintf(v), -128), 127);
    }
    const int wbytes = 2 * NTL;
    a.vec_ok = ((reinterpret_cast<uintptr_t>(y) % wbytes) == 0 && g.OW % wbytes == 0) ? 1 : 0;
    const long long tiles = (long long)g.N * a.bands;
    const int grid = (int)std::min<long long>(tiles, (long long)ctx->sm_count * 4);
    const int MT = g.M / 16;
#define ZB_SMALLC(MTV) (NTL == 4 ? smallc_launch<MTV, 4>(ctx, a, grid, smem, x_u8, lean) : smallc_launch<MTV, 2>(ctx, a, grid, smem, x_u8, lean))
    switch (MT) {
        case 1: return ZB_SMALLC(1);
        case 2: return ZB_SMALLC(2);
        case 3: return ZB_SMALLC(3);
        default: return ZB_SMALLC(4);
    }
#undef ZB_SMALLC
}

}  // namespace zb
