// Tensor-core path for QLinearConv of any geometry with group 1 (and for QLinearMatMul):
//   1. im2col_blocked_kernel gathers the NCHW input into the GEMM-blocked A layout
//      [row tile of 128][K/16][128 rows][16], rows = (image, oh, ow), K = (c, kh, kw) in the
//      weight's own order, padded taps filled with the input zero point, K padded with zeros;
//   2. tc_gemm_i8_kernel<NT, 4, 8, MODE|2> multiplies by the re-blocked weights on tcgen05 and
//      requantises straight into the NCHW output.
// The zero point of x is folded into the bias (bias - x_zp * sum(w)), which is exact because
// padded taps hold x_zp; weight zero points other than 0 are not handled here (generic kernel).
#pragma once
#include <cuda_runtime.h>

#include <cstdint>
#include <vector>

#include "context.cuh"
#include "geometry.hpp"
#include "tc_gemm.cuh"

namespace zb {

struct Im2colArgs {
    const uint8_t* x; uint8_t* a;
    ConvGeom g;
    int K, K16, M;       // K = C*KH*KW, K16 = padded K / 16, M = N*OH*OW
    int pad_value;       // raw byte written for padded taps (the input zero point)
};

__global__ void im2col_blocked_kernel(const Im2colArgs p) {
    const ConvGeom& g = p.g;
    const size_t total = (size_t)((p.M + 127) / 128) * p.K16 * 128;
    const int khw = g.KH * g.KW, ohw = g.OH * g.OW;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int r = (int)(i & 127);
        const size_t t = i >> 7;
        const int k16 = (int)(t % p.K16);
        const int m = (int)(t / p.K16) * 128 + r;
        uint32_t w[4] = {0u, 0u, 0u, 0u};
        if (m < p.M) {
            const int n = m / ohw, pos = m - n * ohw;
            const int oh = pos / g.OW, ow = pos - oh * g.OW;
            const int ih0 = oh * g.sh - g.pt, iw0 = ow * g.sw - g.pl;
            const uint8_t* xn = p.x + (size_t)n * g.C * g.H * g.W;
            int k = k16 * 16;
            int c = k / khw, rem = k - c * khw;
            int kh = rem / g.KW, kw = rem - kh * g.KW;
#pragma unroll
            for (int j = 0; j < 16; ++j, ++k) {
                uint32_t v = 0;
                if (k < p.K) {
                    const int ih = ih0 + kh * g.dh, iw = iw0 + kw * g.dw;
                    v = (ih >= 0 && ih < g.H && iw >= 0 && iw < g.W) ? (uint32_t)__ldg(xn + ((size_t)c * g.H + ih) * g.W + iw) : (uint32_t)(p.pad_value & 255);
                    if (++kw == g.KW) { kw = 0; if (++kh == g.KH) { kh = 0; ++c; } }
                }
                w[j >> 2] |= v << (8 * (j & 3));
            }
        }
        reinterpret_cast<uint4*>(p.a)[i] = make_uint4(w[0], w[1], w[2], w[3]);
    }
}

// 1x1 convolutions (stride 1, no padding) with H*W % 4 == 0: the im2col matrix is the NCHW tensor with
// pixels and channels swapped.  A CTA turns 64 channels x 128 consecutive pixels (image after image) into
// four [128 rows][16] chunks of the GEMM-blocked layout: coalesced 4-byte loads along the pixels into
// shared memory, 4x4 byte transposes with prmt, 16-byte stores.  Rows beyond the last pixel and
// channels beyond C are zero.
struct PwBlockArgs {
    const uint8_t* x; uint8_t* a;
    int C, HW, M, K16;        // M = N * HW rows
};

__global__ void __launch_bounds__(256) pointwise_blocked_kernel(const PwBlockArgs p) {
    __shared__ uint32_t tile[64][33];                 // [channel][32 words of 4 pixels], padded against bank conflicts
    const int tid = threadIdx.x, lane = tid & 31, wrp = tid >> 5;
    const int mt = blockIdx.x, kg = blockIdx.y;       // row tile, group of 4 K chunks (64 channels)
    const int m4 = mt * 128 + lane * 4;               // first of this lane's 4 rows; never straddles an image (H*W % 4 == 0)
    const int n = m4 / p.HW, pix = m4 - n * p.HW;
    const bool row_ok = m4 < p.M;
    const uint8_t* src = p.x + ((size_t)n * p.C) * p.HW + pix;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int cl = wrp * 8 + i, c = kg * 64 + cl;
        tile[cl][lane] = (row_ok && c < p.C) ? __ldg(reinterpret_cast<const uint32_t*>(src + (size_t)c * p.HW)) : 0u;
    }
    __syncthreads();
    // thread = (K chunk q of 4, word w of 32): 16 channels x 4 pixels -> four 16-byte chunks; two rounds cover 4 x 32
    const int q = tid >> 6, w = (tid & 63) >> 1, half = tid & 1;     // half: which 2 of the word's 4 pixels this thread stores
    uint32_t wv[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) wv[j] = tile[q * 16 + j][w];
    uint32_t o[4][4];
#pragma unroll
    for (int g = 0; g < 4; ++g) {
        const uint32_t t0 = __byte_perm(wv[4 * g], wv[4 * g + 1], 0x5140), t1 = __byte_perm(wv[4 * g + 2], wv[4 * g + 3], 0x5140);
        const uint32_t t2 = __byte_perm(wv[4 * g], wv[4 * g + 1], 0x7362), t3 = __byte_perm(wv[4 * g + 2], wv[4 * g + 3], 0x7362);
        o[g][0] = __byte_perm(t0, t1, 0x5410); o[g][1] = __byte_perm(t0, t1, 0x7632);
        o[g][2] = __byte_perm(t2, t3, 0x5410); o[g][3] = __byte_perm(t2, t3, 0x7632);
    }
    const int k16 = kg * 4 + q;
    if (k16 < p.K16) {
        uint4* dst = reinterpret_cast<uint4*>(p.a) + ((size_t)mt * p.K16 + k16) * 128 + w * 4;
#pragma unroll
        for (int px = 0; px < 2; ++px) {
            const int r = half * 2 + px;
            dst[r] = make_uint4(o[0][r], o[1][r], o[2][r], o[3][r]);
        }
    }
}

// Convolutions whose channel count is a multiple of 16 use the K order (tap, channel) instead of the
// weight tensor's (channel, tap): a 16-byte K chunk is then 16 channels of ONE tap, and the im2col
// matrix is built like the 1x1 case, tap by tap.  A CTA takes one tap, 64 channels and 128 output
// pixels: byte loads that are contiguous (or stride-s) along the pixels, out-of-image taps replaced by
// the input zero point, into shared memory, then the same 4x4 byte transposes and 16-byte stores.
struct TapMajorArgs {
    const uint8_t* x; uint8_t* a;
    ConvGeom g;
    int M, K16, cgroups;      // rows, K chunks per row, groups of 64 channels
    int pad_value;
};

__global__ void __launch_bounds__(256) im2col_tapmajor_kernel(const TapMajorArgs p) {
    __shared__ uint32_t tile[64][33];
    uint8_t (*tile8)[132] = reinterpret_cast<uint8_t (*)[132]>(&tile[0][0]);   // the same rows, byte view (33 words = 132 bytes)
    const ConvGeom& g = p.g;
    const int tid = threadIdx.x;
    const int mt = blockIdx.x;
    const int tap = blockIdx.y / p.cgroups, kg = blockIdx.y - tap * p.cgroups;
    const int kh = tap / g.KW, kw = tap - kh * g.KW;
    {
        const int r = tid & 127, half = tid >> 7;
        const int m = mt * 128 + r;
        const int ohw = g.OH * g.OW;
        const int n = m / ohw, pos = m - n * ohw;
        const int oh = pos / g.OW, ow = pos - oh * g.OW;
        const int ih = oh * g.sh - g.pt + kh * g.dh, iw = ow * g.sw - g.pl + kw * g.dw;
        const bool ok = m < p.M && ih >= 0 && ih < g.H && iw >= 0 && iw < g.W;
        const size_t plane = (size_t)g.H * g.W;
        const int c0 = kg * 64 + half * 32;
        const uint8_t* src = p.x + ((size_t)n * g.C + c0) * plane + (size_t)(ok ? ih : 0) * g.W + (ok ? iw : 0);
#pragma unroll 8
        for (int i = 0; i < 32; ++i) {
            uint8_t v = (uint8_t)p.pad_value;
            if (ok && c0 + i < g.C) v = __ldg(src + (size_t)i * plane);
            tile8[half * 32 + i][r] = v;
        }
    }
    __syncthreads();
    const int q = tid >> 6, w = (tid & 63) >> 1, half = tid & 1;
    uint32_t wv[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) wv[j] = tile[q * 16 + j][w];
    uint32_t o[4][4];
#pragma unroll
    for (int gq = 0; gq < 4; ++gq) {
        const uint32_t t0 = __byte_perm(wv[4 * gq], wv[4 * gq + 1], 0x5140), t1 = __byte_perm(wv[4 * gq + 2], wv[4 * gq + 3], 0x5140);
        const uint32_t t2 = __byte_perm(wv[4 * gq], wv[4 * gq + 1], 0x7362), t3 = __byte_perm(wv[4 * gq + 2], wv[4 * gq + 3], 0x7362);
        o[gq][0] = __byte_perm(t0, t1, 0x5410); o[gq][1] = __byte_perm(t0, t1, 0x7632);
        o[gq][2] = __byte_perm(t2, t3, 0x5410); o[gq][3] = __byte_perm(t2, t3, 0x7632);
    }
    if (kg * 64 + q * 16 < g.C) {
        const int k16 = tap * (g.C / 16) + kg * 4 + q;
        uint4* dst = reinterpret_cast<uint4*>(p.a) + ((size_t)mt * p.K16 + k16) * 128 + w * 4;
#pragma unroll
        for (int px = 0; px < 2; ++px) {
            const int r = half * 2 + px;
            dst[r] = make_uint4(o[0][r], o[1][r], o[2][r], o[3][r]);
        }
    }
}

// Host-side preparation of one convolution / matrix product for the tensor-core path.
struct QGemmPrep {
    int NT = 0, N_pad = 0, K = 0, K16 = 0;
    std::vector<int8_t> w_blk;     // [N_pad/NT][K16][NT][16]
    std::vector<float> mult;       // [N_pad]
    std::vector<int32_t> bias;     // [N_pad], includes -x_zp * sum(w)
    bool tap_major = false;        // K order (tap, channel) instead of the weight tensor's (channel, tap)
    bool mult_finite = true;       // every multiplier is finite (the lean epilogue's precondition)
};

// w: [n_out][K] int8 row-major (a convolution's [M][C][KH][KW] weight is exactly that).
// `rows` (when known) lets wide outputs pick the tile width that wastes the least of the last wave of
// 148 persistent CTAs: 256-wide tiles halve the number of tiles but a partly filled wave costs a full one.
inline void qgemm_prepare(const int8_t* w, int n_out, int K, const float* mult, const int32_t* bias, int x_zp, QGemmPrep& p, long long rows = 0) {
    p.NT = n_out <= 64 ? 64 : (n_out <= 128 ? 128 : 256);
    if (p.NT == 256 && rows > 0) {
        const long long mt = (rows + 127) / 128;
        const long long t256 = mt * ((n_out + 255) / 256), t128 = mt * ((n_out + 127) / 128);
        const long long c256 = (t256 + 147) / 148 * 256, c128 = (t128 + 147) / 148 * 128;
        if (c128 < c256) p.NT = 128;
    }
    p.N_pad = (n_out + p.NT - 1) / p.NT * p.NT;
    p.K = K;
    p.K16 = K <= 32 ? 2 : (K + 63) / 64 * 4;      // a stage holds 4 chunks of K (2 when K fits 32: first layers with 3 channels)
    p.w_blk.assign((size_t)p.N_pad * p.K16 * 16, 0);
    p.mult.assign(p.N_pad, 1.0f);
    p.bias.assign(p.N_pad, 0);
    for (int n = 0; n < n_out; ++n) {
        int sum = 0;
        const int8_t* wr = w + (size_t)n * K;
        int8_t* dst_tile = p.w_blk.data() + (size_t)(n / p.NT) * p.K16 * p.NT * 16 + (size_t)(n % p.NT) * 16;
        for (int k = 0; k < K; ++k) {
            dst_tile[(size_t)(k >> 4) * p.NT * 16 + (k & 15)] = wr[k];
            sum += wr[k];
        }
        p.mult[n] = mult[n];
        p.mult_finite = p.mult_finite && std::isfinite(mult[n]);
        p.bias[n] = (bias ? bias[n] : 0) - x_zp * sum;
    }
}

// Convolution weights [M][C][KH][KW]: channel counts that are multiples of 16 (and more than one tap)
// get the (tap, channel) K order that im2col_tapmajor_kernel produces; everything else keeps the
// tensor's own order.
inline void qconv_gemm_prepare(const ConvGeom& g, const int8_t* w, const float* mult, const int32_t* bias, int x_zp, QGemmPrep& p) {
    const int taps = g.KH * g.KW, C = g.Cg, K = C * taps;
    const long long rows = (long long)g.N * g.OH * g.OW;
    if (taps == 1 || C % 16 != 0) { qgemm_prepare(w, g.M, K, mult, bias, x_zp, p, rows); return; }
    std::vector<int8_t> wt((size_t)g.M * K);
    for (int m = 0; m < g.M; ++m)
        for (int c = 0; c < C; ++c)
            for (int t = 0; t < taps; ++t) wt[(size_t)m * K + (size_t)t * C + c] = w[((size_t)m * C + c) * taps + t];
    qgemm_prepare(wt.data(), g.M, K, mult, bias, x_zp, p, rows);
    p.tap_major = true;
}

inline size_t qgemm_a_bytes(size_t rows, const QGemmPrep& p) { return (rows + 127) / 128 * 128 * (size_t)p.K16 * 16; }

template <int NT, int KC, int MODE>
inline int32_t launch_tc_gemm_kc(zant_ctx* ctx, const TcGemmArgs& k, int tiles) {
    using Cfg = TcGemmCfg<NT, KC, 8, MODE>;
    ZB_SMEM_ATTR(ctx, (tc_gemm_i8_kernel<NT, KC, 8, MODE>), Cfg::SMEM_BYTES);
    tc_gemm_i8_kernel<NT, KC, 8, MODE><<<std::min(tiles, ctx->sm_count), Cfg::THREADS, Cfg::SMEM_BYTES, ctx->stream>>>(k);
    return check_launch(ctx, "tc_gemm_i8_kernel");
}

template <int NT, int MODE>
inline int32_t launch_tc_gemm(zant_ctx* ctx, const TcGemmArgs& k, int tiles) {
    if (k.K16 == 2) return launch_tc_gemm_kc<NT, 2, MODE>(ctx, k, tiles);
    return launch_tc_gemm_kc<NT, 4, MODE>(ctx, k, tiles);
}

// im2col + GEMM on device buffers.  `a_blk` is scratch of qgemm_a_bytes(N*OH*OW) bytes.
inline int32_t run_qconv_tc(zant_ctx* ctx, const ConvGeom& g, const void* x, bool x_u8, int x_zp, const QGemmPrep& p,
                            const int8_t* w_blk_dev, const float* mult_dev, const int32_t* bias_dev, uint8_t* a_blk,
                            void* y, bool y_u8, const Requant& rq) {
    const long long M = (long long)g.N * g.OH * g.OW;
    if (M <= 0 || M > 0x7fffff00LL) return fail(ZANT_E_TOO_LARGE, "too many output positions for the tensor-core path");
    Im2colArgs ia{};
    ia.x = (const uint8_t*)x; ia.a = a_blk; ia.g = g; ia.K = p.K; ia.K16 = p.K16; ia.M = (int)M; ia.pad_value = x_zp;
    const bool pointwise = g.KH == 1 && g.KW == 1 && g.sh == 1 && g.sw == 1 && g.pt == 0 && g.pl == 0 && g.pb == 0 && g.pr == 0;
    const int m_tiles = (int)((M + 127) / 128);
    if (pointwise && (g.H * g.W) % 4 == 0 && (reinterpret_cast<uintptr_t>(x) & 3u) == 0 && m_tiles <= 0x7fffffff / 128 && (p.K16 + 3) / 4 <= 65535) {
        PwBlockArgs pa{};
        pa.x = (const uint8_t*)x; pa.a = a_blk; pa.C = g.C; pa.HW = g.H * g.W; pa.M = (int)M; pa.K16 = p.K16;
        pointwise_blocked_kernel<<<dim3((unsigned)m_tiles, (unsigned)((p.K16 + 3) / 4)), 256, 0, ctx->stream>>>(pa);
        ZB_TRY(check_launch(ctx, "pointwise_blocked_kernel"));
    } else if ((p.tap_major || (g.KH * g.KW == 1 && g.C % 16 == 0)) && (long long)g.KH * g.KW * ((g.C + 63) / 64) <= 65535) {
        // (with a single tap the two K orders are the same: 1x1 filters on planes that are not whole words come here)
        TapMajorArgs ta{};
        ta.x = (const uint8_t*)x; ta.a = a_blk; ta.g = g; ta.M = (int)M; ta.K16 = p.K16; ta.cgroups = (g.C + 63) / 64; ta.pad_value = x_zp;
        im2col_tapmajor_kernel<<<dim3((unsigned)m_tiles, (unsigned)(g.KH * g.KW * ta.cgroups)), 256, 0, ctx->stream>>>(ta);
        ZB_TRY(check_launch(ctx, "im2col_tapmajor_kernel"));
    } else {
        if (p.tap_major) return fail(ZANT_E_TOO_LARGE, "too many taps x channel groups for the tap-major gather");
        const size_t chunks = (size_t)m_tiles * p.K16 * 128;
        im2col_blocked_kernel<<<grid_for(chunks, 256, ctx->sm_count, 16), 256, 0, ctx->stream>>>(ia);
        ZB_TRY(check_launch(ctx, "im2col_blocked_kernel"));
    }
    TcGemmArgs k{};
    k.a = (const int8_t*)a_blk; k.w = w_blk_dev; k.mult = mult_dev; k.bias = bias_dev; k.y = (int8_t*)y;
    k.M = (int)M; k.N = p.N_pad; k.K16 = p.K16; k.y_scale = rq.y_scale; k.y_zp = rq.y_zp; k.act = rq.act; k.lut = rq.lut; k.status = ctx->status_word;
    k.n_valid = g.M; k.ohw = g.OH * g.OW; k.out_u8 = y_u8 ? 1 : 0;
    k.lean = (!y_u8 && rq.y_zp == 0 && p.mult_finite) ? 1 : 0;
    if (k.lean) {
        float v6 = 6.0f / rq.y_scale;
        v6 = std::fmin(std::fmax(v6, -512.0f), 511.0f);
        k.six = std::min(std::max((int)std::nearbyintf(v6), -128), 127);
    }
    const int tiles = (int)((M + 127) / 128) * (p.N_pad / p.NT);
    if (p.NT == 64) return x_u8 ? launch_tc_gemm<64, 3>(ctx, k, tiles) : launch_tc_gemm<64, 2>(ctx, k, tiles);
    if (p.NT == 128) return x_u8 ? launch_tc_gemm<128, 3>(ctx, k, tiles) : launch_tc_gemm<128, 2>(ctx, k, tiles);
    return x_u8 ? launch_tc_gemm<256, 3>(ctx, k, tiles) : launch_tc_gemm<256, 2>(ctx, k, tiles);
}

// Work is worth the tensor-core path when there is at least one full row tile and the operands fit.
inline bool qconv_tc_eligible(const ConvGeom& g, bool w_zp_all_zero) {
    const long long M = (long long)g.N * g.OH * g.OW;
    const long long K = (long long)g.Cg * g.KH * g.KW;
    return g.G == 1 && w_zp_all_zero && M >= 256 && g.M <= 2048 && K <= 65536 && (M + 127) / 128 * 128 * ((K + 63) / 64 * 64) <= (8LL << 30);
}

}  // namespace zb
