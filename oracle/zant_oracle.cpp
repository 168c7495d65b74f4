// zant_oracle.cpp — CPU restatement of Z-Ant's TensorMath inference operators.
//
// TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA backend is compared against
// and the timed CPU baseline of the benchmark.  Nothing in the product library includes,
// links or calls it.
//
// Pinning: the FP32 functions are pinned by the golden vectors of the reference's own unit
// tests (tests/golden/reference_goldens.json, each entry citing the Zig test it was read
// from).  The quantized functions have NO counterpart in the reference tree
// (src/Core/Quantization/quantization.zig is empty): for those, parity is UNPINNED — they
// restate the ONNX operator definitions with a fixed arithmetic order and are pinned only by
// hand-computed vectors (tests/golden/quant_goldens.json).
//
// Each function follows the Zig source cited above it step by step (same temporaries, same
// loop order, same order of floating-point operations).  Build with -ffp-contract=off so no
// multiply-add is fused: the reference performs a separate multiply and add.
//
// All paths are into the Z-Ant source tree.

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <string>
#include <vector>

#include "../include/zant_b200.h"

namespace {

using usize = size_t;

inline bool str_eq(const char* s, usize len, const char* lit) {
    return s != nullptr && std::strlen(lit) == len && std::memcmp(s, lit, len) == 0;
}

inline usize ceil_div(usize a, usize b) { return (a + b - 1) / b; }

inline usize prod(const usize* s, usize n) {
    usize p = 1;
    for (usize i = 0; i < n; ++i) p *= s[i];
    return p;
}

// lean_mat_mul, src/Core/Tensor/TensorMath/op_mat_mul.zig:92-172.
// Y[i,j] = ((0 + a_i0*b_0j) + a_i1*b_1j) + ...  (k ascending, separate multiply and add).
// The SIMD column groups of the reference compute the same per-element sequence.
void lean_mat_mul(const float* A, const float* B, float* Y, usize M, usize N, usize K) {
    for (usize i = 0; i < M; ++i) {
        const float* a = A + i * K;
        float* y = Y + i * N;
        for (usize j = 0; j < N; ++j) y[j] = 0.0f;
        for (usize k = 0; k < K; ++k) {
            const float av = a[k];
            const float* b = B + k * N;
            for (usize j = 0; j < N; ++j) {
                const float p = av * b[j];
                y[j] = y[j] + p;
            }
        }
    }
}

// lean_im2col, op_convolution.zig:424-514: row = (n,oh,ow), col = c*KH*KW + kh*KW + kw,
// value X[n,c,oh*s_h+kh*d_h, ow*s_w+kw*d_w]; taps outside the tensor are skipped (stay 0).
void lean_im2col(const float* X, usize N, usize C, usize H, usize W, usize KH, usize KW,
                 usize sh, usize sw, usize dh, usize dw, usize OH, usize OW, float* col) {
    const usize cols = C * KH * KW;
    for (usize row = 0; row < N * OH * OW; ++row) {
        const usize b = row / (OH * OW);
        const usize oh = (row % (OH * OW)) / OW;
        const usize ow = row % OW;
        for (usize c = 0; c < C; ++c) {
            const float* xc = X + (b * C + c) * H * W;
            float* out = col + row * cols + c * KH * KW;
            for (usize kh = 0; kh < KH; ++kh) {
                const usize h = oh * sh + kh * dh;
                if (h >= H) continue;
                for (usize kw = 0; kw < KW; ++kw) {
                    const usize w = ow * sw + kw * dw;
                    if (w >= W) continue;
                    out[kh * KW + kw] = xc[h * W + w];
                }
            }
        }
    }
}

struct ConvGeom {
    usize N, C, H, W, M, KH, KW;
    usize sh, sw, dh, dw;
    usize pt, pl, pb, pr;
    usize OH, OW;
};

// Pad / stride / dilation resolution of OnnxConvLean, op_convolution.zig:44-129.
int32_t conv_resolve(const usize* xs, usize xr, const usize* ws, usize wr,
                     const usize* stride, usize ns, const usize* pads, usize np,
                     const usize* dil, usize nd, usize group,
                     const char* auto_pad, usize apl, ConvGeom& g) {
    if (xr != 4 || wr != 4) return ZANT_E_INVALID_DIMENSIONS;
    if (group != 0 && group != 1) return ZANT_E_INVALID_DIMENSIONS;
    g.N = xs[0]; g.C = xs[1]; g.H = xs[2]; g.W = xs[3];
    g.M = ws[0]; g.KH = ws[2]; g.KW = ws[3];
    g.sh = ns > 0 ? stride[0] : 1;
    g.sw = ns > 1 ? stride[1] : (ns > 0 ? stride[0] : 1);
    g.dh = (dil && nd > 0) ? dil[0] : 1;
    g.dw = dil ? (nd > 1 ? dil[1] : (nd > 0 ? dil[0] : 1)) : 1;
    if (g.sh == 0 || g.sw == 0 || g.KH == 0 || g.KW == 0) return ZANT_E_INVALID_DIMENSIONS;
    const usize dkh = (g.KH - 1) * g.dh + 1;
    const usize dkw = (g.KW - 1) * g.dw + 1;
    g.pt = g.pl = g.pb = g.pr = 0;
    if (auto_pad) {
        if (str_eq(auto_pad, apl, "VALID")) {
        } else if (str_eq(auto_pad, apl, "SAME_UPPER") || str_eq(auto_pad, apl, "SAME_LOWER")) {
            const usize oh = ceil_div(g.H, g.sh), ow = ceil_div(g.W, g.sw);
            // The reference computes these in usize (op_convolution.zig:96-97); a negative
            // total would wrap there, so it is only defined when the total is >= 0.
            const long long th = (long long)((oh - 1) * g.sh + dkh) - (long long)g.H;
            const long long tw = (long long)((ow - 1) * g.sw + dkw) - (long long)g.W;
            if (th < 0 || tw < 0) return ZANT_E_INVALID_PADDING;
            if (str_eq(auto_pad, apl, "SAME_UPPER")) {
                g.pt = (usize)th / 2; g.pb = (usize)th - g.pt;
                g.pl = (usize)tw / 2; g.pr = (usize)tw - g.pl;
            } else {
                g.pb = (usize)th / 2; g.pt = (usize)th - g.pb;
                g.pr = (usize)tw / 2; g.pl = (usize)tw - g.pr;
            }
        } else if (str_eq(auto_pad, apl, "NOTSET")) {
            if (pads) {
                if (np >= 4) { g.pt = pads[0]; g.pl = pads[1]; g.pb = pads[2]; g.pr = pads[3]; }
            } else {
                return ZANT_E_INVALID_PADDING;
            }
        }
        // any other string: no padding (op_convolution.zig:126-128 never reaches its error)
    }
    const usize PH = g.H + g.pt + g.pb, PW = g.W + g.pl + g.pr;
    if (PH < dkh || PW < dkw) return ZANT_E_INVALID_DIMENSIONS;
    g.OH = (PH - dkh) / g.sh + 1;
    g.OW = (PW - dkw) / g.sw + 1;
    return ZANT_OK;
}

inline float rne_clamped(float v) {
    // rne(): nearest-even of v clamped to [-512, 511]; NaN maps to -512 (fmaxf drops the NaN).
    v = std::fmin(std::fmax(v, -512.0f), 511.0f);
    return std::nearbyintf(v);
}

inline int32_t sat_q(int32_t t, int32_t dtype) {
    const int32_t lo = dtype == ZANT_U8 ? 0 : -128;
    const int32_t hi = dtype == ZANT_U8 ? 255 : 127;
    return std::min(std::max(t, lo), hi);
}

inline int32_t load_q(const void* p, usize i, int32_t dtype) {
    if (dtype == ZANT_U8) return ((const uint8_t*)p)[i];
    if (dtype == ZANT_I8) return ((const int8_t*)p)[i];
    return ((const int32_t*)p)[i];
}

inline void store_q(void* p, usize i, int32_t dtype, int32_t v) {
    if (dtype == ZANT_U8) ((uint8_t*)p)[i] = (uint8_t)v;
    else ((int8_t*)p)[i] = (int8_t)v;
}

inline int32_t requant(int32_t acc, float M, int32_t y_zp, int32_t y_dtype, int32_t act,
                       float y_scale) {
    const float f = (float)acc;       // cvt.rn.f32.s32
    const float v = f * M;
    int32_t t = (int32_t)rne_clamped(v) + y_zp;
    t = sat_q(t, y_dtype);
    if (act == ZANT_QACT_RELU || act == ZANT_QACT_RELU6) t = std::max(t, sat_q(y_zp, y_dtype));
    if (act == ZANT_QACT_RELU6) {
        const int32_t six = sat_q((int32_t)rne_clamped(6.0f / y_scale) + y_zp, y_dtype);
        t = std::min(t, six);
    }
    return t;
}

struct PoolGeom { usize pt, pl, pb, pr; };

// Pad resolution of lean_onnx_maxpool, op_pooling.zig:587-618.
int32_t pool_resolve(const usize* xs, const usize* ys, const usize* k, const usize* s,
                     const usize* pads, usize np, int32_t auto_pad, PoolGeom& g) {
    g.pt = g.pl = g.pb = g.pr = 0;
    if (auto_pad == ZANT_PAD_NOTSET) {
        if (np >= 4) { g.pt = pads[0]; g.pl = pads[1]; g.pb = pads[2]; g.pr = pads[3]; }
    } else if (auto_pad == ZANT_PAD_VALID) {
    } else if (auto_pad == ZANT_PAD_SAME_UPPER || auto_pad == ZANT_PAD_SAME_LOWER) {
        const long long th = (long long)((ys[2] - 1) * s[0] + k[0]) - (long long)xs[2];
        const long long tw = (long long)((ys[3] - 1) * s[1] + k[1]) - (long long)xs[3];
        if (th < 0 || tw < 0) return ZANT_E_INVALID_PADDING;  // usize underflow in the reference
        if (auto_pad == ZANT_PAD_SAME_UPPER) {
            g.pt = (usize)th / 2; g.pl = (usize)tw / 2;
            g.pb = (usize)th - g.pt; g.pr = (usize)tw - g.pl;
        } else {
            g.pb = (usize)th / 2; g.pr = (usize)tw / 2;
            g.pt = (usize)th - g.pb; g.pl = (usize)tw - g.pr;
        }
    } else {
        return ZANT_E_INVALID_PADDING;
    }
    return ZANT_OK;
}

}  // namespace

extern "C" {

// ---------------------------------------------------------------------------------------
// Conv
// ---------------------------------------------------------------------------------------

// OnnxConv's expected output shape, op_convolution.zig:647-745 (the allocating wrapper the
// reference's tests call; it then runs OnnxConvLean into a tensor of this shape).
int32_t zo_conv_output_shape(const usize* xs, usize xr, const usize* ws, usize wr,
                             const usize* stride, usize ns, const usize* pads, usize np,
                             const usize* dil, usize nd, const char* auto_pad, usize apl,
                             usize out[4]) {
    if (xr != 4 || wr != 4) return ZANT_E_INVALID_DIMENSIONS;
    const usize H = xs[2], W = xs[3];
    const usize sh = ns > 0 ? stride[0] : 1;
    const usize sw = ns > 1 ? stride[1] : (ns > 0 ? stride[0] : 1);
    const usize dh = (dil && nd > 0) ? dil[0] : 1;
    const usize dw = dil ? (nd > 1 ? dil[1] : (nd > 0 ? dil[0] : 1)) : 1;
    if (sh == 0 || sw == 0 || ws[2] == 0 || ws[3] == 0) return ZANT_E_INVALID_DIMENSIONS;
    const usize dkh = (ws[2] - 1) * dh + 1, dkw = (ws[3] - 1) * dw + 1;
    usize oh, ow;
    if (auto_pad) {
        if (str_eq(auto_pad, apl, "VALID")) {
            if (H < dkh || W < dkw) return ZANT_E_INVALID_DIMENSIONS;
            oh = (H - dkh) / sh + 1; ow = (W - dkw) / sw + 1;
        } else if (str_eq(auto_pad, apl, "SAME_UPPER") || str_eq(auto_pad, apl, "SAME_LOWER")) {
            oh = ceil_div(H, sh); ow = ceil_div(W, sw);
        } else if (str_eq(auto_pad, apl, "NOTSET")) {
            if (pads) {
                if (np < 4) return ZANT_E_INVALID_PADDING;
                if (H + pads[0] + pads[2] < dkh || W + pads[1] + pads[3] < dkw) return ZANT_E_INVALID_DIMENSIONS;
                oh = (H + pads[0] + pads[2] - dkh) / sh + 1;
                ow = (W + pads[1] + pads[3] - dkw) / sw + 1;
            } else {
                if (H < dkh || W < dkw) return ZANT_E_INVALID_DIMENSIONS;
                oh = (H - dkh) / sh + 1; ow = (W - dkw) / sw + 1;
            }
        } else {
            return ZANT_E_INVALID_PADDING;
        }
    } else {
        const usize tph = (pads && np >= 4) ? pads[0] + pads[2] : 0;
        const usize tpw = (pads && np >= 4) ? pads[1] + pads[3] : 0;
        if (H + tph < dkh || W + tpw < dkw) return ZANT_E_INVALID_DIMENSIONS;
        oh = (H + tph - dkh) / sh + 1;
        ow = (W + tpw - dkw) / sw + 1;
    }
    out[0] = xs[0]; out[1] = ws[0]; out[2] = oh; out[3] = ow;
    return ZANT_OK;
}

// OnnxConvLean, op_convolution.zig:42-219, calling convolve_tensor_with_bias :228-331:
// zero-padded copy -> im2col -> kernel matrix [C*KH*KW, M] -> mat_mul -> scatter + bias.
int32_t zo_conv_f32(const float* x, const usize* xs, usize xr,
                    const float* w, const usize* ws, usize wr,
                    const float* bias, usize bias_len,
                    float* y, const usize* ys, usize yr,
                    const usize* stride, usize ns, const usize* pads, usize np,
                    const usize* dil, usize nd, usize group,
                    const char* auto_pad, usize apl) {
    (void)bias_len;
    ConvGeom g;
    int32_t st = conv_resolve(xs, xr, ws, wr, stride, ns, pads, np, dil, nd, group, auto_pad, apl, g);
    if (st != ZANT_OK) return st;
    if (yr != 4) return ZANT_E_INVALID_DIMENSIONS;
    // padded input, op_convolution.zig:134-164
    const usize PH = g.H + g.pt + g.pb, PW = g.W + g.pl + g.pr;
    std::vector<float> xp(g.N * g.C * PH * PW, 0.0f);
    for (usize b = 0; b < g.N; ++b)
        for (usize c = 0; c < g.C; ++c)
            for (usize h = 0; h < g.H; ++h)
                for (usize ww = 0; ww < g.W; ++ww)
                    xp[((b * g.C + c) * PH + h + g.pt) * PW + ww + g.pl] = x[((b * g.C + c) * g.H + h) * g.W + ww];
    // convolve_tensor_with_bias
    const usize K = ws[1] * g.KH * g.KW;  // kernel elements per filter (kernel.shape[1..3])
    const usize rows = g.N * g.OH * g.OW;
    std::vector<float> col(rows * (g.C * g.KH * g.KW), 0.0f);
    lean_im2col(xp.data(), g.N, g.C, PH, PW, g.KH, g.KW, g.sh, g.sw, g.dh, g.dw, g.OH, g.OW, col.data());
    if (K != g.C * g.KH * g.KW) return ZANT_E_INPUT_TENSORS_WRONG_SHAPE;  // mat_mul's shape check
    std::vector<float> km(K * g.M);
    for (usize f = 0; f < g.M; ++f)
        for (usize i = 0; i < K; ++i) km[i * g.M + f] = w[f * K + i];
    std::vector<float> res(rows * g.M);
    lean_mat_mul(col.data(), km.data(), res.data(), rows, g.M, K);
    // result shape must equal the output shape, op_convolution.zig:212-217
    if (ys[0] != g.N || ys[1] != g.M || ys[2] != g.OH || ys[3] != g.OW) return ZANT_E_INVALID_DIMENSIONS;
    usize idx = 0;
    for (usize b = 0; b < g.N; ++b)
        for (usize h = 0; h < g.OH; ++h)
            for (usize ww = 0; ww < g.OW; ++ww) {
                for (usize f = 0; f < g.M; ++f) {
                    const float bv = bias ? bias[f] : 0.0f;
                    y[((b * g.M + f) * g.OH + h) * g.OW + ww] = res[idx * g.M + f] + bv;
                }
                ++idx;
            }
    return ZANT_OK;
}

// ---------------------------------------------------------------------------------------
// MatMul / Gemm
// ---------------------------------------------------------------------------------------

// mat_mul checks (op_mat_mul.zig:22-57) then lean_mat_mul (:92-172) on the last two dims.
int32_t zo_mat_mul_f32(const float* a, const usize* as, usize ar,
                       const float* b, const usize* bs, usize br,
                       float* y, const usize* ys, usize yr) {
    if (ar != br) return ZANT_E_INPUT_TENSOR_DIFFERENT_SHAPE;
    if (ar < 2) return ZANT_E_INPUT_TENSORS_WRONG_SHAPE;
    if (as[ar - 1] != bs[ar - 2]) return ZANT_E_INPUT_TENSORS_WRONG_SHAPE;
    const usize M = as[ar - 2], N = bs[ar - 1], K = as[ar - 1];
    if (M * N == 0 || K == 0) return ZANT_E_INPUT_TENSORS_WRONG_SHAPE;
    if (yr < 2 || ys[yr - 2] != M || ys[yr - 1] != N) return ZANT_E_OUTPUT_TENSOR_DIFFERENT_SIZE;
    lean_mat_mul(a, b, y, M, N, K);
    return ZANT_OK;
}

// gemm checks (op_gemm.zig:15-61) then lean_gemm (:91-185).
int32_t zo_gemm_f32(const float* a, const usize* as, usize ar,
                    const float* b, const usize* bs, usize br,
                    const float* c, const usize* cs, usize cr,
                    float alpha, float beta, int32_t ta, int32_t tb,
                    float* y, const usize* ys, usize yr) {
    if (ar != 4 || br != 4) return ZANT_E_INPUT_TENSORS_WRONG_SHAPE;
    if (as[0] != bs[0] || as[1] != bs[1]) return ZANT_E_INPUT_TENSOR_DIFFERENT_SHAPE;
    const usize condA = ta ? as[2] : as[3], rows = ta ? as[3] : as[2];
    const usize condB = tb ? bs[3] : bs[2], cols = tb ? bs[2] : bs[3];
    if (condA != condB) return ZANT_E_INPUT_TENSOR_DIMENSION_MISMATCH;
    if (c) {
        if (cr != 4) return ZANT_E_INPUT_TENSORS_WRONG_SHAPE;
        if (cs[0] != as[0] || cs[1] != as[1]) return ZANT_E_INPUT_TENSOR_DIFFERENT_SHAPE;
        if ((cs[2] != rows && cs[2] != 1) || (cs[3] != cols && cs[3] != 1)) return ZANT_E_INCOMPATIBLE_BROADCAST_SHAPES;
    }
    if (yr != 4 || ys[2] != rows || ys[3] != cols) return ZANT_E_OUTPUT_TENSOR_DIFFERENT_SIZE;
    const usize K = condA;
    // transposeLastTwo copies (op_gemm.zig:111-124); only the first [rows x K] matrix of the
    // tensor takes part in lean_mat_mul.
    std::vector<float> at, bt;
    const float* A = a;
    const float* B = b;
    if (ta) {
        at.resize(rows * K);
        for (usize i = 0; i < K; ++i) for (usize j = 0; j < rows; ++j) at[j * K + i] = a[i * rows + j];
        A = at.data();
    }
    if (tb) {
        bt.resize(K * cols);
        for (usize i = 0; i < cols; ++i) for (usize j = 0; j < K; ++j) bt[j * cols + i] = b[i * K + j];
        B = bt.data();
    }
    lean_mat_mul(A, B, y, rows, cols, K);
    const usize ysize = prod(ys, 4);
    for (usize i = 0; i < ysize; ++i) y[i] = y[i] * alpha;   // op_gemm.zig:130-132 (whole tensor)
    if (c && beta != 0.0f) {
        const usize csize = prod(cs, 4);
        if (ysize == csize) {
            for (usize i = 0; i < ysize; ++i) { const float t = c[i] * beta; y[i] = y[i] + t; }
        } else {
            const usize crows = cs[2], ccols = cs[3];
            for (usize bb = 0; bb < as[0]; ++bb)
                for (usize ch = 0; ch < as[1]; ++ch)
                    for (usize i = 0; i < rows; ++i)
                        for (usize j = 0; j < cols; ++j) {
                            const usize ci = crows == 1 ? 0 : i, cj = ccols == 1 ? 0 : j;
                            const usize ri = (((bb * ys[1]) + ch) * ys[2] + i) * ys[3] + j;
                            const usize cidx = (((bb * cs[1]) + ch) * cs[2] + ci) * cs[3] + cj;
                            const float t = c[cidx] * beta;
                            y[ri] = y[ri] + t;
                        }
        }
    }
    return ZANT_OK;
}

// ---------------------------------------------------------------------------------------
// Pooling
// ---------------------------------------------------------------------------------------

// get_pooling_output_shape, op_pooling.zig:16-35.
int32_t zo_pooling_output_shape(const usize* xs, usize xr, const usize k[2], const usize s[2], usize out[4]) {
    if (xr != 4) return ZANT_E_INVALID_DIMENSIONS;
    if (k[0] == 0 || k[1] == 0 || s[0] == 0 || s[1] == 0) return ZANT_E_WRONG_STRIDE;
    if (k[0] > xs[2] || k[1] > xs[3]) return ZANT_E_INVALID_DIMENSIONS;
    out[0] = xs[0]; out[1] = xs[1];
    out[2] = (xs[2] - k[0]) / s[0] + 1;
    out[3] = (xs[3] - k[1]) / s[1] + 1;
    return ZANT_OK;
}

// get_onnx_maxpool_output_shape, op_pooling.zig:477-567.
int32_t zo_maxpool_output_shape(const usize* xs, usize xr, const usize* k, const usize* s,
                                const usize* d, const usize* pads, int32_t auto_pad,
                                int32_t ceil_mode, usize out[4]) {
    if (xr != 4) return ZANT_E_INVALID_DIMENSIONS;
    if (s[0] == 0 || s[1] == 0 || k[0] == 0 || k[1] == 0) return ZANT_E_WRONG_STRIDE;
    const usize H = xs[2], W = xs[3];
    const usize ekh = (k[0] - 1) * d[0] + 1, ekw = (k[1] - 1) * d[1] + 1;
    long long ph = 0, pw = 0;
    if (auto_pad == ZANT_PAD_NOTSET) {
        ph = (long long)(pads[0] + pads[2]); pw = (long long)(pads[1] + pads[3]);
    } else if (auto_pad == ZANT_PAD_VALID) {
    } else if (auto_pad == ZANT_PAD_SAME_UPPER || auto_pad == ZANT_PAD_SAME_LOWER) {
        const usize oh = (H + s[0] - 1) / s[0], ow = (W + s[1] - 1) / s[1];
        ph = (long long)((oh - 1) * s[0] + ekh) - (long long)H;
        pw = (long long)((ow - 1) * s[1] + ekw) - (long long)W;
        if (ph < 0 || pw < 0) return ZANT_E_INVALID_PADDING;
    } else {
        return ZANT_E_INVALID_PADDING;
    }
    if ((long long)H + ph < (long long)ekh || (long long)W + pw < (long long)ekw) return ZANT_E_INVALID_DIMENSIONS;
    const usize nh = (usize)((long long)H + ph) - ekh, nw = (usize)((long long)W + pw) - ekw;
    out[0] = xs[0]; out[1] = xs[1];
    if (ceil_mode) {
        out[2] = (nh + s[0] - 1) / s[0] + 1; out[3] = (nw + s[1] - 1) / s[1] + 1;
    } else {
        out[2] = nh / s[0] + 1; out[3] = nw / s[1] + 1;
    }
    return ZANT_OK;
}

// lean_onnx_maxpool, op_pooling.zig:570-659.
int32_t zo_maxpool_f32(const float* x, const usize* xs, usize xr, float* y, const usize* ys, usize yr,
                       const usize* k, usize nk, const usize* s, usize nst, const usize* d, usize nd,
                       const usize* pads, usize np, int32_t auto_pad) {
    if (xr != 4 || yr != 4 || nk < 2 || nst < 2 || nd < 2) return ZANT_E_INVALID_DIMENSIONS;
    PoolGeom g;
    int32_t st = pool_resolve(xs, ys, k, s, pads, np, auto_pad, g);
    if (st != ZANT_OK) return st;
    const usize N = xs[0], C = xs[1], H = xs[2], W = xs[3], OH = ys[2], OW = ys[3];
    for (usize b = 0; b < N; ++b)
        for (usize c = 0; c < C; ++c) {
            const float* xi = x + (b * C + c) * H * W;
            float* yo = y + (b * C + c) * OH * OW;
            for (usize oh = 0; oh < OH; ++oh)
                for (usize ow = 0; ow < OW; ++ow) {
                    const long long ih0 = (long long)(oh * s[0]) - (long long)g.pt;
                    const long long iw0 = (long long)(ow * s[1]) - (long long)g.pl;
                    float m = -std::numeric_limits<float>::infinity();
                    for (usize kh = 0; kh < k[0]; ++kh)
                        for (usize kw = 0; kw < k[1]; ++kw) {
                            const long long ih = ih0 + (long long)(kh * d[0]);
                            const long long iw = iw0 + (long long)(kw * d[1]);
                            if (ih >= 0 && ih < (long long)H && iw >= 0 && iw < (long long)W) {
                                const float v = xi[(usize)ih * W + (usize)iw];
                                m = (v > m) ? v : m;   // @max; inputs are never NaN in the tests
                            }
                        }
                    yo[oh * OW + ow] = m;
                }
        }
    return ZANT_OK;
}

// The same window walk on raw int8/uint8 codes (no reference counterpart: the reference's
// -inf initial value does not exist for integers; the type minimum takes its place).
int32_t zo_maxpool_q8(int32_t dtype, const void* x, const usize* xs, usize xr, void* y, const usize* ys, usize yr,
                      const usize* k, usize nk, const usize* s, usize nst, const usize* d, usize nd,
                      const usize* pads, usize np, int32_t auto_pad) {
    if (xr != 4 || yr != 4 || nk < 2 || nst < 2 || nd < 2) return ZANT_E_INVALID_DIMENSIONS;
    PoolGeom g;
    int32_t st = pool_resolve(xs, ys, k, s, pads, np, auto_pad, g);
    if (st != ZANT_OK) return st;
    const usize N = xs[0], C = xs[1], H = xs[2], W = xs[3], OH = ys[2], OW = ys[3];
    for (usize bc = 0; bc < N * C; ++bc)
        for (usize oh = 0; oh < OH; ++oh)
            for (usize ow = 0; ow < OW; ++ow) {
                int32_t m = dtype == ZANT_U8 ? 0 : -128;
                for (usize kh = 0; kh < k[0]; ++kh)
                    for (usize kw = 0; kw < k[1]; ++kw) {
                        const long long ih = (long long)(oh * s[0]) - (long long)g.pt + (long long)(kh * d[0]);
                        const long long iw = (long long)(ow * s[1]) - (long long)g.pl + (long long)(kw * d[1]);
                        if (ih >= 0 && ih < (long long)H && iw >= 0 && iw < (long long)W)
                            m = std::max(m, load_q(x, bc * H * W + (usize)ih * W + (usize)iw, dtype));
                    }
                store_q(y, bc * OH * OW + oh * OW + ow, dtype, m);
            }
    return ZANT_OK;
}

// ---------------------------------------------------------------------------------------
// Activations
// ---------------------------------------------------------------------------------------

// lean_ReLU, lib_activation_function_math.zig:22-28: writes ONLY where x > 0.  With
// `zero_first` the output is cleared before, which is what ReLU_standard (:14-20, fromShape
// zero-fills) and the generated predict() (resetOutputTensors) arrange.
int32_t zo_relu_f32(const float* x, float* y, usize n, int32_t zero_first) {
    if (zero_first) std::memset(y, 0, n * sizeof(float));
    for (usize i = 0; i < n; ++i)
        if (x[i] > 0) y[i] = x[i];
    return ZANT_OK;
}

// lean_leakyReLU, lib_activation_function_math.zig:68-77.
int32_t zo_leaky_relu_f32(const float* x, float slope, float* y, usize n) {
    for (usize i = 0; i < n; ++i) y[i] = (x[i] <= 0) ? slope * x[i] : x[i];
    return ZANT_OK;
}

// ONNX Clip; not in the reference.
int32_t zo_clip_f32(const float* x, float lo, float hi, float* y, usize n) {
    for (usize i = 0; i < n; ++i) y[i] = std::fmin(std::fmax(x[i], lo), hi);
    return ZANT_OK;
}

// sigmoid_lean, lib_activation_function_math.zig:107-122: 1 / (1 + exp(-x)) element by element.
int32_t zo_sigmoid_f32(const float* x, float* y, usize n) {
    for (usize i = 0; i < n; ++i) y[i] = 1.0f / (1.0f + std::exp(-x[i]));
    return ZANT_OK;
}

// lean_softmax, lib_activation_function_math.zig:154-187: rows of a 2-D tensor; row maximum, exp(x - max)
// stored and summed in index order, then every entry divided by the sum.
int32_t zo_softmax_f32(const float* x, float* y, usize rows, usize cols) {
    for (usize i = 0; i < rows; ++i) {
        if (cols == 0) continue;
        float max_val = x[i * cols];
        for (usize j = 0; j < cols; ++j) { const float v = x[i * cols + j]; if (v > max_val) max_val = v; }
        float sum = 0.0f;
        for (usize j = 0; j < cols; ++j) { const float v = std::exp(x[i * cols + j] - max_val); y[i * cols + j] = v; sum += v; }
        for (usize j = 0; j < cols; ++j) y[i * cols + j] /= sum;
    }
    return ZANT_OK;
}

// tanh_lean, lib_elementWise_math.zig:452-456.
int32_t zo_tanh_f32(const float* x, float* y, usize n) {
    for (usize i = 0; i < n; ++i) y[i] = std::tanh(x[i]);
    return ZANT_OK;
}

// ceil_lean, lib_elementWise_math.zig:471-480: NaN and infinities pass through.
int32_t zo_ceil_f32(const float* x, float* y, usize n) {
    for (usize i = 0; i < n; ++i) y[i] = (std::isnan(x[i]) || std::isinf(x[i])) ? x[i] : std::ceil(x[i]);
    return ZANT_OK;
}

// ---------------------------------------------------------------------------------------
// Transpose / Slice / Gather (lib_shape_math.zig): elements are moved, never interpreted, so the
// functions take the element size in bytes.
// ---------------------------------------------------------------------------------------

// transpose_onnx_lean, lib_shape_math.zig:1628-1753: the output index is decomposed by the output strides and
// coordinate d walks input dimension perm[d]; a missing perm reverses the dimensions.
int32_t zo_transpose_onnx(usize esz, const void* x, const usize* xs, usize xr, const usize* perm, usize np, void* y, const usize* ys, usize yr) {
    if (yr != xr) return ZANT_E_INVALID_RANK;
    std::vector<usize> rp(xr);
    if (perm) {
        if (np != xr) return ZANT_E_INVALID_PERMUTATION;
        std::vector<bool> used(xr, false);
        for (usize i = 0; i < xr; ++i) {
            if (perm[i] >= xr || used[perm[i]]) return ZANT_E_INVALID_PERMUTATION;
            used[perm[i]] = true;
            rp[i] = perm[i];
        }
    } else {
        for (usize i = 0; i < xr; ++i) rp[i] = xr - 1 - i;
    }
    std::vector<usize> istr(xr), oshape(xr), ostr(xr);
    usize st = 1;
    for (usize i = xr; i-- > 0;) { istr[i] = st; st *= xs[i]; }
    for (usize j = 0; j < xr; ++j) oshape[j] = xs[rp[j]];
    st = 1;
    for (usize i = xr; i-- > 0;) { ostr[i] = st; st *= oshape[i]; }
    for (usize j = 0; j < xr; ++j) if (ys[j] != oshape[j]) return ZANT_E_OUTPUT_TENSOR_DIFFERENT_SIZE;
    const usize total = st;
    for (usize flat = 0; flat < total; ++flat) {
        usize tmp = flat, in_idx = 0;
        for (usize d = 0; d < xr; ++d) { const usize c = tmp / ostr[d]; tmp %= ostr[d]; in_idx += c * istr[rp[d]]; }
        std::memcpy((char*)y + flat * esz, (const char*)x + in_idx * esz, esz);
    }
    return ZANT_OK;
}

// The start / end / step normalisation shared by get_slice_output_shape and lean_slice_onnx
// (lib_shape_math.zig:1378-1443).
// `shape_rule`: count the elements of a negative step as get_slice_output_shape does (:1546-1550:
// (start - end) / |step| + 1) instead of as lean_slice_onnx does (:1452-1456).
static int32_t slice_normalise(const usize* xs, usize xr, const int64_t* starts, const int64_t* ends, usize n, const int64_t* axes,
                               const int64_t* steps, std::vector<int64_t>& a_start, std::vector<int64_t>& a_step, std::vector<usize>& odims,
                               bool shape_rule) {
    a_start.assign(xr, 0); a_step.assign(xr, 1); odims.assign(xr, 0);
    std::vector<int64_t> a_end(xr);
    for (usize i = 0; i < xr; ++i) a_end[i] = (int64_t)xs[i];
    for (usize i = 0; i < n; ++i) {
        const int64_t axis = axes ? axes[i] : (int64_t)i;
        const int64_t ax = axis < 0 ? axis + (int64_t)xr : axis;
        if (ax < 0 || (usize)ax >= xr) return ZANT_E_INVALID_SLICE_INDICES;
        const int64_t dim = (int64_t)xs[ax];
        int64_t s0 = starts[i] < 0 ? starts[i] + dim : starts[i];
        s0 = std::max<int64_t>(0, std::min(s0, dim));
        a_start[ax] = s0;
        int64_t e0 = ends[i] < 0 ? ends[i] + dim : ends[i];
        if (steps && steps[i] < 0) e0 = ends[i] < 0 ? -1 : e0;
        else e0 = std::max<int64_t>(0, std::min(e0, dim));
        a_end[ax] = e0;
        if (steps) {
            if (steps[i] == 0) return ZANT_E_INVALID_SLICE_STEP;
            a_step[ax] = steps[i];
        }
    }
    for (usize i = 0; i < xr; ++i) {
        const int64_t st = a_start[i], en = a_end[i], sp = a_step[i];
        usize d = 0;
        if (sp > 0) { if (en > st) d = (usize)(((en - st) + sp - 1) / sp); }
        else if (st > en) {
            const int64_t as = -sp;
            if (shape_rule) d = (usize)((st - en) / as + 1);
            else { const int64_t range = st - (en + 1); d = (usize)((range + as - 1) / as); }
        }
        odims[i] = d;
    }
    return ZANT_OK;
}

// get_slice_output_shape (shape_rule != 0), or the dimensions lean_slice_onnx writes into its output.
int32_t zo_slice_output_shape(const usize* xs, usize xr, const int64_t* starts, const int64_t* ends, usize n, const int64_t* axes,
                              const int64_t* steps, usize* out, int32_t shape_rule) {
    std::vector<int64_t> a, b; std::vector<usize> od;
    const int32_t st = slice_normalise(xs, xr, starts, ends, n, axes, steps, a, b, od, shape_rule != 0);
    if (st != ZANT_OK) return st;
    for (usize i = 0; i < xr; ++i) out[i] = od[i];
    return ZANT_OK;
}

// lean_slice_onnx, lib_shape_math.zig:1445-1495: output coordinates (last dimension fastest) map to
// start + coord * step in every dimension.
int32_t zo_slice_onnx(usize esz, const void* x, const usize* xs, usize xr, const int64_t* starts, const int64_t* ends, usize n,
                      const int64_t* axes, const int64_t* steps, void* y, const usize* ys, usize yr) {
    std::vector<int64_t> a_start, a_step; std::vector<usize> od;
    const int32_t st = slice_normalise(xs, xr, starts, ends, n, axes, steps, a_start, a_step, od, false);
    if (st != ZANT_OK) return st;
    if (yr != xr) return ZANT_E_OUTPUT_TENSOR_DIFFERENT_SIZE;
    usize total = 1;
    for (usize i = 0; i < xr; ++i) { if (ys[i] != od[i]) return ZANT_E_OUTPUT_TENSOR_DIFFERENT_SIZE; total *= od[i]; }
    std::vector<usize> istr(xr);
    usize s = 1;
    for (usize i = xr; i-- > 0;) { istr[i] = s; s *= xs[i]; }
    for (usize o = 0; o < total; ++o) {
        usize tmp = o, in_idx = 0;
        for (usize i = 0; i < xr; ++i) {
            const usize d = xr - 1 - i;
            const usize c = tmp % od[d]; tmp /= od[d];
            in_idx += (usize)(a_start[d] + (int64_t)c * a_step[d]) * istr[d];
        }
        std::memcpy((char*)y + o * esz, (const char*)x + in_idx * esz, esz);
    }
    return ZANT_OK;
}

// gather + lean_gather, lib_shape_math.zig:1217-1330.
int32_t zo_gather(usize esz, const void* x, const usize* xs, usize xr, const usize* indices, const usize* is, usize ir, int64_t axis_in,
                  void* y, const usize* ys, usize yr) {
    if (xr == 0) return ZANT_E_INVALID_RANK;
    const int64_t nd = (int64_t)xr;
    if (axis_in >= nd || axis_in < -nd) return ZANT_E_INVALID_AXIS;
    const usize axis = (usize)(axis_in < 0 ? nd + axis_in : axis_in);
    usize n_idx = 1;
    for (usize i = 0; i < ir; ++i) n_idx *= is[i];
    for (usize i = 0; i < n_idx; ++i) if (indices[i] >= xs[axis]) return ZANT_E_INDEX_OUT_OF_BOUNDS;
    if (yr != xr + ir - 1) return ZANT_E_OUTPUT_TENSOR_DIFFERENT_SIZE;
    for (usize i = 0; i < axis; ++i) if (ys[i] != xs[i]) return ZANT_E_OUTPUT_TENSOR_DIFFERENT_SIZE;
    for (usize i = 0; i < ir; ++i) if (ys[axis + i] != is[i]) return ZANT_E_OUTPUT_TENSOR_DIFFERENT_SIZE;
    for (usize i = axis + 1; i < xr; ++i) if (ys[axis + ir + (i - axis - 1)] != xs[i]) return ZANT_E_OUTPUT_TENSOR_DIFFERENT_SIZE;
    usize outer = 1, inner = 1;
    for (usize i = 0; i < axis; ++i) outer *= xs[i];
    for (usize i = axis + 1; i < xr; ++i) inner *= xs[i];
    for (usize o = 0; o < outer; ++o)
        for (usize k = 0; k < n_idx; ++k)
            std::memcpy((char*)y + ((o * n_idx + k) * inner) * esz, (const char*)x + ((o * xs[axis] + indices[k]) * inner) * esz, inner * esz);
    return ZANT_OK;
}

// get_unsqueeze_output_shape, lib_shape_math.zig:1983-2030: axes refer to the OUTPUT rank; negative axes
// count from its end; out of range -> AxisOutOfBounds, repeated -> DuplicateAxis.
int32_t zo_unsqueeze_output_shape(const usize* xs, usize xr, const int64_t* axes, usize na, usize* out) {
    const usize orank = xr + na;
    std::vector<bool> is_new(orank, false);
    std::vector<usize> seen;
    for (usize i = 0; i < na; ++i) {
        int64_t a = axes[i];
        if (a < 0) a += (int64_t)orank;
        if (a < 0 || a >= (int64_t)orank) return ZANT_E_AXIS_OUT_OF_BOUNDS;
        for (usize j : seen) if (j == (usize)a) return ZANT_E_DUPLICATE_AXIS;
        seen.push_back((usize)a);
        is_new[(usize)a] = true;
    }
    usize k = 0;
    for (usize i = 0; i < orank; ++i) out[i] = is_new[i] ? 1 : xs[k++];
    return ZANT_OK;
}

// get_shape_output_shape (:1903-1931) gives the length; lean_shape_onnx (:1869-1901) the values.  The
// latter clamps the start to rank - 1 (the former to rank); both are restated as they are.
int32_t zo_shape_onnx(const usize* xs, usize xr, int32_t has_start, int64_t start, int32_t has_end, int64_t end, int64_t* out, usize* out_len) {
    if (xr == 0) { *out_len = 0; return ZANT_OK; }
    const int64_t r = (int64_t)xr;
    int64_t s0 = has_start ? start : 0; if (s0 < 0) s0 += r;
    int64_t e0 = has_end ? end : r; if (e0 < 0) e0 += r;
    const int64_t s_len = std::max<int64_t>(0, std::min(s0, r));
    const int64_t e_len = std::max(s_len, std::min(e0, r));
    *out_len = (usize)std::max<int64_t>(0, e_len - s_len);
    const int64_t s_val = std::max<int64_t>(0, std::min(s0, r - 1));
    const int64_t e_val = std::max(s_val, std::min(e0, r));
    if ((usize)std::max<int64_t>(0, e_val - s_val) != *out_len) return ZANT_E_MISMATCHED_SHAPE;   // the reference's ShapeMismatch
    for (usize i = 0; i < *out_len; ++i) out[i] = (int64_t)xs[(usize)s_val + i];
    return ZANT_OK;
}

// ---------------------------------------------------------------------------------------
// Element-wise
// ---------------------------------------------------------------------------------------

// mul_lean / div_lean, lib_elementWise_math.zig:404-408 and 422-426; the callers mul / div reject
// operands of different sizes with MismatchedShape (:393-395, :411-413).
int32_t zo_mul_f32(const float* a, usize na, const float* b, usize nb, float* y) {
    if (na != nb) return ZANT_E_MISMATCHED_SHAPE;
    for (usize i = 0; i < na; ++i) y[i] = a[i] * b[i];
    return ZANT_OK;
}
int32_t zo_div_f32(const float* a, usize na, const float* b, usize nb, float* y) {
    if (na != nb) return ZANT_E_MISMATCHED_SHAPE;
    for (usize i = 0; i < na; ++i) y[i] = a[i] / b[i];
    return ZANT_OK;
}

// lean_sum_tensors, lib_elementWise_math.zig:70-210.
// The broadcasting branch of the reference derives BOTH operands' strides from the OUTPUT
// shape (:160-169).  For an operand whose non-1 dims are followed by a broadcast dim
// (e.g. [C,1,1] against [N,C,H,W]) that index runs past the operand's buffer — the reference
// reads out of bounds there.  `*ref_oob` is set to 1 when that happens; the value returned in
// y is then the NumPy-broadcast result (the behaviour ONNX Add defines), and 0 means y is
// exactly what the reference computes.
int32_t zo_sum_tensors_f32(const float* a, const usize* as, usize ar,
                           const float* b, const usize* bs, usize br,
                           float* y, const usize* ys, usize yr, int32_t* ref_oob) {
    if (ref_oob) *ref_oob = 0;
    const usize asz = prod(as, ar), bsz = prod(bs, br);
    if (asz == bsz) {
        for (usize i = 0; i < asz; ++i) y[i] = a[i] + b[i];
        return ZANT_OK;
    }
    const usize mr = std::max(ar, br);
    if (mr > 4) return ZANT_E_UNSUPPORTED;  // the reference frees its index arrays early above rank 4
    usize s1[4] = {1, 1, 1, 1}, s2[4] = {1, 1, 1, 1}, so[4] = {1, 1, 1, 1};
    for (usize i = 0; i < ar; ++i) s1[mr - ar + i] = as[i];
    for (usize i = 0; i < br; ++i) s2[mr - br + i] = bs[i];
    for (usize d = 0; d < mr; ++d) {
        if (s1[d] != s2[d] && s1[d] != 1 && s2[d] != 1) return ZANT_E_INCOMPATIBLE_BROADCAST_SHAPES;
        so[d] = std::max(s1[d], s2[d]);
    }
    if (yr != mr) return ZANT_E_OUTPUT_TENSOR_DIFFERENT_SIZE;
    for (usize d = 0; d < mr; ++d) if (ys[d] != so[d]) return ZANT_E_OUTPUT_TENSOR_DIFFERENT_SIZE;
    usize ostr[4], rstr1[4], rstr2[4], tstr1[4], tstr2[4];
    usize st = 1, t1 = 1, t2 = 1;
    for (usize i = mr; i-- > 0;) {
        ostr[i] = st;
        rstr1[i] = s1[i] > 1 ? st : 0;   // reference strides (from the output shape)
        rstr2[i] = s2[i] > 1 ? st : 0;
        tstr1[i] = s1[i] > 1 ? t1 : 0;   // true strides of each operand
        tstr2[i] = s2[i] > 1 ? t2 : 0;
        st *= so[i]; t1 *= s1[i]; t2 *= s2[i];
    }
    const usize osz = st;
    for (usize i = 0; i < osz; ++i) {
        usize rem = i, r1 = 0, r2 = 0, i1 = 0, i2 = 0;
        for (usize d = 0; d < mr; ++d) {
            const usize pos = rem / ostr[d];
            rem %= ostr[d];
            r1 += pos * rstr1[d]; r2 += (s2[d] > 1 ? pos % s2[d] : 0) * rstr2[d];
            i1 += pos * tstr1[d]; i2 += pos * tstr2[d];
        }
        if ((r1 != i1 || r2 != i2) && ref_oob) {
            if (r1 >= asz || r2 >= bsz) *ref_oob = 1;
            else if (a[r1] + b[r2] != a[i1] + b[i2]) *ref_oob = 2;  // in bounds but a different element
        }
        y[i] = a[i1] + b[i2];
    }
    return ZANT_OK;
}

// lean_sum_tensor_list, lib_elementWise_math.zig:243-257 (+ the checks of sum_tensor_list :213-241).
int32_t zo_sum_tensor_list_f32(const float* const* ts, usize nt, float* y, usize n) {
    if (nt == 0) return ZANT_E_EMPTY_TENSOR_LIST;
    for (usize i = 0; i < n; ++i) y[i] = ts[0][i];
    for (usize t = 1; t < nt; ++t)
        for (usize i = 0; i < n; ++i) y[i] = y[i] + ts[t][i];
    return ZANT_OK;
}

// add_bias, lib_elementWise_math.zig:22-45 (bias over the last dimension, in place).
int32_t zo_add_bias_f32(float* t, const usize* ts, usize tr, const float* bias, const usize* bs, usize br) {
    const usize n = prod(ts, tr);
    if (n == 0) return ZANT_E_EMPTY_TENSOR;
    if (br != 1) return ZANT_E_INPUT_TENSORS_WRONG_SHAPE;
    if (bs[0] == 0) return ZANT_E_EMPTY_TENSOR;
    const usize len = bs[0];
    if (len != ts[tr - 1]) return ZANT_E_INPUT_TENSOR_DIMENSION_MISMATCH;
    for (usize i = 0; i < n; i += len)
        for (usize j = 0; j < len; ++j) t[i + j] = t[i + j] + bias[j];
    return ZANT_OK;
}

// ---------------------------------------------------------------------------------------
// Shape ops
// ---------------------------------------------------------------------------------------

// Output shape of concatenate, lib_shape_math.zig:463-543 (rank promotion with leading ones).
int32_t zo_concat_output_shape(const usize* const* shapes, const usize* ranks, usize nt, int64_t axis,
                               usize* out, usize* out_rank) {
    if (nt == 0) return ZANT_E_EMPTY_TENSOR_LIST;
    usize mr = ranks[0];
    for (usize t = 0; t < nt; ++t) mr = std::max(mr, ranks[t]);
    int64_t ax = axis;
    if (ax < 0) ax += (int64_t)mr;
    if (ax < 0 || ax >= (int64_t)mr) return ZANT_E_AXIS_OUT_OF_BOUNDS;
    for (usize d = 0; d < mr; ++d) out[d] = 1;
    for (usize d = 0; d < ranks[0]; ++d) out[mr - ranks[0] + d] = shapes[0][d];
    usize sum = 0;
    for (usize t = 0; t < nt; ++t) {
        const usize off = mr - ranks[t];
        sum += ((usize)ax >= off) ? shapes[t][(usize)ax - off] : 1;
    }
    out[(usize)ax] = sum;
    *out_rank = mr;
    return ZANT_OK;
}

// get_concatenate_output_shape, lib_shape_math.zig:582-629 (the generator's shape helper:
// equal ranks required, shapes validated).
int32_t zo_get_concatenate_output_shape(const usize* const* shapes, const usize* ranks, usize nt,
                                        int64_t axis, usize* out) {
    if (nt == 0) return ZANT_E_EMPTY_TENSOR_LIST;
    const usize rank = ranks[0];
    int64_t ax = axis;
    if (ax < 0) ax += (int64_t)rank;
    if (ax < 0 || ax >= (int64_t)rank) return ZANT_E_AXIS_OUT_OF_BOUNDS;
    for (usize t = 0; t < nt; ++t) {
        if (ranks[t] != rank) return ZANT_E_MISMATCHED_RANK;
        for (usize d = 0; d < rank; ++d)
            if (d != (usize)ax && shapes[t][d] != shapes[0][d]) return ZANT_E_MISMATCHED_SHAPE;
    }
    for (usize d = 0; d < rank; ++d) {
        if (d == (usize)ax) {
            usize sum = 0;
            for (usize t = 0; t < nt; ++t) sum += shapes[t][d];
            out[d] = sum;
        } else {
            out[d] = shapes[0][d];
        }
    }
    return ZANT_OK;
}

// lean_concatenate, lib_shape_math.zig:307-445: per outer slice, copy each tensor's
// [concat_dim * slice_size] block in list order.  `esz` = element size in bytes.
int32_t zo_concatenate(usize esz, const void* const* ts, const usize* const* shapes, const usize* ranks,
                       usize nt, int64_t axis, void* y, const usize* ys, usize yr) {
    if (nt == 0) return ZANT_E_EMPTY_TENSOR_LIST;
    usize mr = ranks[0];
    for (usize t = 0; t < nt; ++t) mr = std::max(mr, ranks[t]);
    int64_t ax = axis;
    if (ax < 0) ax += (int64_t)mr;
    if (ax < 0 || ax >= (int64_t)mr) return ZANT_E_AXIS_OUT_OF_BOUNDS;
    if (yr != mr) return ZANT_E_MISMATCHED_RANK;
    std::vector<std::vector<usize>> sh(nt, std::vector<usize>(mr, 1));
    for (usize t = 0; t < nt; ++t)
        for (usize d = 0; d < ranks[t]; ++d) sh[t][mr - ranks[t] + d] = shapes[t][d];
    for (usize t = 0; t < nt; ++t)
        for (usize d = 0; d < mr; ++d)
            if (d != (usize)ax && sh[t][d] != sh[0][d]) return ZANT_E_MISMATCHED_SHAPE;
    usize num_slices = 1, slice = 1;
    for (usize d = 0; d < (usize)ax; ++d) num_slices *= ys[d];
    for (usize d = (usize)ax + 1; d < mr; ++d) slice *= ys[d];
    const usize ysz = prod(ys, yr);
    usize off = 0;
    for (usize s = 0; s < num_slices; ++s)
        for (usize t = 0; t < nt; ++t) {
            const usize cd = sh[t][(usize)ax], cp = cd * slice, src = s * cd * slice;
            if (src + cp > prod(sh[t].data(), mr)) return ZANT_E_INDEX_OUT_OF_BOUNDS;
            if (off + cp > ysz) return ZANT_E_INDEX_OUT_OF_BOUNDS;
            std::memcpy((char*)y + off * esz, (const char*)ts[t] + src * esz, cp * esz);
            off += cp;
        }
    return ZANT_OK;
}

// get_resize_output_shape, lib_shape_math.zig:78-104.
int32_t zo_resize_output_shape(const usize* xs, usize r, const float* scales, usize nsc,
                               const usize* sizes, usize nsz, usize* out) {
    if (!scales && !sizes) return ZANT_E_INVALID_INPUT;
    if (scales && sizes) return ZANT_E_INVALID_INPUT;
    if (scales) {
        if (nsc != r) return ZANT_E_INVALID_INPUT;
        for (usize i = 0; i < r; ++i) out[i] = (usize)std::floor((float)xs[i] * scales[i]);
    } else {
        if (nsz != r) return ZANT_E_INVALID_INPUT;
        for (usize i = 0; i < r; ++i) out[i] = sizes[i];
    }
    return ZANT_OK;
}

// resize + nearest_interpolation, lib_shape_math.zig:22-76, :106-161.
int32_t zo_resize(usize esz, const void* x, const usize* xs, usize r,
                  const char* mode, usize ml, const float* scales, usize nsc,
                  const usize* sizes, usize nsz, const char* cm, usize cml,
                  void* y, const usize* ys, usize yr) {
    std::vector<usize> os(r);
    int32_t st = zo_resize_output_shape(xs, r, scales, nsc, sizes, nsz, os.data());
    if (st != ZANT_OK) return st;
    if (!str_eq(mode, ml, "nearest")) {
        if (str_eq(mode, ml, "linear") || str_eq(mode, ml, "cubic")) return ZANT_E_UNSUPPORTED;
        return ZANT_E_UNSUPPORTED_MODE;
    }
    if (yr != r) return ZANT_E_OUTPUT_TENSOR_DIFFERENT_SIZE;
    for (usize i = 0; i < r; ++i) if (ys[i] != os[i]) return ZANT_E_OUTPUT_TENSOR_DIFFERENT_SIZE;
    std::vector<usize> istr(r), ostr(r), oi(r, 0);
    usize s = 1;
    for (usize i = r; i-- > 0;) { istr[i] = s; s *= xs[i]; }
    s = 1;
    for (usize i = r; i-- > 0;) { ostr[i] = s; s *= os[i]; }
    const usize total = s;
    if (total == 0) return ZANT_OK;
    const bool half = str_eq(cm, cml, "half_pixel"), align = str_eq(cm, cml, "align_corners");
    bool done = false;
    while (!done) {
        usize oidx = 0, iidx = 0;
        for (usize i = 0; i < r; ++i) {
            const float scale = (float)os[i] / (float)xs[i];
            float pos;
            if (half) pos = ((float)oi[i] + 0.5f) / scale - 0.5f;
            else if (align) pos = (float)oi[i] * (float)(xs[i] - 1) / (float)(os[i] - 1);
            else pos = (float)oi[i] / scale;
            const int32_t ii = (int32_t)std::roundf(pos);          // @round: half away from zero
            const int32_t cl = std::min(std::max(ii, 0), (int32_t)(xs[i] - 1));
            iidx += (usize)cl * istr[i];
            oidx += oi[i] * ostr[i];
        }
        std::memcpy((char*)y + oidx * esz, (const char*)x + iidx * esz, esz);
        done = true;
        for (usize i = 0; i < r; ++i) {
            const usize d = r - 1 - i;
            if (++oi[d] < os[d]) { done = false; break; }
            oi[d] = 0;
        }
    }
    return ZANT_OK;
}

// reshape_lean + reshape_lean_common, lib_shape_math.zig:1139-1209.
int32_t zo_reshape(usize esz, const void* x, const usize* xs, usize xr,
                   const usize* ns, usize nr, void* y, usize* ys_out) {
    const usize xsz = prod(xs, xr);
    std::vector<usize> ms(nr);
    long long neg = -1;
    usize known = 1;
    for (usize i = 0; i < nr; ++i) {
        if (ns[i] == 0) {
            if (i >= xr) return ZANT_E_INVALID_INPUT;
            ms[i] = xs[i]; known *= xs[i];
        } else if (ns[i] == std::numeric_limits<usize>::max()) {
            if (neg >= 0) return ZANT_E_INVALID_INPUT;
            neg = (long long)i; ms[i] = 1;
        } else {
            ms[i] = ns[i]; known *= ns[i];
        }
    }
    if (neg >= 0) {
        if (known == 0) return ZANT_E_INVALID_INPUT;
        if (xsz % known != 0) return ZANT_E_INPUT_ARRAY_WRONG_SIZE;
        ms[(usize)neg] = xsz / known;
    }
    if (prod(ms.data(), nr) != xsz) return ZANT_E_INPUT_ARRAY_WRONG_SIZE;
    for (usize i = 0; i < nr; ++i) ys_out[i] = ms[i];
    std::memcpy(y, x, xsz * esz);
    return ZANT_OK;
}

// ---------------------------------------------------------------------------------------
// Reductions
// ---------------------------------------------------------------------------------------

// lean_reduce_mean, lib_reduction_math.zig:87-268.  For each output element the reduced
// coordinates are visited with the LAST listed axis varying fastest (:239-257), summed
// sequentially in fp32, then divided once by the count.
int32_t zo_reduce_mean_f32(const float* x, const usize* xs, usize xr, float* y, const usize* ys, usize yr,
                           const int64_t* axes, usize na, int32_t keepdims, int32_t noop) {
    (void)keepdims;
    const usize xsz = prod(xs, xr), ysz = prod(ys, yr);
    if (!axes || na == 0) {
        if (noop) { std::memcpy(y, x, xsz * sizeof(float)); return ZANT_OK; }
        float sum = 0;
        for (usize i = 0; i < xsz; ++i) sum = sum + x[i];
        y[0] = sum / (float)xsz;
        return ZANT_OK;
    }
    std::vector<usize> ax(na);
    for (usize i = 0; i < na; ++i) {
        const int64_t a = axes[i] < 0 ? (int64_t)xr + axes[i] : axes[i];
        if (a < 0 || a >= (int64_t)xr) return ZANT_E_INVALID_AXES;
        ax[i] = (usize)a;
    }
    usize count = 1;
    for (usize a : ax) count *= xs[a];
    std::vector<usize> istr(xr);
    usize s = 1;
    for (usize i = xr; i-- > 0;) { istr[i] = s; s *= xs[i]; }
    std::vector<usize> rem_dims;
    for (usize d = 0; d < xr; ++d)
        if (std::find(ax.begin(), ax.end(), d) == ax.end()) rem_dims.push_back(d);
    std::vector<usize> ostr(rem_dims.size());
    s = 1;
    for (usize i = rem_dims.size(); i-- > 0;) { ostr[i] = s; s *= xs[rem_dims[i]]; }
    std::vector<usize> rsz(na), rstr(na);
    for (usize i = 0; i < na; ++i) { rsz[na - 1 - i] = xs[ax[i]]; rstr[na - 1 - i] = istr[ax[i]]; }
    for (usize o = 0; o < ysz; ++o) {
        usize rem = o, base = 0;
        for (usize i = 0; i < rem_dims.size(); ++i) {
            const usize cur = rem / ostr[i];
            rem %= ostr[i];
            base += cur * istr[rem_dims[i]];
        }
        float sum = 0;
        for (usize idx = 0; idx < count; ++idx) {
            usize t = idx, ti = base;
            for (usize d = 0; d < na; ++d) { ti += (t % rsz[d]) * rstr[d]; t /= rsz[d]; }
            sum = sum + x[ti];
        }
        y[o] = sum / (float)count;
    }
    return ZANT_OK;
}

// ---------------------------------------------------------------------------------------
// Quantized operators — PARITY UNPINNED against the reference (it has none); these are the
// ONNX operator definitions with the arithmetic order stated in include/zant_b200.h.
// ---------------------------------------------------------------------------------------

int32_t zo_quantize_linear(const float* x, usize n, float scale, int32_t zp, int32_t out_dtype, void* y) {
    if (out_dtype != ZANT_I8 && out_dtype != ZANT_U8) return ZANT_E_INPUT_ARRAY_WRONG_TYPE;
    for (usize i = 0; i < n; ++i) {
        const float v = x[i] / scale;
        store_q(y, i, out_dtype, sat_q((int32_t)rne_clamped(v) + zp, out_dtype));
    }
    return ZANT_OK;
}

int32_t zo_dequantize_linear(int32_t in_dtype, const void* q, usize n, float scale, int32_t zp, float* y) {
    for (usize i = 0; i < n; ++i) y[i] = (float)(load_q(q, i, in_dtype) - zp) * scale;
    return ZANT_OK;
}

// ONNX pad/stride resolution for QLinearConv (ONNX semantics: explicit pads unless auto_pad).
int32_t zo_qconv_geometry(const usize* xs, const usize* ws, const usize* stride, usize ns,
                          const usize* pads, usize np, const usize* dil, usize nd, int32_t auto_pad,
                          usize geom[10] /* sh sw dh dw pt pl pb pr OH OW */) {
    const usize H = xs[2], W = xs[3], KH = ws[2], KW = ws[3];
    const usize sh = ns > 0 ? stride[0] : 1, sw = ns > 1 ? stride[1] : sh;
    const usize dh = nd > 0 ? dil[0] : 1, dw = nd > 1 ? dil[1] : dh;
    if (sh == 0 || sw == 0 || KH == 0 || KW == 0 || dh == 0 || dw == 0) return ZANT_E_INVALID_DIMENSIONS;
    const usize dkh = (KH - 1) * dh + 1, dkw = (KW - 1) * dw + 1;
    usize pt = 0, pl = 0, pb = 0, pr = 0;
    if (auto_pad == ZANT_PAD_NOTSET) {
        if (np >= 4) { pt = pads[0]; pl = pads[1]; pb = pads[2]; pr = pads[3]; }
    } else if (auto_pad == ZANT_PAD_VALID) {
    } else if (auto_pad == ZANT_PAD_SAME_UPPER || auto_pad == ZANT_PAD_SAME_LOWER) {
        const usize oh = ceil_div(H, sh), ow = ceil_div(W, sw);
        const long long th = std::max<long long>((long long)((oh - 1) * sh + dkh) - (long long)H, 0);
        const long long tw = std::max<long long>((long long)((ow - 1) * sw + dkw) - (long long)W, 0);
        if (auto_pad == ZANT_PAD_SAME_UPPER) { pt = th / 2; pb = th - pt; pl = tw / 2; pr = tw - pl; }
        else { pb = th / 2; pt = th - pb; pr = tw / 2; pl = tw - pr; }
    } else {
        return ZANT_E_INVALID_PADDING;
    }
    if (H + pt + pb < dkh || W + pl + pr < dkw) return ZANT_E_INVALID_DIMENSIONS;
    geom[0] = sh; geom[1] = sw; geom[2] = dh; geom[3] = dw;
    geom[4] = pt; geom[5] = pl; geom[6] = pb; geom[7] = pr;
    geom[8] = (H + pt + pb - dkh) / sh + 1;
    geom[9] = (W + pl + pr - dkw) / sw + 1;
    return ZANT_OK;
}

int32_t zo_qlinearconv(int32_t x_dtype, const void* x, const usize* xs, usize xr, float x_scale, int32_t x_zp,
                       const int8_t* w, const usize* ws, usize wr,
                       const float* w_scale, const int32_t* w_zp, usize nws,
                       float y_scale, int32_t y_zp, const int32_t* bias, usize bias_len,
                       int32_t y_dtype, void* y, const usize* ys, usize yr,
                       const usize* stride, usize ns, const usize* pads, usize np,
                       const usize* dil, usize nd, usize group, int32_t auto_pad, int32_t act) {
    if (xr != 4 || wr != 4 || yr != 4) return ZANT_E_INVALID_DIMENSIONS;
    if (x_dtype != ZANT_I8 && x_dtype != ZANT_U8) return ZANT_E_INPUT_ARRAY_WRONG_TYPE;
    if (y_dtype != ZANT_I8 && y_dtype != ZANT_U8) return ZANT_E_INPUT_ARRAY_WRONG_TYPE;
    const usize G = group == 0 ? 1 : group;
    const usize N = xs[0], C = xs[1], H = xs[2], W = xs[3], M = ws[0], Cg = ws[1], KH = ws[2], KW = ws[3];
    if (C % G != 0 || M % G != 0 || Cg != C / G) return ZANT_E_INVALID_DIMENSIONS;
    if (nws != 1 && nws != M) return ZANT_E_INPUT_TENSORS_WRONG_SHAPE;
    if (bias && bias_len != M) return ZANT_E_INPUT_TENSORS_WRONG_SHAPE;
    usize g[10];
    int32_t st = zo_qconv_geometry(xs, ws, stride, ns, pads, np, dil, nd, auto_pad, g);
    if (st != ZANT_OK) return st;
    const usize sh = g[0], sw = g[1], dh = g[2], dw = g[3], pt = g[4], pl = g[5], OH = g[8], OW = g[9];
    if (ys[0] != N || ys[1] != M || ys[2] != OH || ys[3] != OW) return ZANT_E_INVALID_DIMENSIONS;
    const usize Mg = M / G;
    for (usize n = 0; n < N; ++n)
        for (usize m = 0; m < M; ++m) {
            const usize grp = m / Mg;
            const int32_t wz = w_zp ? w_zp[nws == 1 ? 0 : m] : 0;
            const float ws_m = w_scale[nws == 1 ? 0 : m];
            const float xw = x_scale * ws_m;
            const float Mm = xw / y_scale;
            for (usize oh = 0; oh < OH; ++oh)
                for (usize ow = 0; ow < OW; ++ow) {
                    int32_t acc = 0;
                    for (usize c = 0; c < Cg; ++c)
                        for (usize kh = 0; kh < KH; ++kh) {
                            const long long ih = (long long)(oh * sh + kh * dh) - (long long)pt;
                            if (ih < 0 || ih >= (long long)H) continue;
                            for (usize kw = 0; kw < KW; ++kw) {
                                const long long iw = (long long)(ow * sw + kw * dw) - (long long)pl;
                                if (iw < 0 || iw >= (long long)W) continue;
                                const int32_t xv = load_q(x, ((n * C + grp * Cg + c) * H + (usize)ih) * W + (usize)iw, x_dtype) - x_zp;
                                const int32_t wv = (int32_t)w[((m * Cg + c) * KH + kh) * KW + kw] - wz;
                                acc += xv * wv;
                            }
                        }
                    if (bias) acc += bias[m];
                    store_q(y, ((n * M + m) * OH + oh) * OW + ow, y_dtype, requant(acc, Mm, y_zp, y_dtype, act, y_scale));
                }
        }
    return ZANT_OK;
}

int32_t zo_qlinearmatmul(int32_t a_dtype, const void* a, const usize* as, usize ar, float a_scale, int32_t a_zp,
                         const int8_t* b, const usize* bs, usize br,
                         const float* b_scale, const int32_t* b_zp, usize nbs,
                         float y_scale, int32_t y_zp, const int32_t* bias, usize bias_len,
                         int32_t y_dtype, void* y, const usize* ys, usize yr, int32_t act) {
    if (ar != 2 || br != 2 || yr != 2) return ZANT_E_INPUT_TENSORS_WRONG_SHAPE;
    if (a_dtype != ZANT_I8 && a_dtype != ZANT_U8) return ZANT_E_INPUT_ARRAY_WRONG_TYPE;
    const usize M = as[0], K = as[1], N = bs[1];
    if (bs[0] != K) return ZANT_E_INPUT_TENSORS_WRONG_SHAPE;
    if (M * N == 0 || K == 0) return ZANT_E_INPUT_TENSORS_WRONG_SHAPE;
    if (ys[0] != M || ys[1] != N) return ZANT_E_OUTPUT_TENSOR_DIFFERENT_SIZE;
    if (nbs != 1 && nbs != N) return ZANT_E_INPUT_TENSORS_WRONG_SHAPE;
    if (bias && bias_len != N) return ZANT_E_INPUT_TENSORS_WRONG_SHAPE;
    for (usize i = 0; i < M; ++i)
        for (usize j = 0; j < N; ++j) {
            const int32_t bz = b_zp ? b_zp[nbs == 1 ? 0 : j] : 0;
            int32_t acc = 0;
            for (usize k = 0; k < K; ++k)
                acc += (load_q(a, i * K + k, a_dtype) - a_zp) * ((int32_t)b[k * N + j] - bz);
            if (bias) acc += bias[j];
            const float xw = a_scale * b_scale[nbs == 1 ? 0 : j];
            const float Mm = xw / y_scale;
            if (y_dtype == ZANT_I32) ((int32_t*)y)[i * N + j] = acc;
            else store_q(y, i * N + j, y_dtype, requant(acc, Mm, y_zp, y_dtype, act, y_scale));
        }
    return ZANT_OK;
}

int32_t zo_qlinearadd(int32_t dtype, const void* a, float a_s, int32_t a_zp,
                      const void* b, float b_s, int32_t b_zp,
                      float y_s, int32_t y_zp, void* y, usize n, int32_t act) {
    for (usize i = 0; i < n; ++i) {
        const float fa = (float)(load_q(a, i, dtype) - a_zp) * a_s;
        const float fb = (float)(load_q(b, i, dtype) - b_zp) * b_s;
        const float sum = fa + fb;
        const float v = sum / y_s;
        int32_t t = sat_q((int32_t)rne_clamped(v) + y_zp, dtype);
        if (act == ZANT_QACT_RELU || act == ZANT_QACT_RELU6) t = std::max(t, sat_q(y_zp, dtype));
        if (act == ZANT_QACT_RELU6) t = std::min(t, sat_q((int32_t)rne_clamped(6.0f / y_s) + y_zp, dtype));
        store_q(y, i, dtype, t);
    }
    return ZANT_OK;
}

int32_t zo_qlinear_global_avgpool(int32_t dtype, const void* x, const usize* xs, usize xr,
                                  float x_s, int32_t x_zp, float y_s, int32_t y_zp, void* y) {
    if (xr != 4) return ZANT_E_INVALID_DIMENSIONS;
    const usize NC = xs[0] * xs[1], HW = xs[2] * xs[3];
    for (usize i = 0; i < NC; ++i) {
        int32_t sum = 0;
        for (usize j = 0; j < HW; ++j) sum += load_q(x, i * HW + j, dtype) - x_zp;
        const float f = (float)sum * x_s;
        const float mean = f / (float)HW;
        const float v = mean / y_s;
        store_q(y, i, dtype, sat_q((int32_t)rne_clamped(v) + y_zp, dtype));
    }
    return ZANT_OK;
}

int32_t zo_lut_q8(const void* x, const uint8_t lut[256], void* y, usize n) {
    for (usize i = 0; i < n; ++i) ((uint8_t*)y)[i] = lut[((const uint8_t*)x)[i]];
    return ZANT_OK;
}

// Host-side table for LeakyReLU between two QDQ tensors:
// lut[code] = sat(rne(leaky(float(q - zp_in) * s_in) / s_out) + zp_out), q the signed or
// unsigned reading of `code` according to dtype.
int32_t zo_build_leaky_lut(int32_t dtype, float s_in, int32_t zp_in, float slope,
                           float s_out, int32_t zp_out, uint8_t lut[256]) {
    for (int code = 0; code < 256; ++code) {
        const int32_t q = dtype == ZANT_U8 ? code : (int32_t)(int8_t)(uint8_t)code;
        const float f = (float)(q - zp_in) * s_in;
        const float a = (f <= 0) ? slope * f : f;
        const float v = a / s_out;
        lut[code] = (uint8_t)sat_q((int32_t)rne_clamped(v) + zp_out, dtype);
    }
    return ZANT_OK;
}

}  // extern "C"
